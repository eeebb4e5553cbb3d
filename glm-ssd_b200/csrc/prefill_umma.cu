// placeholder until the tcgen05 prefill kernel lands
#include "internal.cuh"
namespace gs {
bool prefill_umma_supported(int, int, int, int, const char **why) { *why = "not built"; return false; }
int launch_prefill_umma(const __half *, const __half *, const __half *, void *, int, int, int, int, int, float, cudaStream_t) { return fail_invalid("tcgen05 prefill not built"); }
}
