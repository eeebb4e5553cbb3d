// placeholder until the tcgen05 decode kernel lands
#include "internal.cuh"
namespace gs {
bool decode_umma_supported(const DecodeProblem &, const char **why) { *why = "not built"; return false; }
int launch_decode_umma(const DecodeProblem &, cudaStream_t) { return fail_invalid("tcgen05 decode not built"); }
}
