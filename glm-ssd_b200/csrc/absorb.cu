// The two per-head matrix products around the attention call of Engine::mla, fused with it into one entry point:
//   absorb   qabs[t][h] = k_b[h] . q[t][h]      (crates/engine/src/forward.rs:900, mm_heads :716-733; [512 x 256] per head)
//   attend   olat[t][h] = attention of qabs over the latent cache (forward.rs:902-906)
//   expand   ov[t][h]   = v_b[h] . olat[t][h]   (forward.rs:907; [256 x 512] per head)
// For a decode or MTP-verify step (T <= 8 tokens) both products are matrix-vector work bound by reading the weights
// once from HBM (16.8 MB each for 64 heads in f16 - as many bytes as a 16K-row cache), so they run as bandwidth
// kernels on the CUDA cores, not on the tensor cores.  What the fusion buys is launches and overlap: four kernels in a
// programmatic-dependent-launch chain (the reference issues 2 T + 2), the attention kernel setting itself up and
// asking its first cache tiles into L2 while the absorb kernel runs, and the expand kernel fetching its weights - which
// depend on nothing - before it waits for the merged attention output.
//
// Weights are taken as f16 [H][rows][K] row-major.  The engine's quantised weight formats (crates/quants) stay
// outside this library.
#include <string.h>

#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {
namespace {

constexpr int HG_WARPS = 8;      // warps per CTA
constexpr int HG_ROWS_W = 4;     // output rows per warp
constexpr int HG_ROWS = HG_WARPS * HG_ROWS_W;
constexpr int HG_TMAX = 8;       // tokens per call

// y[t][h][row] = sum_k W[h][row][k] * x[t][h][k].  grid (ROWS / 32, H); K = 256 * KC.  A lane owns the 8 consecutive
// weights at (c * 32 + lane) * 8 of every row (16-byte loads, a warp reads 512 contiguous bytes); x lies in shared
// memory as f32.  DEP: the kernel is launched behind the producer of x with programmatic dependent launch - the weight
// rows are requested first, then the wait, then x.
template <int KC, typename XT, typename YT, bool DEP>
__global__ void __launch_bounds__(HG_WARPS * 32) k_head_gemv(const __half *__restrict__ W, const XT *__restrict__ x, YT *__restrict__ y,
                                                             int T, int H, int rows) {
    constexpr int K = 256 * KC;
    __shared__ __align__(16) float sx[HG_TMAX][K];
    const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * HG_ROWS + warp * HG_ROWS_W;
    if (!DEP) sm100::griddep_launch_dependents();  // the kernel behind this one may begin its own set-up
    uint4 w[HG_ROWS_W][KC];
#pragma unroll
    for (int r = 0; r < HG_ROWS_W; r++)
#pragma unroll
        for (int c = 0; c < KC; c++) {
            const int row = min(row0 + r, rows - 1);
            w[r][c] = __ldg(reinterpret_cast<const uint4 *>(W + ((int64_t) h * rows + row) * K) + c * 32 + lane);
        }
    if (DEP) {
        sm100::griddep_wait();
        sm100::griddep_launch_dependents();
    }
    for (int i = threadIdx.x; i < T * K; i += blockDim.x) {
        const int t = i / K, k = i - t * K;
        sx[t][k] = (float) x[((int64_t) t * H + h) * K + k];
    }
    __syncthreads();
    for (int t = 0; t < T; t++) {
        float acc[HG_ROWS_W];
#pragma unroll
        for (int r = 0; r < HG_ROWS_W; r++) acc[r] = 0.f;
#pragma unroll
        for (int c = 0; c < KC; c++) {
            const float4 x0 = *reinterpret_cast<const float4 *>(&sx[t][(c * 32 + lane) * 8]);
            const float4 x1 = *reinterpret_cast<const float4 *>(&sx[t][(c * 32 + lane) * 8 + 4]);
#pragma unroll
            for (int r = 0; r < HG_ROWS_W; r++) {
                const __half2 *hw = reinterpret_cast<const __half2 *>(&w[r][c]);
                const float2 a = __half22float2(hw[0]), b = __half22float2(hw[1]), c2 = __half22float2(hw[2]), d = __half22float2(hw[3]);
                acc[r] = fmaf(a.x, x0.x, fmaf(a.y, x0.y, fmaf(b.x, x0.z, fmaf(b.y, x0.w, acc[r]))));
                acc[r] = fmaf(c2.x, x1.x, fmaf(c2.y, x1.y, fmaf(d.x, x1.z, fmaf(d.y, x1.w, acc[r]))));
            }
        }
#pragma unroll
        for (int r = 0; r < HG_ROWS_W; r++) {
            const float v = warp_sum(acc[r]);
            if (lane == r && row0 + r < rows) y[((int64_t) t * H + h) * rows + row0 + r] = (YT) v;
        }
    }
}

template <int KC, typename XT, typename YT, bool DEP>
int launch_head_gemv(const __half *W, const XT *x, YT *y, int T, int H, int rows, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((rows + HG_ROWS - 1) / HG_ROWS, H);
    cfg.blockDim = dim3(HG_WARPS * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = DEP ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GS_TRY(cudaLaunchKernelEx(&cfg, k_head_gemv<KC, XT, YT, DEP>, W, x, y, T, H, rows));
    return 0;
}

int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

}  // namespace
}  // namespace gs

using namespace gs;

GS_EXPORT int64_t gs_mla_fused_workspace_bytes(int T, int H) {
    if (T <= 0 || H <= 0) return 0;
    const int64_t dec = gs_mla_decode_workspace_bytes(1, T, H, 512);
    return align256(dec) + align256((int64_t) T * H * 512 * 2) + align256((int64_t) T * H * 512 * 4);
}

GS_EXPORT int gs_mla_decode_fused(const gs_mla_fused_args *a, void *stream) {
    if (!a) return fail_invalid("gs_mla_decode_fused: args == NULL");
    if (a->T <= 0 || a->H <= 0) return a->T < 0 || a->H < 0 ? fail_invalid("gs_mla_decode_fused: negative size") : 0;
    if (a->T > HG_TMAX) return fail_invalid("gs_mla_decode_fused: at most 8 query tokens (decode and MTP verify); prefill chunks use a GEMM");
    if (a->d_q != 256 || a->d_lat != 512 || a->d_out != 256)
        return fail_invalid("gs_mla_decode_fused: this build takes d_q = 256, d_lat = 512, d_out = 256 (the engine's MLA head sizes)");
    if (!a->q || !a->k_b || !a->v_b || !a->cache || !a->seq_len || !a->ov) return fail_invalid("gs_mla_decode_fused: null pointer");
    if ((reinterpret_cast<uintptr_t>(a->k_b) | reinterpret_cast<uintptr_t>(a->v_b)) & 15)
        return fail_invalid("gs_mla_decode_fused: k_b and v_b must be 16-byte aligned");
    const int64_t need = gs_mla_fused_workspace_bytes(a->T, a->H);
    if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
        set_error("gs_mla_decode_fused: workspace of %lld bytes needed (256-byte aligned), %lld given", (long long) need,
                  (long long) a->workspace_bytes);
        return (int) cudaErrorInvalidValue;
    }
    cudaStream_t st = (cudaStream_t) stream;
    char *ws = (char *) a->workspace;
    const int64_t dec = align256(gs_mla_decode_workspace_bytes(1, a->T, a->H, 512));
    __half *qabs = (__half *) (ws + dec);
    float *olat = (float *) (ws + dec + align256((int64_t) a->T * a->H * 512 * 2));
    // absorb: qabs f16 [T][H][512] = k_b[h] . q[t][h]
    if (int e = launch_head_gemv<1, float, __half, false>((const __half *) a->k_b, (const float *) a->q, qabs, a->T, a->H, 512, st)) return e;
    // attend over the latent rows (V = the same 512 columns), merged output f32 [T][H][512]
    gs_mla_decode_args d;
    memset(&d, 0, sizeof(d));
    d.q = qabs;
    d.cache = a->cache;
    d.cache_rows = a->cache_rows;
    d.seq_lens = a->seq_len;
    d.page_rows = 64;
    d.scale = a->scale;
    d.tail_causal = 1;
    d.o = olat;
    d.workspace = ws;
    d.workspace_bytes = dec;
    d.n_seq = 1;
    d.T = a->T;
    d.H = a->H;
    d.d_qk = 512;
    d.d_v = 512;
    if (int e = gs_mla_decode(&d, stream)) return e;
    // expand: ov f32 [T][H][256] = v_b[h] . olat[t][h]; its weights are fetched before it waits for the merge
    return launch_head_gemv<2, float, float, true>((const __half *) a->v_b, olat, a->ov, a->T, a->H, 256, st);
}
