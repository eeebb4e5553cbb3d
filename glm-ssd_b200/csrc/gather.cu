// Gather of the rows a position list names into contiguous rows, for the tensor-core path of the
// reference-compatible entry point.  The reference's kernel walks `sel` inside its attention loop
// (crates/cuda/kernels/ops.cu:455-480); here the (at most a few thousand) rows of every query token are
// copied once, 16 bytes per thread, and the dense tcgen05 kernel then streams them with TMA.
#include "internal.cuh"

namespace gs {
namespace {

// grid (row blocks + query blocks, T), 256 threads.  A row block copies 4 rows of one token: 64 threads per
// row of R = 512 halves.  Block (0, t) also leaves the token's length and base row, once per head group; the
// query blocks convert the f32 queries.
__global__ void __launch_bounds__(256) k_gather_rows(const __half *__restrict__ C, const __half *__restrict__ C_scales,
                                                     const int *__restrict__ sel, int sel_stride,
                                                     const int *__restrict__ cnt, int max_rows, int row_blocks, int n_groups,
                                                     __half *__restrict__ rows_out, int32_t *lens_out, int32_t *base_out,
                                                     const float *__restrict__ q, __half *__restrict__ q16, int64_t q_elems) {
#if __CUDA_ARCH__ >= 900
    // the attention kernel behind this one may set itself up right away; its dependency wait covers these writes
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
    const int t = blockIdx.y;
    if ((int) blockIdx.x >= row_blocks) {  // query conversion, spread over the remaining blocks of every token row
        const int64_t nb = (int64_t) (gridDim.x - row_blocks) * gridDim.y;
        const int64_t b = (int64_t) (blockIdx.x - row_blocks) * gridDim.y + t;
        for (int64_t i = (b * 256 + threadIdx.x) * 2; i < q_elems; i += nb * 256 * 2) {
            if (i + 1 < q_elems) *reinterpret_cast<__half2 *>(q16 + i) = __floats2half2_rn(q[i], q[i + 1]);
            else q16[i] = __float2half_rn(q[i]);
        }
        return;
    }
    const int n = min(min(max(cnt[t], 0), sel_stride), max_rows);
    // every head group of the token is its own dense "sequence" over the same gathered rows
    if (blockIdx.x == 0 && (int) threadIdx.x < n_groups) {
        lens_out[t * n_groups + threadIdx.x] = n;
        base_out[t * n_groups + threadIdx.x] = t * max_rows;
    }
    const int i = blockIdx.x * 4 + (threadIdx.x >> 6), c = threadIdx.x & 63;
    if (i >= n) return;
    const int64_t src = sel[(int64_t) t * sel_stride + i];
    uint4 *dst = reinterpret_cast<uint4 *>(rows_out + ((int64_t) t * max_rows + i) * 512) + c;
    if (!C_scales) {
        *dst = __ldg(reinterpret_cast<const uint4 *>(C + src * 512) + c);
    } else {
        // Q8 cache (ops.cu:427): int8 rows + one f16 scale per 32 values; the row is rebuilt as half_rn(scale * q),
        // the values the reference's Q8 branch attends over (ops.cu:461-477).  8 values per thread.
        const int8_t *row8 = reinterpret_cast<const int8_t *>(C) + src * 512;
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(row8) + c);
        const float sc = __half2float(C_scales[src * 16 + (c >> 2)]);
        auto pack = [sc](uint32_t w, uint32_t &h01, uint32_t &h23) {
            const __half2 a = __floats2half2_rn(sc * (float) (int8_t) (w), sc * (float) (int8_t) (w >> 8));
            const __half2 b = __floats2half2_rn(sc * (float) (int8_t) (w >> 16), sc * (float) (int8_t) (w >> 24));
            h01 = *reinterpret_cast<const uint32_t *>(&a);
            h23 = *reinterpret_cast<const uint32_t *>(&b);
        };
        uint4 out;
        pack(raw.x, out.x, out.y);
        pack(raw.y, out.z, out.w);
        *dst = out;
    }
}

}  // namespace

int launch_gather_rows(const __half *C, const __half *C_scales, const int *sel, int sel_stride, const int *cnt, int T, int max_rows, int R, int n_groups,
                       __half *rows_out, int32_t *lens_out, int32_t *base_out, const float *q, __half *q16, int64_t q_elems,
                       cudaStream_t st) {
    if (R != 512) return fail_invalid("gather: rows of 512 values only");
    const int rows = sel_stride < max_rows ? sel_stride : max_rows;
    const int row_blocks = (rows + 3) / 4 > 0 ? (rows + 3) / 4 : 1;
    const int q_blocks = 8;
    k_gather_rows<<<dim3(row_blocks + q_blocks, T), 256, 0, st>>>(C, C_scales, sel, sel_stride, cnt, max_rows, row_blocks, n_groups, rows_out,
                                                                 lens_out, base_out, q, q16, q_elems);
    GS_TRY(cudaGetLastError());
    return 0;
}

}  // namespace gs
