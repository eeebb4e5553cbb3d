// DSA k-pool indexer: the kernels that produce the attended position lists (sel, cnt) the attention call
// consumes once the context is longer than top_k positions (crates/engine/src/forward.rs:864-895).  Same entry
// points and arguments as the reference (crates/cuda/kernels/ops.cu:619-791, Rust declarations
// crates/cuda/src/lib.rs:101-113):
//
//   gs_idx_pool    pooled indexer key of every pool of `kpool` positions that completes inside the chunk, plus
//                  the hand-over of the trailing incomplete pool's raw rows to the ring buffers - one launch
//                  (the reference needs two: the pool that straddles the chunk start reads the ring slots the
//                  hand-over then rewrites, so here the same thread does both for its column, in that order);
//   gs_idx_score   score[t][p] = sum_h w[t][h] * relu(scale * q[t][h] . P[p]) over the complete pools;
//   gs_idx_select  exact top-k of the scores (radix select on the order-preserving integer image, as the
//                  reference) and the position list built from it.
//
// One difference in gs_idx_select, on purpose: the reference fills the list in the order its threads reach an
// atomic counter, so the order of the pools inside `sel` - and, among pools whose score equals the k-th largest,
// which of them are taken - changes from run to run there.  Here the list is deterministic: pools in ascending
// index, ties to the lowest indices.  The set of selected pools is the reference's whenever the k-th largest
// score is unique; `cnt` is always the same.
#include "internal.cuh"

namespace gs {
namespace {

// ---- pooling ------------------------------------------------------------------------------------------------
__device__ __forceinline__ const float *idx_row(const float *chunk, const float *ring, int64_t pos, int p0, int Dk, int kpool) {
    return pos >= p0 ? chunk + (pos - p0) * Dk : ring + (pos % kpool) * Dk;
}

// grid (column blocks, max(1, completing pools)); thread = one column of one pool.  Only the first completing pool
// (the one holding position p0) can reach into the rings; its threads also hand the trailing rows over afterwards.
__global__ void __launch_bounds__(128) k_idx_pool(const float *__restrict__ kc, const float *__restrict__ gc, float *rk, float *rg,
                                                  const float *__restrict__ ape, float *__restrict__ P, int p0, int T, int Dk, int kpool) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= Dk) return;
    const int end = p0 + T;
    const int jf = p0 / kpool, jl = end / kpool;
    const int64_t j = (int64_t) jf + blockIdx.y;
    if (j < jl) {
        float mx = -INFINITY;
        for (int m = 0; m < kpool; m++) mx = fmaxf(mx, idx_row(gc, rg, j * kpool + m, p0, Dk, kpool)[c] + ape[m * Dk + c]);
        float sum = 0.f, acc = 0.f;
        for (int m = 0; m < kpool; m++) {
            const int64_t pos = j * kpool + m;
            const float e = expf(idx_row(gc, rg, pos, p0, Dk, kpool)[c] + ape[m * Dk + c] - mx);
            sum += e;
            acc = fmaf(e, idx_row(kc, rk, pos, p0, Dk, kpool)[c], acc);
        }
        P[j * Dk + c] = acc / sum;
    }
    if (blockIdx.y == 0) {
        const int first = max(p0, jl * kpool);
        for (int64_t pos = first; pos < end; pos++) {
            rk[(pos % kpool) * Dk + c] = kc[(pos - p0) * Dk + c];
            rg[(pos % kpool) * Dk + c] = gc[(pos - p0) * Dk + c];
        }
    }
}

// ---- scores -------------------------------------------------------------------------------------------------
// Block = 64 pools x 4 column parts (thread (pool, part) owns columns part, part + 4, part + 8, ... of its pool's key
// in registers); the query's heads sit in shared memory and are read as broadcasts.  Per (pool, head): 32 FMAs per
// thread and two shuffles to join the four parts.
constexpr int SC_POOLS = 64, SC_PARTS = 4, SC_MAXI = 32;  // Dk <= SC_PARTS * SC_MAXI = 128
__global__ void __launch_bounds__(SC_POOLS *SC_PARTS) k_idx_score(const float *__restrict__ q, const float *__restrict__ w,
                                                                  const float *__restrict__ P, float *__restrict__ score,
                                                                  int64_t score_stride, int pos0, int kpool, int Hq, int Dk, float scale) {
    const int t = blockIdx.y;
    const int n_pool = (pos0 + t + 1) / kpool;
    const int p_base = blockIdx.x * SC_POOLS;
    if (p_base >= n_pool) return;
    extern __shared__ float sq[];  // [Hq][Dk] then w [Hq]
    float *sw = sq + Hq * Dk;
    const float *qt = q + (int64_t) t * Hq * Dk;
    for (int i = threadIdx.x; i < Hq * Dk; i += blockDim.x) sq[i] = qt[i];
    for (int i = threadIdx.x; i < Hq; i += blockDim.x) sw[i] = w[(int64_t) t * Hq + i];
    __syncthreads();
    const int part = threadIdx.x & (SC_PARTS - 1);
    const int p = p_base + (threadIdx.x >> 2);
    const int pc = min(p, n_pool - 1);  // lanes past the end work on a valid row and drop the result
    float kreg[SC_MAXI];
    const float *pk = P + (int64_t) pc * Dk;
#pragma unroll
    for (int i = 0; i < SC_MAXI; i++) kreg[i] = (i * SC_PARTS + part) < Dk ? pk[i * SC_PARTS + part] : 0.f;
    float total = 0.f;
    for (int h = 0; h < Hq; h++) {
        const float *qh = sq + h * Dk;
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < SC_MAXI; i++)
            if (i * SC_PARTS < Dk) d = fmaf((i * SC_PARTS + part) < Dk ? qh[i * SC_PARTS + part] : 0.f, kreg[i], d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        total = fmaf(sw[h], fmaxf(d * scale, 0.f), total);
    }
    if (part == 0 && p < n_pool) score[(int64_t) t * score_stride + p] = total;
}

// ---- selection ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2ord(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int SEL_NT = 1024;
// One block per query.  Radix select, 8 bits per pass from the top: after a pass `prefix` holds the leading bits of
// the k-th largest value and `need` how many values are still to be taken among those that share the prefix.  The
// 256 bins are scanned from the top by one warp (8 bins per lane, suffix sums by shuffles).  Then one ordered pass
// over the pools writes the list: block-wide exclusive counts of "greater" and "equal" flags give every taken pool
// its slot, so the pools appear in ascending index and ties go to the lowest indices.
__global__ void __launch_bounds__(SEL_NT) k_idx_select(const float *__restrict__ score, int64_t score_stride, int pos0, int kpool,
                                                       int top_k, int *__restrict__ sel, int sel_stride, int *__restrict__ cnt) {
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = pos0 + t;
    const int n_pool = (pos + 1) / kpool;
    int *out = sel + (int64_t) t * sel_stride;
    if (n_pool <= top_k) {  // everything is attended (ops.cu:728-731)
        for (int i = tid; i <= pos; i += SEL_NT) out[i] = i;
        if (tid == 0) cnt[t] = pos + 1;
        return;
    }
    const float *sc = score + (int64_t) t * score_stride;
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_need;
    __shared__ uint32_t w_gt[SEL_NT / 32], w_eq[SEL_NT / 32];
    __shared__ uint32_t run_gt, run_eq;
    uint32_t prefix = 0, mask = 0, need = (uint32_t) top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int p = tid; p < n_pool; p += SEL_NT) {
            const uint32_t u = f2ord(sc[p]);
            if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1u);
        }
        __syncthreads();
        if (warp == 0) {
            // lane L owns bins 255 - 8L .. 248 - 8L (descending); above[L] = count in all bins above lane L's
            uint32_t mine[8], tot = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                mine[i] = hist[255 - (lane * 8 + i)];
                tot += mine[i];
            }
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            uint32_t acc = incl - tot;  // values in bins above this lane's
            // the digit: the highest bin at which the running count reaches `need`
            int found = -1;
            uint32_t acc_at = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (found < 0 && acc + mine[i] >= need) {
                    found = 255 - (lane * 8 + i);
                    acc_at = acc;
                }
                acc += mine[i];
            }
            const uint32_t has = __ballot_sync(0xffffffffu, found >= 0);
            const int src = __ffs(has) - 1;  // the first lane (highest bins) that reached it; always exists: need <= count
            const int d = __shfl_sync(0xffffffffu, found, src < 0 ? 0 : src);
            const uint32_t a = __shfl_sync(0xffffffffu, acc_at, src < 0 ? 0 : src);
            if (lane == 0) {
                s_prefix = prefix | ((uint32_t) (d < 0 ? 0 : d) << shift);
                s_need = need - a;
            }
        }
        __syncthreads();
        prefix = s_prefix;
        need = s_need;
        mask |= 255u << shift;
    }
    const uint32_t U = prefix, need_eq = need;  // take every value above U and the first need_eq values equal to it
    if (tid == 0) run_gt = run_eq = 0;
    __syncthreads();
    for (int p0 = 0; p0 < n_pool; p0 += SEL_NT) {
        const int p = p0 + tid;
        const uint32_t u = p < n_pool ? f2ord(sc[p]) : 0u;
        const bool gt = p < n_pool && u > U, eq = p < n_pool && u == U;
        const uint32_t b_gt = __ballot_sync(0xffffffffu, gt), b_eq = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) {
            w_gt[warp] = __popc(b_gt);
            w_eq[warp] = __popc(b_eq);
        }
        __syncthreads();
        uint32_t before_gt = run_gt, before_eq = run_eq;
        for (int w = 0; w < warp; w++) {
            before_gt += w_gt[w];
            before_eq += w_eq[w];
        }
        const uint32_t lt_mask = (1u << lane) - 1u;
        const uint32_t my_eq = before_eq + __popc(b_eq & lt_mask);  // equal values in front of this one
        const uint32_t my_gt = before_gt + __popc(b_gt & lt_mask);
        const bool take = gt || (eq && my_eq < need_eq);
        if (take) {
            const uint32_t slot = my_gt + min(my_eq, need_eq);  // taken pools in front of this one
            for (int m = 0; m < kpool; m++) out[(int64_t) slot * kpool + m] = p * kpool + m;
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t g = 0, e = 0;
            for (int w = 0; w < SEL_NT / 32; w++) {
                g += w_gt[w];
                e += w_eq[w];
            }
            run_gt += g;
            run_eq += e;
        }
        __syncthreads();
    }
    const int base = top_k * kpool, tail0 = n_pool * kpool;
    for (int i = tid; tail0 + i <= pos; i += SEL_NT) out[base + i] = tail0 + i;
    if (tid == 0) cnt[t] = base + (pos + 1 - tail0);
}

}  // namespace
}  // namespace gs

using namespace gs;

GS_EXPORT int gs_idx_pool(const float *kc, const float *gc, float *rk, float *rg, const float *ape, float *P, int p0, int T,
                          int Dk, int kpool, void *stream) {
    if (T <= 0) return 0;
    if (p0 < 0 || Dk <= 0 || kpool <= 0) return fail_invalid("gs_idx_pool: need p0 >= 0, Dk > 0, kpool > 0");
    if (!kc || !gc || !rk || !rg || !ape || !P) return fail_invalid("gs_idx_pool: null pointer");
    const int jf = p0 / kpool, jl = (p0 + T) / kpool;
    const int n_pools = jl - jf;
    if (n_pools > 65535) return fail_invalid("gs_idx_pool: more than 65535 pools complete in one call");
    dim3 grid((Dk + 127) / 128, n_pools > 0 ? n_pools : 1);
    k_idx_pool<<<grid, 128, 0, (cudaStream_t) stream>>>(kc, gc, rk, rg, ape, P, p0, T, Dk, kpool);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_idx_score(const float *q, const float *w, const float *P, float *score, int64_t score_stride, int pos0, int T,
                           int kpool, int Hq, int Dk, float scale, void *stream) {
    if (kpool <= 0) return fail_invalid("gs_idx_score: kpool <= 0");
    const int max_pool = (pos0 + T) / kpool;
    if (max_pool <= 0 || T <= 0) return 0;  // ops.cu:703
    if (Dk > 128 || Dk <= 0) return fail_invalid("gs_idx_score: Dk must be 1..128");  // ops.cu:704
    if (Hq <= 0 || (int64_t) Hq * (Dk + 1) * 4 > 48 * 1024) return fail_invalid("gs_idx_score: Hq * Dk beyond 12288");
    if (T > 65535) return fail_invalid("gs_idx_score: T > 65535");
    if (!q || !w || !P || !score) return fail_invalid("gs_idx_score: null pointer");
    dim3 grid((max_pool + SC_POOLS - 1) / SC_POOLS, T);
    k_idx_score<<<grid, SC_POOLS * SC_PARTS, (size_t) Hq * (Dk + 1) * sizeof(float), (cudaStream_t) stream>>>(
        q, w, P, score, score_stride, pos0, kpool, Hq, Dk, scale);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_idx_select(const float *score, int64_t score_stride, int pos0, int T, int kpool, int top_k, int *sel,
                            int sel_stride, int *cnt, void *stream) {
    if (T <= 0) return 0;  // ops.cu:788
    if (kpool <= 0 || top_k < 0 || pos0 < 0) return fail_invalid("gs_idx_select: need kpool > 0, top_k >= 0, pos0 >= 0");
    if (!sel || !cnt) return fail_invalid("gs_idx_select: null pointer");
    k_idx_select<<<T, SEL_NT, 0, (cudaStream_t) stream>>>(score, score_stride, pos0, kpool, top_k, sel, sel_stride, cnt);
    GS_TRY(cudaGetLastError());
    return 0;
}
