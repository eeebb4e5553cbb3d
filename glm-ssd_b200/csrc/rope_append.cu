// Fused RoPE + KV-append, plain append, and in-place RoPE for prefill inputs.
//
// The reference appends the new latent rows with a bare f32 -> f16 conversion
// (crates/cuda/kernels/gemm.cu:155-163, called from crates/engine/src/forward.rs:857-860).  The fused
// kernel does the same rounding and, for cache rows that carry a rotary part, rotates the last d_rope
// columns at the row's absolute position in the same pass, so the rotated f32 row never exists in
// memory.  Convention: adjacent pairs (2i, 2i+1), angle = pos * base^(-2i/d_rope); the inverse
// frequencies are computed on the host in double and rounded to f32, cos/sin are the full-range
// f32 functions (this file must not be built with fast-math).
#include <math.h>

#include <new>

#include "internal.cuh"

namespace gs {
namespace {

constexpr int ROPE_MAX_PAIRS = 64;
struct RopeTable {
    float inv_freq[ROPE_MAX_PAIRS];
};

static void fill_table(RopeTable &t, int d_rope, float base) {
    for (int i = 0; i < d_rope / 2; i++) t.inv_freq[i] = (float) pow((double) base, -2.0 * i / (double) d_rope);
}

// Separately rounded products (no fused multiply-add) so the result matches a plain C evaluation.
__device__ __forceinline__ float2 rotate(float2 v, float cs, float sn) {
    return make_float2(__fsub_rn(__fmul_rn(v.x, cs), __fmul_rn(v.y, sn)), __fadd_rn(__fmul_rn(v.x, sn), __fmul_rn(v.y, cs)));
}

__global__ void k_f32_to_f16_scalar(const float *__restrict__ x, __half *__restrict__ y, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}

__global__ void k_f32_to_f16_rows(const float *__restrict__ x, __half *__restrict__ y, int64_t n) {
    // two values per thread, 4-byte stores
    const int64_t i = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i + 1 < n) {
        const float2 v = *reinterpret_cast<const float2 *>(x + i);
        *reinterpret_cast<__half2 *>(y + i) = __floats2half2_rn(v.x, v.y);
    } else if (i < n) {
        y[i] = __float2half_rn(x[i]);
    }
}

// Q8 latent rows: per block of 32 values d = amax / 127, q = round-to-nearest-even(x / d), d kept as f16.
// One warp per block.  (Exact division and reciprocal: this file is not built with fast-math.)
__global__ void k_quant_q8(const float *__restrict__ x, int8_t *__restrict__ q, __half *__restrict__ d, int64_t n_blocks) {
    const int64_t b = (int64_t) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x & 31;
    if (b >= n_blocks) return;
    const float v = x[b * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float dd = __fdiv_rn(amax, 127.f);
    const float inv = dd > 0.f ? __fdiv_rn(1.f, dd) : 0.f;
    q[b * 32 + lane] = (int8_t) __float2int_rn(__fmul_rn(v, inv));
    if (lane == 0) d[b] = __float2half_rn(dd);
}

struct AppendParams {
    const float *kv;
    __half *cache;
    const int32_t *pos0, *seq_base, *page_table;
    int64_t pos0_host;
    int page_table_stride, page_rows;
    int T, d_row, d_rope;
    int32_t *len_out;  // optional: receives len_val (the sequence length after the append), for the decode that follows
    int32_t len_val;
    // checked form (cache_rows > 0): a position, page-table slot or cache row out of range is not followed; the row is
    // skipped and bit 17 of *status is set
    int64_t cache_rows;
    int32_t *status;
    RopeTable tab;
};

// grid (T, n_seq); thread j handles column pair (2j, 2j+1)
__global__ void k_rope_append(const AppendParams P) {
    const int t = blockIdx.x, b = blockIdx.y;
    if (P.len_out && t == 0 && b == 0 && threadIdx.x == 0) *P.len_out = P.len_val;
    const int64_t pos = (P.pos0 ? (int64_t) P.pos0[b] : P.pos0_host) + t;
    int64_t row;
    const bool checked = P.cache_rows > 0;
    bool bad = checked && pos < 0;
    if (P.page_table) {
        const int64_t slot = pos / P.page_rows;
        if (checked && (bad || slot >= P.page_table_stride)) {
            bad = true;
            row = 0;
        } else {
            row = (int64_t) P.page_table[(int64_t) b * P.page_table_stride + slot] * P.page_rows + pos % P.page_rows;
        }
    } else if (P.pos0) {
        row = (P.seq_base ? (int64_t) P.seq_base[b] : 0) + pos;
    } else {
        row = t;  // host-position form: `cache` already points at the first new row
    }
    if (checked && (bad || row < 0 || row >= P.cache_rows)) {
        if (threadIdx.x == 0) atomicOr(P.status, 1 << 17);
        return;
    }
    const float *src = P.kv + ((int64_t) b * P.T + t) * P.d_row;
    __half *dst = P.cache + row * P.d_row;
    const int d0 = P.d_row - P.d_rope;
    for (int j = threadIdx.x; j < P.d_row / 2; j += blockDim.x) {
        const int c = 2 * j;
        float2 v = *reinterpret_cast<const float2 *>(src + c);
        if (c >= d0) {
            const float ang = (float) pos * P.tab.inv_freq[(c - d0) >> 1];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            v = rotate(v, cs, sn);
        }
        *reinterpret_cast<__half2 *>(dst + c) = __floats2half2_rn(v.x, v.y);
    }
}

// RMSNorm of the latent columns fused into the append: y[c] = x[c] * rsqrt(mean(x[0..d0)^2) + eps) * w[c] for the
// first d0 = d_row - d_rope columns (the reference runs gs_rmsnorm over the new latent rows and then appends them,
// forward.rs:850 then :857-860; ops.cu:43-50), the last d_rope columns rotated at position pos0 + t; everything
// rounded to f16.  One block of 128 threads per row; division and square root are IEEE (no fast-math in this file).
__global__ void __launch_bounds__(128) k_norm_rope_append(const AppendParams P, const float *__restrict__ w, float eps) {
    __shared__ float red[4];
    const int t = blockIdx.x;
    const int64_t pos = P.pos0_host + t;
    const float *src = P.kv + (int64_t) t * P.d_row;
    __half *dst = P.cache + (int64_t) t * P.d_row;
    const int d0 = P.d_row - P.d_rope;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d0; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float tot = (red[0] + red[1]) + (red[2] + red[3]);
    const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float) d0), eps)));
    for (int j = threadIdx.x; j < P.d_row / 2; j += blockDim.x) {
        const int c = 2 * j;
        float2 v = *reinterpret_cast<const float2 *>(src + c);
        if (c >= d0) {
            const float ang = (float) pos * P.tab.inv_freq[(c - d0) >> 1];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            v = rotate(v, cs, sn);
        } else {
            v.x = __fmul_rn(__fmul_rn(v.x, r), w ? w[c] : 1.f);
            v.y = __fmul_rn(__fmul_rn(v.y, r), w ? w[c + 1] : 1.f);
        }
        *reinterpret_cast<__half2 *>(dst + c) = __floats2half2_rn(v.x, v.y);
    }
}

// First kernel of a replayed step.  Block 0 reads the position from a page-locked host word (so the launch
// itself carries no per-step argument and can be replayed from a CUDA graph), appends the T rows of one
// dense sequence there and leaves the new length in *len_dev for the attention kernel.  A step that would
// run past the cache writes nothing, sets bit 17 of the status word and reports through host_words[1].
// `kv` is page-locked host memory read in place.  The other blocks bring the query rows over from
// page-locked host memory (16-byte words); a step then needs no copy-engine operation.
constexpr int STAGE_T_MAX = 4;   // new rows per replayed step
constexpr int STAGE_PAIRS = 3;   // column pairs per thread: rows of up to 768 values
__global__ void __launch_bounds__(128) k_stage_append(const AppendParams P, volatile int64_t *host_words, int32_t *len_dev,
                                                      int64_t cache_rows, int32_t *status, const uint4 *q_src, uint4 *q_dst,
                                                      int q_words) {
#if __CUDA_ARCH__ >= 900
    // Let the attention kernel behind this one be scheduled right away: while this kernel waits for its reads
    // over PCIe, that one sets itself up and asks the first cache tiles of its range into L2; its own dependency
    // wait still covers everything written here.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
    if (blockIdx.x > 0) {
        const int nb = gridDim.x - 1;
        for (int i = (blockIdx.x - 1) * blockDim.x + threadIdx.x; i < q_words; i += nb * blockDim.x) q_dst[i] = q_src[i];
        return;
    }
    // every read that crosses to the host is issued before any is used: the position and the new rows arrive in
    // one round trip (STAGE_T_MAX rows of up to STAGE_PAIRS * 128 column pairs)
    const int pairs = P.d_row / 2;
    float2 v[STAGE_T_MAX][STAGE_PAIRS];
#pragma unroll
    for (int t = 0; t < STAGE_T_MAX; t++)
#pragma unroll
        for (int k = 0; k < STAGE_PAIRS; k++) {
            const int j = threadIdx.x + k * 128;
            v[t][k] = (t < P.T && j < pairs) ? *reinterpret_cast<const float2 *>(P.kv + (int64_t) t * P.d_row + 2 * j)
                                             : make_float2(0.f, 0.f);
        }
    const int64_t pos0 = host_words[0];
    if (pos0 < 0 || pos0 + P.T > cache_rows) {
        if (threadIdx.x == 0) {
            atomicOr(status, 1 << 17);
            host_words[1] = 1;
            *len_dev = 0;  // the attention that follows sees an empty sequence
        }
        return;
    }
    if (threadIdx.x == 0) *len_dev = (int32_t) (pos0 + P.T);
    const int d0 = P.d_row - P.d_rope;
#pragma unroll
    for (int t = 0; t < STAGE_T_MAX; t++) {
        if (t >= P.T) break;
        const int64_t pos = pos0 + t;
        __half *dst = P.cache + pos * P.d_row;
#pragma unroll
        for (int k = 0; k < STAGE_PAIRS; k++) {
            const int j = threadIdx.x + k * 128;
            if (j >= pairs) break;
            const int c = 2 * j;
            float2 u = v[t][k];
            if (c >= d0) {
                const float ang = (float) pos * P.tab.inv_freq[(c - d0) >> 1];
                float sn, cs;
                sincosf(ang, &sn, &cs);
                u = rotate(u, cs, sn);
            }
            *reinterpret_cast<__half2 *>(dst + c) = __floats2half2_rn(u.x, u.y);
        }
    }
}

// x f16 [S][H][d]: rotate the last d_rope columns of every head in place
__global__ void k_rope_f16(__half *x, int64_t n_pairs, int H, int d, int d_rope, int64_t pos0, const RopeTable tab) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int ppr = d_rope / 2;
    const int pair = (int) (i % ppr);
    const int64_t sh = i / ppr;  // s * H + h
    const int64_t s = sh / H;
    __half2 *p = reinterpret_cast<__half2 *>(x + sh * d + (d - d_rope)) + pair;
    const float2 v = __half22float2(*p);
    const float ang = (float) (pos0 + s) * tab.inv_freq[pair];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float2 r = rotate(v, cs, sn);
    *p = __floats2half2_rn(r.x, r.y);
}

int check_rope(int d_row, int d_rope) {
    if (d_row <= 0 || d_row % 2 != 0) return fail_invalid("append: d_row must be positive and even");
    if (d_rope < 0 || d_rope % 2 != 0 || d_rope > d_row || d_rope / 2 > ROPE_MAX_PAIRS)
        return fail_invalid("append: d_rope must be even, <= d_row and <= 128");
    return 0;
}

}  // namespace
}  // namespace gs

using namespace gs;

GS_EXPORT int gs_f32_to_f16(const float *x, void *y, int64_t n, void *stream) {
    if (n <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(y) & 3)) {
        // odd alignment: one value per thread
        k_f32_to_f16_scalar<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, (__half *) y, n);
        GS_TRY(cudaGetLastError());
        return 0;
    }
    const int64_t pairs = (n + 1) / 2;
    k_f32_to_f16_rows<<<(unsigned) ((pairs + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, (__half *) y, n);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_quant_q8_rows(const float *x, void *q, void *d, int64_t n, void *stream) {
    if (n % 32 != 0) return fail_invalid("gs_quant_q8_rows: n must be a multiple of 32");  // ops.cu:612
    const int64_t nb = n / 32;
    if (nb <= 0) return 0;
    k_quant_q8<<<(unsigned) ((nb + 7) / 8), 256, 0, (cudaStream_t) stream>>>(x, (int8_t *) q, (__half *) d, nb);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_rope_kv_append_at(const float *kv, void *cache_row0, int64_t pos0, int T, int d_row, int d_rope,
                                   float rope_base, void *stream) {
    if (int e = check_rope(d_row, d_rope)) return e;
    if (T <= 0) return 0;
    if (pos0 < 0) return fail_invalid("append: pos0 < 0");
    AppendParams P{};
    P.kv = kv;
    P.cache = (__half *) cache_row0;
    P.pos0 = nullptr;
    P.pos0_host = pos0;
    P.page_rows = 1;
    P.T = T;
    P.d_row = d_row;
    P.d_rope = d_rope;
    fill_table(P.tab, d_rope, rope_base);
    k_rope_append<<<dim3(T, 1), 128, 0, (cudaStream_t) stream>>>(P);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_norm_rope_kv_append_at(const float *kv, const float *w, float eps, void *cache_row0, int64_t pos0, int T,
                                        int d_row, int d_rope, float rope_base, void *stream) {
    if (int e = check_rope(d_row, d_rope)) return e;
    if (T <= 0) return 0;
    if (pos0 < 0) return fail_invalid("append: pos0 < 0");
    if ((d_row - d_rope) % 2 != 0 || d_row == d_rope) return fail_invalid("append: need an even, non-empty run of latent columns");
    if (!(eps >= 0.f)) return fail_invalid("append: eps must be non-negative");
    AppendParams P{};
    P.kv = kv;
    P.cache = (__half *) cache_row0;
    P.pos0_host = pos0;
    P.page_rows = 1;
    P.T = T;
    P.d_row = d_row;
    P.d_rope = d_rope;
    fill_table(P.tab, d_rope, rope_base);
    k_norm_rope_append<<<T, 128, 0, (cudaStream_t) stream>>>(P, w, eps);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_rope_kv_append(const float *kv, void *cache, const int32_t *pos0, const int32_t *seq_base,
                                const int32_t *page_table, int page_table_stride, int page_rows, int n_seq, int T,
                                int d_row, int d_rope, float rope_base, void *stream) {
    if (int e = check_rope(d_row, d_rope)) return e;
    if (n_seq <= 0 || T <= 0) return 0;
    if (!pos0) return fail_invalid("append: pos0 (device) is required; use gs_rope_kv_append_at for a host position");
    if (page_table && page_rows <= 0) return fail_invalid("append: page_rows must be positive");
    if (n_seq > 65535) return fail_invalid("append: n_seq > 65535");
    AppendParams P{};
    P.kv = kv;
    P.cache = (__half *) cache;
    P.pos0 = pos0;
    P.seq_base = seq_base;
    P.page_table = page_table;
    P.page_table_stride = page_table_stride;
    P.page_rows = page_rows > 0 ? page_rows : 1;
    P.T = T;
    P.d_row = d_row;
    P.d_rope = d_rope;
    fill_table(P.tab, d_rope, rope_base);
    k_rope_append<<<dim3(T, n_seq), 128, 0, (cudaStream_t) stream>>>(P);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_rope_kv_append_checked(const float *kv, void *cache, int64_t cache_rows, const int32_t *pos0,
                                        const int32_t *seq_base, const int32_t *page_table, int page_table_stride,
                                        int page_rows, int n_seq, int T, int d_row, int d_rope, float rope_base,
                                        int32_t *status, void *stream) {
    if (int e = check_rope(d_row, d_rope)) return e;
    if (n_seq <= 0 || T <= 0) return 0;
    if (!pos0 || !status) return fail_invalid("append: pos0 and status (device) are required");
    if (cache_rows <= 0) return fail_invalid("append: cache_rows <= 0");
    if (page_table && (page_rows <= 0 || page_table_stride <= 0)) return fail_invalid("append: page_rows and page_table_stride must be positive");
    if (n_seq > 65535) return fail_invalid("append: n_seq > 65535");
    AppendParams P{};
    P.kv = kv;
    P.cache = (__half *) cache;
    P.pos0 = pos0;
    P.seq_base = seq_base;
    P.page_table = page_table;
    P.page_table_stride = page_table_stride;
    P.page_rows = page_rows > 0 ? page_rows : 1;
    P.T = T;
    P.d_row = d_row;
    P.d_rope = d_rope;
    P.cache_rows = cache_rows;
    P.status = status;
    fill_table(P.tab, d_rope, rope_base);
    k_rope_append<<<dim3(T, n_seq), 128, 0, (cudaStream_t) stream>>>(P);
    GS_TRY(cudaGetLastError());
    return 0;
}

GS_EXPORT int gs_rope_f16_inplace(void *x, int S, int H, int d, int d_rope, int64_t pos0, float rope_base,
                                  void *stream) {
    if (d <= 0 || d_rope < 0 || d_rope % 2 != 0 || d_rope > d || d % 2 != 0 || d_rope / 2 > ROPE_MAX_PAIRS)
        return fail_invalid("rope: need even d, even d_rope <= d, d_rope <= 128");
    if (S <= 0 || H <= 0 || d_rope == 0) return 0;
    RopeTable tab;
    fill_table(tab, d_rope, rope_base);
    const int64_t n_pairs = (int64_t) S * H * (d_rope / 2);
    k_rope_f16<<<(unsigned) ((n_pairs + 255) / 256), 256, 0, (cudaStream_t) stream>>>((__half *) x, n_pairs, H, d, d_rope,
                                                                                     pos0, tab);
    GS_TRY(cudaGetLastError());
    return 0;
}

// ---- one decode step of a layer with host buffers ---------------------------------------------------
GS_EXPORT int gs_mla_layer_step_host(const gs_mla_layer_step *s, void *stream) {
    if (!s) return fail_invalid("gs_mla_layer_step_host: args == NULL");
    if (s->T <= 0 || s->H <= 0) return 0;
    if (!s->q_host || !s->kv_host || !s->o_host || !s->q_dev || !s->kv_dev || !s->o_dev || !s->cache || !s->seq_len_dev ||
        !s->workspace)
        return fail_invalid("gs_mla_layer_step_host: null pointer");
    if (int e = check_rope(s->d_qk, s->d_rope)) return e;
    if (s->pos0 < 0 || s->pos0 + s->T > s->cache_rows) {
        set_error("context full (%lld tokens)", (long long) s->cache_rows);  // forward.rs:839-841
        return (int) cudaErrorInvalidValue;
    }
    cudaStream_t st = (cudaStream_t) stream;
    const size_t q_bytes = (size_t) s->T * s->H * s->d_qk * 2, kv_bytes = (size_t) s->T * s->d_qk * 4;
    GS_TRY(cudaMemcpyAsync(s->q_dev, s->q_host, q_bytes, cudaMemcpyHostToDevice, st));
    GS_TRY(cudaMemcpyAsync(s->kv_dev, s->kv_host, kv_bytes, cudaMemcpyHostToDevice, st));
    AppendParams P{};
    P.kv = (const float *) s->kv_dev;
    P.cache = (__half *) s->cache + s->pos0 * s->d_qk;
    P.pos0 = nullptr;
    P.pos0_host = s->pos0;
    P.page_rows = 1;
    P.T = s->T;
    P.d_row = s->d_qk;
    P.d_rope = s->d_rope;
    P.len_out = s->seq_len_dev;
    P.len_val = (int32_t) (s->pos0 + s->T);
    fill_table(P.tab, s->d_rope, s->rope_base);
    k_rope_append<<<dim3(s->T, 1), 128, 0, st>>>(P);
    GS_TRY(cudaGetLastError());
    gs_mla_decode_args a{};
    a.q = s->q_dev;
    a.cache = s->cache;
    a.cache_rows = s->cache_rows;
    a.seq_lens = s->seq_len_dev;
    a.page_rows = 64;
    a.scale = s->scale;
    a.tail_causal = 1;
    a.o = (float *) s->o_dev;
    a.workspace = s->workspace;
    a.workspace_bytes = s->workspace_bytes;
    a.n_seq = 1;
    a.T = s->T;
    a.H = s->H;
    a.d_qk = s->d_qk;
    a.d_v = s->d_v;
    a.max_seq_len = (int32_t) (s->pos0 + s->T);
    if (int e = gs_mla_decode(&a, stream)) return e;
    GS_TRY(cudaMemcpyAsync(s->o_host, s->o_dev, (size_t) s->T * s->H * s->d_v * 4, cudaMemcpyDeviceToHost, st));
    return 0;
}

// ---- the same step as a replayable CUDA graph ---------------------------------------------------------
struct gs_mla_layer_graph {
    cudaGraphExec_t exec;
    int64_t *host_words;  // page-locked: [0] position of the step (host -> device), [1] refusal flag (device -> host)
    int64_t cache_rows;
    int T;
};

GS_EXPORT int gs_mla_layer_graph_create(const gs_mla_layer_step *s, void *stream, gs_mla_layer_graph **out) {
    if (!s || !out) return fail_invalid("gs_mla_layer_graph_create: null argument");
    *out = nullptr;
    if (s->T <= 0 || s->H <= 0) return fail_invalid("gs_mla_layer_graph_create: T and H must be positive");
    if (s->T > STAGE_T_MAX || s->d_qk > STAGE_PAIRS * 256)
        return fail_invalid("gs_mla_layer_graph_create: at most 4 new rows of at most 768 values per step");
    if (!s->q_host || !s->kv_host || !s->o_host || !s->q_dev || !s->cache || !s->seq_len_dev || !s->workspace)
        return fail_invalid("gs_mla_layer_graph_create: null pointer");
    if (!stream) return fail_invalid("gs_mla_layer_graph_create: stream capture needs a stream other than the default one");
    if (int e = check_rope(s->d_qk, s->d_rope)) return e;
    if (s->cache_rows <= 0 || s->cache_rows >= (1ll << 31)) return fail_invalid("gs_mla_layer_graph_create: cache_rows out of range");
    cudaStream_t st = (cudaStream_t) stream;
    // the page-locked host buffers as the device sees them: the kernels read q / kv and write o in place
    void *q_map = nullptr, *kv_map = nullptr, *o_map = nullptr, *w_map = nullptr;
    GS_TRY(cudaHostGetDevicePointer(&q_map, const_cast<void *>(s->q_host), 0));
    GS_TRY(cudaHostGetDevicePointer(&kv_map, const_cast<float *>(s->kv_host), 0));
    GS_TRY(cudaHostGetDevicePointer(&o_map, s->o_host, 0));
    const size_t q_bytes = (size_t) s->T * s->H * s->d_qk * 2;
    if (q_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(q_map) & 15) || (reinterpret_cast<uintptr_t>(s->q_dev) & 15) ||
        (reinterpret_cast<uintptr_t>(kv_map) & 7) || (reinterpret_cast<uintptr_t>(o_map) & 15))
        return fail_invalid("gs_mla_layer_graph_create: host buffers must be 16-byte aligned");
    int64_t *words = nullptr;
    GS_TRY(cudaHostAlloc((void **) &words, 2 * sizeof(int64_t), cudaHostAllocMapped));
    words[0] = words[1] = 0;
    cudaError_t ce = cudaHostGetDevicePointer(&w_map, words, 0);
    if (ce == cudaSuccess) ce = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    if (ce != cudaSuccess) {
        cudaFreeHost(words);
        GS_TRY(ce);
    }
    auto enqueue = [&]() -> int {
        AppendParams P{};
        P.kv = (const float *) kv_map;
        P.cache = (__half *) s->cache;
        P.T = s->T;
        P.d_row = s->d_qk;
        P.d_rope = s->d_rope;
        fill_table(P.tab, s->d_rope, s->rope_base);
        const int q_words = (int) (q_bytes / 16);
        const int copy_blocks = (q_words + 127) / 128 < 24 ? (q_words + 127) / 128 : 24;
        k_stage_append<<<1 + copy_blocks, 128, 0, st>>>(P, (volatile int64_t *) w_map, s->seq_len_dev, s->cache_rows,
                                                        (int32_t *) s->workspace, (const uint4 *) q_map, (uint4 *) s->q_dev,
                                                        q_words);
        GS_TRY(cudaGetLastError());
        gs_mla_decode_args a{};
        a.q = s->q_dev;
        a.cache = s->cache;
        a.cache_rows = s->cache_rows;
        a.seq_lens = s->seq_len_dev;
        a.page_rows = 64;
        a.scale = s->scale;
        a.tail_causal = 1;
        a.o = (float *) o_map;  // the combine kernel stores the result straight into the host buffer
        a.workspace = s->workspace;
        a.workspace_bytes = s->workspace_bytes;
        a.n_seq = 1;
        a.T = s->T;
        a.H = s->H;
        a.d_qk = s->d_qk;
        a.d_v = s->d_v;
        a.max_seq_len = (int32_t) s->cache_rows;
        return gs_mla_decode(&a, stream);
    };
    const int e = enqueue();
    cudaGraph_t graph = nullptr;
    ce = cudaStreamEndCapture(st, &graph);  // always ends the capture, also after an error
    cudaGraphExec_t exec = nullptr;
    if (!e && ce == cudaSuccess) ce = cudaGraphInstantiate(&exec, graph, 0);
    if (graph) cudaGraphDestroy(graph);
    gs_mla_layer_graph *g = (!e && ce == cudaSuccess) ? new (std::nothrow) gs_mla_layer_graph : nullptr;
    if (!g) {
        if (exec) cudaGraphExecDestroy(exec);
        cudaFreeHost(words);
        if (e) {
            (void) cudaGetLastError();
            return e;
        }
        GS_TRY(ce);
        set_error("gs_mla_layer_graph_create: out of host memory");
        return (int) cudaErrorMemoryAllocation;
    }
    g->exec = exec;
    g->host_words = words;
    g->cache_rows = s->cache_rows;
    g->T = s->T;
    *out = g;
    return 0;
}

GS_EXPORT int gs_mla_layer_graph_step(gs_mla_layer_graph *g, int64_t pos0, void *stream, int wait) {
    if (!g) return fail_invalid("gs_mla_layer_graph_step: null handle");
    if (pos0 < 0 || pos0 + g->T > g->cache_rows) {
        set_error("context full (%lld tokens)", (long long) g->cache_rows);  // forward.rs:839-841
        return (int) cudaErrorInvalidValue;
    }
    *(volatile int64_t *) g->host_words = pos0;
    GS_TRY(cudaGraphLaunch(g->exec, (cudaStream_t) stream));
    if (wait) {
        GS_TRY(cudaStreamSynchronize((cudaStream_t) stream));
        if (((volatile int64_t *) g->host_words)[1] != 0) {
            set_error("gs_mla_layer_graph_step: the device refused a step past the end of the cache");
            return (int) cudaErrorInvalidValue;
        }
    }
    return 0;
}

GS_EXPORT int gs_mla_layer_graph_destroy(gs_mla_layer_graph *g) {
    if (!g) return 0;
    const cudaError_t e = cudaGraphExecDestroy(g->exec);
    const cudaError_t f = cudaFreeHost(g->host_words);
    delete g;
    GS_TRY(e);
    GS_TRY(f);
    return 0;
}
