// CUDA-core split-KV decode ("gather" kernel) and the partial combine.
//
// This kernel takes any addressing (explicit position lists as in the reference ABI, dense ranges,
// paged), any head count, f32 or f16 queries and any number of query tokens.  It is the path for
// shapes the tcgen05 kernel does not cover (position lists, f32 queries, T > 2) and the second
// opinion the tcgen05 kernel is tested against; it is not the fast path.
//
// Arithmetic follows the reference kernel's contract (crates/cuda/kernels/ops.cu:420-424):
//   score = scale * q . K[row]; online softmax over the attended rows; o = sum p V[row] / sum p,
// with split-KV partials (unnormalised acc, m, l) merged as in ops.cu:552-574.
#include <type_traits>

#include "combine.cuh"
#include "sm100_prims.cuh"
#include "internal.cuh"

namespace gs {

namespace {

constexpr int KT = 16;   // keys per shared-memory tile
constexpr int HG_MAX = 32;  // heads per CTA: 32, 16 or 8 (template parameter), fewer when the grid would not fill the GPU
constexpr int NT = 256;  // threads per CTA

struct SimtParams {
    const void *q;
    const __half *cache;        // f16 rows, or int8 rows when `scales` is set
    const __half *scales;       // Q8 cache: one f16 scale per 32 values, [rows][d_qk/32]; nullptr = f16 cache
    const int32_t *seq_lens, *seq_base, *page_table, *sel;
    int page_table_stride, page_rows, sel_stride;
    float scale;
    int tail_causal;
    float *ws_acc, *ws_ml;
    float *o_direct;            // splits == 1: the normalised output [groups][H][d_v] is stored here and no record is written
    int T, H, d_qk, d_v, splits;
};

template <typename QT, bool Q8, int HG>
__global__ void __launch_bounds__(NT) k_decode_gather(const SimtParams P) {
    static_assert(HG <= HG_MAX && HG <= 32, "a lane per head in the score reduction");
    const int split = blockIdx.x, hg = blockIdx.y, bt = blockIdx.z;
    const int b = bt / P.T, t = bt % P.T;
    const int h0 = hg * HG;
    const int nh = min(HG, P.H - h0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int d_qk = P.d_qk, d_v = P.d_v;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *sq = reinterpret_cast<float *>(smem_raw);             // [HG][d_qk]
    __half *tile = reinterpret_cast<__half *>(sq + HG * d_qk);   // [KT][d_qk]
    float *sp = reinterpret_cast<float *>(tile + KT * d_qk);     // [HG][KT]
    float *s_m = sp + HG * KT, *s_l = s_m + HG, *s_f = s_l + HG;  // [HG] each

    // attended rows of this (sequence, token)
    RowMap rows;
    int n;
    if (P.sel) {
        rows = RowMap{P.sel + (int64_t) t * P.sel_stride, nullptr, 0, 1};
        n = P.seq_lens[t];
    } else {
        const int len = P.seq_lens[b];
        n = P.tail_causal ? len - (P.T - 1 - t) : len;
        rows = RowMap{nullptr, P.page_table ? P.page_table + (int64_t) b * P.page_table_stride : nullptr,
                      P.seq_base ? (int64_t) P.seq_base[b] : 0, P.page_rows};
    }
    n = max(n, 0);
    const int per = (n + P.splits - 1) / P.splits;
    const int s0 = min(n, split * per), s1 = min(n, s0 + per);

    const QT *qg = reinterpret_cast<const QT *>(P.q) + ((int64_t) bt * P.H + h0) * d_qk;
    for (int i = tid; i < nh * d_qk; i += NT) sq[i] = (float) qg[i];
    for (int i = nh * d_qk + tid; i < HG * d_qk; i += NT) sq[i] = 0.f;
    if (tid < HG) {
        s_m[tid] = -INFINITY;
        s_l[tid] = 0.f;
    }
    float acc[HG][2];
#pragma unroll
    for (int h = 0; h < HG; h++) acc[h][0] = acc[h][1] = 0.f;
    __syncthreads();

    const int vec_per_row = d_qk / 8;
    for (int kb = s0; kb < s1; kb += KT) {
        const int nk = min(KT, s1 - kb);
        if (Q8) {
            // int8 rows with one f16 scale per 32 values: rebuild the f16 tile as half_rn(scale * q), the
            // values the reference's Q8 branch attends over (crates/cuda/kernels/ops.cu:461-477)
            const int chunks = d_qk / 16;  // one 16-byte load of int8 -> two 16-byte stores of f16
            const int8_t *c8 = reinterpret_cast<const int8_t *>(P.cache);
            for (int i = tid; i < KT * chunks; i += NT) {
                const int kk = i / chunks, c = i - kk * chunks;
                uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
                if (kk < nk) {
                    const int64_t row = rows(kb + kk);
                    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(c8 + row * d_qk) + c);
                    const float sc = __half2float(P.scales[row * (d_qk / 32) + (c >> 1)]);
                    auto pack = [sc](uint32_t w, uint32_t &h01, uint32_t &h23) {
                        const float f0 = sc * (float) (int8_t) (w), f1 = sc * (float) (int8_t) (w >> 8);
                        const float f2 = sc * (float) (int8_t) (w >> 16), f3 = sc * (float) (int8_t) (w >> 24);
                        const __half2 a = __floats2half2_rn(f0, f1), b2 = __floats2half2_rn(f2, f3);
                        h01 = *reinterpret_cast<const uint32_t *>(&a);
                        h23 = *reinterpret_cast<const uint32_t *>(&b2);
                    };
                    pack(raw.x, lo.x, lo.y);
                    pack(raw.y, lo.z, lo.w);
                    pack(raw.z, hi.x, hi.y);
                    pack(raw.w, hi.z, hi.w);
                }
                uint4 *dst = reinterpret_cast<uint4 *>(tile + kk * d_qk + c * 16);
                dst[0] = lo;
                dst[1] = hi;
            }
        } else {
            for (int i = tid; i < KT * vec_per_row; i += NT) {
                const int kk = i / vec_per_row, c = i % vec_per_row;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (kk < nk) val = reinterpret_cast<const uint4 *>(P.cache + rows(kb + kk) * d_qk)[c];
                reinterpret_cast<uint4 *>(tile + kk * d_qk)[c] = val;
            }
        }
        __syncthreads();
        // scores: each warp takes two keys, every lane a strided slice of the row
        for (int kk = warp * 2; kk < warp * 2 + 2; kk++) {
            float d[HG];
#pragma unroll
            for (int h = 0; h < HG; h++) d[h] = 0.f;
            const __half2 *krow = reinterpret_cast<const __half2 *>(tile + kk * d_qk);
            for (int r2 = lane; r2 < d_qk / 2; r2 += 32) {
                const float2 kf = __half22float2(krow[r2]);
#pragma unroll
                for (int h = 0; h < HG; h++) {
                    const float2 qf = reinterpret_cast<const float2 *>(sq + h * d_qk)[r2];
                    d[h] = fmaf(qf.x, kf.x, fmaf(qf.y, kf.y, d[h]));
                }
            }
#pragma unroll
            for (int h = 0; h < HG; h++) {
                const float v = warp_sum(d[h]);
                if (lane == h) sp[h * KT + kk] = kk < nk ? v * P.scale : -INFINITY;
            }
        }
        __syncthreads();
        // online softmax: one warp per head, lanes over the tile's keys
        for (int h = warp; h < nh; h += NT / 32) {
            const float s = lane < KT ? sp[h * KT + lane] : -INFINITY;
            const float m_old = s_m[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float p = s == -INFINITY ? 0.f : expf(s - m_new);
            const float psum = warp_sum(p);
            if (lane < KT) sp[h * KT + lane] = p;
            if (lane == 0) {
                const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                s_f[h] = f;
                s_l[h] = s_l[h] * f + psum;
                s_m[h] = m_new;
            }
        }
        __syncthreads();
        // PV: thread owns value columns tid and tid + 256
        {
            float v0[KT], v1[KT];
#pragma unroll
            for (int k = 0; k < KT; k++) {
                v0[k] = tid < d_v ? __half2float(tile[k * d_qk + tid]) : 0.f;
                v1[k] = tid + NT < d_v ? __half2float(tile[k * d_qk + tid + NT]) : 0.f;
            }
#pragma unroll
            for (int h = 0; h < HG; h++) {
                if (h < nh) {
                    const float f = s_f[h];
                    float a0 = acc[h][0] * f, a1 = acc[h][1] * f;
#pragma unroll
                    for (int k = 0; k < KT; k++) {
                        const float p = sp[h * KT + k];
                        a0 = fmaf(p, v0[k], a0);
                        a1 = fmaf(p, v1[k], a1);
                    }
                    acc[h][0] = a0;
                    acc[h][1] = a1;
                }
            }
        }
        __syncthreads();
    }
    if (P.o_direct) {
        // a single split needs no merge: normalise here and leave the workspace alone, as the reference does
        // (crates/cuda/kernels/ops.cu:531-538; zeros for a query that attends nothing)
#pragma unroll
        for (int h = 0; h < HG; h++) {
            if (h < nh) {
                const float l = s_l[h];
                const float inv = l > 0.f ? 1.f / l : 0.f;
                float *dst = P.o_direct + ((int64_t) bt * P.H + h0 + h) * d_v;
                if (tid < d_v) dst[tid] = acc[h][0] * inv;
                if (tid + NT < d_v) dst[tid + NT] = acc[h][1] * inv;
            }
        }
        return;
    }
    // one (acc, m, l) record per (sequence, token, split, head)
    const int64_t seg = (int64_t) bt * P.splits + split;
#pragma unroll
    for (int h = 0; h < HG; h++) {
        if (h < nh) {
            float *dst = P.ws_acc + (seg * P.H + h0 + h) * d_v;
            if (tid < d_v) dst[tid] = acc[h][0];
            if (tid + NT < d_v) dst[tid + NT] = acc[h][1];
        }
    }
    if (tid < nh) {
        float *ml = P.ws_ml + (seg * P.H + h0 + tid) * 2;
        ml[0] = s_m[tid];
        ml[1] = s_l[tid];
    }
}

// ---- combine --------------------------------------------------------------------------------------
// Stand-alone combine: one CTA per item.  Launched with programmatic dependent launch: the launch
// overlaps the tail of the kernel that writes the partials.
__global__ void __launch_bounds__(CB_NT) k_combine(const CombinePlan C) {
    __shared__ CombineSmem S;
    long long *prof = nullptr;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    if (C.status && C.status[1] != 0 && cta < 256 && threadIdx.x == 0)
        prof = reinterpret_cast<long long *>(const_cast<char *>(reinterpret_cast<const char *>(C.status)) + kCombineProfOffsetBytes) + cta * 8;
    if (prof) prof[0] = sm100::global_timer_ns();
#if __CUDA_ARCH__ >= 900
    // the kernel behind this one may be scheduled as soon as every CTA of this grid is running: its CTAs
    // then start on each SM as this grid's leave it, and their own dependency wait still covers our stores
    cudaTriggerProgrammaticLaunchCompletion();
#endif
    const bool early = combine_locate_is_early(C);
    SegRange R;
    if (early) R = combine_locate(C, blockIdx.x, S);
#if __CUDA_ARCH__ >= 900
    cudaGridDependencySynchronize();  // the partial records (and desc) are written by the preceding kernel
#endif
    if (prof) prof[1] = sm100::global_timer_ns();
    if (!early) R = combine_locate(C, blockIdx.x, S);
    combine_item(C, R, blockIdx.x, blockIdx.y * CB_COLS, S);
    if (prof) prof[2] = sm100::global_timer_ns();
}

// Combine of the tcgen05 kernel's records with one tiled TMA copy per item (combine_item_fetch_tma): the copy engine
// keeps the L2 read at full rate with no address arithmetic in the threads.
__global__ void __launch_bounds__(CB_NT) k_combine_bulk(const __grid_constant__ CombineBulk CBk) {
    const CombinePlan &C = CBk.c;
    extern __shared__ unsigned char bulk_raw[];
    // [n_ctas][32] column quads, 128-byte aligned for the TMA
    float4 *tile = reinterpret_cast<float4 *>((reinterpret_cast<uintptr_t>(bulk_raw) + 127) & ~(uintptr_t) 127);
    __shared__ CombineSmem S;
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    long long *prof = nullptr;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    if (C.status && C.status[1] != 0 && cta < 256 && tid == 0)
        prof = reinterpret_cast<long long *>(const_cast<char *>(reinterpret_cast<const char *>(C.status)) + kCombineProfOffsetBytes) + cta * 8;
    if (prof) prof[0] = sm100::global_timer_ns();
    cudaTriggerProgrammaticLaunchCompletion();
    if (tid == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::fence_barrier_init();
        s_abort = 0;
    }
    const int row = blockIdx.x, col0 = blockIdx.y * CB_COLS;
    const SegRange R = combine_locate(C, row, S);  // from the sequence lengths only: nothing the kernel in front writes
    __syncthreads();
    cudaGridDependencySynchronize();  // the records are written by the preceding kernel
    if (prof) prof[1] = sm100::global_timer_ns();
    float4 a;
    float M, L;
    if (!combine_item_fetch_tma(C, &CBk.tm, R, col0, tile, &bar, &s_abort, S, a, M, L)) return;  // the status word says why; nothing is written
    const int col = col0 + lane * 4;
    if (warp == 0 && col < C.d_v) {
        int H_out;
        const int64_t orow = combine_out_row(C, row, H_out);
        if (C.part_out) {
            const int64_t rows_total = (int64_t) (C.seq_div > 1 ? C.n_seq / C.seq_div : C.n_seq) * C.T * H_out;
            *reinterpret_cast<float4 *>(C.part_out + orow * C.d_v + col) = a;
            if (col == 0) {
                C.part_out[rows_total * C.d_v + orow * 2] = M;
                C.part_out[rows_total * C.d_v + orow * 2 + 1] = L;
            }
        }
        if (C.o) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4 *>(C.o + orow * C.d_v + col) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
    if (prof) prof[2] = sm100::global_timer_ns();
}

// Combine for large batches: a sequence then has only a few segments (about n_ctas / n_seq + 1), and one CTA per
// (row, 128 columns) with block-wide reductions costs far more than the merge itself.  Here one thread owns four
// columns of one output row and walks the row's segments; (m, l) loads are the same for the whole block.
__global__ void __launch_bounds__(128) k_combine_rows(const CombinePlan C) {
#if __CUDA_ARCH__ >= 900
    cudaTriggerProgrammaticLaunchCompletion();
    cudaGridDependencySynchronize();  // the partial records and desc are written by the preceding kernel
#endif
    const int row = blockIdx.x;
    const int h = row % C.H, t = (row / C.H) % C.T, b = row / (C.H * C.T);
    int first, nseg, row_in_seg;
    if (C.desc) {
        const int2 d = __ldcg(C.desc + b);
        first = d.x;
        nseg = d.y;
        row_in_seg = t * C.H + h;
    } else {
        first = (b * C.T + t) * C.regular_segments;
        nseg = C.regular_segments;
        row_in_seg = h;
    }
    const float *ml0 = combine_ml_ptr(C, first, row_in_seg);
    float M = -INFINITY;
    for (int s = 0; s < nseg; s++) M = fmaxf(M, __ldcg(ml0 + (int64_t) s * C.seg_stride_ml));
    int H_out;
    const int64_t orow = combine_out_row(C, row, H_out);
    const int64_t rows_total = (int64_t) (C.seq_div > 1 ? C.n_seq / C.seq_div : C.n_seq) * C.T * H_out;
    for (int col = threadIdx.x * 4; col < C.d_v; col += blockDim.x * 4) {
        const float *acc0 = combine_acc_ptr(C, first, row_in_seg, col);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
        for (int s = 0; s < nseg; s++) {
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(ml0 + (int64_t) s * C.seg_stride_ml));
            const float w = ml.x == -INFINITY ? 0.f : expf(ml.x - M);
            L += ml.y * w;
            if (w != 0.f) {  // an empty segment's accumulator never enters the sum
                const float4 u = __ldcg(reinterpret_cast<const float4 *>(acc0 + (int64_t) s * C.seg_stride_acc));
                a.x = fmaf(u.x, w, a.x);
                a.y = fmaf(u.y, w, a.y);
                a.z = fmaf(u.z, w, a.z);
                a.w = fmaf(u.w, w, a.w);
            }
        }
        if (C.part_out) {
            *reinterpret_cast<float4 *>(C.part_out + orow * C.d_v + col) = a;
            if (col == 0) {
                C.part_out[rows_total * C.d_v + orow * 2] = M;
                C.part_out[rows_total * C.d_v + orow * 2 + 1] = L;
            }
        }
        if (C.o) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4 *>(C.o + orow * C.d_v + col) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
}

}  // namespace

int launch_combine(const CombinePlan &c, cudaStream_t st) {
    const int rows = c.n_seq * c.T * c.H;
    if (rows <= 0) return 0;
    if (c.d_v % 4 != 0) return fail_invalid("combine: d_v must be a multiple of 4");
    cudaLaunchConfig_t cfg = {};
    // many sequences: few segments each (the attention kernel spreads n_ctas + n_seq segments over them)
    const bool by_rows = c.desc != nullptr && c.n_seq >= 16;
    cfg.gridDim = by_rows ? dim3(rows) : dim3(rows, (c.d_v + CB_COLS - 1) / CB_COLS);
    cfg.blockDim = by_rows ? dim3(128) : dim3(CB_NT);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // records of the tcgen05 kernel ([segment][row][d_v], at most one segment per CTA and sequence): tiled TMA fetch
    const bool bulk = c.bulk && !by_rows && c.desc != nullptr && c.seq_lens != nullptr && c.n_ctas > 0 && c.n_ctas <= CB_NT &&
                      c.d_v % CB_COLS == 0 && c.n_segments > 0 && c.seg_stride_acc % 4 == 0 && !(reinterpret_cast<uintptr_t>(c.acc) & 15);
    if (bulk) {
        CombineBulk cb;
        cb.c = c;
        const int rows_seg = (int) (c.seg_stride_acc / c.d_v);  // query rows per record
        if (int e = encode_tmap_3d_f32(&cb.tm, c.acc, (uint64_t) c.d_v, (uint64_t) rows_seg, (uint64_t) c.n_segments, (uint64_t) c.d_v * 4,
                                       (uint64_t) c.seg_stride_acc * 4, CB_COLS, 1, (uint32_t) c.n_ctas))
            return e;
        const int smem = c.n_ctas * CB_COLS * 4 + 128;
        // attributes are set on every call: a cached flag would go stale across a device reset
        GS_TRY(cudaFuncSetAttribute(k_combine_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        cfg.dynamicSmemBytes = smem;
        GS_TRY(cudaLaunchKernelEx(&cfg, k_combine_bulk, cb));
    } else if (by_rows) {
        GS_TRY(cudaLaunchKernelEx(&cfg, k_combine_rows, c));
    } else {
        GS_TRY(cudaLaunchKernelEx(&cfg, k_combine, c));
    }
    return 0;
}

int launch_decode_simt(const DecodeProblem &p, cudaStream_t st) {
    if (p.d_qk % 8 != 0 || p.d_qk > 576 || p.d_v > 512 || p.d_v > p.d_qk || p.d_v % 4 != 0)
        return fail_invalid("decode: need d_qk % 8 == 0, d_qk <= 576, d_v <= min(512, d_qk), d_v % 4 == 0");
    const int groups = p.n_seq * p.T;
    if (groups <= 0 || p.H <= 0) return 0;
    // Heads per CTA.  When the caller fixes the number of splits (the reference's entry point; a decode call there is
    // small), fewer heads per CTA are the only way to give every SM a CTA; otherwise the splits provide the CTAs.
    int HG = HG_MAX;
    if (p.splits > 0) {
        const int64_t per_hg = (int64_t) groups * p.splits;
        while (HG > 8 && per_hg * ((p.H + HG - 1) / HG) < p.sm_count) HG >>= 1;
    }
    const int n_hg = (p.H + HG - 1) / HG;
    int splits = p.splits;
    if (splits <= 0) {
        // enough CTAs for two waves, but no split shorter than four tiles of the longest sequence
        const int want = (2 * p.sm_count + groups * n_hg - 1) / (groups * n_hg);
        const int max_len = p.max_seq_len > 0 ? p.max_seq_len : (int) (p.cache_rows > (1 << 30) ? (1 << 30) : p.cache_rows);
        const int by_len = (max_len + 4 * KT - 1) / (4 * KT);
        splits = want < by_len ? want : by_len;
        if (splits < 1) splits = 1;
        if (splits > kSimtMaxSplits) splits = kSimtMaxSplits;
    }
    // One split and a plain output wanted: the kernel normalises and stores o itself, no record, no combine launch.
    const bool direct = splits == 1 && p.o && !p.part_out && !p.exchange && !p.no_combine;
    if (!direct && (int64_t) groups * splits > p.max_segments) return fail_invalid("decode: workspace too small for the splits");
    if (!direct && (!p.ws_acc || !p.ws_ml)) return fail_invalid("decode: a workspace for the split records is required");
    SimtParams P;
    P.q = p.q;
    P.cache = p.cache;
    P.seq_lens = p.seq_lens;
    P.seq_base = p.seq_base;
    P.page_table = p.page_table;
    P.sel = p.sel;
    P.page_table_stride = p.page_table_stride;
    P.page_rows = p.page_rows > 0 ? p.page_rows : 1;
    P.sel_stride = p.sel_stride;
    P.scale = p.scale;
    P.tail_causal = p.tail_causal;
    P.ws_acc = p.ws_acc;
    P.ws_ml = p.ws_ml;
    P.o_direct = direct ? p.o : nullptr;
    P.T = p.T;
    P.H = p.H;
    P.d_qk = p.d_qk;
    P.d_v = p.d_v;
    P.splits = splits;
    const size_t smem = (size_t) HG * p.d_qk * 4 + (size_t) KT * p.d_qk * 2 + (size_t) HG * KT * 4 + 3 * HG * 4;
    dim3 grid(splits, n_hg, groups);
    // attributes are set on every call: a cached flag would go stale across a device reset
    P.scales = p.cache_scales;
    auto launch = [&](auto kernel) -> int {
        GS_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        kernel<<<grid, NT, smem, st>>>(P);
        return 0;
    };
    auto pick = [&](auto qtag, auto q8tag) -> int {
        using QT = decltype(qtag);
        constexpr bool Q8 = decltype(q8tag)::value;
        if (HG == 32) return launch(k_decode_gather<QT, Q8, 32>);
        if (HG == 16) return launch(k_decode_gather<QT, Q8, 16>);
        return launch(k_decode_gather<QT, Q8, 8>);
    };
    int e;
    if (p.cache_scales) {
        if (p.d_qk % 32 != 0) return fail_invalid("decode: a Q8 cache needs d_qk % 32 == 0");
        e = p.q_is_f32 ? pick(float{}, std::true_type{}) : pick(__half{}, std::true_type{});
    } else {
        e = p.q_is_f32 ? pick(float{}, std::false_type{}) : pick(__half{}, std::false_type{});
    }
    if (e) return e;
    GS_TRY(cudaGetLastError());
    if (p.ev_after_main) GS_TRY(cudaEventRecord(p.ev_after_main, st));
    if (p.no_combine || direct) return 0;
    CombinePlan c{};
    c.acc = p.ws_acc;
    c.ml = p.ws_ml;
    c.desc = nullptr;
    c.regular_segments = splits;
    c.seg_stride_acc = (int64_t) p.H * p.d_v;
    c.seg_stride_ml = (int64_t) p.H * 2;
    c.n_seq = p.n_seq;
    c.T = p.T;
    c.H = p.H;
    c.d_v = p.d_v;
    c.o = p.o;
    c.part_out = p.part_out;
    if (p.exchange) return launch_exchange_combine(c, *p.exchange, p.o, p.status, p.sm_count, st);
    return launch_combine(c, st);
}

}  // namespace gs
