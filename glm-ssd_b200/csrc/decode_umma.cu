// Absorbed-MLA decode on the Blackwell tensor cores (tcgen05 + TMEM), fed by TMA.
//
// What it computes is the contract of the reference kernel (crates/cuda/kernels/ops.cu:420-424):
// scores of every query row against the attended cache rows, softmax, and the probability-weighted
// sum of the same rows' first d_v columns, emitted as split partials (unnormalised acc, m, l) that
// the combine kernel merges (ops.cu:539-574).  How it computes it is specific to sm_100a:
//
//  * One persistent CTA per SM.  The 16-row units (64-row pages when paged) of all sequences are
//    cut into equal contiguous chunks, one per CTA; the part of a sequence inside a chunk is a
//    "segment" and yields one partial record.  The cache is read from HBM exactly once.
//  * A producer warp streams 64-row cache tiles into a two-stage shared-memory ring with TMA
//    (128-byte swizzle, one 64x64 box per 64-column block); the ragged last tile of a segment is
//    fetched in 16-row boxes so no row outside the segment is read.
//  * The contraction is small on the query side (T*H = 20..48 rows; 64 in the position-list form for 64
//    heads over 512-column rows, with two issuing warps instead of three), so the cache rows fill the
//    128-lane datapath and the packed query rows (all heads of all query tokens) ride on the MMA's
//    N side:  S^T[64 x NQ] = C_tile[64 x d_qk] . Q^T   (M = 64 cache rows, K-major operands),
//             O^T[128 x NQ] += V^T[128 x 64] . P^T     (M = 128 value columns; the SAME shared-memory
//    tile, now read MN-major), with both accumulators in tensor memory.  Padding 20 query rows to
//    the 64/128 rows of an M tile instead would spend 3-6x the tensor time on zeros and push the
//    kernel from the HBM roofline to the tensor roofline.
//  * A 4-warp group reads S^T from TMEM (one cache row per thread), does the online softmax with
//    warp-shuffle column maxima and a lazily updated reference maximum (the O accumulators are
//    rescaled only when a maximum grows by more than 2^6; in the common case one vote barrier per tile
//    replaces the reduction), writes P^T as f16 into shared memory in the canonical MN-major operand
//    layout, and at the end of a segment drains O^T from TMEM.
//  * Three warps issue the MMAs concurrently, each into its own accumulators (a single issuing thread
//    cannot keep the tensor pipe busy with MMAs this small); the softmax group adds the S^T partials.
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word and leaves
// through the common exit, which frees tensor memory.
#include <string.h>

#include <atomic>

#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {

typedef CUresult (*tmap_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The entry point is a host function of the driver library: it stays valid for the life of the process
// (also across a device reset), so it is looked up once.  Racing first calls store the same value.
static int tmap_encoder(tmap_encode_fn *out) {
    static std::atomic<void *> cached{nullptr};
    void *fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        cudaDriverEntryPointQueryResult qres;
        GS_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) {
            set_error("cuTensorMapEncodeTiled is not available from this driver");
            return (int) cudaErrorNotSupported;
        }
        cached.store(fn, std::memory_order_release);
    }
    *out = (tmap_encode_fn) fn;
    return 0;
}

int encode_tmap_2d_f16(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                       uint32_t box_rows, uint32_t box_cols, int swizzle) {
    tmap_encode_fn fn;
    if (int e = tmap_encoder(&fn)) return e;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, (CUtensorMapSwizzle) swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows %llu cols %llu box %ux%u)", (int) r,
                  (unsigned long long) rows, (unsigned long long) cols, box_rows, box_cols);
        return (int) cudaErrorInvalidValue;
    }
    return 0;
}

int encode_tmap_3d_f32(CUtensorMap *out, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                       uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
    tmap_encode_fn fn;
    if (int e = tmap_encoder(&fn)) return e;
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    const cuuint32_t box[3] = {b0, b1, b2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (3-D) failed with CUresult %d (dims %llu %llu %llu box %u %u %u)", (int) r,
                  (unsigned long long) d0, (unsigned long long) d1, (unsigned long long) d2, b0, b1, b2);
        return (int) cudaErrorInvalidValue;
    }
    return 0;
}

namespace {
using namespace sm100;

constexpr int TILE = 64;                 // cache rows per tile
constexpr int BLK_BYTES = TILE * 128;    // one 64-column block of a tile: 64 rows x 128 B
constexpr int NBLK_MAX = 9;              // 576 / 64
constexpr int STAGES = 2;
// A tile's blocks may complete separate barriers (groups of GRP blocks) so that the score MMAs of a group are issued as
// soon as it has landed.  Measured on the B200 with three groups of three: the boxes of a tile are requested together and
// land together, nothing starts earlier, and the extra barrier traffic costs 0.6 us per step at 32K rows (2.5 us at 128K).
// One group per tile it is.
constexpr int GRP = NBLK_MAX;
constexpr int NGRP = (NBLK_MAX + GRP - 1) / GRP;
constexpr int AHEAD = 2;                 // tiles of a CTA's range asked into L2 before the inputs are final (1-3 measured: 2 best)
constexpr int N_MMA_WARPS = 3;           // MMA warp slots (warps 1-3); a kernel form issues from the first NI of them
constexpr int NTHREADS = 32 * (1 + N_MMA_WARPS + 4);  // warp 0 producer, warps 1-3 MMA, warps 4-7 softmax group
constexpr int TMEM_COLS = 512;
// TMEM columns (slots of NQ columns): S^T partials [2 buffers][NI issuers], then the 4 O^T tiles:
// 10 x 48 = 480 of the 512 columns for NQ = 48 with three issuers, 8 x 64 = 512 for NQ = 64 with two
__host__ __device__ constexpr int issuers_for(int nq) { return nq > 48 ? 2 : 3; }
constexpr int NVT = 4;                   // 128-column value tiles (d_v = 512)
constexpr int MAX_SEQ = 1024;
constexpr int UNIT_CAP = 1 << 29;         // the running sum of units saturates here (two such values still add in an int)
constexpr float RESCALE_LOG2 = 6.0f;     // lazy rescale threshold, in log2 units
constexpr float LN2 = 0.6931471805599453f;

// status codes (bit flags) left in the workspace when a bounded wait gives up
enum { ST_PRODUCER = 1, ST_MMA = 2, ST_SOFTMAX = 4 };
// clock-stamp slots (tuning aid)
enum { PF_LOAD_ISSUE = 0, PF_KV_FULL = 1, PF_S_ISSUED = 2, PF_S_FULL = 3, PF_S_LOADED = 4, PF_VOTED = 5,
       PF_P_WRITTEN = 6, PF_P_FULL_SEEN = 7, PF_PV_ISSUED = 8, PF_SLOW_PATH = 9 };

// Sticky status word of the position-list form: the reference's entry point has no workspace that could carry one.
__device__ int32_t g_list_status[2];

struct UmmaParams {
    CUtensorMap tm_kv64, tm_kv16, tm_q;
    const int32_t *seq_lens, *seq_base, *page_table;
    int page_table_stride, paged;
    float scale_log2;
    int tail_causal;
    float *ws_acc, *ws_ml;
    int2 *ws_desc;
    int32_t *status;
    int n_seq, T, H, rows_q, d_v;  // H: heads handled by this launch (a group of the H_full heads of q)
    int H_full, h0;                // q holds H_full heads per token; this launch takes heads h0 .. h0+H-1
    // position-list form (the reference's sel / cnt): kernel sequence b attends rows sel[(b / seq_div) * sel_stride + i],
    // i < seq_lens[b / seq_div]; the rows are fetched by the producer warp with 16-byte asynchronous copies
    const void *list_cache;        // the cache as a plain pointer (rows of d_qk f16, or of d_qk int8 when list_scales is set)
    const __half *list_scales;     // Q8 cache (crates/cuda/kernels/ops.cu:427): one f16 scale per 32 values, [rows][d_qk / 32]
    const int32_t *sel;
    int sel_stride;
    const float *q_f32;            // list form: f32 queries [tokens][H_full][d_qk], rounded to f16 inside the kernel
    int whole_seq;                 // list form: every sequence is attended by one CTA, which normalises and stores o itself
    float *o;                      // whole_seq: output f32 [tokens][H_out][d_v]
    int H_out;
    int seg_cap;                   // segments the record arrays hold
    int seq_div;                   // >= 1: kernel sequence b reads the length / base / pages of caller sequence b / seq_div
                                   // (T = 1 only: the head groups of a sequence as sequences of their own)
    int64_t cache_rows;
};

struct Barriers {
    uint64_t kv_full[STAGES][NGRP], kv_empty[STAGES];
    uint64_t kv_raw[STAGES];  // Q8 list form: the int8 rows and scales of a tile have landed (not yet widened)
    uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2];
    uint64_t q_full, q_empty, o_full, o_empty;
};

// NQ <= 48: stages and query rows sized for the widest row (576 columns), one layout for both row widths.  NQ = 64 (only
// built for 512-column rows): sized by the row width, or two stages, the query rows and P would not fit.
template <int NQ, int NBLK = NBLK_MAX, bool Q8 = false>
struct Smem {
    static constexpr int SBLK = (NQ > 48 || Q8) ? NBLK : NBLK_MAX;   // 64-column blocks a stage and the query rows are sized for
    static constexpr int STAGE = SBLK * BLK_BYTES;
    static constexpr int Q_BYTES = SBLK * NQ * 128;
    static constexpr int P_BYTES = NQ * TILE * 2;
    static constexpr int OFF_Q = STAGES * STAGE;
    static constexpr int OFF_P = OFF_Q + Q_BYTES;
    static constexpr int QS_BYTES = Q8 ? TILE * (NBLK * 2) * 2 : 0;  // Q8: the tile's scales, NBLK * 2 halves per row
    static constexpr int OFF_QS = OFF_P + 2 * P_BYTES;
    static constexpr int OFF_MISC = OFF_QS + STAGES * QS_BYTES;
    struct Misc {
        Barriers bar;
        uint32_t tmem_base;
        int abort_flag;
        int flag[2];
        int cum[MAX_SEQ + 1];
        int len[MAX_SEQ];
        int base[MAX_SEQ];
        float smax[4][NQ];
        float sl[4][NQ];
        float mref[NQ];
        float f[NQ];
        int lim[NQ];
    };
    static constexpr int TOTAL = OFF_MISC + (int) sizeof(Misc) + 1024;  // + slack for the 1024-byte alignment
    static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

struct Segment {
    int b, r0, r1, len, n_tiles, seg_id;
};

// The schedule as every thread holds it.  With one sequence (the decode and MTP-verify calls) it lives in registers:
// no shared-memory arrays, no scan, no search and no block barrier between reading the length and the first copy.
struct Sched {
    int total, chunk, start, end, b0;
    int len0, base0;  // single sequence: its (capped) length and first row
    bool single;
    bool whole;       // sequences are not cut: CTA c attends sequences c, c + grid, ... from their first row to their last
};

// Walks the segments of this CTA's unit range [pos, end); `b` is a cursor over sequences.
__device__ __forceinline__ bool next_segment(int &pos, int &b, int end, const int *cum, int unit_rows,
                                             const int *seq_lens, Segment &sg, const Sched &sc) {
    if (sc.whole) {
        // `b` walks this CTA's sequences; empty ones yield no segment (their output rows are zeroed up front)
        int len = 0;
        while (b < sc.total && (len = sc.single ? sc.len0 : seq_lens[b]) <= 0) b += (int) gridDim.x;
        if (b >= sc.total) return false;
        sg.b = b;
        sg.len = len;
        sg.r0 = 0;
        sg.r1 = len;
        sg.n_tiles = (len + TILE - 1) / TILE;
        sg.seg_id = 0;
        b += (int) gridDim.x;
        return true;
    }
    if (pos >= end) return false;
    if (sc.single) {
        sg.b = 0;
        sg.len = sc.len0;
        sg.r0 = pos * unit_rows;
        sg.r1 = min(sc.len0, end * unit_rows);
        sg.n_tiles = (sg.r1 - sg.r0 + TILE - 1) / TILE;
        sg.seg_id = blockIdx.x;
        pos = end;
        return true;
    }
    while (cum[b + 1] <= pos) b++;
    const int u_lo = pos - cum[b];
    const int u_hi = min(end, cum[b + 1]) - cum[b];
    sg.b = b;
    sg.len = seq_lens[b];
    sg.r0 = u_lo * unit_rows;
    sg.r1 = min(sg.len, u_hi * unit_rows);
    sg.n_tiles = (sg.r1 - sg.r0 + TILE - 1) / TILE;
    sg.seg_id = blockIdx.x + b;
    pos = cum[b] + u_hi;
    return true;
}

// barrier among the softmax group that also ORs a predicate over its threads
__device__ __forceinline__ bool group_any(int id, int n_threads, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .pred p, r;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.or.pred r, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, r;\n\t"
        "}\n"
        : "=r"(out)
        : "r"((uint32_t) pred), "r"(id), "r"(n_threads)
        : "memory");
    return out != 0;
}

// P.V for the O^T tiles [MT_LO, MT_HI): nk 16-row k-steps, fully unrolled
template <int NQ, int MT_LO, int MT_HI, int O_SLOT0>
__device__ __forceinline__ void issue_pv(uint32_t tmem, uint64_t d_vt, uint64_t d_pt, uint32_t kv_lo, uint32_t p_lo,
                                         uint32_t idesc, int nk, bool acc0) {
    if (nk == 4) {
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int mt = MT_LO; mt < MT_HI; mt++)
                umma_ss(tmem + (O_SLOT0 + mt) * NQ, d_vt + (kv_lo + 2 * mt * (BLK_BYTES >> 4) + ks * 128), d_pt + (p_lo + ks * 16),
                        idesc, acc0 || ks > 0);
    } else {
#pragma unroll
        for (int ks = 0; ks < 3; ks++)
            if (ks < nk) {
#pragma unroll
                for (int mt = MT_LO; mt < MT_HI; mt++)
                    umma_ss(tmem + (O_SLOT0 + mt) * NQ, d_vt + (kv_lo + 2 * mt * (BLK_BYTES >> 4) + ks * 128),
                            d_pt + (p_lo + ks * 16), idesc, acc0 || ks > 0);
            }
    }
}

template <int NQ, int NBLK, bool LIST, bool Q8 = false>
__global__ void __launch_bounds__(NTHREADS, 1) k_decode_umma(const __grid_constant__ UmmaParams P) {
    static_assert(!Q8 || LIST, "the Q8 cache comes with position lists only");
    using SM = Smem<NQ, NBLK, Q8>;
    constexpr int NI = issuers_for(NQ);   // issuing MMA warps
    constexpr int O_SLOT0 = 2 * NI;       // first O^T slot in tensor memory
    constexpr int STAGE_BYTES = SM::STAGE;
    static_assert((O_SLOT0 + 4) * NQ <= TMEM_COLS, "tensor memory columns");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t *kv_smem = smem;
    uint8_t *q_smem = smem + SM::OFF_Q;
    uint8_t *p_smem = smem + SM::OFF_P;
    uint8_t *qs_smem = smem + SM::OFF_QS;
    typename SM::Misc &M = *reinterpret_cast<typename SM::Misc *>(smem + SM::OFF_MISC);
    Barriers &B = M.bar;
    volatile int *abort_flag = &M.abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit_rows = P.paged ? TILE : 16;
    int32_t *const status_w = LIST ? g_list_status : P.status;  // where a wait that gives up leaves its code

    // optional clock stamps of CTA 0's first tiles
    long long *prof = nullptr;
    if (blockIdx.x == 0 && P.status && P.status[1] != 0)
        prof = reinterpret_cast<long long *>(reinterpret_cast<char *>(P.status) + kProfOffsetBytes);
#define GS_STAMP(tile, slot)                                                                     \
    do {                                                                                         \
        if (prof && (tile) < (uint32_t) kProfTiles) prof[(tile) * kProfSlots + (slot)] = clock64(); \
    } while (0)

    long long *cta_prof = nullptr;  // wall-clock stamps of every CTA
    if (P.status && P.status[1] != 0)
        cta_prof = reinterpret_cast<long long *>(reinterpret_cast<char *>(P.status) + kCtaProfOffsetBytes) + blockIdx.x * 8;
#define GS_CTA_STAMP(slot)                              \
    do {                                                \
        if (cta_prof) cta_prof[slot] = global_timer_ns(); \
    } while (0)
    if (tid == 0) GS_STAMP(kProfTiles - 1, 0);  // kernel-level stamps live in the last row
    if (tid == 0) {
        GS_CTA_STAMP(0);
        if (cta_prof) cta_prof[6] = sm_id();
    }
    // ---- set-up: barriers, tensor memory, the unit schedule -------------------------------------------
    if (tid == 0) {
        tma_prefetch_desc(&P.tm_kv64);
        tma_prefetch_desc(&P.tm_kv16);
        tma_prefetch_desc(&P.tm_q);
        for (int s = 0; s < STAGES; s++) {
            // list form: one arrival per producer lane; Q8 list form: one per softmax warp, after the widening
            for (int g = 0; g < NGRP; g++) mbar_init(&B.kv_full[s][g], Q8 ? 4 : LIST ? 32 : 1);
            mbar_init(&B.kv_raw[s], 32);
            mbar_init(&B.kv_empty[s], NI);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(&B.s_full[s], NI);
            mbar_init(&B.s_empty[s], 4);
            mbar_init(&B.p_full[s], 4);
            mbar_init(&B.p_empty[s], NI);
        }
        mbar_init(&B.q_full, (LIST && P.q_f32) ? 4 : 1);  // f32 queries are converted by the four softmax warps
        mbar_init(&B.q_empty, NI);
        mbar_init(&B.o_full, NI);
        mbar_init(&B.o_empty, 4);
        M.abort_flag = 0;
        M.flag[0] = M.flag[1] = 0;
        M.cum[0] = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(&M.tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    // The schedule: units per sequence, their running sum, this CTA's chunk and the sequence it starts in.
    Sched sc;
    sc.single = P.n_seq == 1;
    sc.whole = LIST && P.whole_seq;
    sc.total = 0;
    sc.chunk = 1;
    sc.start = sc.end = sc.b0 = 0;
    sc.len0 = sc.base0 = 0;
    auto build_schedule = [&]() {
        // the small per-sequence inputs are read by every CTA on every call: ask L2 to keep them
        const uint64_t pol_keep = l2_policy_evict_last();
        // A length is taken as at most what the cache (or the sequence's row of the page table) can hold,
        // and the running sum below saturates: whatever the arrays contain - they are read once before they
        // are final - the schedule stays monotone and every index derived from it stays in range.
        const int64_t len_cap = min(P.paged ? (int64_t) P.page_table_stride * TILE : P.cache_rows,
                                    (int64_t) 0x7fffffff - 64);  // the rounding up to units below stays in an int
        if (sc.single) {
            // one sequence: every thread reads the one length word itself and derives its CTA's range in registers
            sc.len0 = (int) min((int64_t) max(ld_global_hint(P.seq_lens, pol_keep), 0), len_cap);
            sc.base0 = P.seq_base ? ld_global_hint(P.seq_base, pol_keep) : 0;
            sc.total = (sc.len0 + unit_rows - 1) / unit_rows;
        } else {
            for (int b = tid; b < P.n_seq; b += NTHREADS) {
                const int len = (int) min((int64_t) max(ld_global_hint(P.seq_lens + b / P.seq_div, pol_keep), 0), len_cap);
                M.base[b] = P.seq_base ? ld_global_hint(P.seq_base + b / P.seq_div, pol_keep) : 0;
                M.len[b] = len;
                M.cum[b + 1] = (len + unit_rows - 1) / unit_rows;  // < 2^27
            }
            tc_fence_before();
            __syncthreads();
            if (warp == 0) {  // inclusive scan of cum[1..n_seq], 32 entries per step
                int carry = 0;
                for (int base = 1; base <= P.n_seq; base += 32) {
                    const int i = base + lane;
                    int v = i <= P.n_seq ? M.cum[i] : 0;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int u = __shfl_up_sync(0xffffffffu, v, o);
                        if (lane >= o) v = min(v + u, UNIT_CAP);
                    }
                    v = min(v + carry, UNIT_CAP);
                    if (i <= P.n_seq) M.cum[i] = v;
                    carry = __shfl_sync(0xffffffffu, v, 31);
                }
            }
            __syncthreads();
            tc_fence_after();
            sc.total = M.cum[P.n_seq];
        }
        sc.chunk = max(1, (sc.total + (int) gridDim.x - 1) / (int) gridDim.x);
        sc.start = min(sc.total, (int) blockIdx.x * sc.chunk);
        sc.end = min(sc.total, sc.start + sc.chunk);
        sc.b0 = 0;
        if (sc.whole) {  // sequences dealt round-robin; `total` counts sequences, the cursor starts at this CTA's first
            sc.total = P.n_seq;
            sc.b0 = (int) blockIdx.x;
            return;
        }
        if (!sc.single) {
            // first sequence of this CTA's range (binary search: largest b with cum[b] <= start)
            int lo = 0, hi = P.n_seq - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (M.cum[mid] <= sc.start) lo = mid; else hi = mid - 1;
            }
            sc.b0 = lo;
        }
    };
    // Everything above touched only this CTA's own resources.  While the kernel in front of this one is still
    // running (programmatic dependent launch), the schedule is built once from whatever the length / base /
    // page arrays hold at the moment - the values of the previous step when that kernel is about to update
    // them - and the first tiles of this CTA's range are asked into L2.  Nothing read here is used for a
    // result: a stale value costs a useless prefetch, and every index is checked before it is followed.
    build_schedule();
    if (!LIST && warp == 0) {
        int pp = sc.start, bb = sc.b0, asked = 0;
        Segment s2;
        while (asked < AHEAD && next_segment(pp, bb, sc.end, M.cum, unit_rows, M.len, s2, sc)) {
            for (int j = 0; j < s2.n_tiles && asked < AHEAD; j++, asked++) {
                const int row = s2.r0 + j * TILE;
                int64_t grow = -1;
                if (!P.paged) grow = (int64_t) (sc.single ? sc.base0 : M.base[s2.b]) + row;
                else if (row >= 0 && row / TILE < P.page_table_stride)
                    grow = (int64_t) P.page_table[(int64_t) (s2.b / P.seq_div) * P.page_table_stride + row / TILE] * TILE;
                if (grow >= 0 && grow < P.cache_rows && elect_one()) {
#pragma unroll
                    for (int k = 0; k < NBLK; k++) tma_prefetch_2d(&P.tm_kv64, k * 64, (int) grow);
                }
                __syncwarp();
            }
        }
    }
    // barrier initialisation and the tensor-memory address become visible to every warp here; with several
    // sequences it is also the barrier in front of rebuilding the shared-memory arrays
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();
    if (tid == 0) GS_CTA_STAMP(1);
    build_schedule();
    const uint32_t tmem = M.tmem_base;
    if (blockIdx.x == 0 && P.ws_desc && !sc.whole) {  // where the combine kernel finds each sequence's segments
        if (sc.single) {
            if (tid == 0) P.ws_desc[0] = sc.total > 0 ? make_int2(0, (sc.total - 1) / sc.chunk + 1) : make_int2(0, 0);
        } else {
            for (int b = tid; b < P.n_seq; b += NTHREADS) {
                const int u0 = M.cum[b], u1 = M.cum[b + 1];
                int2 d = make_int2(0, 0);
                if (u1 > u0) {
                    const int c_first = u0 / sc.chunk, c_last = (u1 - 1) / sc.chunk;
                    d = make_int2(c_first + b, c_last - c_first + 1);
                }
                P.ws_desc[b] = d;
            }
        }
    }
    griddep_launch_dependents();
    if (tid == 0) GS_STAMP(kProfTiles - 1, 1);
    int pos = sc.start, b_cur = sc.b0;
    const int end = sc.end;
    uint32_t it = 0, sgc = 0;  // running tile and segment counters (identical in every role)
    Segment sg;

    if (warp == 0) {
        // =================================== TMA producer ==================================================
        // The whole warp runs the loop (uniform control flow); one elected lane issues each copy.
        bool ok = true;
        const uint64_t pol_stream = l2_policy_evict_first();  // every cache row is read once per step
        while (ok && next_segment(pos, b_cur, end, M.cum, unit_rows, M.len, sg, sc)) {
            const int64_t base_row = sc.single ? sc.base0 : M.base[sg.b];
            for (int j = 0; j < sg.n_tiles; j++, it++) {
                const int s = it & 1;
                ok = mbar_wait(&B.kv_empty[s], ((it >> 1) & 1) ^ 1, abort_flag, status_w, ST_PRODUCER);
                if (!ok) break;
                if (lane == 0) GS_STAMP(it, PF_LOAD_ISSUE);
                if (lane == 0 && it == 0) GS_CTA_STAMP(7);
                const int row = sg.r0 + j * TILE;
                const int valid = min(TILE, sg.r1 - row);
                uint8_t *dst = kv_smem + s * STAGE_BYTES;
                if (LIST && Q8) {
                    // Q8 cache: the listed rows arrive as they are - 512 bytes of int8 per row (one 16-byte copy per lane)
                    // into the upper half of the stage, their scales (32 bytes per row) beside the stages - and the
                    // softmax warps widen them to f16 in place before the MMAs see the stage (see there).
                    const int32_t *lp = P.sel + (int64_t) (sg.b / P.seq_div) * P.sel_stride + row;
                    const int ra = lane < valid ? max(lp[lane], 0) : 0, rb = lane + 32 < valid ? max(lp[lane + 32], 0) : 0;
                    const char *qbase = reinterpret_cast<const char *>(P.list_cache);
                    const char *sbase = reinterpret_cast<const char *>(P.list_scales);
                    uint8_t *raw = dst + STAGE_BYTES / 2;
                    uint8_t *qs = qs_smem + s * SM::QS_BYTES;
#pragma unroll 4
                    for (int r = 0; r < valid; r++) {
                        const int grow = __shfl_sync(0xffffffffu, r < 32 ? ra : rb, r & 31);
                        cp_async16_hint(raw + r * (NBLK * 64) + lane * 16, qbase + (int64_t) grow * (NBLK * 64) + lane * 16, pol_stream);
                    }
#pragma unroll
                    for (int k = 0; k < TILE / 16; k++) {  // scales: two 16-byte halves per row, sixteen rows per instruction
                        const int r = k * 16 + (lane >> 1);
                        const int ga = __shfl_sync(0xffffffffu, ra, r & 31), gb = __shfl_sync(0xffffffffu, rb, r & 31);
                        const int grow = r < 32 ? ga : gb;
                        if (r < valid)
                            cp_async16_hint(qs + r * (NBLK * 4) + (lane & 1) * 16, sbase + (int64_t) grow * (NBLK * 4) + (lane & 1) * 16, pol_stream);
                    }
                    cp_async_mbar_arrive(&B.kv_raw[s]);
                    __syncwarp();
                } else if (LIST) {
                    // Rows named by the position list.  Lane l holds the cache rows of tile rows l and l + 32; every warp
                    // instruction copies 512 contiguous bytes of one listed row (16 bytes per lane) to the place the tiled
                    // copy of the dense form would have put them: 64-column block c / 8, 16-byte chunk (c % 8) xor (r % 8)
                    // of row r.  Each lane's arrival on the stage's barrier follows its own copies.
                    // (Measured per 64-row tile of 64 KB, rows already in L2: these copies 2.6 us, the same when four warps
                    // share the issuing; TMA gather copies of four rows x 64 columns, 128 per tile, 5.9 us issued lane by
                    // lane from one warp, 3.6 us with one copy per lane from four warps.  A listed row is 1 KB somewhere:
                    // about 20-25 GB/s per SM whatever issues the requests, against 44 GB/s and more for the tiled copies
                    // of consecutive rows.  Splitting a tile between the two paths does not add them up: with 16, 24 or 32
                    // of the 64 rows on gather copies and the rest on these copies the T = 256 shape took 468, 549 and 589 us
                    // against 343 us, and an evict-last hint on the listed rows 367 us.  Asking for the next tile's list
                    // entries a tile ahead (346 us) or dropping the eviction hint (339 us) changes nothing either: for that
                    // shape the profiler shows L2 at 7 %, DRAM at 4 % and the L1 fill path at 8 % of their peaks - the
                    // copies are bound by what one SM keeps in flight, two 64 KB tiles against 3.2 us of latency each.)
                    const int32_t *lp = P.sel + (int64_t) (sg.b / P.seq_div) * P.sel_stride + row;
                    const int ra = lane < valid ? max(lp[lane], 0) : 0, rb = lane + 32 < valid ? max(lp[lane + 32], 0) : 0;
                    constexpr int CPR = NBLK * 8;  // 16-byte chunks per row
                    const char *cbase = reinterpret_cast<const char *>(P.list_cache);
#pragma unroll 4
                    for (int r = 0; r < valid; r++) {
                        const int grow = __shfl_sync(0xffffffffu, r < 32 ? ra : rb, r & 31);
                        const char *src = cbase + (int64_t) grow * (NBLK * 128);
                        uint8_t *drow = dst + r * 128;
#pragma unroll
                        for (int c0 = 0; c0 < CPR; c0 += 32) {
                            const int c = c0 + lane;
                            if (c < CPR) cp_async16_hint(drow + (c >> 3) * BLK_BYTES + (((c & 7) ^ (r & 7)) << 4), src + c * 16, pol_stream);
                        }
                    }
                    cp_async_mbar_arrive(&B.kv_full[s][0]);
                    __syncwarp();
                } else if (P.paged || valid == TILE) {
                    const int grow = P.paged ? P.page_table[(int64_t) (sg.b / P.seq_div) * P.page_table_stride +
                                                            min(max(row / TILE, 0), P.page_table_stride - 1)] * TILE
                                             : (int) (base_row + row);
                    if (elect_one()) {
#pragma unroll
                        for (int g = 0; g < NGRP; g++) {
                            const int k_lo = g * GRP, k_hi = min(NBLK, g * GRP + GRP);
                            mbar_arrive_expect_tx(&B.kv_full[s][g], (uint32_t) ((k_hi - k_lo) * BLK_BYTES));
#pragma unroll
                            for (int k = 0; k < GRP; k++)
                                if (k_lo + k < k_hi)
                                    tma_load_2d_hint(dst + (k_lo + k) * BLK_BYTES, &P.tm_kv64, &B.kv_full[s][g], (k_lo + k) * 64, grow, pol_stream);
                        }
                    }
                } else {
                    const int ng = (valid + 15) >> 4;
                    if (elect_one()) {
#pragma unroll
                        for (int g = 0; g < NGRP; g++) {
                            const int k_lo = g * GRP, k_hi = min(NBLK, g * GRP + GRP);
                            mbar_arrive_expect_tx(&B.kv_full[s][g], (uint32_t) (ng * (k_hi - k_lo) * 2048));
                            for (int r = 0; r < ng; r++) {
#pragma unroll
                                for (int k = 0; k < GRP; k++)
                                    if (k_lo + k < k_hi)
                                        tma_load_2d_hint(dst + (k_lo + k) * BLK_BYTES + r * 2048, &P.tm_kv16, &B.kv_full[s][g], (k_lo + k) * 64,
                                                         (int) (base_row + row + r * 16), pol_stream);
                            }
                        }
                    }
                }
                if (j == 0 && !(LIST && P.q_f32)) {  // the query rows of this sequence, after the first (larger, farther) cache tile
                    ok = mbar_wait(&B.q_empty, (sgc & 1) ^ 1, abort_flag, status_w, ST_PRODUCER);
                    if (!ok) break;
                    if (elect_one()) {
                        if (P.H_full == P.H) {  // the sequence's T*H query rows are contiguous: one box per block
                            mbar_arrive_expect_tx(&B.q_full, (uint32_t) (NBLK * NQ * 128));
#pragma unroll
                            for (int k = 0; k < NBLK; k++)
                                tma_load_2d(q_smem + k * NQ * 128, &P.tm_q, &B.q_full, k * 64, sg.b * P.rows_q);
                        } else {  // a head group: H rows per token (H % 8 == 0, so every box starts on a swizzle atom)
                            mbar_arrive_expect_tx(&B.q_full, (uint32_t) (NBLK * P.rows_q * 128));
                            for (int t = 0; t < P.T; t++) {
#pragma unroll
                                for (int k = 0; k < NBLK; k++)
                                    tma_load_2d(q_smem + k * NQ * 128 + t * P.H * 128, &P.tm_q, &B.q_full, k * 64,
                                                ((sg.b / P.seq_div) * P.T + t) * P.H_full + P.h0 + (sg.b % P.seq_div) * P.H);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            sgc++;
        }
    } else if (warp <= NI) {
        // =================================== MMA issuers ====================================================
        // Three warps issue concurrently: one issuer cannot keep the tensor pipe busy with MMAs this
        // small.  Each warp owns its accumulators: a third of the 16-column k-steps of S^T (partial sums,
        // added by the softmax group) and one or two of the four 128-column O^T tiles.  The whole warp runs
        // the loop; one elected lane (the same one every time) issues the MMAs and their commits.
        const int mw = warp - 1;
        constexpr uint32_t idesc_s = make_idesc_f16(64, NQ, 0, 0);    // A, B K-major
        constexpr uint32_t idesc_pv = make_idesc_f16(128, NQ, 1, 1);  // A (V^T) and B (P^T) MN-major
        constexpr int KSTEPS = NBLK * 4;
        constexpr int K_PER = (KSTEPS + NI - 1) / NI;
        // the landing groups this warp's score k-steps read
        const int g_lo = ((mw * K_PER) >> 2) / GRP, g_hi = ((min(KSTEPS, (mw + 1) * K_PER) - 1) >> 2) / GRP;
        constexpr int g_all = NGRP;
        const uint64_t d_kmaj = make_smem_desc(0, 16, 1024, kSwizzle128B);         // cache tile / Q, K-major
        const uint64_t d_vt = make_smem_desc(0, BLK_BYTES, 1024, kSwizzle128B);    // cache tile, MN-major
        const uint64_t d_pt = make_smem_desc(0, 128, 1024, kSwizzleNone);          // P^T, MN-major
        const uint32_t q_lo = smem_u32(q_smem) >> 4, p_lo0 = smem_u32(p_smem) >> 4, kv_lo0 = smem_u32(kv_smem) >> 4;
        bool ok = true;
        while (ok && next_segment(pos, b_cur, end, M.cum, unit_rows, M.len, sg, sc)) {
            ok = mbar_wait(&B.q_full, sgc & 1, abort_flag, status_w, ST_MMA);
            // S of tile j+1 is issued ahead of P.V of tile j whenever its data has already landed, so it
            // runs on the tensor pipe while the softmax of tile j is computed.
            auto issue_s = [&](uint32_t i) {
                const int s = i & 1;
                const uint32_t kv_lo = kv_lo0 + s * (STAGE_BYTES >> 4);
                tc_fence_after();
                if (LIST) fence_proxy_async_smem();  // the stage was filled by ordinary asynchronous copies, not by the TMA
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < K_PER; k++) {
                        const int kidx = mw * K_PER + k;
                        if (kidx < KSTEPS) {
                            const int kb = kidx >> 2, ks = kidx & 3;
                            umma_ss(tmem + (s * NI + mw) * NQ, d_kmaj + (kv_lo + kb * (BLK_BYTES >> 4) + ks * 2),
                                    d_kmaj + (q_lo + kb * (NQ * 128 >> 4) + ks * 2), idesc_s, k != 0);
                        }
                    }
                    umma_commit(&B.s_full[s]);
                }
                __syncwarp();
            };
            bool s_ahead = false;  // S of the current tile was already issued during the previous iteration
            for (int j = 0; ok && j < sg.n_tiles; j++, it++) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const uint32_t kv_lo = kv_lo0 + s * (STAGE_BYTES >> 4);
                if (!s_ahead) {
                    ok = mbar_wait(&B.s_empty[s], ph ^ 1, abort_flag, status_w, ST_MMA);
                    for (int g = g_lo; ok && g <= g_hi; g++) ok = mbar_wait(&B.kv_full[s][g], ph, abort_flag, status_w, ST_MMA);
                    if (!ok) break;
                    if (mw == 0 && lane == 0) GS_STAMP(it, PF_KV_FULL);
                    if (mw == 0 && lane == 0 && it == 0) GS_CTA_STAMP(2);
                    issue_s(it);
                    if (mw == 0 && lane == 0) GS_STAMP(it, PF_S_ISSUED);
                }
                s_ahead = false;
                if (j + 1 < sg.n_tiles) {
                    const uint32_t i1 = it + 1;
                    const uint32_t ph1 = (i1 >> 1) & 1;
                    // uniform over the warp: every lane polls the same barriers
                    bool landed = mbar_test(&B.s_empty[i1 & 1], ph1 ^ 1);
                    for (int g = g_lo; g <= g_hi; g++) landed = landed && mbar_test(&B.kv_full[i1 & 1][g], ph1);
                    if (__all_sync(0xffffffffu, landed)) {
                        if (mw == 0 && lane == 0) GS_STAMP(i1, PF_KV_FULL);
                        issue_s(i1);
                        if (mw == 0 && lane == 0) GS_STAMP(i1, PF_S_ISSUED);
                        s_ahead = true;
                    }
                }
                // ---- O^T[my tiles] += V^T . P^T ----
                ok = mbar_wait(&B.p_full[s], ph, abort_flag, status_w, ST_MMA);
                // P.V reads every value block of the tile: all groups (they have landed: the scores the softmax
                // just turned into P needed them; the waits return at once and make that landing visible here)
                for (int g = 0; ok && g < g_all; g++) ok = mbar_wait(&B.kv_full[s][g], ph, abort_flag, status_w, ST_MMA);
                if (ok && j == 0) ok = mbar_wait(&B.o_empty, (sgc & 1) ^ 1, abort_flag, status_w, ST_MMA);
                if (!ok) break;
                if (mw == 0 && lane == 0) GS_STAMP(it, PF_P_FULL_SEEN);
                tc_fence_after();
                if (LIST) fence_proxy_async_smem();
                const int valid = min(TILE, sg.r1 - (sg.r0 + j * TILE));
                const int nk = (valid + 15) >> 4;
                const uint32_t p_lo = p_lo0 + s * (SM::P_BYTES >> 4);
                const bool acc0 = j > 0;
                const bool last = j == sg.n_tiles - 1;
                if (elect_one()) {
                    if (mw == 0) issue_pv<NQ, 0, 2, O_SLOT0>(tmem, d_vt, d_pt, kv_lo, p_lo, idesc_pv, nk, acc0);
                    else if (NI == 2) issue_pv<NQ, 2, 4, O_SLOT0>(tmem, d_vt, d_pt, kv_lo, p_lo, idesc_pv, nk, acc0);
                    else if (mw == 1) issue_pv<NQ, 2, 3, O_SLOT0>(tmem, d_vt, d_pt, kv_lo, p_lo, idesc_pv, nk, acc0);
                    else issue_pv<NQ, 3, 4, O_SLOT0>(tmem, d_vt, d_pt, kv_lo, p_lo, idesc_pv, nk, acc0);
                    umma_commit(&B.kv_empty[s]);
                    umma_commit(&B.p_empty[s]);
                    if (last) {
                        umma_commit(&B.o_full);
                        umma_commit(&B.q_empty);
                    }
                }
                __syncwarp();
                if (mw == 0 && lane == 0) GS_STAMP(it, PF_PV_ISSUED);
            }
            sgc++;
        }
    } else if (warp > N_MMA_WARPS) {  // (with two issuers warp 3 has no part)
        // =================================== softmax / epilogue group ==========================================
        const int wg_tid = tid - 32 * (1 + N_MMA_WARPS);
        const int qt = warp & 3;                      // TMEM lane quarter this warp may touch
        const uint32_t lane_base = (uint32_t) (qt * 32) << 16;
        const int my_row = qt * 16 + (lane & 15);     // cache row (within the tile) this lane works on
        constexpr float UNSET = 1e30f;                // "-reference" of a column that has seen no attended row
        // After the scores are read (one cache row per thread, lanes 0..15), the upper half of the query
        // rows is handed to lanes 16..31, so every lane works on HQ = NQ/2 query rows of one cache row.
        constexpr int HQ = NQ / 2;
        const int hi = lane >> 4;                     // which half of the query rows this lane handles
        const int col0 = hi * HQ;
        const uint64_t pol_keep = l2_policy_evict_last();  // the partial records are read next, by the combine kernel
        float l_part[HQ];                             // row sums of this thread's cache row, per query row
        float nm[HQ];                                 // minus the reference maximum (log2 units) per query row
        bool ok = true;
        if (LIST && sc.whole) {
            // a query that attends nothing gets zeros (crates/cuda/kernels/ops.cu:535); such sequences yield no segment
            for (int b = (int) blockIdx.x; b < P.n_seq; b += (int) gridDim.x) {
                if ((sc.single ? sc.len0 : M.len[b]) > 0) continue;
                float *dst = P.o + ((int64_t) (b / P.seq_div) * P.H_out + (b % P.seq_div) * P.H) * P.d_v;
                for (int i = wg_tid; i < P.rows_q * P.d_v; i += 128) dst[i] = 0.f;
            }
        }
        while (ok && next_segment(pos, b_cur, end, M.cum, unit_rows, M.len, sg, sc)) {
            if (LIST && P.q_f32) {
                // f32 queries: the four warps round this sequence's rows to f16 straight into the operand layout the
                // TMA would have produced (64-column blocks of [NQ rows][128 bytes], 16-byte chunk j of row r at chunk
                // position j ^ (r % 8)), once the MMAs of the previous sequence have finished with the old rows
                (void) mbar_wait(&B.q_empty, (sgc & 1) ^ 1, abort_flag, status_w, ST_SOFTMAX);
                const float *qsrc = P.q_f32 + ((int64_t) (sg.b / P.seq_div) * P.H_full + (int64_t) (sg.b % P.seq_div) * P.H) * (NBLK * 64);
                constexpr int CPR = NBLK * 8;  // 16-byte chunks (8 columns) per row
                for (int i = wg_tid; i < NQ * CPR; i += 128) {
                    const int r = i / CPR, cc = i - r * CPR;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (r < P.rows_q) {
                        const float4 a = __ldg(reinterpret_cast<const float4 *>(qsrc + (int64_t) r * (NBLK * 64) + cc * 8));
                        const float4 b4 = __ldg(reinterpret_cast<const float4 *>(qsrc + (int64_t) r * (NBLK * 64) + cc * 8 + 4));
                        __half2 h;
                        h = __floats2half2_rn(a.x, a.y); v.x = *reinterpret_cast<uint32_t *>(&h);
                        h = __floats2half2_rn(a.z, a.w); v.y = *reinterpret_cast<uint32_t *>(&h);
                        h = __floats2half2_rn(b4.x, b4.y); v.z = *reinterpret_cast<uint32_t *>(&h);
                        h = __floats2half2_rn(b4.z, b4.w); v.w = *reinterpret_cast<uint32_t *>(&h);
                    }
                    const int kb = cc >> 3, jj = cc & 7;
                    *reinterpret_cast<uint4 *>(q_smem + kb * (NQ * 128) + r * 128 + ((jj ^ (r & 7)) << 4)) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.q_full);
            }
            if (wg_tid < NQ) {
                const int q = wg_tid, t = q / P.H;
                int lim = 0;
                if (q < P.rows_q) lim = P.tail_causal ? min(sg.r1, sg.len - (P.T - 1 - t)) : sg.r1;
                M.lim[q] = lim;
                M.mref[q] = -INFINITY;
            }
            // rows below lim_min are attended by every query row of the sequence
            const int lim_min = P.tail_causal ? min(sg.r1, sg.len - (P.T - 1)) : sg.r1;
#pragma unroll
            for (int i = 0; i < HQ; i++) {
                l_part[i] = 0.f;
                nm[i] = UNSET;
            }
            named_bar_sync(1, 128);
            // Q8 cache: widen tile i (the jj-th of this segment): int8 rows (upper half of the stage) x f16 scales ->
            // half_rn(scale * q) in the operand layout the f16 form's copies produce (crates/cuda/kernels/ops.cu:461-477 attends over
            // these values).  Each of the four warps takes 16 rows into registers; only when every raw row is in
            // registers are the f16 rows written, since they cover the raw area.  Rows past the segment's end become
            // zeros.  Done for the segment's first tile before its scores are awaited and for every further tile right
            // after the probabilities of the tile before are handed over, so that it runs beside that tile's P.V.
            // (Measured on 2052-row lists, 64 heads, T = 1 / 2 / 256: 24.9 / 53.4 / 473 us this way; 26.7 / 66.7 / 684 us
            // with the three issuing warps widening instead - fewer threads, two more barriers, and their MMAs late;
            // 24.2 / 55.1 / 484 us with one f16 stage filled from a ring of three stand-alone raw buffers - the copies
            // then never wait for a stage, but widening, scores, softmax and P.V of consecutive tiles no longer
            // overlap: the chain of hand-overs per tile, not the copies, is what the time follows.)
            auto widen_tile = [&](uint32_t i, int jj) {
                const int s = i & 1;
                (void) mbar_wait(&B.kv_raw[s], (i >> 1) & 1, abort_flag, status_w, ST_SOFTMAX);
                const int valid_q = min(TILE, sg.r1 - (sg.r0 + jj * TILE));
                uint8_t *stage = kv_smem + s * STAGE_BYTES;
                const uint8_t *raw = stage + STAGE_BYTES / 2;
                const uint8_t *qs = qs_smem + s * SM::QS_BYTES;
                uint4 rv[16];
#pragma unroll
                for (int k = 0; k < 16; k++) rv[k] = *reinterpret_cast<const uint4 *>(raw + (qt * 16 + k) * (NBLK * 64) + lane * 16);
                named_bar_sync(1, 128);
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const int r = qt * 16 + k;
                    // scale * q as an f16 product: q (|q| <= 127) is exact in f16 and the product of an 11-bit by a 7-bit
                    // significand is exact before the one rounding, so this is half_rn(scale * q) bit for bit.  The bytes
                    // become f16 through the 1024-offset trick: 0x6400 | (q + 128) is the f16 number 1152 + q.
                    const __half sc = r < valid_q ? *reinterpret_cast<const __half *>(qs + r * (NBLK * 4) + (lane >> 1) * 2) : __ushort_as_half(0);
                    const __half2 sc2 = __half2half2(sc), off2 = __half2half2(__ushort_as_half(0x6480));  // 1152
                    auto widen4 = [&](uint32_t w, uint32_t &h01, uint32_t &h23) {
                        const uint32_t u = w ^ 0x80808080u;
                        uint32_t a = __byte_perm(u, 0x64646464u, 0x5140), b2 = __byte_perm(u, 0x64646464u, 0x7362);
                        const __half2 x = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&a), off2), sc2);
                        const __half2 y = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&b2), off2), sc2);
                        h01 = *reinterpret_cast<const uint32_t *>(&x);
                        h23 = *reinterpret_cast<const uint32_t *>(&y);
                    };
                    uint4 lo, hi;
                    widen4(rv[k].x, lo.x, lo.y);
                    widen4(rv[k].y, lo.z, lo.w);
                    widen4(rv[k].z, hi.x, hi.y);
                    widen4(rv[k].w, hi.z, hi.w);
                    if (r >= valid_q) lo = hi = make_uint4(0, 0, 0, 0);  // (a stale byte times a zero scale is zero too; this says so)
                    // 16-byte chunks 2 * lane and 2 * lane + 1 of the row.  Lanes of every other 64-column block store
                    // their odd chunk first, so that one store instruction covers all eight chunk positions of the
                    // 128-byte lines (four lanes each) instead of four positions (eight lanes each).
                    const int flip = (lane >> 2) & 1;
                    const int c0 = lane * 2 + flip, c1 = lane * 2 + 1 - flip;
                    *reinterpret_cast<uint4 *>(stage + (c0 >> 3) * BLK_BYTES + r * 128 + (((c0 & 7) ^ (r & 7)) << 4)) = flip ? hi : lo;
                    *reinterpret_cast<uint4 *>(stage + (c1 >> 3) * BLK_BYTES + r * 128 + (((c1 & 7) ^ (r & 7)) << 4)) = flip ? lo : hi;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.kv_full[s][0]);
            };
            for (int j = 0; j < sg.n_tiles; j++, it++) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                if (Q8 && j == 0) widen_tile(it, 0);
                (void) mbar_wait(&B.s_full[s], ph, abort_flag, status_w, ST_SOFTMAX);
                GS_STAMP(it, PF_S_FULL);
                tc_fence_after();
                const int row0 = sg.r0 + j * TILE;
                const int rpos = row0 + my_row;
                const bool boundary = row0 + TILE > lim_min;  // some query row must not see some row of this tile
                // S^T row = sum of the issuers' partial accumulators; then split the query rows over the lane halves
                float sv[HQ];
#pragma unroll
                for (int c = 0; c < NQ / 16; c++) {
                    uint32_t r0[16], r1[16], r2[16];
                    tmem_ld16(tmem + lane_base + (s * NI + 0) * NQ + c * 16, r0);
                    tmem_ld16(tmem + lane_base + (s * NI + 1) * NQ + c * 16, r1);
                    if (NI > 2) tmem_ld16(tmem + lane_base + (s * NI + 2) * NQ + c * 16, r2);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int q = c * 16 + i;
                        float v = __uint_as_float(r0[i]) + __uint_as_float(r1[i]);
                        if (NI > 2) v += __uint_as_float(r2[i]);
                        // lanes 0..15 keep query rows [0, HQ), lanes 16..31 fetch [HQ, NQ) from lane - 16
                        if (q < HQ) {
                            if (!hi) sv[q] = v;
                        } else {
                            const float u = __shfl_sync(0xffffffffu, v, lane & 15);
                            if (hi) sv[q - HQ] = u;
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.s_empty[s]);
                GS_STAMP(it, PF_S_LOADED);
                if (boundary) {
#pragma unroll
                    for (int i = 0; i < HQ; i++)
                        if (rpos >= M.lim[col0 + i]) sv[i] = -INFINITY;
                }
                // does any score exceed its column's reference by the threshold (or meet an unset column)?
                bool exceed = false;
#pragma unroll
                for (int i = 0; i < HQ; i++) exceed |= fmaf(sv[i], P.scale_log2, nm[i]) > RESCALE_LOG2;
                // one barrier per tile: combines the vote and orders the group; on abort every thread leaves together
                const bool slow = group_any(2, 128, exceed);
                if (*abort_flag) { ok = false; break; }
                GS_STAMP(it, PF_VOTED);
                bool rescale = false;
                if (slow) {
                    // some column's maximum moved: exact column maxima, new references, rescale factors
                    GS_STAMP(it, PF_SLOW_PATH);
#pragma unroll
                    for (int i = 0; i < HQ; i++) {
                        float mx = sv[i] * P.scale_log2;
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                        if ((lane & 15) == 0) M.smax[qt][col0 + i] = mx;
                    }
                    named_bar_sync(1, 128);
                    if (wg_tid < NQ) {
                        const int q = wg_tid;
                        const float mt = fmaxf(fmaxf(M.smax[0][q], M.smax[1][q]), fmaxf(M.smax[2][q], M.smax[3][q]));
                        const float mr = M.mref[q];
                        float f = 1.f;
                        if (mt > mr + RESCALE_LOG2) {  // also true for mr = -inf and any finite mt
                            if (mr == -INFINITY) {
                                f = 0.f;
                            } else {
                                f = exp2f(mr - mt);
                                if (j > 0) M.flag[it & 1] = 1;  // accumulators hold data scaled by the old reference
                            }
                            M.mref[q] = mt;
                        }
                        M.f[q] = f;
                    }
                    if (wg_tid == 0) M.flag[(it + 1) & 1] = 0;
                    named_bar_sync(1, 128);
                    rescale = M.flag[it & 1] != 0;
#pragma unroll
                    for (int i = 0; i < HQ; i++) {
                        l_part[i] *= M.f[col0 + i];
                        const float mr = M.mref[col0 + i];
                        nm[i] = mr == -INFINITY ? UNSET : -mr;
                    }
                }
                (void) mbar_wait(&B.p_empty[s], ph ^ 1, abort_flag, status_w, ST_SOFTMAX);
                // probabilities: row sums in registers; P^T as f16, 8 query rows per 16-byte store, in the
                // MN-major operand layout [q/8][row/8][row%8][q%8].  A masked score is -inf and gives 0; an
                // unset column holds only masked scores.
                uint8_t *pbuf = p_smem + s * SM::P_BYTES + (my_row >> 3) * 128 + (my_row & 7) * 16 + (col0 >> 3) * 1024;
#pragma unroll
                for (int g = 0; g < HQ / 8; g++) {
                    float p[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        p[i] = ex2_approx(fmaf(sv[g * 8 + i], P.scale_log2, nm[g * 8 + i]));
                        l_part[g * 8 + i] += p[i];
                    }
                    uint4 v;
                    __half2 h;
                    h = __floats2half2_rn(p[0], p[1]); v.x = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2half2_rn(p[2], p[3]); v.y = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2half2_rn(p[4], p[5]); v.z = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2half2_rn(p[6], p[7]); v.w = *reinterpret_cast<uint32_t *>(&h);
                    *reinterpret_cast<uint4 *>(pbuf + g * 1024) = v;
                }
                if (rescale) {
                    // S of this tile may have been issued ahead of P.V of the previous one: wait for that P.V
                    (void) mbar_wait(&B.p_empty[s ^ 1], ((it - 1) >> 1) & 1, abort_flag, status_w, ST_SOFTMAX);
                    tc_fence_after();
#pragma unroll 1
                    for (int mt = 0; mt < NVT; mt++) {
#pragma unroll
                        for (int c = 0; c < NQ / 16; c++) {
                            uint32_t r[16];
                            const uint32_t addr = tmem + lane_base + (O_SLOT0 + mt) * NQ + c * 16;
                            tmem_ld16(addr, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 16; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * M.f[c * 16 + i]);
                            tmem_st16(addr, r);
                        }
                    }
                    tmem_wait_st();
                }
                // rows of the last 16-row group past the segment's end must not feed NaNs into P.V
                const int valid = min(TILE, sg.r1 - row0);
                if (valid & 15) {
                    const int r_lo = valid, r_hi = (valid + 15) & ~15;
                    const int n_vec = (r_hi - r_lo) * NBLK * 8;  // 16-byte vectors
                    uint8_t *stage = kv_smem + s * STAGE_BYTES;
                    for (int i = wg_tid; i < n_vec; i += 128) {
                        const int v = i & 7, rk = i >> 3;
                        const int k = rk % NBLK, r = r_lo + rk / NBLK;
                        *reinterpret_cast<uint4 *>(stage + k * BLK_BYTES + r * 128 + v * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
                fence_proxy_async_smem();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.p_full[s]);
                GS_STAMP(it, PF_P_WRITTEN);
                if (Q8 && j + 1 < sg.n_tiles) widen_tile(it + 1, j + 1);
            }
            if (!ok) break;
            // ---- end of segment: drain the accumulators into this segment's partial record ----------------
            (void) mbar_wait(&B.o_full, sgc & 1, abort_flag, status_w, ST_SOFTMAX);
            named_bar_sync(2, 128);
            if (*abort_flag) { ok = false; break; }
            tc_fence_after();
            if (wg_tid == 0) GS_STAMP(kProfTiles - 1, 2);
            if (wg_tid == 0) GS_CTA_STAMP(3);
#pragma unroll
            for (int i = 0; i < HQ; i++) {
                float v = l_part[i];
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                if ((lane & 15) == 0) M.sl[qt][col0 + i] = v;
            }
            named_bar_sync(1, 128);
            if (LIST && sc.whole) {
                // the whole sequence was attended here: no record, no merge - normalise and store (ops.cu:531-538)
                if (wg_tid < NQ) {
                    const float l = (M.sl[0][wg_tid] + M.sl[1][wg_tid]) + (M.sl[2][wg_tid] + M.sl[3][wg_tid]);
                    M.f[wg_tid] = l > 0.f ? 1.f / l : 0.f;
                }
                named_bar_sync(1, 128);
                float *dst = P.o + ((int64_t) (sg.b / P.seq_div) * P.H_out + (sg.b % P.seq_div) * P.H) * P.d_v + qt * 32 + lane;
#pragma unroll 1
                for (int mt = 0; mt < NVT; mt++) {
#pragma unroll
                    for (int c = 0; c < NQ / 16; c++) {
                        uint32_t r[16];
                        tmem_ld16(tmem + lane_base + (O_SLOT0 + mt) * NQ + c * 16, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            if (c * 16 + i < P.rows_q) dst[(int64_t) (c * 16 + i) * P.d_v + mt * 128] = __uint_as_float(r[i]) * M.f[c * 16 + i];
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.o_empty);
                sgc++;
                continue;
            }
            if (wg_tid < P.rows_q) {
                const int q = wg_tid;
                const float m = M.mref[q];
                float *ml = P.ws_ml + ((int64_t) sg.seg_id * P.rows_q + q) * 2;
                ml[0] = m == -INFINITY ? -INFINITY : m * LN2;
                ml[1] = (M.sl[0][q] + M.sl[1][q]) + (M.sl[2][q] + M.sl[3][q]);
            }
            // one record per segment, [query row][d_v] f32: a CTA's stores stay inside one contiguous block
            float *acc = P.ws_acc + (int64_t) sg.seg_id * P.rows_q * P.d_v + qt * 32 + lane;
            // one value tile (NQ columns of this lane's row) per step; the loads of the next tile are in flight
            // while the current one is stored
            constexpr int NB = NQ > 48 ? 1 : 2;  // (64 columns twice over would not leave the registers for the rest)
            uint32_t rbuf[NB][NQ];
            if (NB == 2) {
#pragma unroll
                for (int c = 0; c < NQ / 16; c++) tmem_ld16(tmem + lane_base + O_SLOT0 * NQ + c * 16, *reinterpret_cast<uint32_t(*)[16]>(rbuf[0] + c * 16));
            }
            {
#pragma unroll
                for (int mt = 0; mt < NVT; mt++) {
                    if (NB == 1) {
#pragma unroll
                        for (int c = 0; c < NQ / 16; c++)
                            tmem_ld16(tmem + lane_base + (O_SLOT0 + mt) * NQ + c * 16, *reinterpret_cast<uint32_t(*)[16]>(rbuf[0] + c * 16));
                    }
                    tmem_wait_ld();
                    if (NB == 2 && mt + 1 < NVT) {
#pragma unroll
                        for (int c = 0; c < NQ / 16; c++)
                            tmem_ld16(tmem + lane_base + (O_SLOT0 + mt + 1) * NQ + c * 16,
                                      *reinterpret_cast<uint32_t(*)[16]>(rbuf[(mt + 1) & (NB - 1)] + c * 16));
                    }
#pragma unroll
                    for (int q = 0; q < NQ; q++)
                        if (q < P.rows_q) st_global_hint(acc + (int64_t) q * P.d_v + mt * 128, __uint_as_float(rbuf[mt & (NB - 1)][q]), pol_keep);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B.o_empty);
            if (wg_tid == 0) GS_STAMP(kProfTiles - 1, 3);
            if (wg_tid == 0) GS_CTA_STAMP(4);
            sgc++;
        }
    }

    // ---- common exit -----------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) {
        // loads that were issued but never consumed may still be landing in this CTA's shared memory
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    if (tid == 32) GS_STAMP(kProfTiles - 1, 4);
    if (tid == 32) GS_CTA_STAMP(5);
#undef GS_STAMP
#undef GS_CTA_STAMP
}

template <int NQ, int NBLK, bool LIST = false, bool Q8 = false>
int launch_cfg(const UmmaParams &P, int grid, cudaStream_t st) {
    const int smem = Smem<NQ, NBLK, Q8>::TOTAL;
    // attributes are set on every call: a cached flag would go stale across a device reset
    GS_TRY(cudaFuncSetAttribute(k_decode_umma<NQ, NBLK, LIST, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    // programmatic dependent launch: the CTA-local set-up may overlap the tail of the preceding kernel
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GS_TRY(cudaLaunchKernelEx(&cfg, k_decode_umma<NQ, NBLK, LIST, Q8>, P));
    return 0;
}

}  // namespace

int read_list_status(int32_t *out) {
    GS_TRY(cudaMemcpyFromSymbol(out, g_list_status, sizeof(int32_t)));
    return 0;
}

// Position lists on the tensor cores.  Head groups of at most 48 heads (a multiple of 8 each): 0 = not cut that way.
// (49..64 heads may also run as one group of 64 query columns, see launch_decode_umma_list.)
static int list_head_groups(int H) {
    const int n = (H + 47) / 48;
    return (n > 0 && H % n == 0 && (H / n) % 8 == 0) ? n : 0;
}

// Returns 0 when launched, -1 when the shape is not taken by the tcgen05 kernel (the caller then runs the CUDA-core
// kernel), or a cudaError_t.  Every (token, head group) is a kernel sequence over the token's list.  With one split, or
// when the caller's `part` cannot hold enough records, every sequence is attended by one CTA that stores o itself;
// otherwise the rows are dealt to CTAs as in the dense form and the records live in `part`
// (T*H*splits*(R+2) floats, crates/cuda/kernels/ops.cu:578): accumulators [segment][row][R], then (m, l) [segment][row][2], then
// the per-sequence descriptors.
// What a cut into n_groups head groups gives: the grid, whether every (token, group) is attended whole by one CTA, and
// the longest run of tiles one CTA walks (what the call's time follows).
struct ListPlan {
    int n_groups, grid, grid_rec, grid_whole;
    bool whole;
    int64_t depth;
};
static ListPlan list_plan(int n_groups, int T, int H, int R, int sel_stride, int splits, const float *part, int grid_max) {
    ListPlan L{};
    L.n_groups = n_groups;
    const int Hg = H / n_groups;
    const int64_t n_seq_k = (int64_t) T * n_groups;
    const int64_t tiles_seq = (sel_stride + TILE - 1) / TILE;
    // records that fit the caller's buffer
    if (splits > 1 && part && !(reinterpret_cast<uintptr_t>(part) & 15)) {
        const int64_t part_floats = (int64_t) T * H * splits * (R + 2);
        const int64_t desc_floats = (n_seq_k * 2 + 3) / 4 * 4;
        const int64_t segs = (part_floats - desc_floats) / ((int64_t) Hg * (R + 2));
        const int64_t tiles = n_seq_k * tiles_seq;
        int64_t g = segs - n_seq_k;
        if (g > grid_max) g = grid_max;
        if (g > tiles) g = tiles;
        L.grid_rec = (int) (g > 0 ? g : 0);
    }
    L.grid_whole = (int) (n_seq_k < grid_max ? n_seq_k : grid_max);
    L.whole = L.grid_rec <= L.grid_whole;
    L.grid = L.whole ? L.grid_whole : L.grid_rec;
    L.depth = L.whole ? (n_seq_k + L.grid - 1) / L.grid * tiles_seq : (n_seq_k * tiles_seq + L.grid - 1) / L.grid;
    return L;
}

int launch_decode_umma_list(const float *q, const void *C, const __half *C_scales, const int32_t *sel, int sel_stride, const int32_t *cnt,
                            float scale, float *o, float *part, int T, int H, int R, int splits, int sm_count, cudaStream_t st) {
    const int g48 = list_head_groups(H);
    if (R != 512 || g48 == 0 || sel_stride <= 0 || !(scale > 0.f)) return -1;
    if ((reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(C_scales) & 15)) return -1;
    int grid_max = sm_count < kMaxCtas ? sm_count : kMaxCtas;
    if (grid_max < 1) grid_max = 1;
    // 49..64 heads: two groups of at most 32 heads (the listed rows are copied once per group), or all heads in one
    // pass with 64 query columns and two issuing warps.  Listed rows arrive at a latency-bound rate per SM, so the
    // cut with the shorter longest run of tiles wins; the two-group form on a tie.
    ListPlan L = list_plan(g48, T, H, R, sel_stride, splits, part, grid_max);
    if (H > 48 && H <= 64 && !C_scales) {  // (the 64-column form is built for the f16 cache only)
        const ListPlan L1 = list_plan(1, T, H, R, sel_stride, splits, part, grid_max);
        if (L1.depth < L.depth) L = L1;
    }
    const int n_groups = L.n_groups;
    const int64_t n_seq_k = (int64_t) T * n_groups;
    if (n_seq_k > MAX_SEQ) return -1;
    const int Hg = H / n_groups;
    UmmaParams P;
    memset(&P, 0, sizeof(P));
    // The entry point is not told how many rows the cache holds: the lists are trusted as the reference trusts them
    // (a negative index is read as 0).  The tensor maps are unused in this form; one valid map keeps the descriptor
    // prefetches of the set-up harmless.
    if (encode_tmap_2d_f16(&P.tm_kv64, C, (uint64_t) 64, (uint64_t) R, (uint64_t) R * 2, 16, 64, (int) CU_TENSOR_MAP_SWIZZLE_128B))
        return -1;
    P.tm_kv16 = P.tm_kv64;
    P.tm_q = P.tm_kv64;
    P.list_cache = C;
    P.list_scales = C_scales;
    P.seq_lens = cnt;
    P.sel = sel;
    P.sel_stride = sel_stride;
    P.q_f32 = q;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.tail_causal = 0;
    P.n_seq = (int) n_seq_k;
    P.T = 1;
    P.H = Hg;
    P.H_full = H;
    P.H_out = H;
    P.h0 = 0;
    P.rows_q = Hg;
    P.d_v = R;
    P.seq_div = n_groups;
    P.cache_rows = sel_stride;  // caps a length word: a list holds at most sel_stride entries
    P.o = o;
    P.status = nullptr;
    const bool whole = L.whole;
    const int grid = L.grid;
    P.whole_seq = whole ? 1 : 0;
    CombinePlan c{};
    if (!whole) {
        P.seg_cap = grid + (int) n_seq_k;
        P.ws_acc = part;
        P.ws_ml = part + (int64_t) Hg * P.seg_cap * R;
        P.ws_desc = reinterpret_cast<int2 *>(P.ws_ml + (int64_t) Hg * P.seg_cap * 2);
        c.acc = P.ws_acc;
        c.ml = P.ws_ml;
        c.desc = P.ws_desc;
        c.seg_stride_acc = (int64_t) Hg * R;
        c.seg_stride_ml = (int64_t) Hg * 2;
        c.n_segments = P.seg_cap;
        c.n_seq = (int) n_seq_k;
        c.T = 1;
        c.H = Hg;
        c.H_out = H;
        c.h0 = 0;
        c.seq_div = n_groups;
        c.d_v = R;
        c.o = o;
        c.seq_lens = cnt;
        c.unit_rows = 16;
        c.n_ctas = grid;
        c.len_cap = sel_stride;
        c.bulk = true;
    }
    int e;
    if (C_scales) e = Hg <= 32 ? launch_cfg<32, 8, true, true>(P, grid, st) : launch_cfg<48, 8, true, true>(P, grid, st);
    else if (Hg <= 32) e = launch_cfg<32, 8, true>(P, grid, st);
    else if (Hg <= 48) e = launch_cfg<48, 8, true>(P, grid, st);
    else e = launch_cfg<64, 8, true>(P, grid, st);
    if (e) return e;
    if (!whole) return launch_combine(c, st);
    return 0;
}

bool decode_umma_supported(const DecodeProblem &p, const char **why) {
    if (p.q_is_f32) { *why = "f32 queries"; return false; }
    if (p.sel) { *why = "explicit position lists"; return false; }
    if (!((p.d_qk == 576 || p.d_qk == 512) && p.d_v == 512)) { *why = "row widths other than 576/512 or 512/512"; return false; }
    const bool one64 = p.d_qk == 512 && p.T * p.H <= 64;  // 512-column rows: up to 64 query rows ride in one pass
    if (p.T * p.H > 48 && !one64) {
        // wider blocks run as head groups of at most 48 rows, one launch each (the cache is read once per group)
        if (p.T > 4 || p.H % 8 != 0) { *why = "more than 48 query rows per sequence with T > 4 or H % 8 != 0"; return false; }
        if (p.exchange) { *why = "more than 48 query rows per sequence together with a cross-GPU exchange"; return false; }
    }
    if (!(p.scale > 0.f)) { *why = "non-positive softmax scale"; return false; }
    if (p.n_seq > MAX_SEQ) { *why = "more than 1024 sequences"; return false; }
    if (p.page_table && p.page_rows != TILE) { *why = "page size other than 64"; return false; }
    if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (reinterpret_cast<uintptr_t>(p.cache) & 15)) { *why = "q and cache must be 16-byte aligned"; return false; }
    if ((int64_t) p.n_seq * p.T * p.H >= (1ll << 31) || p.cache_rows >= (1ll << 31)) { *why = "row counts beyond 2^31"; return false; }
    return true;
}

int launch_decode_umma(const DecodeProblem &p, cudaStream_t st) {
    // Head groups: up to 48 query rows (T tokens x Hg heads) ride on the N side of one launch; up to 64 over
    // 512-column rows (the stages and the query rows are then sized by the row width, see Smem).
    int Hg = p.H, n_groups = 1, seq_div = 1;
    const bool one64 = p.d_qk == 512 && p.T * p.H <= 64;
    if (p.T * p.H > 48 && !one64) {
        const int hg_max = (48 / p.T) & ~7;          // a multiple of 8 heads
        n_groups = (p.H + hg_max - 1) / hg_max;
        Hg = (((p.H + n_groups - 1) / n_groups) + 7) & ~7;  // balanced, rounded up to 8
        // Equal groups can run as sequences of their own over the same rows - kernel sequence b is head group
        // b % groups of caller sequence b / groups - so that one launch covers them.  Take the group count that
        // divides the heads into multiples of 8 if it is the minimum or one more (each group reads the cache again).
        for (int n = n_groups; n <= n_groups + 1 && n <= 8; n++) {
            if (p.H % n == 0 && (p.H / n) % 8 == 0 && p.T * (p.H / n) <= 48) {
                if ((int64_t) p.n_seq * n <= MAX_SEQ) {
                    seq_div = n;
                    Hg = p.H / n;
                    n_groups = 1;
                }
                break;
            }
        }
    }
    const int n_seq_k = p.n_seq * seq_div;  // sequences as the kernel sees them
    UmmaParams P;
    memset(&P, 0, sizeof(P));
    const int kSw128 = (int) CU_TENSOR_MAP_SWIZZLE_128B;
    if (int e = encode_tmap_2d_f16(&P.tm_kv64, p.cache, (uint64_t) p.cache_rows, (uint64_t) p.d_qk, (uint64_t) p.d_qk * 2,
                                   TILE, 64, kSw128)) return e;
    if (int e = encode_tmap_2d_f16(&P.tm_kv16, p.cache, (uint64_t) p.cache_rows, (uint64_t) p.d_qk, (uint64_t) p.d_qk * 2,
                                   16, 64, kSw128)) return e;
    P.seq_lens = p.seq_lens;
    P.seq_base = p.seq_base;
    P.page_table = p.page_table;
    P.page_table_stride = p.page_table_stride;
    P.paged = p.page_table != nullptr;
    P.scale_log2 = p.scale * 1.4426950408889634f;
    P.tail_causal = p.tail_causal;
    P.ws_acc = p.ws_acc;
    P.ws_ml = p.ws_ml;
    P.ws_desc = p.ws_desc;
    P.status = p.status;
    P.n_seq = n_seq_k;
    P.T = p.T;
    P.H_full = (seq_div > 1 && p.T == 1) ? Hg : p.H;  // one token: the groups' query rows are contiguous, no per-token boxes
    P.seq_div = seq_div;
    P.d_v = p.d_v;
    P.cache_rows = p.cache_rows;
    int grid = p.sm_count < kMaxCtas ? p.sm_count : kMaxCtas;
    if (p.max_ctas > 0 && grid > p.max_ctas) grid = p.max_ctas;
    if (grid < 1) grid = 1;
    // every CTA and every sequence can add one segment, each with the query rows of one launch
    if (((int64_t) grid + n_seq_k) * p.T * (seq_div > 1 || n_groups > 1 ? Hg : p.H) > p.max_record_rows)
        return fail_invalid("decode: workspace too small for the segment records");
    P.seg_cap = grid + n_seq_k;

    for (int g = 0; g < n_groups; g++) {
        const int h0 = g * Hg;
        const int hg = p.H - h0 < Hg ? p.H - h0 : Hg;
        if (hg <= 0) break;
        const int rows_q = p.T * hg;
        const int NQ = rows_q <= 32 ? 32 : rows_q <= 48 ? 48 : 64;
        // one box of NQ rows when the rows of a sequence are contiguous, else one box of hg rows per token
        if (int e = encode_tmap_2d_f16(&P.tm_q, p.q, (uint64_t) p.n_seq * p.T * p.H, (uint64_t) p.d_qk, (uint64_t) p.d_qk * 2,
                                       (uint32_t) (P.H_full == hg ? NQ : hg), 64, kSw128)) return e;
        P.H = hg;
        P.h0 = h0;
        P.rows_q = rows_q;
        CombinePlan c{};
        c.acc = p.ws_acc;
        c.ml = p.ws_ml;
        c.desc = p.ws_desc;
        c.regular_segments = 0;
        c.seg_stride_acc = (int64_t) rows_q * p.d_v;  // records as [segment][row][d_v], (m, l) as [segment][row][2]
        c.seg_stride_ml = (int64_t) rows_q * 2;
        c.n_segments = P.seg_cap;
        c.n_seq = n_seq_k;
        c.T = p.T;
        c.H = hg;
        c.H_out = p.H;
        c.h0 = h0;
        c.seq_div = seq_div;
        c.d_v = p.d_v;
        c.o = p.o;
        c.part_out = p.part_out;
        c.status = p.status;
        c.seq_lens = p.seq_lens;
        c.unit_rows = P.paged ? TILE : 16;
        c.n_ctas = grid;
        c.len_cap = P.paged ? (int64_t) P.page_table_stride * TILE : P.cache_rows;
        c.bulk = true;
        int e;
        if (p.d_qk == 576) e = NQ == 32 ? launch_cfg<32, 9>(P, grid, st) : launch_cfg<48, 9>(P, grid, st);
        else e = NQ == 32 ? launch_cfg<32, 8>(P, grid, st) : NQ == 48 ? launch_cfg<48, 8>(P, grid, st) : launch_cfg<64, 8>(P, grid, st);
        if (e) return e;
        if (p.ev_after_main && g == n_groups - 1) GS_TRY(cudaEventRecord(p.ev_after_main, st));
        if (p.no_combine) continue;
        if (p.exchange) return launch_exchange_combine(c, *p.exchange, p.o, p.status, p.sm_count, st);
        if (int ce = launch_combine(c, st)) return ce;
    }
    return 0;
}

}  // namespace gs
