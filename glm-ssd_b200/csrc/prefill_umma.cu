// Causal prefill attention on the Blackwell tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Semantics (what the reference reaches through its absorbed kernel with one launch per 256
// queries, crates/engine/src/forward.rs:61, :898-908): query i of head h attends keys 0 .. p0+i,
// score = scale * q.k over d = 256, softmax, o = P V.
//
// One CTA per (128-query block, head).  Per 64-key tile:
//   S[128 x 64]   = Q[128 x 256] . K_tile^T      16 MMAs (M = 128, N = 64, K = 16), both operands
//                                                 K-major in 128-byte-swizzled shared memory
//   P = exp2(S*c - m) as f16, written back into the tensor memory columns of S (one query row per
//       thread, so the row maximum and row sum need no shuffles)
//   O[128 x 256] += P . V_tile                    4 MMAs (M = 128, N = 256, K = 16) with P read from
//                                                 tensor memory and V_tile read MN-major
// Tensor memory holds four score / probability buffers (4 x 64 columns) and the accumulator (256 columns), so
// the scores run up to three tiles ahead of the softmax.  Shared memory holds the 64 KB query tile, three 32 KB
// K stages and two 32 KB V stages, fed by two independent TMA producers: every load has more than a tile period
// to land (128-key tiles in single buffers left the tensor pipe waiting for every load).  Three warps issue
// MMAs (scores of even tiles, scores of odd tiles, P.V): an issuing thread is held while the pipe works off its
// MMAs, so one thread cannot keep the queue filled with both kinds.  What bounds the tensor time is the pipe itself: an M = 128, N = 64 MMA with both operands in shared memory occupies it for ~49
// cycles (it is bound by reading (M + N) x 32 operand bytes, not by the math, which would take 32), so a
// tile takes about 16 x 49 + 4 x 129 = 1300 cycles (measured 1240) against 1049 at peak.
// Measured on the heaviest CTA with all SMs busy (clock stamps, GS_PF_PROF): a tile takes 1240-1330 cycles; the
// softmax threads are busy 1130 of them (80 reading the scores, 255 row maximum, 630 exponentials - 64 per thread at
// the special-function rate of 4 per cycle and quarter - and 160 writing P), and a hand-over through an mbarrier
// (MMA done -> waiting warp runs on) costs 200-300 cycles.  So the tensor time and the softmax time nearly coincide,
// and what keeps both busy is the depth of the score buffers.  Measured alternatives, all with correct results:
//  * score MMAs over 128 keys (N = 128: 65 cycles where two N = 64 take 98), fed by a ring of [128 keys x 64 columns]
//    blocks: 7 % slower with the probabilities written over two double-width score buffers (the next scores then wait
//    for the P.V of the pair before), 12 % slower with one double-width score buffer and four probability buffers;
//  * the query block kept in tensor memory (128 columns; an N = 64 MMA then takes 33 cycles instead of 49), which
//    leaves room for one score buffer and two probability buffers: the same speed with P.V issued as soon as its
//    probabilities are there, 6 % slower with P.V held back until the scores two tiles on are issued, 7 % slower
//    with one thread issuing both kinds (an issuing thread is held while the pipe works off its MMAs).
//  * the first half of the query block in tensor memory (64 columns) beside three score buffers: a tile takes 1168
//    cycles instead of 1245, and the S = 8192, H = 20 chunk takes the same 0.60 ms.  During back-to-back launches of
//    this kernel the SM clock reads 1567 MHz of 1965 with the software power cap as the only reason: at the board's
//    power limit fewer cycles buy a lower clock, not a shorter time.
// Cycles per MMA from one issuing thread, long runs: M = 128, K = 16, both operands in shared memory N = 64 49,
// N = 128 65, N = 256 129; A in tensor memory N = 32 24, N = 64 33, N = 128 65, N = 256 129.
// The accumulator is rescaled lazily (only when a row maximum grows by more than 2^8), decided per warp.
// Every mbarrier wait is bounded and ends in an error status instead of a hang.
#include <string.h>

#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {
namespace {
using namespace sm100;

constexpr int BM = 128;                  // query rows per CTA
constexpr int BN = 64;                   // keys per tile
constexpr int HD = 256;                  // head width
constexpr int NDB = HD / 64;             // 64-column blocks per row
constexpr int QBLK = BM * 128;           // bytes of one [128 query rows][64 cols] block
constexpr int KBLK = BN * 128;           // bytes of one [64 key rows][64 cols] block
constexpr int Q_BYTES = NDB * QBLK;      // 64 KB
constexpr int KV_BYTES = NDB * KBLK;     // 32 KB: a K or V tile
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int S_BUFS = 4;                // score / probability buffers in tensor memory: 4 x 64 columns + 256 of O
// warp 0 K producer, 1 score MMAs of even tiles, 2-5 softmax, 6 V producer, 7 score MMAs of odd tiles, 8 P.V MMAs
constexpr int PF_THREADS = 288;
constexpr int S_COLS = 64, O_COL = 256;
constexpr float PF_RESCALE = 8.0f;

struct PrefillParams {
    CUtensorMap tm_q, tm_k, tm_v;
    void *o;
    int o_f16;
    int S, H, p0;
    float scale_log2;
    int32_t *status;  // may be nullptr
};

// Tuning aid, compiled in only for the timing probe: clock stamps of the heaviest CTA's first tiles.
#ifdef GS_PF_PROF
__device__ long long g_pf_prof[32 * 8];
#define PF_STAMP(j, slot)                                                                                  \
    do {                                                                                                   \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (j) >= 8 && (j) < 40) g_pf_prof[((j) - 8) * 8 + (slot)] = clock64(); \
    } while (0)
#else
#define PF_STAMP(j, slot) do { } while (0)
#endif

struct PfBarriers {
    uint64_t q_full, k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
    uint64_t s_full[S_BUFS], p_full[S_BUFS], p_free[S_BUFS];  // p_free[b]: P.V has read the probabilities in buffer b
};

struct PfSmemMisc {
    PfBarriers bar;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int PF_SMEM = Q_BYTES + (K_STAGES + V_STAGES) * KV_BYTES + (int) sizeof(PfSmemMisc) + 1024;

__global__ void __launch_bounds__(PF_THREADS, 1) k_prefill_umma(const __grid_constant__ PrefillParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t *q_smem = smem, *k_smem = smem + Q_BYTES, *v_smem = k_smem + K_STAGES * KV_BYTES;
    PfSmemMisc &M = *reinterpret_cast<PfSmemMisc *>(v_smem + V_STAGES * KV_BYTES);
    PfBarriers &B = M.bar;
    volatile int *abort_flag = &M.abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // heavier (later) query blocks first
    const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
    const int q0 = qb * BM;
    const int k_end = min(P.p0 + P.S, P.p0 + q0 + BM);  // keys any row of this block attends
    const int n_tiles = (k_end + BN - 1) / BN;
    const int col0 = h * HD;

    if (tid == 0) {
        tma_prefetch_desc(&P.tm_q);
        tma_prefetch_desc(&P.tm_k);
        tma_prefetch_desc(&P.tm_v);
        mbar_init(&B.q_full, 1);
        for (int i = 0; i < K_STAGES; i++) {
            mbar_init(&B.k_full[i], 1);
            mbar_init(&B.k_empty[i], 1);
        }
        for (int i = 0; i < V_STAGES; i++) {
            mbar_init(&B.v_full[i], 1);
            mbar_init(&B.v_empty[i], 1);
        }
        for (int i = 0; i < S_BUFS; i++) {
            mbar_init(&B.s_full[i], 1);
            mbar_init(&B.p_full[i], 4);
            mbar_init(&B.p_free[i], 1);
        }
        M.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(&M.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = M.tmem_base;

    if (warp == 0) {
        // ---- Q once, then the K tiles -------------------------------------------------------------------
        if (elect_one()) {
            mbar_arrive_expect_tx(&B.q_full, Q_BYTES);
#pragma unroll
            for (int b = 0; b < NDB; b++) tma_load_2d(q_smem + b * QBLK, &P.tm_q, &B.q_full, col0 + b * 64, q0);
        }
        __syncwarp();
        for (int j = 0; j < n_tiles; j++) {
            const int st = j % K_STAGES;
            if (!mbar_wait(&B.k_empty[st], ((j / K_STAGES) & 1) ^ 1, abort_flag, P.status, 1)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&B.k_full[st], KV_BYTES);
#pragma unroll
                for (int b = 0; b < NDB; b++)
                    tma_load_2d(k_smem + st * KV_BYTES + b * KBLK, &P.tm_k, &B.k_full[st], col0 + b * 64, j * BN);
            }
            __syncwarp();
        }
    } else if (warp == 6) {
        // ---- the V tiles ------------------------------------------------------------------------------------
        for (int j = 0; j < n_tiles; j++) {
            const int st = j & 1;
            if (!mbar_wait(&B.v_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, P.status, 1)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&B.v_full[st], KV_BYTES);
#pragma unroll
                for (int b = 0; b < NDB; b++)
                    tma_load_2d(v_smem + st * KV_BYTES + b * KBLK, &P.tm_v, &B.v_full[st], col0 + b * 64, j * BN);
            }
            __syncwarp();
        }
    } else if (warp == 1 || warp == 7) {
        // ---- score MMA issuers: S = Q . K^T, warp 1 the even tiles, warp 7 the odd ones --------------------------
        // An issuing thread is held while the pipe works off its MMAs; a tile needs 16 of these (N = 64) besides the
        // 4 P.V MMAs: three issuing warps keep the pipe's queue filled.
        constexpr uint32_t idesc_s = make_idesc_f16(BM, BN, 0, 0);
        const uint64_t d_kmaj = make_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint32_t q_lo = smem_u32(q_smem) >> 4, k_lo = smem_u32(k_smem) >> 4;
        bool ok = mbar_wait(&B.q_full, 0, abort_flag, P.status, 2);
        // Scores run up to three tiles ahead of the softmax: S(j) goes into tensor-memory buffer j & 3, where
        // P(j-4) lives until P.V(j-4) has read it.  Two MMAs are only ordered with respect to each other on the
        // same accumulator, so that P.V is awaited explicitly.
        for (int j = warp == 1 ? 0 : 1; ok && j < n_tiles; j += 2) {
            const int st = j % K_STAGES, sb = j & (S_BUFS - 1);
            ok = mbar_wait(&B.k_full[st], (j / K_STAGES) & 1, abort_flag, P.status, 2) &&
                 mbar_wait(&B.p_free[sb], ((j / S_BUFS) & 1) ^ 1, abort_flag, P.status, 2);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) PF_STAMP(j, 0);
            if (elect_one()) {
#pragma unroll
                for (int b = 0; b < NDB; b++)
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_ss(tmem + sb * S_COLS, d_kmaj + (q_lo + b * (QBLK >> 4) + ks * 2),
                                d_kmaj + (k_lo + st * (KV_BYTES >> 4) + b * (KBLK >> 4) + ks * 2), idesc_s, (b | ks) != 0);
                umma_commit(&B.s_full[sb]);
                umma_commit(&B.k_empty[st]);
            }
            __syncwarp();
        }
    } else if (warp == 8) {
        // ---- P.V MMA issuer: O += P . V ----------------------------------------------------------------------------
        constexpr uint32_t idesc_pv = make_idesc_f16(BM, HD, 0, 1);  // A = P from tensor memory, B = V MN-major
        const uint64_t d_v = make_smem_desc(0, KBLK, 1024, kSwizzle128B);
        const uint32_t v_lo = smem_u32(v_smem) >> 4;
        bool ok = true;
        for (int j = 0; ok && j < n_tiles; j++) {
            const int sb = j & (S_BUFS - 1);
            ok = mbar_wait(&B.p_full[sb], (j / S_BUFS) & 1, abort_flag, P.status, 2) &&
                 mbar_wait(&B.v_full[j & 1], (j >> 1) & 1, abort_flag, P.status, 2);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) PF_STAMP(j, 1);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < BN / 16; ks++)
                    umma_ts(tmem + O_COL, tmem + sb * S_COLS + ks * 8, d_v + (v_lo + (j & 1) * (KV_BYTES >> 4) + ks * 128),
                            idesc_pv, j > 0 || ks > 0);
                umma_commit(&B.v_empty[j & 1]);
                umma_commit(&B.p_free[sb]);
            }
            __syncwarp();
        }
    } else {
        // ---- softmax / correction / epilogue: one query row per thread ------------------------------------------
        if (warp >= 2 && warp <= 5) {
            const int qt = warp & 3;
            const uint32_t lane_base = (uint32_t) (qt * 32) << 16;
            const int row = qt * 32 + lane;
            const int qi = q0 + row;                 // query index within the chunk
            const int k_lim = P.p0 + qi;             // last key this row attends
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < n_tiles; j++) {
                const int sb = j & (S_BUFS - 1);
                const uint32_t s_addr = tmem + lane_base + sb * S_COLS;
                ok = mbar_wait(&B.s_full[sb], (j / S_BUFS) & 1, abort_flag, P.status, 4);
                if (!ok) break;
                tc_fence_after();
                if (warp == 2 && lane == 0) PF_STAMP(j, 3);
                const int k0 = j * BN;
                const bool need_mask = k0 + BN - 1 > P.p0 + q0;  // some row of the block must not see some key
                // the whole score row of this thread (128 keys) is read once and kept in registers: one
                // tensor-memory round trip per tile instead of eight
                uint32_t r[BN];
#pragma unroll
                for (int c = 0; c < BN / 16; c++) tmem_ld16(s_addr + c * 16, *reinterpret_cast<uint32_t(*)[16]>(r + c * 16));
                tmem_wait_ld();
                if (warp == 2 && lane == 0) PF_STAMP(j, 4);
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < BN; i++)
                        if (k0 + i > k_lim) r[i] = __float_as_uint(-INFINITY);
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < BN; i += 4) {
                    mx4[0] = fmaxf(mx4[0], __uint_as_float(r[i]));
                    mx4[1] = fmaxf(mx4[1], __uint_as_float(r[i + 1]));
                    mx4[2] = fmaxf(mx4[2], __uint_as_float(r[i + 2]));
                    mx4[3] = fmaxf(mx4[3], __uint_as_float(r[i + 3]));
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                mx *= P.scale_log2;  // scale > 0
                // lazy reference update, decided per warp (tensor-memory accesses are warp-wide)
                const bool grow = mx > m_run + PF_RESCALE;
                if (__any_sync(0xffffffffu, grow)) {
                    const float m_new = grow ? mx : m_run;
                    const float f = m_run == -INFINITY ? 0.f : exp2f(m_run - m_new);
                    if (j > 0) {
                        // the accumulator holds tiles 0..j-1: wait for P.V(j-1), then scale this row.  (Its
                        // barrier is the one of buffer (j-1) & 3, whose previous phase, P.V(j-5), was over before
                        // S(j-1) could be issued: the parity cannot be mistaken.)
                        ok = mbar_wait(&B.p_free[(j - 1) & (S_BUFS - 1)], ((j - 1) / S_BUFS) & 1, abort_flag, P.status, 4);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < HD / 16; c++) {
                            uint32_t r[16];
                            tmem_ld16(tmem + lane_base + O_COL + c * 16, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 16; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
                            tmem_st16(tmem + lane_base + O_COL + c * 16, r);
                        }
                        tmem_wait_st();
                    }
                    l_run *= f;
                    m_run = m_new;
                }
                // probabilities, row sum, P as packed f16 pairs (keys 2i, 2i+1 -> column i of this S buffer)
                if (warp == 2 && lane == 0) PF_STAMP(j, 5);
                const float nm = -m_run;
                float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < BN / 2; i++) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), P.scale_log2, nm));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), P.scale_log2, nm));
                    l4[i & 3] += p0 + p1;
                    const __half2 hh = __floats2half2_rn(p0, p1);
                    r[i] = *reinterpret_cast<const uint32_t *>(&hh);
                }
                l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                if (warp == 2 && lane == 0) PF_STAMP(j, 6);
#pragma unroll
                for (int c = 0; c < BN / 32; c++) tmem_st16(s_addr + c * 16, *reinterpret_cast<const uint32_t(*)[16]>(r + c * 16));
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.p_full[sb]);
                if (warp == 2 && lane == 0) PF_STAMP(j, 7);
            }
            // ---- epilogue: O / l -> global ------------------------------------------------------------------------
            // The P.V MMAs come from one thread and share one accumulator, so they complete in order: the last one
            // done means all done.  Its barrier's previous phase, P.V(n-5), was over before S(n-1) was issued.
            if (ok) ok = mbar_wait(&B.p_free[(n_tiles - 1) & (S_BUFS - 1)], ((n_tiles - 1) / S_BUFS) & 1, abort_flag, P.status, 4);
            if (ok) {
                tc_fence_after();
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                const int64_t off = ((int64_t) qi * P.H + h) * HD;
#pragma unroll 1
                for (int c = 0; c < HD / 16; c++) {
                    uint32_t r[16];
                    tmem_ld16(tmem + lane_base + O_COL + c * 16, r);  // warp-wide: executed by rows past S too
                    tmem_wait_ld();
                    if (qi < P.S) {
                        if (P.o_f16) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const __half2 hh = __floats2half2_rn(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                                w[i] = *reinterpret_cast<const uint32_t *>(&hh);
                            }
                            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(P.o) + off + c * 16);
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
                            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(P.o) + off + c * 16);
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                dst[i] = make_float4(__uint_as_float(r[4 * i]) * inv, __uint_as_float(r[4 * i + 1]) * inv,
                                                     __uint_as_float(r[4 * i + 2]) * inv, __uint_as_float(r[4 * i + 3]) * inv);
                        }
                    }
                }
            }
        }
    }
    // ---- common exit ---------------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

bool prefill_umma_supported(int S, int H, int d, int p0, const char **why) {
    if (d != HD) { *why = "head width other than 256"; return false; }
    if ((int64_t) H * d >= (1ll << 31) || (int64_t) p0 + S >= (1ll << 31)) { *why = "sizes beyond 2^31"; return false; }
    if (H > 65535) { *why = "more than 65535 heads"; return false; }
    return true;
}

int launch_prefill_umma(const __half *q, const __half *k, const __half *v, void *o, int o_f16, int S, int H, int d,
                        int p0, float scale, int32_t *status, cudaStream_t st) {
    if (!(scale > 0.f)) return fail_invalid("prefill: the tcgen05 kernel needs a positive softmax scale");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(o)) & 15)
        return fail_invalid("prefill: q, k, v and o must be 16-byte aligned");
    PrefillParams P;
    memset(&P, 0, sizeof(P));
    const int sw = (int) CU_TENSOR_MAP_SWIZZLE_128B;
    const uint64_t cols = (uint64_t) H * d, pitch = cols * 2;
    if (int e = encode_tmap_2d_f16(&P.tm_q, q, (uint64_t) S, cols, pitch, BM, 64, sw)) return e;
    if (int e = encode_tmap_2d_f16(&P.tm_k, k, (uint64_t) p0 + S, cols, pitch, BN, 64, sw)) return e;
    if (int e = encode_tmap_2d_f16(&P.tm_v, v, (uint64_t) p0 + S, cols, pitch, BN, 64, sw)) return e;
    P.o = o;
    P.o_f16 = o_f16;
    P.S = S;
    P.H = H;
    P.p0 = p0;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.status = status;  // may be nullptr: a wait that gives up is then not reported
    GS_TRY(cudaFuncSetAttribute(k_prefill_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
    dim3 grid((S + BM - 1) / BM, H);
    k_prefill_umma<<<grid, PF_THREADS, PF_SMEM, st>>>(P);
    GS_TRY(cudaGetLastError());
    return 0;
}

}  // namespace gs

#ifdef GS_PF_PROF
// timing probe only: copies the clock stamps of the heaviest CTA to the host
extern "C" __attribute__((visibility("default"))) int gs_pf_prof_read(long long *host) {
    return (int) cudaMemcpyFromSymbol(host, gs::g_pf_prof, sizeof(long long) * 32 * 8);
}
#endif
