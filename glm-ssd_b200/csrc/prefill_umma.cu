// Causal prefill attention on the Blackwell tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Semantics (what the reference reaches through its absorbed kernel with one launch per 256
// queries, crates/engine/src/forward.rs:61, :898-908): query i of head h attends keys 0 .. p0+i,
// score = scale * q.k over d = 256, softmax, o = P V.
//
// One CTA per (128-query block, head).  Per 128-key tile:
//   S[128 x 128]  = Q[128 x 256] . K_tile^T      16 MMAs (M = 128, N = 128, K = 16), both operands
//                                                 K-major in 128-byte-swizzled shared memory
//   P = exp2(S*c - m) as f16, written back into the tensor memory columns of S (one query row per
//       thread, so the row maximum and row sum need no shuffles)
//   O[128 x 256] += P . V_tile                    8 MMAs (M = 128, N = 256, K = 16) with P read from
//                                                 tensor memory and V_tile read MN-major
// S is double-buffered in tensor memory (2 x 128 columns + 256 columns of O = all 512), so the
// scores of tile j+1 are computed while the softmax of tile j runs.  K and V tiles are single
// 64 KB buffers fed by two independent TMA producers; K of tile j+1 is fetched as soon as S of tile j
// has been computed, V of tile j+1 as soon as P.V of tile j has.  The accumulator is rescaled lazily
// (only when a row maximum grows by more than 2^8), decided per warp.
// Every mbarrier wait is bounded and ends in an error status instead of a hang.
#include <string.h>

#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {
namespace {
using namespace sm100;

constexpr int BM = 128;                  // query rows per CTA
constexpr int BN = 128;                  // keys per tile
constexpr int HD = 256;                  // head width
constexpr int NDB = HD / 64;             // 64-column blocks per row
constexpr int TBLK = 128 * 128;          // bytes of one [128 rows][64 cols] block
constexpr int TILE_BYTES = NDB * TBLK;   // 64 KB: a Q, K or V tile
constexpr int PF_THREADS = 224;          // warp 0 K producer, 1 MMA, 2-5 softmax, 6 V producer
constexpr int S_COLS = 128, O_COL = 256;
constexpr float PF_RESCALE = 8.0f;

struct PrefillParams {
    CUtensorMap tm_q, tm_k, tm_v;
    void *o;
    int o_f16;
    int S, H, p0;
    float scale_log2;
    int32_t *status;  // may be nullptr
};

struct PfBarriers {
    uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full[2], p_full[2], pv_done;
};

struct PfSmemMisc {
    PfBarriers bar;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int PF_SMEM = 3 * TILE_BYTES + (int) sizeof(PfSmemMisc) + 1024;

__global__ void __launch_bounds__(PF_THREADS, 1) k_prefill_umma(const __grid_constant__ PrefillParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t *q_smem = smem, *k_smem = smem + TILE_BYTES, *v_smem = smem + 2 * TILE_BYTES;
    PfSmemMisc &M = *reinterpret_cast<PfSmemMisc *>(smem + 3 * TILE_BYTES);
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
        mbar_init(&B.k_full, 1);
        mbar_init(&B.k_empty, 1);
        mbar_init(&B.v_full, 1);
        mbar_init(&B.v_empty, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&B.s_full[i], 1);
            mbar_init(&B.p_full[i], 4);
        }
        mbar_init(&B.pv_done, 1);
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
            mbar_arrive_expect_tx(&B.q_full, TILE_BYTES);
#pragma unroll
            for (int b = 0; b < NDB; b++) tma_load_2d(q_smem + b * TBLK, &P.tm_q, &B.q_full, col0 + b * 64, q0);
        }
        __syncwarp();
        for (int j = 0; j < n_tiles; j++) {
            if (j > 0 && !mbar_wait(&B.k_empty, (j - 1) & 1, abort_flag, P.status, 1)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&B.k_full, TILE_BYTES);
#pragma unroll
                for (int b = 0; b < NDB; b++) tma_load_2d(k_smem + b * TBLK, &P.tm_k, &B.k_full, col0 + b * 64, j * BN);
            }
            __syncwarp();
        }
    } else if (warp == 6) {
        // ---- the V tiles ------------------------------------------------------------------------------------
        for (int j = 0; j < n_tiles; j++) {
            if (j > 0 && !mbar_wait(&B.v_empty, (j - 1) & 1, abort_flag, P.status, 1)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&B.v_full, TILE_BYTES);
#pragma unroll
                for (int b = 0; b < NDB; b++) tma_load_2d(v_smem + b * TBLK, &P.tm_v, &B.v_full, col0 + b * 64, j * BN);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------------------------------
        constexpr uint32_t idesc_s = make_idesc_f16(BM, BN, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_f16(BM, HD, 0, 1);  // A = P from tensor memory, B = V MN-major
        const uint64_t d_kmaj = make_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint64_t d_v = make_smem_desc(0, TBLK, 1024, kSwizzle128B);
        const uint32_t q_lo = smem_u32(q_smem) >> 4, k_lo = smem_u32(k_smem) >> 4, v_lo = smem_u32(v_smem) >> 4;
        bool ok = mbar_wait(&B.q_full, 0, abort_flag, P.status, 2);
        auto issue_s = [&](int j) {
            if (elect_one()) {
#pragma unroll
                for (int b = 0; b < NDB; b++)
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_ss(tmem + (j & 1) * S_COLS, d_kmaj + (q_lo + b * (TBLK >> 4) + ks * 2),
                                d_kmaj + (k_lo + b * (TBLK >> 4) + ks * 2), idesc_s, (b | ks) != 0);
                umma_commit(&B.s_full[j & 1]);
                umma_commit(&B.k_empty);
            }
            __syncwarp();
        };
        if (ok) ok = mbar_wait(&B.k_full, 0, abort_flag, P.status, 2);
        if (ok) {
            tc_fence_after();
            issue_s(0);
        }
        for (int j = 0; ok && j < n_tiles; j++) {
            if (j + 1 < n_tiles) {
                ok = mbar_wait(&B.k_full, (j + 1) & 1, abort_flag, P.status, 2);
                // S(j+1) overwrites the tensor-memory columns P(j-1) lives in.  Two MMAs are only ordered with
                // respect to each other on the same accumulator, so P.V(j-1) must have completed first.
                if (ok && j > 0) ok = mbar_wait(&B.pv_done, (j - 1) & 1, abort_flag, P.status, 2);
                if (!ok) break;
                tc_fence_after();
                issue_s(j + 1);
            }
            ok = mbar_wait(&B.p_full[j & 1], (j >> 1) & 1, abort_flag, P.status, 2) &&
                 mbar_wait(&B.v_full, j & 1, abort_flag, P.status, 2);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < BN / 16; ks++)
                    umma_ts(tmem + O_COL, tmem + (j & 1) * S_COLS + ks * 8, d_v + (v_lo + ks * 128), idesc_pv, j > 0 || ks > 0);
                umma_commit(&B.v_empty);
                umma_commit(&B.pv_done);
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
                const uint32_t s_addr = tmem + lane_base + (j & 1) * S_COLS;
                ok = mbar_wait(&B.s_full[j & 1], (j >> 1) & 1, abort_flag, P.status, 4);
                if (!ok) break;
                tc_fence_after();
                const int k0 = j * BN;
                const bool need_mask = k0 + BN - 1 > P.p0 + q0;  // some row of the block must not see some key
                // the whole score row of this thread (128 keys) is read once and kept in registers: one
                // tensor-memory round trip per tile instead of eight
                uint32_t r[BN];
#pragma unroll
                for (int c = 0; c < BN / 16; c++) tmem_ld16(s_addr + c * 16, *reinterpret_cast<uint32_t(*)[16]>(r + c * 16));
                tmem_wait_ld();
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
                        // the accumulator holds tiles 0..j-1: wait for P.V(j-1), then scale this row
                        ok = mbar_wait(&B.pv_done, (j - 1) & 1, abort_flag, P.status, 4);
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
#pragma unroll
                for (int c = 0; c < BN / 32; c++) tmem_st16(s_addr + c * 16, *reinterpret_cast<const uint32_t(*)[16]>(r + c * 16));
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&B.p_full[j & 1]);
            }
            // ---- epilogue: O / l -> global ------------------------------------------------------------------------
            // A parity wait only tells phases apart when the waiter is at most one phase behind.  These warps last
            // saw P.V(n-3) complete (through S(n-1), which was issued after it), so P.V(n-2) is awaited first:
            // asking for the parity of P.V(n-1) while P.V(n-2) is still running would return at once.
            if (ok && n_tiles >= 2) ok = mbar_wait(&B.pv_done, (n_tiles - 2) & 1, abort_flag, P.status, 4);
            if (ok) ok = mbar_wait(&B.pv_done, (n_tiles - 1) & 1, abort_flag, P.status, 4);
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
                        int p0, float scale, cudaStream_t st) {
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
    P.status = nullptr;
    GS_TRY(cudaFuncSetAttribute(k_prefill_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
    dim3 grid((S + BM - 1) / BM, H);
    k_prefill_umma<<<grid, PF_THREADS, PF_SMEM, st>>>(P);
    GS_TRY(cudaGetLastError());
    return 0;
}

}  // namespace gs
