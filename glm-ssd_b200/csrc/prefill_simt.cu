// CUDA-core causal prefill attention: the general-shape path (any S, prior context p0 > 0, head
// widths other than 256) and the second opinion for the tcgen05 prefill kernel.
//
// Semantics: query i of head h attends keys 0 .. p0+i; score = scale * q.k, softmax, o = P V.  The
// reference reaches the same result through its absorbed kernel with one launch per 256 queries
// (crates/engine/src/forward.rs:61, :898-908).
#include "internal.cuh"

namespace gs {
namespace {

constexpr int BQ = 32;    // queries per CTA
constexpr int BK = 32;    // keys per tile
constexpr int PNT = 256;  // threads: 8 per query row
constexpr int DMAX = 256;

template <bool OUT_F16>
__global__ void __launch_bounds__(PNT) k_prefill_simt(const __half *__restrict__ Q, const __half *__restrict__ K,
                                                      const __half *__restrict__ V, void *__restrict__ O, int S, int H,
                                                      int d, int p0, float scale) {
    // heavier (later) query blocks first so the tail of the grid is short
    const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
    const int q0 = qb * BQ;
    const int tid = threadIdx.x;
    const int qi = tid >> 3, sub = tid & 7;  // query row in the block, lane within the row's group of 8

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *sq = reinterpret_cast<float *>(smem_raw);           // [BQ][d]
    __half *sk = reinterpret_cast<__half *>(sq + BQ * d);      // [BK][d]
    __half *sv = sk + BK * d;                                  // [BK][d]
    float *sp = reinterpret_cast<float *>(sv + BK * d);        // [BQ][BK]

    const int64_t hs = (int64_t) H * d;  // stride between consecutive positions
    for (int i = tid; i < BQ * d; i += PNT) {
        const int r = i / d, c = i % d;
        sq[i] = q0 + r < S ? __half2float(Q[(int64_t) (q0 + r) * hs + (int64_t) h * d + c]) : 0.f;
    }
    float acc[DMAX / 8];
#pragma unroll
    for (int j = 0; j < DMAX / 8; j++) acc[j] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int my_q = q0 + qi;
    const int n_keys_cta = min(p0 + q0 + BQ, p0 + S);  // keys any query of this block may see
    const int vec = d / 8;
    __syncthreads();

    for (int k0 = 0; k0 < n_keys_cta; k0 += BK) {
        for (int i = tid; i < BK * vec; i += PNT) {
            const int r = i / vec, c = i % vec;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
            if (k0 + r < p0 + S) {
                kv = reinterpret_cast<const uint4 *>(K + (int64_t) (k0 + r) * hs + (int64_t) h * d)[c];
                vv = reinterpret_cast<const uint4 *>(V + (int64_t) (k0 + r) * hs + (int64_t) h * d)[c];
            }
            reinterpret_cast<uint4 *>(sk + r * d)[c] = kv;
            reinterpret_cast<uint4 *>(sv + r * d)[c] = vv;
        }
        __syncthreads();
        // scores for keys sub, sub+8, sub+16, sub+24 of this tile
        float s[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int kk = sub + 8 * j;
            const __half2 *kr = reinterpret_cast<const __half2 *>(sk + kk * d);
            const float2 *qr = reinterpret_cast<const float2 *>(sq + qi * d);
            float a = 0.f;
            for (int c = 0; c < d / 2; c++) {
                const float2 kf = __half22float2(kr[c]);
                const float2 qf = qr[c];
                a = fmaf(qf.x, kf.x, fmaf(qf.y, kf.y, a));
            }
            const bool ok = my_q < S && k0 + kk <= p0 + my_q;
            s[j] = ok ? a * scale : -INFINITY;
        }
        float mx = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run, mx);
        const float f = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        float ps = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p = s[j] == -INFINITY ? 0.f : expf(s[j] - m_new);
            sp[qi * BK + sub + 8 * j] = p;
            ps += p;
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l_run = l_run * f + ps;
        m_run = m_new;
        __syncwarp();
        // PV: this thread owns value columns sub + 8*j of its query row
#pragma unroll
        for (int j = 0; j < DMAX / 8; j++) acc[j] *= f;
        for (int kk = 0; kk < BK; kk++) {
            const float p = sp[qi * BK + kk];
            if (p != 0.f) {
#pragma unroll
                for (int j = 0; j < DMAX / 8; j++) {
                    const int c = sub + 8 * j;
                    if (c < d) acc[j] = fmaf(p, __half2float(sv[kk * d + c]), acc[j]);
                }
            }
        }
        __syncthreads();
    }
    if (my_q < S) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const int64_t off = (int64_t) my_q * hs + (int64_t) h * d;
#pragma unroll
        for (int j = 0; j < DMAX / 8; j++) {
            const int c = sub + 8 * j;
            if (c < d) {
                if (OUT_F16)
                    reinterpret_cast<__half *>(O)[off + c] = __float2half_rn(acc[j] * inv);
                else
                    reinterpret_cast<float *>(O)[off + c] = acc[j] * inv;
            }
        }
    }
}

}  // namespace

int launch_prefill_simt(const __half *q, const __half *k, const __half *v, void *o, int o_f16, int S, int H, int d,
                        int p0, float scale, cudaStream_t st) {
    if (d % 8 != 0 || d > DMAX || d <= 0) return fail_invalid("prefill: need d % 8 == 0 and d <= 256");
    if (S <= 0 || H <= 0) return 0;
    const size_t smem = (size_t) BQ * d * 4 + 2 * (size_t) BK * d * 2 + (size_t) BQ * BK * 4;
    dim3 grid((S + BQ - 1) / BQ, H);
    if (o_f16) {
        GS_TRY(cudaFuncSetAttribute(k_prefill_simt<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        k_prefill_simt<true><<<grid, PNT, smem, st>>>(q, k, v, o, S, H, d, p0, scale);
    } else {
        GS_TRY(cudaFuncSetAttribute(k_prefill_simt<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        k_prefill_simt<false><<<grid, PNT, smem, st>>>(q, k, v, o, S, H, d, p0, scale);
    }
    GS_TRY(cudaGetLastError());
    return 0;
}

}  // namespace gs
