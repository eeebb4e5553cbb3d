// Merge of split-KV partial records (unnormalised acc, m, l) into outputs: the arithmetic of the
// reference's k_mla_combine (crates/cuda/kernels/ops.cu:552-574):
//   M = max m_s;  w_s = e^(m_s - M) (0 for an empty segment, m_s = -inf);  L = sum l_s w_s;
//   o = sum acc_s w_s / L, zeros when L == 0.
// One "item" is (output row, 128-column chunk), worked on by 256 threads: 32 column quads x 8 segment
// lanes.  The accumulator loads are issued before the weights are known, so an item costs one round
// trip to memory.  
#pragma once
#include "internal.cuh"

namespace gs {

constexpr int CB_COLS = 128;
constexpr int CB_LANES = 8;
constexpr int CB_NT = (CB_COLS / 4) * CB_LANES;  // 256
constexpr int CB_MAX_SEG = 1024;
constexpr int CB_REG_SEG = 20;                   // segments per lane held in registers (covers 160 segments)

struct CombineSmem {
    float m[CB_MAX_SEG], l[CB_MAX_SEG];
    float red[CB_NT / 32];
    float M, L;
    float4 part[CB_LANES][CB_COLS / 4];
};

// All CB_NT threads of the CTA call this with the same (row, col0).  Returns true in the threads that hold a
// result: `a` = 4 merged (unnormalised) accumulator columns starting at `col`, with the row's M and L.
__device__ __forceinline__ bool combine_item_compute(const CombinePlan &C, int row, int col0, CombineSmem &S, float4 &a_out,
                                                     float &M_out, float &L_out, int &col_out) {
    const int h = row % C.H, t = (row / C.H) % C.T, b = row / (C.H * C.T);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int quad = tid % (CB_COLS / 4), sl = tid / (CB_COLS / 4);
    const int col = col0 + quad * 4;
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
    nseg = min(nseg, CB_MAX_SEG);
    const float *acc0 = C.acc + (int64_t) first * C.seg_stride_acc + (int64_t) row_in_seg * C.d_v + col;
    const bool in_regs = nseg <= CB_LANES * CB_REG_SEG;
    float4 v[CB_REG_SEG];
    if (in_regs && col < C.d_v) {
#pragma unroll
        for (int i = 0; i < CB_REG_SEG; i++) {
            const int s = sl + i * CB_LANES;
            v[i] = s < nseg ? __ldcg(reinterpret_cast<const float4 *>(acc0 + (int64_t) s * C.seg_stride_acc))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float mx = -INFINITY;
    for (int s = tid; s < nseg; s += CB_NT) {
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(C.ml + (int64_t) (first + s) * C.seg_stride_ml + row_in_seg * 2));
        S.m[s] = ml.x;
        S.l[s] = ml.y;
        mx = fmaxf(mx, ml.x);
    }
    mx = warp_max(mx);
    if (lane == 0) S.red[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = -INFINITY;
        for (int w = 0; w < CB_NT / 32; w++) m = fmaxf(m, S.red[w]);
        S.M = m;
    }
    __syncthreads();
    const float M = S.M;
    // weights e^(m-M) replace m in shared memory; L = sum l w
    float lsum = 0.f;
    for (int s = tid; s < nseg; s += CB_NT) {
        const float m = S.m[s];
        const float w = m == -INFINITY ? 0.f : expf(m - M);
        S.m[s] = w;
        lsum += S.l[s] * w;
    }
    lsum = warp_sum(lsum);
    if (lane == 0) S.red[warp] = lsum;
    __syncthreads();
    if (tid == 0) {
        float l = 0.f;
        for (int w = 0; w < CB_NT / 32; w++) l += S.red[w];
        S.L = l;
    }
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < C.d_v) {
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < CB_REG_SEG; i++) {
                const int s = sl + i * CB_LANES;
                const float w = s < nseg ? S.m[s] : 0.f;
                if (w != 0.f) {  // an empty segment's accumulator never enters the sum
                    a.x = fmaf(v[i].x, w, a.x);
                    a.y = fmaf(v[i].y, w, a.y);
                    a.z = fmaf(v[i].z, w, a.z);
                    a.w = fmaf(v[i].w, w, a.w);
                }
            }
        } else {
            for (int s = sl; s < nseg; s += CB_LANES) {
                const float w = S.m[s];
                if (w != 0.f) {
                    const float4 u = __ldcg(reinterpret_cast<const float4 *>(acc0 + (int64_t) s * C.seg_stride_acc));
                    a.x = fmaf(u.x, w, a.x);
                    a.y = fmaf(u.y, w, a.y);
                    a.z = fmaf(u.z, w, a.z);
                    a.w = fmaf(u.w, w, a.w);
                }
            }
        }
    }
    S.part[sl][quad] = a;
    __syncthreads();
    const float L = S.L;
    bool holds = false;
    if (sl == 0 && col < C.d_v) {
#pragma unroll
        for (int j = 1; j < CB_LANES; j++) {
            const float4 u = S.part[j][quad];
            a.x += u.x;
            a.y += u.y;
            a.z += u.z;
            a.w += u.w;
        }
        holds = true;
    }
    a_out = a;
    M_out = M;
    L_out = L;
    col_out = col;
    __syncthreads();  // shared memory is reused by the next item
    return holds;
}

// Merge one item and write it: normalised output and/or the merged record.
__device__ __forceinline__ void combine_item(const CombinePlan &C, int row, int col0, CombineSmem &S) {
    float4 a;
    float M, L;
    int col;
    if (combine_item_compute(C, row, col0, S, a, M, L, col)) {
        if (C.part_out) {
            const int64_t rows_total = (int64_t) C.n_seq * C.T * C.H;
            *reinterpret_cast<float4 *>(C.part_out + (int64_t) row * C.d_v + col) = a;
            if (col == 0) {
                C.part_out[rows_total * C.d_v + (int64_t) row * 2] = M;
                C.part_out[rows_total * C.d_v + (int64_t) row * 2 + 1] = L;
            }
        }
        if (C.o) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4 *>(C.o + (int64_t) row * C.d_v + col) =
                make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
}

}  // namespace gs
