// Merge of split-KV partial records (unnormalised acc, m, l) into outputs: the arithmetic of the
// reference's k_mla_combine (crates/cuda/kernels/ops.cu:552-574):
//   M = max m_s;  w_s = e^(m_s - M) (0 for an empty segment, m_s = -inf);  L = sum l_s w_s;
//   o = sum acc_s w_s / L, zeros when L == 0.
// One "item" is (output row, 128-column chunk), worked on by 256 threads: 32 column quads x 8 segment
// lanes.  The accumulator loads are issued before the weights are known, so an item costs one round
// trip to memory.
#pragma once
#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {

constexpr int CB_COLS = 128;
constexpr int CB_LANES = 8;
constexpr int CB_NT = (CB_COLS / 4) * CB_LANES;  // 256: warp w is segment lane w, its 32 lanes are the column quads
constexpr int CB_MAX_SEG = 1024;
constexpr int CB_REG_SEG = 20;                   // segments per lane held in registers (covers 160 segments)
static_assert(CB_COLS / 4 == 32 && CB_REG_SEG <= 32, "a warp is one segment lane; lane j also owns the weight of segment j");

struct CombineSmem {
    float m[CB_MAX_SEG], l[CB_MAX_SEG];  // only the path for more than 160 segments
    float red[CB_NT / 32], lred[CB_NT / 32];
    long long lred2[2][CB_NT / 32];
    float M, L;
    float4 part[CB_LANES][CB_COLS / 4];
};

// Address helpers of the generalised record layout (see CombinePlan).
__device__ __forceinline__ int64_t combine_row_stride_acc(const CombinePlan &C) { return C.row_stride_acc ? C.row_stride_acc : C.d_v; }
__device__ __forceinline__ int64_t combine_chunk_stride_acc(const CombinePlan &C) { return C.chunk_stride_acc ? C.chunk_stride_acc : CB_COLS; }
__device__ __forceinline__ int64_t combine_row_stride_ml(const CombinePlan &C) { return C.row_stride_ml ? C.row_stride_ml : 2; }
// column `col` of row `row_in_seg` of segment `seg`
__device__ __forceinline__ const float *combine_acc_ptr(const CombinePlan &C, int64_t seg, int row_in_seg, int col) {
    return C.acc + seg * C.seg_stride_acc + (int64_t) row_in_seg * combine_row_stride_acc(C) +
           (int64_t) (col / CB_COLS) * combine_chunk_stride_acc(C) + (col % CB_COLS);
}
__device__ __forceinline__ const float *combine_ml_ptr(const CombinePlan &C, int64_t seg, int row_in_seg) {
    return C.ml + seg * C.seg_stride_ml + (int64_t) row_in_seg * combine_row_stride_ml(C);
}

// Where the segments of output row `row` lie.
struct SegRange {
    int first, nseg, row_in_seg;
};

// True when combine_locate() needs nothing the preceding kernel writes, so it may run before the
// grid-dependency wait of a programmatic dependent launch.  (seq_lens is an input of the attention kernel,
// complete before that kernel's own dependency wait returned in any of its CTAs, and a dependent kernel
// starts only after every CTA of the attention kernel has passed that point.)
__device__ __forceinline__ bool combine_locate_is_early(const CombinePlan &C) { return C.desc == nullptr || C.seq_lens != nullptr; }

// All CB_NT threads call this.  The schedule of the tcgen05 kernel is recomputed from the sequence lengths:
// sequences are cut into units of `unit_rows` rows, the units are dealt in equal contiguous chunks to the
// n_ctas CTAs, and CTA c keeps the record of sequence b in segment c + b.
__device__ __forceinline__ SegRange combine_locate(const CombinePlan &C, int row, CombineSmem &S) {
    const int h = row % C.H, t = (row / C.H) % C.T, b = row / (C.H * C.T);
    SegRange r;
    if (!C.desc) {
        r.first = (b * C.T + t) * C.regular_segments;
        r.nseg = C.regular_segments;
        r.row_in_seg = h;
        return r;
    }
    r.row_in_seg = t * C.H + h;
    if (!C.seq_lens) {
        const int2 d = __ldcg(C.desc + b);
        r.first = d.x;
        r.nseg = d.y;
        return r;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The attention kernel caps every length at what the cache can hold and lets its running sum of units
    // saturate at 2^29; capped non-negative terms make that sum min(plain sum, 2^29).  The terms fit an int
    // (a length below 2^31 is at most 2^27 units of 16 rows); only the sums are kept in 64 bits, and the
    // divisions below run on the saturated 32-bit values.  unit_rows is 16 or 64: a shift.
    constexpr int kUnitCap = 1 << 29;
    const int shift = __ffs(C.unit_rows) - 1, div = C.seq_div > 1 ? C.seq_div : 1;
    const int len_cap = (int) min(C.len_cap, (int64_t) 0x7fffffff - 64);
    auto units_of = [&](int i) -> int {
        const int len = min(max(__ldg(C.seq_lens + (div == 1 ? i : i / div)), 0), len_cap);
        return (len + C.unit_rows - 1) >> shift;
    };
    long long before64 = 0, total64 = 0;
    for (int i = tid; i < C.n_seq; i += CB_NT) {
        const int u = units_of(i);
        total64 += u;
        if (i < b) before64 += u;
    }
    if (C.n_seq > 1) {  // one sequence: thread 0 alone holds the (single) term, nothing to add up
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            total64 += __shfl_xor_sync(0xffffffffu, total64, o);
            before64 += __shfl_xor_sync(0xffffffffu, before64, o);
        }
        if (lane == 0) {
            S.lred2[0][warp] = total64;
            S.lred2[1][warp] = before64;
        }
        __syncthreads();
        total64 = before64 = 0;
#pragma unroll
        for (int w = 0; w < CB_NT / 32; w++) {
            total64 += S.lred2[0][w];
            before64 += S.lred2[1][w];
        }
    }
    const int mine = units_of(b);
    if (C.n_seq == 1) total64 = mine;
    const int after = (int) min(before64 + mine, (long long) kUnitCap);  // saturated running sums, as the kernel holds them
    const int before = (int) min(before64, (long long) kUnitCap);
    const int total = (int) min(total64, (long long) kUnitCap);
    const int chunk = max(1, (total + C.n_ctas - 1) / C.n_ctas);
    r.first = b;
    r.nseg = 0;
    if (after > before) {
        const int c_first = before / chunk, c_last = (after - 1) / chunk;
        // CTA indices are below n_ctas by construction; the clamp only keeps absurd inputs inside the workspace
        const int cf = min(c_first, C.n_ctas - 1);
        r.first = cf + b;
        r.nseg = min(c_last - c_first + 1, C.n_ctas - cf);
    }
    return r;
}

// All CB_NT threads of the CTA call this with the same (row, col0).  Returns true in the threads that hold a
// result: `a` = 4 merged (unnormalised) accumulator columns starting at `col`, with the row's M and L.
__device__ __forceinline__ bool combine_item_compute(const CombinePlan &C, const SegRange &R, int col0, CombineSmem &S,
                                                     float4 &a_out, float &M_out, float &L_out, int &col_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int quad = lane, sl = warp;
    const int col = col0 + quad * 4;
    const int first = R.first, row_in_seg = R.row_in_seg;
    const int nseg = min(R.nseg, CB_MAX_SEG);
    const float *acc0 = combine_acc_ptr(C, first, row_in_seg, col < C.d_v ? col : 0);
    const float *ml0 = combine_ml_ptr(C, first, row_in_seg);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    float M, L;
    if (nseg <= CB_LANES * CB_REG_SEG) {
        // One round trip: lane j of segment lane sl fetches (m, l) of segment sl + 8 j, and every lane the four
        // columns of all the segments of its segment lane, before any weight is known.
        const int sj = sl + CB_LANES * lane;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (lane < CB_REG_SEG && sj < nseg) ml = __ldcg(reinterpret_cast<const float2 *>(ml0 + (int64_t) sj * C.seg_stride_ml));
        float4 v[CB_REG_SEG];
#pragma unroll
        for (int i = 0; i < CB_REG_SEG; i++) {
            const int s = sl + i * CB_LANES;
            v[i] = (s < nseg && col < C.d_v) ? __ldcg(reinterpret_cast<const float4 *>(acc0 + (int64_t) s * C.seg_stride_acc))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const float mx = warp_max(ml.x);
        if (lane == 0) S.red[warp] = mx;
        __syncthreads();
        M = S.red[0];
#pragma unroll
        for (int w = 1; w < CB_NT / 32; w++) M = fmaxf(M, S.red[w]);
        const float wj = ml.x == -INFINITY ? 0.f : expf(ml.x - M);
        const float ls = warp_sum(ml.y * wj);
        if (lane == 0) S.lred[warp] = ls;
#pragma unroll
        for (int i = 0; i < CB_REG_SEG; i++) {
            const float w = __shfl_sync(0xffffffffu, wj, i);
            if (w != 0.f) {  // an empty segment's accumulator never enters the sum
                a.x = fmaf(v[i].x, w, a.x);
                a.y = fmaf(v[i].y, w, a.y);
                a.z = fmaf(v[i].z, w, a.z);
                a.w = fmaf(v[i].w, w, a.w);
            }
        }
        S.part[sl][quad] = a;
        __syncthreads();
        L = 0.f;
#pragma unroll
        for (int w = 0; w < CB_NT / 32; w++) L += S.lred[w];
    } else {
        float mx = -INFINITY;
        for (int s = tid; s < nseg; s += CB_NT) {
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(ml0 + (int64_t) s * C.seg_stride_ml));
            S.m[s] = ml.x;
            S.l[s] = ml.y;
            mx = fmaxf(mx, ml.x);
        }
        mx = warp_max(mx);
        if (lane == 0) S.red[warp] = mx;
        __syncthreads();
        M = S.red[0];
#pragma unroll
        for (int w = 1; w < CB_NT / 32; w++) M = fmaxf(M, S.red[w]);
        // weights e^(m-M) replace m in shared memory; L = sum l w
        float lsum = 0.f;
        for (int s = tid; s < nseg; s += CB_NT) {
            const float m = S.m[s];
            const float w = m == -INFINITY ? 0.f : expf(m - M);
            S.m[s] = w;
            lsum += S.l[s] * w;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) S.lred[warp] = lsum;
        __syncthreads();
        if (col < C.d_v) {
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
        S.part[sl][quad] = a;
        __syncthreads();
        L = 0.f;
#pragma unroll
        for (int w = 0; w < CB_NT / 32; w++) L += S.lred[w];
    }
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

// The records of the tcgen05 kernel ([segment][row][d_v]) fetched by ONE tiled 3-D TMA copy: what an item (output row,
// 128 columns) needs is one 512-byte piece per segment, a whole record apart from the next - a box
// {128, 1, n_ctas} of the tensor {d_v, rows, segments}.  The box always spans n_ctas segments (a sequence has at most
// one per CTA); segments past the sequence's last one belong to other sequences or lie outside the tensor (zero-filled)
// and get weight 0.
constexpr int32_t ST_COMBINE = 1 << 18;  // status bit: the copy of the records did not complete in time
struct CombineBulk {
    CUtensorMap tm;
    CombinePlan c;
};

// All CB_NT threads call this with the same arguments.  `tile` is 128-byte aligned shared memory of n_ctas x 512 bytes,
// `bar` an initialised mbarrier (count 1) in its first phase, *abort_flag zero.  Thread 0 issues the copy; meanwhile
// thread i fetches (m, l) of segment i and the block forms M, the weights and L; after the copy has landed 8 segment
// lanes x 32 column quads sum from shared memory.  Returns false when the copy did not complete in time (status bit
// set, nothing may be written); else the threads of warp 0 hold the four merged (unnormalised) columns col0 + 4 lane
// in `a`, and every thread M and L.
__device__ __forceinline__ bool combine_item_fetch_tma(const CombinePlan &C, const CUtensorMap *tm, const SegRange &R, int col0,
                                                       float4 *tile, uint64_t *bar, int *abort_flag, CombineSmem &S, float4 &a,
                                                       float &M, float &L) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nseg = min(R.nseg, min(C.n_ctas, CB_NT));
    if (tid == 0 && nseg > 0) {
        sm100::mbar_arrive_expect_tx(bar, (uint32_t) C.n_ctas * CB_COLS * 4);  // the whole box, zero-filled rows included
        sm100::tma_load_3d(tile, tm, bar, col0, R.row_in_seg, R.first);
    }
    float2 ml = make_float2(-INFINITY, 0.f);
    if (tid < nseg) ml = __ldcg(reinterpret_cast<const float2 *>(combine_ml_ptr(C, R.first + tid, R.row_in_seg)));
    const float mx = warp_max(ml.x);
    if (lane == 0) S.red[warp] = mx;
    __syncthreads();
    M = S.red[0];
#pragma unroll
    for (int w = 1; w < CB_NT / 32; w++) M = fmaxf(M, S.red[w]);
    const float wgt = ml.x == -INFINITY ? 0.f : expf(ml.x - M);
    S.m[tid] = wgt;
    const float ls = warp_sum(ml.y * wgt);
    if (lane == 0) S.lred[warp] = ls;
    if (nseg > 0 && !sm100::mbar_wait(bar, 0, abort_flag, const_cast<int32_t *>(C.status), ST_COMBINE)) *abort_flag = 1;
    __syncthreads();
    if (*abort_flag) return false;
    L = 0.f;
#pragma unroll
    for (int w = 0; w < CB_NT / 32; w++) L += S.lred[w];
    a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = warp; s < nseg; s += CB_LANES) {
        const float w = S.m[s];
        if (w != 0.f) {  // an empty segment's accumulator never enters the sum
            const float4 u = tile[s * (CB_COLS / 4) + lane];
            a.x = fmaf(u.x, w, a.x);
            a.y = fmaf(u.y, w, a.y);
            a.z = fmaf(u.z, w, a.z);
            a.w = fmaf(u.w, w, a.w);
        }
    }
    S.part[warp][lane] = a;
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int j = 1; j < CB_LANES; j++) {
            const float4 u = S.part[j][lane];
            a.x += u.x;
            a.y += u.y;
            a.z += u.z;
            a.w += u.w;
        }
    }
    return true;
}

// Output row of record row `row` = (sequence b, token t, head h of the records).  The records may cover a group of
// the output's heads (h0), or - seq_div > 1 - sequence b of the records is head group b % seq_div of caller
// sequence b / seq_div.
__device__ __forceinline__ int64_t combine_out_row(const CombinePlan &C, int row, int &H_out) {
    H_out = C.H_out > 0 ? C.H_out : C.H;
    if (C.seq_div > 1) {
        const int h = row % C.H, t = (row / C.H) % C.T, b = row / (C.H * C.T);
        return ((int64_t) (b / C.seq_div) * C.T + t) * H_out + (b % C.seq_div) * C.H + h;
    }
    return (int64_t) (row / C.H) * H_out + C.h0 + row % C.H;
}

// Merge one item and write it: normalised output and/or the merged record.
__device__ __forceinline__ void combine_item(const CombinePlan &C, const SegRange &R, int row, int col0, CombineSmem &S) {
    float4 a;
    float M, L;
    int col;
    if (combine_item_compute(C, R, col0, S, a, M, L, col)) {
        // the records may cover a group of the output's heads: row (b, t, h) of the group is row (b, t, h0 + h) there
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
            *reinterpret_cast<float4 *>(C.o + orow * C.d_v + col) =
                make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
}

}  // namespace gs
