// Shared host/device helpers of the attention library.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/glmssd_attn.h"

#define GS_EXPORT extern "C" __attribute__((visibility("default")))

namespace gs {

// Last-error text, per host thread (gs_attn_last_error_string).
void set_error(const char *fmt, ...);

inline int fail_invalid(const char *what) {
    set_error("%s", what);
    return (int) cudaErrorInvalidValue;
}

#define GS_TRY(expr)                                                          \
    do {                                                                      \
        cudaError_t _e = (expr);                                              \
        if (_e != cudaSuccess) {                                              \
            gs::set_error("%s: %s", #expr, cudaGetErrorString(_e));           \
            return (int) _e;                                                  \
        }                                                                     \
    } while (0)

// ---- decode workspace layout -------------------------------------------------------------------
// [0, 32768)               status block: int32 status word (sticky, kernels only OR into it);
//                           int32 at byte 4: when non-zero, CTA 0 of the tcgen05 kernel writes clock64
//                           stamps of its first tiles as int64 from byte 256 on (a tuning aid, off by default)
//   [4096, 16384)           with the same switch every CTA of the tcgen05 kernel writes eight int64 %globaltimer
//                           stamps (entry, inputs visible, first tile landed, drain start/end, exit, SM id)
//   [16384, 32768)          and every CTA of the combine kernel eight stamps of its own
// [32768, ...)             per-sequence segment descriptors, then
//                           partial accumulators f32 [n_segments][rows_q][d_v]
// then                     partial (m, l)       f32 [n_segments][rows_q][2]
// A "segment" is the share of one sequence handled by one CTA (tcgen05 kernel: at most
// n_ctas + n_seq of them) or one (sequence, token, split) triple (CUDA-core kernel).
constexpr int kStatusBytes = 32768;
constexpr int kCtaProfOffsetBytes = 4096;       // [cta][8] int64
constexpr int kCombineProfOffsetBytes = 16384;  // [cta][8] int64, first 256 CTAs
constexpr int kProfOffsetBytes = 256;
constexpr int kProfSlots = 16;   // stamps per tile
constexpr int kProfTiles = 24;   // tiles recorded
constexpr int kMaxCtas = 160;       // persistent grid never exceeds this (B200 has 148 SMs)
constexpr int kSimtMaxSplits = 64;  // CUDA-core kernel: splits per (sequence, token)

inline int64_t decode_segments_bound(int n_seq, int T) {
    const int64_t umma = (int64_t) kMaxCtas + n_seq;
    const int64_t simt = (int64_t) n_seq * T * kSimtMaxSplits;
    return umma > simt ? umma : simt;
}

// Row addressing shared by the kernels: explicit list, paged or dense.
struct RowMap {
    const int32_t *list;   // explicit positions (legacy `sel` row) or nullptr
    const int32_t *pages;  // page ids of this sequence or nullptr
    int64_t base;          // dense: first row
    int page_rows;
    __device__ __forceinline__ int64_t operator()(int64_t i) const {
        if (list) return list[i];
        if (pages) return (int64_t) pages[i / page_rows] * page_rows + (i % page_rows);
        return base + i;
    }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace gs
