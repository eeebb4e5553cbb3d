// Internal launch interfaces between the translation units of the attention library.
#pragma once
#include "common.cuh"

namespace gs {

// A decode call with every argument resolved (see gs_mla_decode_args for the meaning).
struct DecodeProblem {
    const void *q;        // f16, or f32 when q_is_f32
    bool q_is_f32;
    const __half *cache;
    const __half *cache_scales;  // Q8 cache: `cache` holds int8 rows and this one f16 scale per 32 values
    int64_t cache_rows;
    const int32_t *seq_lens;
    const int32_t *seq_base;
    const int32_t *page_table;
    int page_table_stride, page_rows;
    const int32_t *sel;   // legacy explicit position lists [T][sel_stride] (n_seq == 1), lengths in seq_lens[T]
    int sel_stride;
    float scale;
    int tail_causal;
    float *o;
    float *part_out;
    // workspace pieces
    int32_t *status;
    float *ws_acc;
    float *ws_ml;
    int2 *ws_desc;        // per-sequence (first_segment, n_segments), written by the tcgen05 kernel
    int64_t max_segments;
    int64_t max_record_rows;  // query rows of partial records the workspace holds (segments x rows per segment)
    int n_seq, T, H, d_qk, d_v;
    int max_seq_len;
    int splits;           // CUDA-core kernel: splits per (sequence, token); 0 = choose
    int sm_count;
    int max_ctas;         // tcgen05 kernel: upper bound of the persistent grid (0 = one CTA per SM)
    bool no_combine;      // stop after the attention kernel (timing aid)
    const gs_shard_exchange *exchange;  // cross-GPU merge of the records instead of a local output, or nullptr
    cudaEvent_t ev_after_main;  // recorded between the attention kernel and the combine, or nullptr
};

// Combine descriptor: how the segments of an output row are found.
struct CombinePlan {
    const float *acc;      // accumulators of the records (addressing below)
    const float *ml;       // their (m, l) pairs
    const int2 *desc;      // per sequence (first_segment, n_segments), or nullptr => regular
    int regular_segments;  // desc == nullptr: segments per (sequence, token) group, consecutive
    int64_t seg_stride_acc;  // floats between the accumulator blocks of consecutive segments
    int64_t seg_stride_ml;   // floats between the (m, l) blocks of consecutive segments
    // Generalised addressing (0 = the plain record layout [segment][row][d_v] / [segment][row][2]): column c of row r of
    // segment s lies at acc + s*seg_stride_acc + r*row_stride_acc + (c/128)*chunk_stride_acc + c%128, its (m, l) pair at
    // ml + s*seg_stride_ml + r*row_stride_ml.  The tcgen05 kernel keeps its records as [row][128-column chunk][segment][128],
    // so that everything one (row, chunk) item of the combine needs is one contiguous run of memory.
    int64_t row_stride_acc, chunk_stride_acc, row_stride_ml;
    bool bulk;             // fetch an item's accumulators with one tiled TMA copy into shared memory (k_combine_bulk)
    int n_segments;        // bulk: segments the record arrays hold (extent of the tensor map)
    int n_seq, T, H, d_v;  // H: heads in the records being merged
    int H_out, h0;         // the output has H_out heads per token and these are heads h0 .. h0+H-1 (0, 0: H_out = H)
    float *o;              // may be nullptr
    float *part_out;       // may be nullptr
    const int32_t *status; // workspace status block (stamps switch at word 1) or nullptr
    // with desc: when seq_lens is set, the (first_segment, n_segments) pairs are recomputed from the lengths
    // (unit_rows rows per unit, units dealt in equal chunks to n_ctas CTAs) instead of being read from desc
    const int32_t *seq_lens;
    int unit_rows, n_ctas;
    int64_t len_cap;       // a length counts as at most this many rows, exactly as in the attention kernel
    int seq_div;           // > 1: sequence b of the records has the length of caller sequence b / seq_div (0 or 1: itself)
};

int launch_decode_simt(const DecodeProblem &p, cudaStream_t st);
int launch_combine(const CombinePlan &c, cudaStream_t st);
// local merge + peer-to-peer exchange of the merged records + final merge (exchange.cu)
int launch_exchange_combine(CombinePlan c, const gs_shard_exchange &x, float *o, int32_t *status, int sm_count,
                            cudaStream_t st);
bool decode_umma_supported(const DecodeProblem &p, const char **why);
// position lists (the reference's sel / cnt) with f32 queries on the tcgen05 kernel: 0 launched, -1 shape not taken, else an error
int launch_decode_umma_list(const float *q, const void *C, const __half *C_scales, const int32_t *sel, int sel_stride, const int32_t *cnt,
                            float scale, float *o, float *part, int T, int H, int R, int splits, int sm_count, cudaStream_t st);
int read_list_status(int32_t *out);
int launch_decode_umma(const DecodeProblem &p, cudaStream_t st);

int launch_prefill_simt(const __half *q, const __half *k, const __half *v, void *o, int o_f16, int S, int H, int d,
                        int p0, float scale, cudaStream_t st);
bool prefill_umma_supported(int S, int H, int d, int p0, const char **why);
int launch_prefill_umma(const __half *q, const __half *k, const __half *v, void *o, int o_f16, int S, int H, int d,
                        int p0, float scale, int32_t *status, cudaStream_t st);

}  // namespace gs
