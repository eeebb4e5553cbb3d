/* CPU oracle for the attention hot path: test infrastructure, never part of the product library.
 * See oracle.c for the reference lines each function follows. */
#ifndef GLMSSD_ORACLE_H
#define GLMSSD_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

float oracle_f16_to_f32(uint16_t h);
uint16_t oracle_f32_to_f16(float f);
void oracle_f16_to_f32_array(const uint16_t *x, float *y, int64_t n);
void oracle_f32_to_f16_array(const float *x, uint16_t *y, int64_t n);
int oracle_host_cores(void);

/* Every threaded entry point returns the number of threads it used. threads <= 0: all host cores. */
int oracle_mla_attn_ref(const float *q, const uint16_t *C, const int32_t *sel, int sel_stride, const int32_t *cnt,
                        float scale, float *o, int T, int H, int R, int threads);
void oracle_combine(const float *part, int64_t n_rows, int n_parts, int d_v, float *o);
int oracle_mla_decode(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens, const int32_t *seq_base,
                      const int32_t *page_table, int page_table_stride, int page_rows, float scale, float *o,
                      int n_seq, int T, int H, int d_qk, int d_v, int threads);
/* oracle_mla_decode with every row's attended range cut into key_splits work items (all host cores busy); scratch:
 * n_seq*T*H*key_splits*(d_v+2) floats */
int oracle_mla_decode_split(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens, const int32_t *seq_base,
                            const int32_t *page_table, int page_table_stride, int page_rows, float scale, float *o,
                            int n_seq, int T, int H, int d_qk, int d_v, int key_splits, float *scratch, int threads);
int oracle_mla_decode_partial(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens,
                              const int32_t *seq_base, const int32_t *page_table, int page_table_stride,
                              int page_rows, float scale, float *parts, int64_t part_lo, int64_t part_hi, int n_seq,
                              int T, int H, int d_qk, int d_v, int threads);
int oracle_prefill(const uint16_t *Q, const uint16_t *K, const uint16_t *V, float scale, float *o, int S, int H, int d,
                   int dv, int p0, const int32_t *rows_subset, int n_subset, int threads);
void oracle_quant_q8_rows(const float *x, int8_t *q, uint16_t *d, int64_t n_blocks);
void oracle_dequant_q8(const int8_t *q, const uint16_t *d, uint16_t *out, int64_t n_blocks);
void oracle_rope_inv_freq(float *inv_freq, int d_rope, double base);
void oracle_rope_append(const float *x, uint16_t *y, int T, int d_row, int d_rope, int64_t pos0, double base);
void oracle_norm_rope_append(const float *x, const float *w, float eps, uint16_t *y, int T, int d_row, int d_rope,
                             int64_t pos0, double base);
void oracle_rope_f16(uint16_t *x, int S, int H, int d, int d_rope, int64_t pos0, double base);

/* attention with its two per-head products (forward.rs:900-907), fp32 */
int oracle_mla_fused(const float *q, const uint16_t *k_b, const uint16_t *v_b, const uint16_t *cache, int seq_len, float scale,
                     float *ov, int T, int H, int d_q, int R, int d_out, int threads);
/* DSA k-pool indexer (ops.cu:619-791) */
void oracle_idx_pool(const float *kc, const float *gc, float *rk, float *rg, const float *ape, float *P, int p0, int T,
                     int Dk, int kpool);
void oracle_idx_score(const float *q, const float *w, const float *P, float *score, int64_t score_stride, int pos0, int T,
                      int kpool, int Hq, int Dk, float scale);
void oracle_idx_select(const float *score, int64_t score_stride, int pos0, int T, int kpool, int top_k, int32_t *sel,
                       int sel_stride, int32_t *cnt);

#ifdef __cplusplus
}
#endif
#endif
