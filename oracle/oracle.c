/*
 * CPU oracle for the GLM-SSD attention hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C fp32 restatement of the attention semantics of the reference engine's
 * CUDA kernels, used by the test-suite as the checker and by the benchmark as the timed CPU
 * baseline.  It is never linked into, imported by, or called from the product library.
 *
 * Parity status: the reference repository holds no golden vector, known-answer test or CPU
 * implementation for its attention path, so this restatement is pinned in two other ways:
 *   (1) the f16 conversion pair is checked against the reference's own pin, the exhaustive
 *       65 536-value round trip of crates/quants/src/lib.rs:361-370;
 *   (2) the attention functions are checked against outputs of the reference's own CUDA kernel
 *       (crates/cuda/kernels/ops.cu gs_mla_attn, gemm.cu gs_f32_to_f16) compiled unmodified and
 *       run on a B200; those outputs are committed as fixtures under tests/golden/.
 * The 576-wide score / 512-wide value split, RoPE and the non-absorbed prefill are extensions the
 * reference does not have; for them parity is unpinned by the reference and rests on (2)'s shared
 * core plus an independent float64 numpy check in the tests.
 *
 * Each function cites the reference lines it follows (paths relative to the reference project).
 */
#define _GNU_SOURCE
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "oracle.h"

/* ------------------------------------------------------------------------------------------
 * f16 <-> f32, round-to-nearest-even.  Follows crates/quants/src/lib.rs:15-38 (f16_to_f32) and
 * :41-74 (f32_to_f16); the CUDA side of the reference uses __float2half (gemm.cu:157), which is
 * the same rounding.
 * ------------------------------------------------------------------------------------------ */
float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t) (h >> 15)) << 31;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal half: shift the mantissa up until its leading one reaches bit 10 */
            uint32_t e = 113;
            while ((man & 0x400) == 0) {
                man <<= 1;
                e -= 1;
            }
            bits = sign | (e << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t) ((x >> 16) & 0x8000);
    int32_t exp = (int32_t) ((x >> 23) & 0xff);
    uint32_t man = x & 0x7fffff;
    if (exp == 0xff) return (uint16_t) (sign | 0x7c00 | (man ? 0x200 : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t) (sign | 0x7c00);
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = man | 0x800000;
        uint32_t shift = (uint32_t) (14 - e);
        uint32_t half = 1u << (shift - 1);
        uint32_t rem = m & ((1u << shift) - 1);
        uint32_t r = m >> shift;
        if (rem > half || (rem == half && (r & 1))) r += 1;
        return (uint16_t) (sign | r);
    }
    uint32_t rem = man & 0x1fff;
    uint32_t r = ((uint32_t) e << 10) | (man >> 13);
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r += 1;
    return (uint16_t) (sign | r);
}

static float g_h2f[65536];
static pthread_once_t g_h2f_once = PTHREAD_ONCE_INIT;
static void h2f_init(void) {
    for (uint32_t i = 0; i < 65536; i++) g_h2f[i] = oracle_f16_to_f32((uint16_t) i);
}
static inline const float *h2f_table(void) {
    pthread_once(&g_h2f_once, h2f_init);
    return g_h2f;
}

void oracle_f16_to_f32_array(const uint16_t *x, float *y, int64_t n) {
    const float *lut = h2f_table();
    for (int64_t i = 0; i < n; i++) y[i] = lut[x[i]];
}

/* KV-append of the reference: cache[i] = half_rn(x[i]) for i < n (gemm.cu:155-163). */
void oracle_f32_to_f16_array(const float *x, uint16_t *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = oracle_f32_to_f16(x[i]);
}

/* ------------------------------------------------------------------------------------------
 * Thread pool helper: run fn(item) for item in [0, n_items) on up to `threads` pthreads.
 * ------------------------------------------------------------------------------------------ */
typedef void (*item_fn)(void *ctx, int64_t item);
typedef struct {
    item_fn fn;
    void *ctx;
    int64_t n_items;
    volatile int64_t next;
} pool_t;

static void *pool_worker(void *arg) {
    pool_t *p = (pool_t *) arg;
    for (;;) {
        int64_t i = __atomic_fetch_add(&p->next, 1, __ATOMIC_RELAXED);
        if (i >= p->n_items) break;
        p->fn(p->ctx, i);
    }
    return NULL;
}

int oracle_host_cores(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int) n : 1;
}

static int run_pool(item_fn fn, void *ctx, int64_t n_items, int threads) {
    if (threads <= 0) threads = oracle_host_cores();
    if (threads > 256) threads = 256;
    if ((int64_t) threads > n_items) threads = n_items > 0 ? (int) n_items : 1;
    pool_t p = {fn, ctx, n_items, 0};
    if (threads == 1) {
        pool_worker(&p);
        return 1;
    }
    pthread_t th[256];
    int started = 0;
    for (int t = 0; t < threads - 1; t++) {
        if (pthread_create(&th[started], NULL, pool_worker, &p) == 0) started++;
    }
    pool_worker(&p);
    for (int t = 0; t < started; t++) pthread_join(th[t], NULL);
    return started + 1;
}

/* ------------------------------------------------------------------------------------------
 * One attention row.  Semantics of k_mla_flash (crates/cuda/kernels/ops.cu:420-424, :487-538):
 *   score_s = scale * q . K[row_s]          (fp32 accumulate over d_qk)
 *   p_s     = exp(score_s - max_s score)     (softmax over the n attended rows)
 *   o       = sum_s p_s * V[row_s] / sum_s p_s, over d_v columns; an empty set gives zeros
 *             (ops.cu:535, :565).
 * In the reference K and V are the same latent row (d_qk = d_v = 512); the absorbed-MLA extension
 * scores over 576 columns and takes V = the first 512 of the same row; the non-absorbed prefill
 * passes separate K and V rows.  `rows` (may be NULL = identity) is the position list sel[t]
 * (ops.cu:455, :459).  Also returns the softmax statistics (m = max score, l = sum p) so that
 * split partials in the layout of ops.cu:539-549 can be formed.
 * ------------------------------------------------------------------------------------------ */
#if defined(__F16C__) && defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
/* 8-wide helpers; the f16 -> f32 widening is exact, so these give the same products as the table. */
static inline float dot_f32_f16(const float *q, const uint16_t *k, int d) {
    __m256 a0 = _mm256_setzero_ps(), a1 = _mm256_setzero_ps();
    int r = 0;
    for (; r + 16 <= d; r += 16) {
        a0 = _mm256_fmadd_ps(_mm256_loadu_ps(q + r), _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (k + r))), a0);
        a1 = _mm256_fmadd_ps(_mm256_loadu_ps(q + r + 8), _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (k + r + 8))),
                             a1);
    }
    float tmp[8];
    _mm256_storeu_ps(tmp, _mm256_add_ps(a0, a1));
    float acc = ((tmp[0] + tmp[1]) + (tmp[2] + tmp[3])) + ((tmp[4] + tmp[5]) + (tmp[6] + tmp[7]));
    const float *lut = h2f_table();
    for (; r < d; r++) acc += q[r] * lut[k[r]];
    return acc;
}
static inline void axpy_f16(float *o, float p, const uint16_t *v, int d) {
    const __m256 pp = _mm256_set1_ps(p);
    int c = 0;
    for (; c + 8 <= d; c += 8)
        _mm256_storeu_ps(o + c, _mm256_fmadd_ps(pp, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (v + c))),
                                                _mm256_loadu_ps(o + c)));
    const float *lut = h2f_table();
    for (; c < d; c++) o[c] += p * lut[v[c]];
}
#else
static inline float dot_f32_f16(const float *q, const uint16_t *k, int d) {
    const float *lut = h2f_table();
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int r = 0;
    for (; r + 4 <= d; r += 4) {
        a0 += q[r] * lut[k[r]];
        a1 += q[r + 1] * lut[k[r + 1]];
        a2 += q[r + 2] * lut[k[r + 2]];
        a3 += q[r + 3] * lut[k[r + 3]];
    }
    for (; r < d; r++) a0 += q[r] * lut[k[r]];
    return (a0 + a1) + (a2 + a3);
}
static inline void axpy_f16(float *o, float p, const uint16_t *v, int d) {
    const float *lut = h2f_table();
    for (int c = 0; c < d; c++) o[c] += p * lut[v[c]];
}
#endif

/* Register-blocked forms used by the timed CPU baseline only: four query rows against one key row (the key row is widened
 * once), and four weighted key rows into one output row (the output row is loaded and stored once). */
#if defined(__F16C__) && defined(__AVX2__) && defined(__FMA__)
static inline float hsum8(__m256 v) {
    float t[8];
    _mm256_storeu_ps(t, v);
    return ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
}
static inline void dot4_f32_f16(const float *q, int64_t q_stride, const uint16_t *k, int d, float out[4]) {
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0, b0 = a0, b1 = a0, b2 = a0, b3 = a0;
    int r = 0;
    for (; r + 16 <= d; r += 16) {
        const __m256 k0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (k + r)));
        const __m256 k1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (k + r + 8)));
        a0 = _mm256_fmadd_ps(_mm256_loadu_ps(q + r), k0, a0);
        b0 = _mm256_fmadd_ps(_mm256_loadu_ps(q + r + 8), k1, b0);
        a1 = _mm256_fmadd_ps(_mm256_loadu_ps(q + q_stride + r), k0, a1);
        b1 = _mm256_fmadd_ps(_mm256_loadu_ps(q + q_stride + r + 8), k1, b1);
        a2 = _mm256_fmadd_ps(_mm256_loadu_ps(q + 2 * q_stride + r), k0, a2);
        b2 = _mm256_fmadd_ps(_mm256_loadu_ps(q + 2 * q_stride + r + 8), k1, b2);
        a3 = _mm256_fmadd_ps(_mm256_loadu_ps(q + 3 * q_stride + r), k0, a3);
        b3 = _mm256_fmadd_ps(_mm256_loadu_ps(q + 3 * q_stride + r + 8), k1, b3);
    }
    out[0] = hsum8(_mm256_add_ps(a0, b0));
    out[1] = hsum8(_mm256_add_ps(a1, b1));
    out[2] = hsum8(_mm256_add_ps(a2, b2));
    out[3] = hsum8(_mm256_add_ps(a3, b3));
    const float *lut = h2f_table();
    for (; r < d; r++)
        for (int i = 0; i < 4; i++) out[i] += q[i * q_stride + r] * lut[k[r]];
}
static inline void axpy4_f16(float *o, const float p[4], const uint16_t *const v[4], int d) {
    const __m256 p0 = _mm256_set1_ps(p[0]), p1 = _mm256_set1_ps(p[1]), p2 = _mm256_set1_ps(p[2]), p3 = _mm256_set1_ps(p[3]);
    int c = 0;
    for (; c + 8 <= d; c += 8) {
        __m256 a = _mm256_loadu_ps(o + c);
        a = _mm256_fmadd_ps(p0, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (v[0] + c))), a);
        a = _mm256_fmadd_ps(p1, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (v[1] + c))), a);
        a = _mm256_fmadd_ps(p2, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (v[2] + c))), a);
        a = _mm256_fmadd_ps(p3, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *) (v[3] + c))), a);
        _mm256_storeu_ps(o + c, a);
    }
    const float *lut = h2f_table();
    for (; c < d; c++)
        for (int i = 0; i < 4; i++) o[c] += p[i] * lut[v[i][c]];
}
#else
static inline void dot4_f32_f16(const float *q, int64_t q_stride, const uint16_t *k, int d, float out[4]) {
    for (int i = 0; i < 4; i++) out[i] = dot_f32_f16(q + i * q_stride, k, d);
}
static inline void axpy4_f16(float *o, const float p[4], const uint16_t *const v[4], int d) {
    for (int i = 0; i < 4; i++) axpy_f16(o, p[i], v[i], d);
}
#endif

static void attend_row(const float *q, int d_qk, int d_v, const uint16_t *K, int64_t k_stride, const uint16_t *V,
                       int64_t v_stride, const int32_t *rows, int64_t row0, int64_t n, float scale, int normalise,
                       float *o, float *m_out, float *l_out, float *score_buf) {
    float m = -INFINITY;
    for (int64_t s = 0; s < n; s++) {
        const int64_t row = rows ? (int64_t) rows[s] : row0 + s;
        const float sc = dot_f32_f16(q, K + row * k_stride, d_qk) * scale;
        score_buf[s] = sc;
        if (sc > m) m = sc;
    }
    for (int c = 0; c < d_v; c++) o[c] = 0.f;
    float l = 0.f;
    for (int64_t s = 0; s < n; s++) {
        const int64_t row = rows ? (int64_t) rows[s] : row0 + s;
        const float p = expf(score_buf[s] - m);
        l += p;
        axpy_f16(o, p, V + row * v_stride, d_v);
    }
    if (normalise) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        for (int c = 0; c < d_v; c++) o[c] *= inv;
    }
    if (m_out) *m_out = m;
    if (l_out) *l_out = l;
}

/* ------------------------------------------------------------------------------------------
 * Reference-ABI attention: gs_mla_attn (ops.cu:579-597) with an f16 cache (C_scales == NULL).
 *   q   f32 [T][H][R]     sel int32 [T][sel_stride]   cnt int32 [T]    o f32 [T][H][R]
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const float *q;
    const uint16_t *C;
    const int32_t *sel;
    int sel_stride;
    const int32_t *cnt;
    float scale;
    float *o;
    int T, H, R;
} ref_ctx_t;

static void ref_item(void *vctx, int64_t item) {
    ref_ctx_t *c = (ref_ctx_t *) vctx;
    const int t = (int) (item / c->H), h = (int) (item % c->H);
    const int64_t n = c->cnt[t];
    float *buf = (float *) malloc(sizeof(float) * (size_t) (n > 0 ? n : 1));
    attend_row(c->q + ((int64_t) t * c->H + h) * c->R, c->R, c->R, c->C, c->R, c->C, c->R,
               c->sel + (int64_t) t * c->sel_stride, 0, n, c->scale, 1, c->o + ((int64_t) t * c->H + h) * c->R, NULL,
               NULL, buf);
    free(buf);
}

int oracle_mla_attn_ref(const float *q, const uint16_t *C, const int32_t *sel, int sel_stride, const int32_t *cnt,
                        float scale, float *o, int T, int H, int R, int threads) {
    ref_ctx_t c = {q, C, sel, sel_stride, cnt, scale, o, T, H, R};
    return run_pool(ref_item, &c, (int64_t) T * H, threads);
}

/* ------------------------------------------------------------------------------------------
 * Split partials and their combine, as the reference forms them:
 *   key range of split s: per = ceil(n / splits), [s*per, min(n, s*per + per))  (ops.cu:447-449)
 *   partial = (unnormalised acc[R], m, l)                                       (ops.cu:539-549)
 *   combine: M = max m_s; L = sum l_s e^{m_s-M} (skipping m_s = -inf);
 *            o = sum acc_s e^{m_s-M} / L, zeros when L == 0                      (ops.cu:558-573)
 * The oracle keeps one record per (t, h, split): part[((t*H+h)*splits+s)*(R_v+2)] = acc.., m, l.
 * ------------------------------------------------------------------------------------------ */
void oracle_combine(const float *part, int64_t n_rows, int n_parts, int d_v, float *o) {
    const int64_t rec = d_v + 2;
    float *w = (float *) malloc(sizeof(float) * (size_t) (n_parts > 0 ? n_parts : 1));
    for (int64_t r = 0; r < n_rows; r++) {
        const float *base = part + r * n_parts * rec;
        float M = -INFINITY;
        for (int s = 0; s < n_parts; s++) M = fmaxf(M, base[s * rec + d_v]);
        float L = 0.f;
        for (int s = 0; s < n_parts; s++) { /* the weight of a part, once per part; an empty part (m = -inf) has none */
            const float m = base[s * rec + d_v];
            w[s] = m != -INFINITY ? expf(m - M) : 0.f;
            if (m != -INFINITY) L += base[s * rec + d_v + 1] * w[s];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        float *out = o + r * d_v;
        for (int c = 0; c < d_v; c++) out[c] = 0.f;
        for (int s = 0; s < n_parts; s++) {
            if (base[s * rec + d_v] == -INFINITY) continue;
            const float ws = w[s];
            const float *a = base + s * rec;
            for (int c = 0; c < d_v; c++) out[c] += a[c] * ws;
        }
        for (int c = 0; c < d_v; c++) out[c] *= inv;
    }
    free(w);
}

/* ------------------------------------------------------------------------------------------
 * Absorbed-MLA decode over the latent cache (extension of gs_mla_attn to the benchmark shapes):
 *   q      f16 [n_seq][T][H][d_qk]
 *   cache  f16 rows of d_qk; dense: sequence b owns rows seq_base[b] .. ; paged: row i of sequence
 *          b is row (i % page_rows) of page page_table[b][i / page_rows]
 *   seq_lens[b] = rows attended by the LAST of the T query tokens; token t attends
 *          seq_lens[b] - (T-1-t) rows, i.e. the T tokens are causal among themselves.  This is the
 *          dense list of ops.cu:728-731 (query t sees 0..=pos0+t) with the new rows already
 *          appended (crates/engine/src/forward.rs:849-860 precede :902).
 *   V = first d_v columns of the same row; o f32 [n_seq][T][H][d_v].
 * With parts != NULL the rows [part_lo, part_hi) of every sequence are attended only and the
 * unnormalised (acc, m, l) record is written instead of o (the per-GPU shard partial).
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const uint16_t *q;
    const uint16_t *cache;
    const int32_t *seq_lens, *seq_base, *page_table;
    int page_table_stride, page_rows;
    float scale;
    float *o;
    float *parts;
    int64_t part_lo, part_hi;
    int n_seq, T, H, d_qk, d_v;
} dec_ctx_t;

static void dec_item(void *vctx, int64_t item) {
    dec_ctx_t *c = (dec_ctx_t *) vctx;
    const int h = (int) (item % c->H);
    const int t = (int) ((item / c->H) % c->T);
    const int b = (int) (item / ((int64_t) c->H * c->T));
    int64_t n = (int64_t) c->seq_lens[b] - (c->T - 1 - t);
    if (n < 0) n = 0;
    int64_t lo = 0, hi = n;
    if (c->parts) {
        lo = c->part_lo < n ? c->part_lo : n;
        hi = c->part_hi < n ? c->part_hi : n;
    }
    const int64_t cnt = hi - lo;
    float *qf = (float *) malloc(sizeof(float) * (size_t) c->d_qk);
    oracle_f16_to_f32_array(c->q + (((int64_t) b * c->T + t) * c->H + h) * c->d_qk, qf, c->d_qk);
    float *buf = (float *) malloc(sizeof(float) * (size_t) (cnt > 0 ? cnt : 1));
    int32_t *rows = NULL;
    int64_t row0 = 0;
    if (c->page_table) {
        rows = (int32_t *) malloc(sizeof(int32_t) * (size_t) (cnt > 0 ? cnt : 1));
        const int32_t *pt = c->page_table + (int64_t) b * c->page_table_stride;
        for (int64_t i = 0; i < cnt; i++) {
            const int64_t pos = lo + i;
            rows[i] = pt[pos / c->page_rows] * c->page_rows + (int32_t) (pos % c->page_rows);
        }
    } else {
        row0 = (c->seq_base ? (int64_t) c->seq_base[b] : 0) + lo;
    }
    const int64_t orow = ((int64_t) b * c->T + t) * c->H + h;
    if (c->parts) {
        float *rec = c->parts + orow * (c->d_v + 2);
        attend_row(qf, c->d_qk, c->d_v, c->cache, c->d_qk, c->cache, c->d_qk, rows, row0, cnt, c->scale, 0, rec,
                   rec + c->d_v, rec + c->d_v + 1, buf);
    } else {
        attend_row(qf, c->d_qk, c->d_v, c->cache, c->d_qk, c->cache, c->d_qk, rows, row0, cnt, c->scale, 1,
                   c->o + orow * c->d_v, NULL, NULL, buf);
    }
    free(rows);
    free(buf);
    free(qf);
}

int oracle_mla_decode(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens, const int32_t *seq_base,
                      const int32_t *page_table, int page_table_stride, int page_rows, float scale, float *o,
                      int n_seq, int T, int H, int d_qk, int d_v, int threads) {
    dec_ctx_t c = {q, cache, seq_lens, seq_base, page_table, page_table_stride, page_rows, scale, o, NULL, 0, 0,
                   n_seq, T, H, d_qk, d_v};
    return run_pool(dec_item, &c, (int64_t) n_seq * T * H, threads);
}

int oracle_mla_decode_partial(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens,
                              const int32_t *seq_base, const int32_t *page_table, int page_table_stride,
                              int page_rows, float scale, float *parts, int64_t part_lo, int64_t part_hi, int n_seq,
                              int T, int H, int d_qk, int d_v, int threads) {
    dec_ctx_t c = {q, cache, seq_lens, seq_base, page_table, page_table_stride, page_rows, scale, NULL, parts,
                   part_lo, part_hi, n_seq, T, H, d_qk, d_v};
    return run_pool(dec_item, &c, (int64_t) n_seq * T * H, threads);
}

/* The same decode with the attended rows of every (sequence, token, head) cut into `key_splits` ranges by the
 * reference's split rule (per = ceil(n / splits), ops.cu:447-449) and merged by oracle_combine (ops.cu:558-573).
 * One work item is (sequence, key range): it walks the range in blocks of 32 keys and passes all T*H query rows over each
 * block with an online softmax (running maximum and rescale, ops.cu:503-517), so every cache row is read from memory
 * once and serves every head from the core's cache - the order a CPU wants, and the form that keeps every host core
 * busy when n_seq*T*H is small.  `scratch` holds n_seq*T*H*key_splits*(d_v+2) floats. */
typedef struct {
    dec_ctx_t d;
    int key_splits;
    float *scratch;
} dec_split_ctx_t;

static void dec_split_item(void *vctx, int64_t item) {
    dec_split_ctx_t *sc = (dec_split_ctx_t *) vctx;
    const dec_ctx_t *c = &sc->d;
    const int ks = sc->key_splits;
    const int b = (int) (item / ks);
    const int split = (int) (item % ks);
    const int64_t len = c->seq_lens[b] > 0 ? c->seq_lens[b] : 0;
    const int n_q = c->T * c->H;
    enum { KB = 32 }; /* keys per block: a block's rows stay in the core's cache while all query rows pass over them */
    float *qf = (float *) malloc(sizeof(float) * (size_t) n_q * c->d_qk);
    float *acc = (float *) calloc((size_t) n_q * c->d_v, sizeof(float));
    float *m = (float *) malloc(sizeof(float) * (size_t) n_q);
    float *l = (float *) calloc((size_t) n_q, sizeof(float));
    float *sc_blk = (float *) malloc(sizeof(float) * (size_t) n_q * KB);
    int64_t *lo_q = (int64_t *) malloc(sizeof(int64_t) * (size_t) c->T), *hi_q = (int64_t *) malloc(sizeof(int64_t) * (size_t) c->T);
    oracle_f16_to_f32_array(c->q + (int64_t) b * n_q * c->d_qk, qf, (int64_t) n_q * c->d_qk);
    int64_t lo_all = len, hi_all = 0;
    for (int t = 0; t < c->T; t++) { /* the key range of this split for every query token (ops.cu:447-449) */
        int64_t n = len - (c->T - 1 - t);
        if (n < 0) n = 0;
        const int64_t per = (n + ks - 1) / ks;
        lo_q[t] = split * per < n ? split * per : n;
        hi_q[t] = lo_q[t] + per < n ? lo_q[t] + per : n;
        if (lo_q[t] < lo_all) lo_all = lo_q[t];
        if (hi_q[t] > hi_all) hi_all = hi_q[t];
    }
    for (int i = 0; i < n_q; i++) m[i] = -INFINITY;
    const int32_t *pt = c->page_table ? c->page_table + (int64_t) b * c->page_table_stride : NULL;
    const int64_t base = c->page_table ? 0 : (c->seq_base ? (int64_t) c->seq_base[b] : 0);
    for (int64_t k0 = lo_all; k0 < hi_all; k0 += KB) {
        const int64_t k1 = k0 + KB < hi_all ? k0 + KB : hi_all;
        const uint16_t *rows[KB];
        for (int64_t k = k0; k < k1; k++) {
            const int64_t row = pt ? (int64_t) pt[k / c->page_rows] * c->page_rows + k % c->page_rows : base + k;
            rows[k - k0] = c->cache + row * c->d_qk;
        }
        /* scores of the block: four query rows at a time against each key row; a row's keys outside its own causal
         * range are computed and then ignored */
        for (int q0 = 0; q0 < n_q; q0 += 4) {
            if (q0 + 4 <= n_q) {
                for (int64_t k = k0; k < k1; k++) {
                    float s4[4];
                    dot4_f32_f16(qf + (int64_t) q0 * c->d_qk, c->d_qk, rows[k - k0], c->d_qk, s4);
                    for (int i = 0; i < 4; i++) sc_blk[(q0 + i) * KB + (k - k0)] = s4[i] * c->scale;
                }
            } else {
                for (int qi = q0; qi < n_q; qi++)
                    for (int64_t k = k0; k < k1; k++)
                        sc_blk[qi * KB + (k - k0)] = dot_f32_f16(qf + (int64_t) qi * c->d_qk, rows[k - k0], c->d_qk) * c->scale;
            }
        }
        for (int qi = 0; qi < n_q; qi++) {
            const int t = qi / c->H;
            const int64_t a0 = k0 > lo_q[t] ? k0 : lo_q[t], a1 = k1 < hi_q[t] ? k1 : hi_q[t];
            if (a1 <= a0) continue;
            const float *sc_k = sc_blk + qi * KB;
            float mx = m[qi];
            for (int64_t k = a0; k < a1; k++)
                if (sc_k[k - k0] > mx) mx = sc_k[k - k0];
            float *o = acc + (int64_t) qi * c->d_v;
            if (mx > m[qi]) { /* running maximum moved: rescale what was summed so far (ops.cu:503-517) */
                const float f = m[qi] == -INFINITY ? 0.f : expf(m[qi] - mx);
                for (int d = 0; d < c->d_v; d++) o[d] *= f;
                l[qi] *= f;
                m[qi] = mx;
            }
            int64_t k = a0;
            for (; k + 4 <= a1; k += 4) {
                float p4[4];
                for (int i = 0; i < 4; i++) {
                    p4[i] = expf(sc_k[k + i - k0] - mx);
                    l[qi] += p4[i];
                }
                axpy4_f16(o, p4, rows + (k - k0), c->d_v);
            }
            for (; k < a1; k++) {
                const float p = expf(sc_k[k - k0] - mx);
                l[qi] += p;
                axpy_f16(o, p, rows[k - k0], c->d_v);
            }
        }
    }
    for (int qi = 0; qi < n_q; qi++) {
        const int64_t row_item = (int64_t) b * n_q + qi;
        float *rec = sc->scratch + (row_item * ks + split) * (c->d_v + 2);
        memcpy(rec, acc + (int64_t) qi * c->d_v, sizeof(float) * (size_t) c->d_v);
        rec[c->d_v] = m[qi];
        rec[c->d_v + 1] = l[qi];
    }
    free(hi_q);
    free(lo_q);
    free(sc_blk);
    free(l);
    free(m);
    free(acc);
    free(qf);
}

int oracle_mla_decode_split(const uint16_t *q, const uint16_t *cache, const int32_t *seq_lens, const int32_t *seq_base,
                            const int32_t *page_table, int page_table_stride, int page_rows, float scale, float *o,
                            int n_seq, int T, int H, int d_qk, int d_v, int key_splits, float *scratch, int threads) {
    if (key_splits < 1) key_splits = 1;
    dec_split_ctx_t c = {{q, cache, seq_lens, seq_base, page_table, page_table_stride, page_rows, scale, NULL, NULL, 0,
                          0, n_seq, T, H, d_qk, d_v},
                         key_splits, scratch};
    const int64_t n_rows = (int64_t) n_seq * T * H;
    const int used = run_pool(dec_split_item, &c, (int64_t) n_seq * key_splits, threads);
    oracle_combine(scratch, n_rows, key_splits, d_v, o);
    return used;
}

/* ------------------------------------------------------------------------------------------
 * Causal prefill attention, non-absorbed form.  The reference runs prefill through the same
 * absorbed kernel with T <= 256 queries and splits = 1 (forward.rs:61, :898-908); with
 * q.(k_b c) = (k_b^T q).c that equals per-head causal attention with head width 256
 * (forward.rs:900, :907), which is what is restated here:
 *   Q f16 [S][H][d], K f16 [p0+S][H][d], V f16 [p0+S][H][dv]; query i attends keys 0 .. p0+i.
 * rows_subset (may be NULL) restricts the computed query rows (for spot checks at full size).
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const uint16_t *Q, *K, *V;
    float scale;
    float *o;
    int S, H, d, dv, p0;
    const int32_t *rows_subset;
    int n_subset;
} pf_ctx_t;

static void pf_item(void *vctx, int64_t item) {
    pf_ctx_t *c = (pf_ctx_t *) vctx;
    const int h = (int) (item % c->H);
    const int64_t idx = item / c->H;
    const int i = c->rows_subset ? c->rows_subset[idx] : (int) idx;
    const int64_t n = (int64_t) c->p0 + i + 1;
    float *qf = (float *) malloc(sizeof(float) * (size_t) c->d);
    oracle_f16_to_f32_array(c->Q + ((int64_t) i * c->H + h) * c->d, qf, c->d);
    float *buf = (float *) malloc(sizeof(float) * (size_t) n);
    attend_row(qf, c->d, c->dv, c->K + (int64_t) h * c->d, (int64_t) c->H * c->d, c->V + (int64_t) h * c->dv,
               (int64_t) c->H * c->dv, NULL, 0, n, c->scale, 1, c->o + (idx * c->H + h) * c->dv, NULL, NULL, buf);
    free(buf);
    free(qf);
}

int oracle_prefill(const uint16_t *Q, const uint16_t *K, const uint16_t *V, float scale, float *o, int S, int H, int d,
                   int dv, int p0, const int32_t *rows_subset, int n_subset, int threads) {
    pf_ctx_t c = {Q, K, V, scale, o, S, H, d, dv, p0, rows_subset, n_subset};
    const int64_t n_rows = rows_subset ? n_subset : S;
    return run_pool(pf_item, &c, n_rows * H, threads);
}

/* ------------------------------------------------------------------------------------------
 * RoPE.  The reference model has no rotary embedding; the benchmark configs add one: base 10000 on
 * the last `d_rope` columns of a row at its absolute position.  Convention fixed here (and matched
 * by the CUDA kernels): adjacent pairs (2i, 2i+1) rotate by angle pos * base^(-2i/d_rope);
 * the inverse frequency is computed in double and rounded to f32, the angle is an f32 product,
 * cos/sin are evaluated in f32.
 * ------------------------------------------------------------------------------------------ */
void oracle_rope_inv_freq(float *inv_freq, int d_rope, double base) {
    for (int i = 0; i < d_rope / 2; i++) inv_freq[i] = (float) pow(base, -2.0 * i / (double) d_rope);
}

static inline void rope_pair(float *x0, float *x1, float pos, float inv_freq) {
    const float ang = pos * inv_freq;
    const float c = cosf(ang), s = sinf(ang);
    const float a = *x0, b = *x1;
    *x0 = a * c - b * s;
    *x1 = a * s + b * c;
}

/* Fused RoPE + KV-append: the reference appends half_rn(kv) to cache rows p0.. (gemm.cu:155-163,
 * forward.rs:857-860); here the last d_rope columns are rotated at position pos0+t first.
 * x f32 [T][d_row] -> y f16 [T][d_row]. */
void oracle_rope_append(const float *x, uint16_t *y, int T, int d_row, int d_rope, int64_t pos0, double base) {
    float inv[256];
    oracle_rope_inv_freq(inv, d_rope, base);
    for (int t = 0; t < T; t++) {
        const float *xr = x + (int64_t) t * d_row;
        uint16_t *yr = y + (int64_t) t * d_row;
        const int d0 = d_row - d_rope;
        for (int c = 0; c < d0; c++) yr[c] = oracle_f32_to_f16(xr[c]);
        for (int i = 0; i < d_rope / 2; i++) {
            float a = xr[d0 + 2 * i], b = xr[d0 + 2 * i + 1];
            rope_pair(&a, &b, (float) (pos0 + t), inv[i]);
            yr[d0 + 2 * i] = oracle_f32_to_f16(a);
            yr[d0 + 2 * i + 1] = oracle_f32_to_f16(b);
        }
    }
}

/* Latent RMSNorm (crates/cuda/kernels/ops.cu:43-50, called at forward.rs:850) followed by the fused RoPE + append:
 * the first d_row - d_rope columns become x * rsqrt(mean(x^2) + eps) * w (w may be NULL), then the row goes through
 * oracle_rope_append.  The sum of squares is accumulated in double, so this is the reference for any summation
 * order. */
void oracle_norm_rope_append(const float *x, const float *w, float eps, uint16_t *y, int T, int d_row, int d_rope,
                             int64_t pos0, double base) {
    const int d0 = d_row - d_rope;
    float *tmp = (float *) malloc((size_t) d_row * sizeof(float));
    for (int t = 0; t < T; t++) {
        const float *xr = x + (int64_t) t * d_row;
        double ss = 0.0;
        for (int c = 0; c < d0; c++) ss += (double) xr[c] * xr[c];
        const float r = (float) (1.0 / sqrt(ss / d0 + (double) eps));
        for (int c = 0; c < d0; c++) tmp[c] = xr[c] * r * (w ? w[c] : 1.f);
        for (int c = d0; c < d_row; c++) tmp[c] = xr[c];
        oracle_rope_append(tmp, y + (int64_t) t * d_row, 1, d_row, d_rope, pos0 + t, base);
    }
    free(tmp);
}

/* RoPE in place on f16 rows [S][H][d] (prefill Q and K): last d_rope columns of every head at
 * position pos0 + s; computed in f32 and rounded back to f16. */
void oracle_rope_f16(uint16_t *x, int S, int H, int d, int d_rope, int64_t pos0, double base) {
    float inv[256];
    oracle_rope_inv_freq(inv, d_rope, base);
    const int d0 = d - d_rope;
    for (int s = 0; s < S; s++)
        for (int h = 0; h < H; h++) {
            uint16_t *r = x + ((int64_t) s * H + h) * d + d0;
            for (int i = 0; i < d_rope / 2; i++) {
                float a = oracle_f16_to_f32(r[2 * i]), b = oracle_f16_to_f32(r[2 * i + 1]);
                rope_pair(&a, &b, (float) (pos0 + s), inv[i]);
                r[2 * i] = oracle_f32_to_f16(a);
                r[2 * i + 1] = oracle_f32_to_f16(b);
            }
        }
}

/* ------------------------------------------------------------------------------------------
 * Q8 latent cache (the engine's --kv-cache q8).  Quantiser: per block of 32 values d = amax / 127,
 * q = round_to_nearest_even(x / d) stored as int8, d stored as f16 (crates/cuda/kernels/ops.cu:599-610).
 * Reader: the attention kernel rebuilds an f16 tile as half_rn(float(d) * q) (ops.cu:461-477) and
 * then proceeds as with an f16 cache, so the Q8 oracle is dequantise-to-f16 + the f16 oracle.
 * ------------------------------------------------------------------------------------------ */
void oracle_quant_q8_rows(const float *x, int8_t *q, uint16_t *d, int64_t n_blocks) {
    for (int64_t b = 0; b < n_blocks; b++) {
        float amax = 0.f;
        for (int i = 0; i < 32; i++) {
            const float a = fabsf(x[b * 32 + i]);
            if (a > amax) amax = a;
        }
        const float dd = amax / 127.f;
        const float inv = dd > 0.f ? 1.f / dd : 0.f;
        for (int i = 0; i < 32; i++) q[b * 32 + i] = (int8_t) lrintf(x[b * 32 + i] * inv);
        d[b] = oracle_f32_to_f16(dd);
    }
}

void oracle_dequant_q8(const int8_t *q, const uint16_t *d, uint16_t *out, int64_t n_blocks) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const float dd = oracle_f16_to_f32(d[b]);
        for (int i = 0; i < 32; i++) out[b * 32 + i] = oracle_f32_to_f16(dd * (float) q[b * 32 + i]);
    }
}

/* ------------------------------------------------------------------------------------------
 * DSA k-pool indexer (crates/cuda/kernels/ops.cu:619-791): the kernels that produce the position
 * lists (sel, cnt) the attention call consumes beyond top_k positions of context
 * (crates/engine/src/forward.rs:864-895).
 *
 * oracle_idx_pool (ops.cu:622-672): raw indexer keys kc / gates gc of the chunk's T positions
 * p0..p0+T-1, [T][Dk] f32; older positions of an unfinished pool live in the rings rk / rg
 * ([kpool][Dk], row pos % kpool).  For every pool j of kpool positions that completes inside
 * [p0, p0+T):  P[j][c] = sum_m softmax_m(gate[m][c] + ape[m][c]) * key[m][c]  (softmax over the pool's
 * kpool positions, per column c); afterwards the rows of the trailing incomplete pool are copied
 * into the rings.
 * ------------------------------------------------------------------------------------------ */
static inline const float *idx_row_cpu(const float *chunk, const float *ring, int64_t pos, int p0, int Dk, int kpool) {
    return pos >= p0 ? chunk + (pos - p0) * Dk : ring + (pos % kpool) * Dk; /* ops.cu:622-625 */
}

void oracle_idx_pool(const float *kc, const float *gc, float *rk, float *rg, const float *ape, float *P, int p0, int T,
                     int Dk, int kpool) {
    const int end = p0 + T;
    const int jf = p0 / kpool, jl = end / kpool; /* ops.cu:656-657 */
    for (int64_t j = jf; j < jl; j++) {
        for (int c = 0; c < Dk; c++) {
            float mx = -INFINITY;
            for (int m = 0; m < kpool; m++) {
                const int64_t pos = j * kpool + m;
                mx = fmaxf(mx, idx_row_cpu(gc, rg, pos, p0, Dk, kpool)[c] + ape[m * Dk + c]);
            }
            float sum = 0.f, acc = 0.f;
            for (int m = 0; m < kpool; m++) {
                const int64_t pos = j * kpool + m;
                const float e = expf(idx_row_cpu(gc, rg, pos, p0, Dk, kpool)[c] + ape[m * Dk + c] - mx);
                sum += e;
                acc += e * idx_row_cpu(kc, rk, pos, p0, Dk, kpool)[c];
            }
            P[j * Dk + c] = acc / sum;
        }
    }
    const int first = p0 > jl * kpool ? p0 : jl * kpool; /* ops.cu:662-666 */
    for (int64_t pos = first; pos < end; pos++) {
        for (int c = 0; c < Dk; c++) {
            rk[(pos % kpool) * Dk + c] = kc[(pos - p0) * Dk + c];
            rg[(pos % kpool) * Dk + c] = gc[(pos - p0) * Dk + c];
        }
    }
}

/* oracle_idx_score (ops.cu:675-712): score[t][p] = sum_h w[t][h] * relu(scale * q[t][h] . P[p]) for the
 * p < (pos0 + t + 1) / kpool pools complete at query position pos0 + t; other entries are left alone. */
void oracle_idx_score(const float *q, const float *w, const float *P, float *score, int64_t score_stride, int pos0, int T,
                      int kpool, int Hq, int Dk, float scale) {
    for (int t = 0; t < T; t++) {
        const int n_pool = (pos0 + t + 1) / kpool;
        for (int p = 0; p < n_pool; p++) {
            float total = 0.f;
            for (int h = 0; h < Hq; h++) {
                const float *qh = q + ((int64_t) t * Hq + h) * Dk;
                float d = 0.f;
                for (int c = 0; c < Dk; c++) d += qh[c] * P[(int64_t) p * Dk + c];
                total += w[(int64_t) t * Hq + h] * fmaxf(d * scale, 0.f);
            }
            score[(int64_t) t * score_stride + p] = total;
        }
    }
}

/* oracle_idx_select (ops.cu:714-791): the attended position list of query t (position pos = pos0 + t).
 *   n_pool = (pos+1)/kpool <= top_k : every position 0..pos, cnt = pos + 1            (ops.cu:728-731)
 *   else: the kpool positions of each of the top_k highest-scoring pools, then the positions of the
 *         incomplete tail pool n_pool*kpool..pos; cnt = top_k*kpool + (pos + 1 - n_pool*kpool).
 * Top-k is exact on the order-preserving uint32 image of the scores (ops.cu:718-721), i.e. all pools
 * above the k-th largest value and as many of the pools equal to it as are still needed (ops.cu:770-777).
 * The reference fills the slots in the order its threads reach an atomic counter, so neither the order of
 * the pools inside the list nor which of several equal-valued pools are taken is fixed there; this
 * restatement fixes both: pools in ascending index, ties to the lowest indices. */
static inline uint32_t f2ord_cpu(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

static int cmp_u32_desc(const void *a, const void *b) {
    const uint32_t x = *(const uint32_t *) a, y = *(const uint32_t *) b;
    return x < y ? 1 : x > y ? -1 : 0;
}

void oracle_idx_select(const float *score, int64_t score_stride, int pos0, int T, int kpool, int top_k, int32_t *sel,
                       int sel_stride, int32_t *cnt) {
    for (int t = 0; t < T; t++) {
        const int pos = pos0 + t;
        const int n_pool = (pos + 1) / kpool;
        int32_t *out = sel + (int64_t) t * sel_stride;
        if (n_pool <= top_k) {
            for (int i = 0; i <= pos && i < sel_stride; i++) out[i] = i;
            cnt[t] = pos + 1;
            continue;
        }
        const float *sc = score + (int64_t) t * score_stride;
        uint32_t *ord = (uint32_t *) malloc(sizeof(uint32_t) * (size_t) n_pool);
        for (int p = 0; p < n_pool; p++) ord[p] = f2ord_cpu(sc[p]);
        uint32_t *sorted = (uint32_t *) malloc(sizeof(uint32_t) * (size_t) n_pool);
        memcpy(sorted, ord, sizeof(uint32_t) * (size_t) n_pool);
        qsort(sorted, (size_t) n_pool, sizeof(uint32_t), cmp_u32_desc);
        const uint32_t U = top_k > 0 ? sorted[top_k - 1] : 0xffffffffu; /* the k-th largest value; nothing is taken when top_k is 0 */
        int above = 0;
        for (int p = 0; p < n_pool; p++) above += ord[p] > U;
        int need_eq = top_k - above, slot = 0;
        for (int p = 0; p < n_pool; p++) {
            int take = ord[p] > U;
            if (ord[p] == U && need_eq > 0) {
                take = 1;
                need_eq--;
            }
            if (take && slot < top_k) { /* never more than top_k pools, whatever the scores hold */
                for (int m = 0; m < kpool; m++)
                    if ((int64_t) slot * kpool + m < sel_stride) out[slot * kpool + m] = p * kpool + m;
                slot++;
            }
        }
        const int base = top_k * kpool, tail0 = n_pool * kpool;
        for (int i = 0; tail0 + i <= pos; i++)
            if (base + i < sel_stride) out[base + i] = tail0 + i;
        cnt[t] = base + (pos + 1 - tail0);
        free(sorted);
        free(ord);
    }
}

/* ------------------------------------------------------------------------------------------
 * The attention call with its two per-head products (crates/engine/src/forward.rs:900-907):
 *   qabs[t][h][r] = sum_k k_b[h][r][k] * q[t][h][k]        mm_heads(&w.k_b, ...), forward.rs:900, :716-733
 *   olat[t][h]    = attention of qabs over latent rows 0 .. n_t-1, n_t = seq_len - (T-1-t)   (forward.rs:902-906;
 *                   dense list of ops.cu:728-731, new rows already appended)
 *   ov[t][h][j]   = sum_r v_b[h][j][r] * olat[t][h][r]      mm_heads(&w.v_b, ...), forward.rs:907
 * everything in fp32 as in the reference (its weights are quantised formats read into fp32 products; here they are
 * f16 values widened exactly).  q f32 [T][H][d_q]; k_b f16 [H][R][d_q]; v_b f16 [H][d_out][R]; cache f16 [rows][R].
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const float *q;
    const uint16_t *k_b, *v_b, *cache;
    int seq_len;
    float scale;
    float *ov;
    int T, H, d_q, R, d_out;
} fused_ctx_t;

static void fused_item(void *vctx, int64_t item) {
    fused_ctx_t *c = (fused_ctx_t *) vctx;
    const int t = (int) (item / c->H), h = (int) (item % c->H);
    const float *lut = h2f_table();
    float *qabs = (float *) malloc(sizeof(float) * (size_t) c->R);
    float *olat = (float *) malloc(sizeof(float) * (size_t) c->R);
    const float *qh = c->q + ((int64_t) t * c->H + h) * c->d_q;
    for (int r = 0; r < c->R; r++) {
        const uint16_t *w = c->k_b + ((int64_t) h * c->R + r) * c->d_q;
        float a = 0.f;
        for (int k = 0; k < c->d_q; k++) a += lut[w[k]] * qh[k];
        qabs[r] = a;
    }
    int64_t n = (int64_t) c->seq_len - (c->T - 1 - t);
    if (n < 0) n = 0;
    float *buf = (float *) malloc(sizeof(float) * (size_t) (n > 0 ? n : 1));
    attend_row(qabs, c->R, c->R, c->cache, c->R, c->cache, c->R, NULL, 0, n, c->scale, 1, olat, NULL, NULL, buf);
    float *out = c->ov + ((int64_t) t * c->H + h) * c->d_out;
    for (int j = 0; j < c->d_out; j++) {
        const uint16_t *w = c->v_b + ((int64_t) h * c->d_out + j) * c->R;
        float a = 0.f;
        for (int r = 0; r < c->R; r++) a += lut[w[r]] * olat[r];
        out[j] = a;
    }
    free(buf);
    free(olat);
    free(qabs);
}

int oracle_mla_fused(const float *q, const uint16_t *k_b, const uint16_t *v_b, const uint16_t *cache, int seq_len, float scale,
                     float *ov, int T, int H, int d_q, int R, int d_out, int threads) {
    fused_ctx_t c = {q, k_b, v_b, cache, seq_len, scale, ov, T, H, d_q, R, d_out};
    return run_pool(fused_item, &c, (int64_t) T * H, threads);
}
