/*
 * glmssd_attn.h - C ABI of the B200 (sm_100a) attention library for the GLM-SSD engine.
 *
 * Conventions (those of the reference's kernel crate, crates/cuda/kernels/common.cuh:6-14):
 *   - every function is extern "C", returns a cudaError_t as int (0 = success), never throws;
 *   - bad arguments return cudaErrorInvalidValue (1), like crates/cuda/kernels/ops.cu:581;
 *   - calls only enqueue work on the caller's stream (`void *stream` is a cudaStream_t) and never
 *     synchronise; results are valid in stream order;
 *   - the caller owns all device memory, including workspaces; the library allocates nothing and
 *     keeps no state between calls (safe across cudaDeviceReset, cf. ops.cu:583-587) - except where an
 *     entry point says otherwise.  Those are: gs_peer_alloc / gs_peer_open (allocate or map an exchange
 *     buffer), gs_mla_layer_graph_create (allocates a handle with a recorded graph), and
 *     gs_mla_decode_static (keeps the device address of its built-in scratch array per device).  After a
 *     cudaDeviceReset (the engine's idle unload, runtime.cu:51-53) a layer-graph handle and every peer
 *     mapping are gone with the context and must be created again, and gs_mla_decode_static must not
 *     be used in a process that resets the device.
 * All pointers are device pointers unless a comment says "host".
 */
#ifndef GLMSSD_ATTN_H
#define GLMSSD_ATTN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------
 * Reference-compatible entry points (same names, argument order and meaning).
 * ---------------------------------------------------------------------------------------------- */

/* Replaces gs_mla_attn, crates/cuda/kernels/ops.cu:579-597 (Rust declaration crates/cuda/src/lib.rs:97-100;
 * only caller crates/engine/src/forward.rs:902-906).
 *   q    f32 [T][H][R]  absorbed queries           C    f16 [ctx][R] latent cache
 *   sel  i32 [T][sel_stride] attended rows         cnt  i32 [T] rows attended by query t
 *   o    f32 [T][H][R]                             part f32 workspace, T*H*splits*(R+2) floats
 *                                                       when splits > 1 (same size as ops.cu:578)
 *   C_scales NULL: f16 cache.  Non-NULL: the Q8 cache of ops.cu:427 - C is int8 [ctx][R] and C_scales one
 *   f16 scale per 32 values, [ctx][R/32]; rows are rebuilt as half_rn(scale * q) exactly as ops.cu:461-477.
 * Returns cudaErrorInvalidValue for R != 512, H % 16 != 0, splits < 1 (as the reference). */
int gs_mla_attn(const float *q, const void *C, const void *C_scales, const int *sel, int sel_stride, const int *cnt,
                float scale, float *o, float *part, int T, int H, int R, int splits, void *stream);

/* Which kernel gs_mla_attn runs (no counterpart in the reference).  The call runs on the tcgen05 decode kernel whenever
 * that kernel takes the shape: the rows a list names are fetched straight from the cache by the kernel's producer warp
 * (f16 rows, or the int8 rows and scales of a Q8 cache, which the kernel widens to half_rn(scale * q) in shared
 * memory), the f32 queries are rounded to f16 inside the kernel (the precision
 * of the f16-query entry points; outputs stay within max-abs 2e-3 of the f32-query result), and nothing beyond the
 * reference's own arguments is needed: with splits > 1 the split records live in `part` (as many segments as fit its
 * T*H*splits*(R+2) floats), with splits == 1 every (token, head group) is attended by one CTA that stores o itself.
 * Head counts that cannot be cut into groups of 8..48 heads and misaligned q / C / C_scales run on the CUDA-core
 * kernel, which keeps the queries in f32.
 *   gs_mla_attn_set_impl(impl): 0 = automatic (default), 1 = always the CUDA-core kernel, 2 = the tcgen05 kernel or
 *     cudaErrorInvalidValue.  A process-wide setting; it changes no result beyond the rounding described above.
 *   gs_mla_attn_status(status_out, stream): synchronises `stream` and reads the sticky status word of the tcgen05
 *     path (the reference's argument list has no workspace that could carry one): 0 = ok, else a bounded wait inside
 *     the kernel gave up and cudaErrorLaunchTimeout is returned. */
int gs_mla_attn_set_impl(int impl);
int gs_mla_attn_status(int32_t *status_out /* host, may be NULL */, void *stream);

/* Replaces gs_quant_q8_rows, crates/cuda/kernels/ops.cu:599-617 (Rust declaration crates/cuda/src/lib.rs:96;
 * caller crates/engine/src/forward.rs:852-856): the KV-append of the Q8 cache.  Per block of 32 values
 * d = amax / 127 (stored as f16), q = round-to-nearest-even(x / d) as int8.  n % 32 != 0 is rejected. */
int gs_quant_q8_rows(const float *x, void *q, void *d, int64_t n, void *stream);

/* Replaces gs_f32_to_f16, crates/cuda/kernels/gemm.cu:159-163 (Rust declaration crates/cuda/src/lib.rs:123;
 * caller crates/engine/src/forward.rs:857-860): y[i] = half_rn(x[i]) for i < n.  This is the reference's
 * KV-append. */
int gs_f32_to_f16(const float *x, void *y, int64_t n, void *stream);

/* ------------------------------------------------------------------------------------------------
 * DSA k-pool indexer: produces the attended position lists (sel, cnt) gs_mla_attn consumes once the context is
 * longer than top_k positions (caller crates/engine/src/forward.rs:864-895).  Same names, argument order and
 * meaning as the reference.
 * ---------------------------------------------------------------------------------------------- */
/* Replaces gs_idx_pool, crates/cuda/kernels/ops.cu:627-672 (Rust declaration crates/cuda/src/lib.rs:101-104).
 *   kc, gc f32 [T][Dk]   raw indexer keys / gates of positions p0 .. p0+T-1
 *   rk, rg f32 [kpool][Dk] rings holding the rows of the pool that is still incomplete (row pos % kpool)
 *   ape    f32 [kpool][Dk]  P f32 [pools][Dk]
 * For every pool j of kpool positions completing inside the chunk: P[j][c] = sum_m softmax_m(gate + ape)[m][c] *
 * key[m][c]; afterwards the rows of the trailing incomplete pool go to the rings.  One launch (the reference: two). */
int gs_idx_pool(const float *kc, const float *gc, float *rk, float *rg, const float *ape, float *P, int p0, int T, int Dk,
                int kpool, void *stream);
/* Replaces gs_idx_score, ops.cu:675-712 (lib.rs:105-108): score[t][p] = sum_h w[t][h] * relu(scale * q[t][h] . P[p])
 * for the p < (pos0 + t + 1) / kpool complete pools; q f32 [T][Hq][Dk], w f32 [T][Hq], score f32 [T][score_stride].
 * Dk > 128 is rejected as in the reference. */
int gs_idx_score(const float *q, const float *w, const float *P, float *score, int64_t score_stride, int pos0, int T,
                 int kpool, int Hq, int Dk, float scale, void *stream);
/* Replaces gs_idx_select, ops.cu:714-791 (lib.rs:109-112).  Query t (position pos0 + t) with n_pool = (pos+1)/kpool
 * complete pools: n_pool <= top_k -> every position 0..pos; else the kpool positions of each of the top_k
 * highest-scoring pools followed by the positions of the incomplete tail pool.  sel i32 [T][sel_stride], cnt i32 [T].
 * The top-k is exact (radix select on the order-preserving integer image of the scores, as the reference).  Unlike
 * the reference, whose list order and choice among pools tied at the k-th largest score depend on thread timing,
 * the list here is deterministic: pools in ascending index, ties to the lowest indices. */
int gs_idx_select(const float *score, int64_t score_stride, int pos0, int T, int kpool, int top_k, int *sel,
                  int sel_stride, int *cnt, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Absorbed-MLA decode over the f16 latent cache.  Generalises gs_mla_attn (ops.cu:420-597) to
 * score width d_qk != value width d_v (V = the first d_v columns of the same cache row), f16
 * queries, any head count, several sequences per call, and dense-range or paged addressing
 * instead of a materialised position list (the dense list of ops.cu:728-731).
 * ---------------------------------------------------------------------------------------------- */
/* Cross-GPU merge for a context sharded by sequence ranges over `world` GPUs of one node (one
 * process per GPU).  Every rank attends its own rows; instead of a local output each rank's merged
 * (acc, m, l) record is stored straight into every rank's exchange buffer over NVLink (plain peer
 * stores), a per-item flag is released, and each rank merges the `world` records it received - the
 * reference's split/combine algebra (ops.cu:539-574) with "split" = GPU.  No counterpart in the
 * reference, which is single-GPU.  All ranks must make the same call with the same epoch. */
typedef struct gs_shard_exchange {
    int32_t world, rank;       /* 2..8 ranks */
    uint32_t epoch;            /* 1, 2, 3, ... : consecutive - every call's epoch is the previous call's plus one, on
                                  every rank (the record slots alternate with the epoch's parity, so a skipped
                                  value would reuse the slot a slower rank is still reading and end in a wait
                                  that runs out); or 0 on every call of every rank: the epoch is then kept in
                                  the exchange buffers themselves, which lets the call be captured in a CUDA
                                  graph and replayed.  After a call whose wait ran out (status bit 16), all
                                  ranks carry on with the next consecutive epoch */
    void *const *peer_bufs;    /* host array [world]: every rank's exchange buffer as mapped in THIS process
                                  (gs_peer_alloc / gs_peer_export / gs_peer_open); peer_bufs[rank] is local */
    int64_t buf_bytes;         /* size of each buffer, >= gs_shard_exchange_bytes() */
    int64_t wait_limit_cycles; /* bound of the wait for the other ranks' flags; 0 = about one second.  When
                                  it runs out the kernel sets bit 16 of the workspace status word and
                                  returns without writing o */
} gs_shard_exchange;

typedef struct gs_mla_decode_args {
    const void *q;             /* f16 [n_seq][T][H][d_qk] */
    const void *cache;         /* f16 [cache_rows][d_qk] row-major (the layout of forward.rs:388-404) */
    int64_t cache_rows;        /* rows in the cache allocation (for paged: n_pages * page_rows) */
    const int32_t *seq_lens;   /* [n_seq] rows attended by the LAST query token of each sequence */
    const int32_t *seq_base;   /* dense: [n_seq] first cache row of each sequence; NULL = all 0 */
    const int32_t *page_table; /* paged: [n_seq][page_table_stride] page ids; NULL = dense */
    int32_t page_table_stride;
    int32_t page_rows;         /* rows per page; 64 when paged */
    float scale;               /* softmax scale, 1/sqrt(256) in the engine (forward.rs:904) */
    int32_t tail_causal;       /* 1: query token t attends seq_lens[b] - (T-1-t) rows (the T new rows are
                                  causal among themselves, ops.cu:728-731); 0: every token attends
                                  seq_lens[b] rows (a shard that does not hold the end of the sequence) */
    float *o;                  /* f32 [n_seq][T][H][d_v]; NULL when only part_out is wanted */
    float *part_out;           /* optional: one merged (acc, m, l) record per query row instead of / besides
                                  o, for a cross-GPU combine: floats [rows*d_v acc][rows*2 (m,l)],
                                  rows = n_seq*T*H; the unnormalised form of ops.cu:539-549 */
    void *workspace;           /* gs_mla_decode_workspace_bytes() bytes, 256-byte aligned; zero it once after
                                  allocating (its first word is a sticky status the kernels only OR into) */
    int64_t workspace_bytes;
    int32_t n_seq, T, H, d_qk, d_v;
    int32_t max_seq_len;       /* host-side upper bound of seq_lens[] (sizing only; 0 = cache_rows) */
    int32_t impl;              /* 0 = automatic; 1 = force the CUDA-core gather kernel; 2 = force the
                                  tcgen05 kernel (returns cudaErrorInvalidValue if the shape is outside it) */
    void *ev_after_main;       /* optional cudaEvent_t recorded on the stream between the attention kernel and
                                  the combine kernel, so a caller can time the two apart; NULL = none */
    int32_t flags;             /* bit 0 (GS_DECODE_NO_COMBINE): run the attention kernel only and leave the split
                                  partials in the workspace (o / part_out are not written); for timing that
                                  kernel alone */
    const gs_shard_exchange *exchange; /* host; NULL = single GPU.  When set, o receives the result merged
                                  over all ranks (on every rank) and part_out is ignored */
} gs_mla_decode_args;
#define GS_DECODE_NO_COMBINE 1

/* Bytes of workspace gs_mla_decode needs on the current device for these sizes (host function). */
int64_t gs_mla_decode_workspace_bytes(int n_seq, int T, int H, int d_v);

/* Enqueue the decode.  New entry point; the call it stands in for is forward.rs:902-906. */
int gs_mla_decode(const gs_mla_decode_args *args /* host */, void *stream);

/* One decode step's attention with the two per-head products around it (no counterpart as a single call in the
 * reference, which issues them one by one: crates/engine/src/forward.rs:900 mm_heads(k_b), :902-906 gs_mla_attn,
 * :907 mm_heads(v_b); mm_heads :716-733):
 *   qabs[t][h] = k_b[h] . q[t][h];   olat[t][h] = attention of qabs over the latent rows;   ov[t][h] = v_b[h] . olat[t][h]
 * for one sequence and T <= 8 query tokens (causal among themselves, the new rows already appended).  Four kernels in a
 * programmatic-dependent-launch chain.  The weights are f16; the engine's quantised weight formats are not read here. */
typedef struct gs_mla_fused_args {
    const float *q;          /* f32 [T][H][d_q] queries before absorption (forward.rs:848) */
    const void *k_b;         /* f16 [H][d_lat][d_q], 16-byte aligned */
    const void *v_b;         /* f16 [H][d_out][d_lat], 16-byte aligned */
    const void *cache;       /* f16 [cache_rows][d_lat] latent cache */
    int64_t cache_rows;
    const int32_t *seq_len;  /* device: rows attended by the last query token */
    float scale;             /* 1/sqrt(d_q) in the engine (forward.rs:904) */
    float *ov;               /* f32 [T][H][d_out] */
    void *workspace;         /* gs_mla_fused_workspace_bytes(T, H) bytes, 256-byte aligned, zeroed once */
    int64_t workspace_bytes;
    int32_t T, H, d_q, d_lat, d_out; /* d_q = 256, d_lat = 512, d_out = 256 */
} gs_mla_fused_args;
int64_t gs_mla_fused_workspace_bytes(int T, int H);
int gs_mla_decode_fused(const gs_mla_fused_args *args /* host */, void *stream);

/* gs_mla_decode for callers that cannot allocate device memory.  It has no counterpart in the
 * reference, whose engine owns and passes every buffer (forward.rs:496-500).  Some hosts of this
 * library cannot: a plugin running inside another runtime's memory pool, a call issued while that
 * runtime forbids cudaMalloc (for instance between the capture and the replay set-up of its own
 * graphs), or a caller with no place to keep a workspace between calls.  For them the split-KV
 * partials and the status block live in a fixed scratch array inside the library image
 * (GS_MLA_DECODE_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process
 * exits); args->workspace and args->workspace_bytes are ignored, everything else is as for
 * gs_mla_decode.
 *   - Sizes whose workspace (gs_mla_decode_workspace_bytes) exceeds the scratch array are rejected
 *     with cudaErrorInvalidValue and a message; one sequence with T <= 2 and H <= 24 fits.
 *   - The first call on each device looks the array's device address up (with that device
 *     current) and keeps it; make that first call outside any stream capture.  A cudaDeviceReset
 *     invalidates the kept address: this entry point is not for processes that reset the device.
 *   - All calls share the one array.  Each call clears the status block on `stream` first; the
 *     partial records are overwritten before they are read.  Two calls whose kernels overlap on
 *     the GPU (different streams, or different host threads) race on it: serialise them.
 *   - Calls neither cudaMalloc nor cudaFree nor any allocating library routine. */
#define GS_MLA_DECODE_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int gs_mla_decode_static(const gs_mla_decode_args *args /* host */, void *stream);
/* gs_mla_decode_status for the built-in array of the current device (its address is not exposed): synchronises
 * `stream`, reads the status word the last gs_mla_decode_static call left there and returns cudaErrorLaunchTimeout
 * when a bounded wait inside the kernels gave up (the output of that call is then not valid).  Read it before the
 * next gs_mla_decode_static call on the device: every call starts by clearing the word.  Allocates nothing. */
int gs_mla_decode_static_status(int32_t *status_out /* host, may be NULL */, void *stream);

/* Bytes of one rank's exchange buffer for `rows` = n_seq*T*H query rows (host function). */
int64_t gs_shard_exchange_bytes(int world, int rows, int d_v);
/* Exchange-buffer plumbing (host functions; the only entry points that allocate): a zeroed device
 * buffer that other processes on the node can map, its 64-byte handle, mapping a peer's handle
 * (enables peer access on first use), and the matching releases. */
int gs_peer_alloc(void **ptr, int64_t bytes);
int gs_peer_free(void *ptr);
int gs_peer_export(const void *ptr, void *handle64);
int gs_peer_open(const void *handle64, void **ptr);
int gs_peer_close(void *ptr);

/* Merge n_parts record blocks (each [rows*d_v acc][rows*2 (m,l)] floats, consecutive blocks
 * part_stride floats apart) into o f32 [rows][d_v]:  M = max m, L = sum l e^(m-M),
 * o = sum acc e^(m-M) / L, zeros when L == 0; the arithmetic of k_mla_combine, ops.cu:552-574,
 * with "split" = shard/GPU. */
int gs_mla_combine_parts(const float *parts, int n_parts, int64_t part_stride, int rows, int d_v, float *o,
                         void *stream);

/* ------------------------------------------------------------------------------------------------
 * Causal prefill attention (non-absorbed).  The reference runs prefill through gs_mla_attn with
 * T <= 256 and splits = 1 (forward.rs:61, :898-908), which equals per-head causal attention of
 * width 256 (forward.rs:900, :907).
 *   q f16 [S][H][d]   k f16 [p0+S][H][d]   v f16 [p0+S][H][d]   query i attends keys 0 .. p0+i
 *   o: f32 [S][H][d] (o_f16 == 0) or f16 (o_f16 == 1)
 * ---------------------------------------------------------------------------------------------- */
int gs_prefill_attn(const void *q, const void *k, const void *v, void *o, int o_f16, int S, int H, int d, int p0,
                    float scale, int impl, void *stream);
/* The same call with a status word: `status` is one int32 on the device, zeroed by the caller once; when a bounded
 * wait inside the tcgen05 kernel gives up (o is then not valid) the kernel ORs a code into it instead of failing
 * silently.  Read it with gs_mla_decode_status(status, ...), which treats any device word that way. */
int gs_prefill_attn_checked(const void *q, const void *k, const void *v, void *o, int o_f16, int S, int H, int d, int p0,
                            float scale, int impl, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Fused RoPE + KV-append: replaces the gs_f32_to_f16 call of forward.rs:857-860 when the cache row
 * carries a rotary part.  Row t of kv (f32 [n_seq][T][d_row]) is rounded to f16 (RNE, as
 * gemm.cu:157) and stored at position pos0 + t of its sequence, after rotating its last d_rope
 * columns (adjacent pairs, angle pos * base^(-2i/d_rope)).  d_rope = 0 gives the plain append.
 * ---------------------------------------------------------------------------------------------- */
/* Host-known position, one sequence, dense cache: `cache_row0` points at row pos0 (as the
 * reference passes latent + p0*R*2, forward.rs:858). */
int gs_rope_kv_append_at(const float *kv, void *cache_row0, int64_t pos0, int T, int d_row, int d_rope,
                         float rope_base, void *stream);
/* Batched, positions on the device: pos0[b] is the position of sequence b's first new row. */
/* The same append with the latent RMSNorm in front of it folded in (the reference runs gs_rmsnorm over the new
 * rows, forward.rs:850 / ops.cu:43-50, and then appends them, :857-860): the first d_row - d_rope columns become
 * x * rsqrt(mean(x^2) + eps) * w (w may be NULL = all ones), the last d_rope columns are rotated, all rounded to f16. */
int gs_norm_rope_kv_append_at(const float *kv, const float *w, float eps, void *cache_row0, int64_t pos0, int T,
                              int d_row, int d_rope, float rope_base, void *stream);
int gs_rope_kv_append(const float *kv, void *cache, const int32_t *pos0, const int32_t *seq_base,
                      const int32_t *page_table, int page_table_stride, int page_rows, int n_seq, int T, int d_row,
                      int d_rope, float rope_base, void *stream);
/* gs_rope_kv_append that never follows a bad index: a negative position, a position beyond the sequence's
 * page_table_stride * page_rows rows, or a cache row outside [0, cache_rows) writes nothing for that row and sets
 * bit 17 of *status (one int32 on the device, zeroed by the caller once; read it with gs_mla_decode_status).
 * gs_rope_kv_append itself trusts pos0, seq_base and the page table, as the reference trusts p0 (forward.rs:858). */
int gs_rope_kv_append_checked(const float *kv, void *cache, int64_t cache_rows, const int32_t *pos0,
                              const int32_t *seq_base, const int32_t *page_table, int page_table_stride, int page_rows,
                              int n_seq, int T, int d_row, int d_rope, float rope_base, int32_t *status, void *stream);
/* RoPE in place on f16 rows x [S][H][d] (prefill Q and K): last d_rope columns of every head at
 * position pos0 + s. */
int gs_rope_f16_inplace(void *x, int S, int H, int d, int d_rope, int64_t pos0, float rope_base, void *stream);

/* One decode step of one MLA layer with HOST buffers: the sequence of Engine::mla around the
 * attention call (forward.rs:849-860 then :900-906) enqueued by a single call - copy the queries and
 * the new latent rows in (pinned host memory for true asynchrony), append the rows at pos0 with
 * RoPE, attend seq_len = pos0 + T rows with the new rows visible, copy the output back.  Nothing is
 * synchronised: the result is in o_host once `stream` has drained.  The caller owns every buffer. */
typedef struct gs_mla_layer_step {
    const void *q_host;   /* f16 [T][H][d_qk] */
    const float *kv_host; /* f32 [T][d_qk] new latent rows */
    float *o_host;        /* f32 [T][H][d_v] */
    void *q_dev, *kv_dev, *o_dev; /* device staging of the same sizes */
    void *cache;          /* f16 [cache_rows][d_qk] */
    int64_t cache_rows;
    int32_t *seq_len_dev; /* one int32 on the device, written by the step */
    void *workspace;      /* gs_mla_decode_workspace_bytes(1, T, H, d_v) */
    int64_t workspace_bytes;
    int64_t pos0;         /* position of the first new row */
    int32_t T, H, d_qk, d_v, d_rope;
    float rope_base, scale;
} gs_mla_layer_step;
int gs_mla_layer_step_host(const gs_mla_layer_step *step /* host */, void *stream);

/* The same step recorded once as a CUDA graph of three kernels and replayed (no counterpart in the reference,
 * which enqueues every call separately).  q_host / kv_host / o_host must be page-locked, 16-byte aligned and
 * stay where they are: the first kernel reads the inputs from them in place, the combine kernel stores the
 * result into o_host in place (no copy-engine operation; kv_dev / o_dev are unused), and the caller refills
 * them between steps.  The position of a step travels through a page-locked word the handle owns, so one
 * graph serves every step with the same T; step->pos0 is ignored at creation.  One step may be in flight per
 * handle.  `stream` must not be the default stream.
 *   gs_mla_layer_graph_step(g, pos0, stream, wait): rejects pos0 + T > cache_rows ("context full",
 *   forward.rs:839-841) before launching; wait != 0 also synchronises the stream, after which o_host is valid.
 *   Moving pos0 back (a rejected MTP draft, forward.rs:1564-1575) needs no other call. */
typedef struct gs_mla_layer_graph gs_mla_layer_graph;
int gs_mla_layer_graph_create(const gs_mla_layer_step *step /* host */, void *stream, gs_mla_layer_graph **out);
int gs_mla_layer_graph_step(gs_mla_layer_graph *g, int64_t pos0, void *stream, int wait);
int gs_mla_layer_graph_destroy(gs_mla_layer_graph *g);

/* ------------------------------------------------------------------------------------------------
 * Cache persistence for paged caches.  The reference saves and restores every per-position buffer of a layer as
 * `unit` bytes per position, positions 0 .. upto-1 back to back (crates/engine/src/forward.rs:654-668
 * position_caches, :672-681 save_state, :683-695 load_state; crates/engine/src/session.rs:152-204).  These two
 * calls move a sequence between that layout and a paged pool (or a dense cache: pages == NULL, rows row0 ..),
 * byte for byte: f16 latent rows (unit_bytes = 2 * row width), or the int8 rows and f16 scales of a Q8 cache
 * (unit_bytes = row width, and row width / 32 * 2).
 *   pool      [pool_rows][unit_bytes]          pages  i32 [n_pages] page ids of the sequence (device)
 *   dst / src [upto][unit_bytes], device memory or page-locked host memory
 *   status    optional int32 on the device: bit 19 is set (and the position skipped) when a page id points outside
 *             the pool; read it with gs_mla_decode_status. */
int gs_cache_export_rows(const void *pool, int64_t pool_rows, const int32_t *pages, int32_t n_pages, int32_t page_rows,
                         int64_t row0, int64_t upto, int32_t unit_bytes, void *dst, int32_t *status, void *stream);
int gs_cache_import_rows(void *pool, int64_t pool_rows, const int32_t *pages, int32_t n_pages, int32_t page_rows,
                         int64_t row0, int64_t upto, int32_t unit_bytes, const void *src, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Diagnostics.
 * ---------------------------------------------------------------------------------------------- */
/* Text of the last error this thread's calls produced (host; like gs_error_string, lib.rs:169-175). */
const char *gs_attn_last_error_string(void);
/* Library build tag, e.g. "glmssd_attn sm_100a". */
const char *gs_attn_version(void);
/* Reads (synchronously, after synchronising `stream`) the device status word a decode left in its
 * workspace: 0 = ok, non-zero = a bounded wait inside the kernel gave up (code identifies which).
 * Returns cudaErrorLaunchTimeout when the word is non-zero. */
int gs_mla_decode_status(const void *workspace, int32_t *status_out /* host, may be NULL */, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GLMSSD_ATTN_H */
