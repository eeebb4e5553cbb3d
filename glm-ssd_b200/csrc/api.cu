// extern "C" entry points: argument validation, workspace carving and kernel selection.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "internal.cuh"

namespace gs {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

struct WsLayout {
    int64_t off_desc, off_acc, off_ml, total, max_segments, record_rows;
};

static WsLayout ws_layout(int n_seq, int T, int H, int d_v) {
    WsLayout w;
    w.max_segments = decode_segments_bound(n_seq, T);
    // a tcgen05 segment carries all T*H rows of a sequence, a CUDA-core segment H rows; size for the larger
    const int64_t rows_umma = ((int64_t) kMaxCtas + n_seq) * T * H;
    const int64_t rows_simt = (int64_t) n_seq * T * kSimtMaxSplits * H;
    const int64_t rows = rows_umma > rows_simt ? rows_umma : rows_simt;
    w.off_desc = kStatusBytes;
    // descriptors: up to 8 head groups of a sequence may run as sequences of their own
    w.off_acc = align_up(w.off_desc + (int64_t) n_seq * 8 * (int64_t) sizeof(int2), 256);
    w.record_rows = rows;
    w.off_ml = align_up(w.off_acc + rows * d_v * 4, 256);
    w.total = align_up(w.off_ml + rows * 2 * 4, 256);
    return w;
}

static int device_sm_count(int *out) {
    int dev = 0;
    GS_TRY(cudaGetDevice(&dev));
    GS_TRY(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev));
    return 0;
}

}  // namespace gs

using namespace gs;

GS_EXPORT const char *gs_attn_last_error_string(void) { return g_err; }
GS_EXPORT const char *gs_attn_version(void) { return "glmssd_attn sm_100a"; }

GS_EXPORT int64_t gs_mla_decode_workspace_bytes(int n_seq, int T, int H, int d_v) {
    if (n_seq <= 0 || T <= 0 || H <= 0 || d_v <= 0) return kStatusBytes;
    return ws_layout(n_seq, T, H, d_v).total;
}

GS_EXPORT int gs_mla_decode(const gs_mla_decode_args *a, void *stream) {
    if (!a) return fail_invalid("gs_mla_decode: args == NULL");
    if (a->n_seq < 0 || a->T < 0 || a->H < 0) return fail_invalid("gs_mla_decode: negative size");
    if (a->n_seq == 0 || a->T == 0 || a->H == 0) return 0;
    if (!a->q || !a->cache || !a->seq_lens) return fail_invalid("gs_mla_decode: q, cache and seq_lens are required");
    if (!a->o && !a->part_out) return fail_invalid("gs_mla_decode: o or part_out is required");
    if (a->d_qk <= 0 || a->d_v <= 0 || a->d_v > a->d_qk) return fail_invalid("gs_mla_decode: need 0 < d_v <= d_qk");
    if (a->page_table && a->page_rows != 64) return fail_invalid("gs_mla_decode: paged caches use 64-row pages");
    if (a->page_table && a->page_table_stride <= 0) return fail_invalid("gs_mla_decode: page_table_stride <= 0");
    if (a->cache_rows <= 0) return fail_invalid("gs_mla_decode: cache_rows <= 0");
    if (a->impl < 0 || a->impl > 2) return fail_invalid("gs_mla_decode: impl must be 0, 1 or 2");
    const WsLayout w = ws_layout(a->n_seq, a->T, a->H, a->d_v);
    if (!a->workspace || a->workspace_bytes < w.total) {
        set_error("gs_mla_decode: workspace of %lld bytes needed, %lld given", (long long) w.total,
                  (long long) a->workspace_bytes);
        return (int) cudaErrorInvalidValue;
    }
    if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return fail_invalid("gs_mla_decode: workspace must be 256-byte aligned");
    DecodeProblem p{};
    p.q = a->q;
    p.q_is_f32 = false;
    p.cache = (const __half *) a->cache;
    p.cache_rows = a->cache_rows;
    p.seq_lens = a->seq_lens;
    p.seq_base = a->seq_base;
    p.page_table = a->page_table;
    p.page_table_stride = a->page_table_stride;
    p.page_rows = a->page_table ? a->page_rows : 1;
    p.sel = nullptr;
    p.sel_stride = 0;
    p.scale = a->scale;
    p.tail_causal = a->tail_causal;
    p.o = a->o;
    p.part_out = a->part_out;
    char *ws = (char *) a->workspace;
    p.status = (int32_t *) ws;
    p.ws_desc = (int2 *) (ws + w.off_desc);
    p.ws_acc = (float *) (ws + w.off_acc);
    p.ws_ml = (float *) (ws + w.off_ml);
    p.max_segments = w.max_segments;
    p.max_record_rows = w.record_rows;
    p.n_seq = a->n_seq;
    p.T = a->T;
    p.H = a->H;
    p.d_qk = a->d_qk;
    p.d_v = a->d_v;
    p.max_seq_len = a->max_seq_len;
    p.splits = 0;
    p.ev_after_main = (cudaEvent_t) a->ev_after_main;
    p.exchange = a->exchange;
    if (p.exchange && !a->o) return fail_invalid("gs_mla_decode: the cross-GPU merge writes o; o is required");
    p.no_combine = (a->flags & GS_DECODE_NO_COMBINE) != 0;
    if (int e = device_sm_count(&p.sm_count)) return e;
    const char *why = "";
    const bool umma_ok = decode_umma_supported(p, &why);
    if (a->impl == 2 && !umma_ok) {
        set_error("gs_mla_decode: tcgen05 kernel does not take this shape: %s", why);
        return (int) cudaErrorInvalidValue;
    }
    if (umma_ok && a->impl != 1) return launch_decode_umma(p, (cudaStream_t) stream);
    return launch_decode_simt(p, (cudaStream_t) stream);
}

// ---- kernel choice of the reference-compatible entry point ---------------------------------------------------
// 0 = automatic (the tcgen05 kernel whenever it takes the shape), 1 = always the CUDA-core kernel (bit-level second
// opinion: f32 queries stay f32), 2 = the tcgen05 kernel or an error.  A process-wide setting, read once per call.
static std::atomic<int> g_attn_impl{0};

GS_EXPORT int gs_mla_attn_set_impl(int impl) {
    if (impl < 0 || impl > 2) return fail_invalid("gs_mla_attn_set_impl: impl must be 0, 1 or 2");
    g_attn_impl.store(impl, std::memory_order_relaxed);
    return 0;
}

GS_EXPORT int gs_mla_attn_status(int32_t *status_out, void *stream) {
    GS_TRY(cudaStreamSynchronize((cudaStream_t) stream));
    int32_t st = 0;
    if (int e = read_list_status(&st)) return e;
    if (status_out) *status_out = st;
    if (st != 0) {
        set_error("gs_mla_attn: a bounded wait inside the tcgen05 kernel gave up (status 0x%x)", st);
        return (int) cudaErrorLaunchTimeout;
    }
    return 0;
}

GS_EXPORT int gs_mla_attn(const float *q, const void *C, const void *C_scales, const int *sel, int sel_stride,
                          const int *cnt, float scale, float *o, float *part, int T, int H, int R, int splits,
                          void *stream) {
    // same rejections as the reference launcher (ops.cu:581)
    if (R != 512 || H % 16 != 0 || splits < 1) return fail_invalid("gs_mla_attn: need R == 512, H % 16 == 0, splits >= 1");
    if (T <= 0 || H <= 0) return 0;
    if (!q || !C || !sel || !cnt || !o) return fail_invalid("gs_mla_attn: null pointer");
    if (splits > 1 && !part) return fail_invalid("gs_mla_attn: part workspace required when splits > 1");
    DecodeProblem p{};
    if (int e = device_sm_count(&p.sm_count)) return e;
    // The tcgen05 kernel's producer warp fetches the listed rows itself (f16 rows, or int8 rows and their scales, which
    // the kernel widens in shared memory) and the kernel rounds the queries to f16 itself; it needs nothing beyond the
    // reference's own arguments.  Shapes it does not take run on the CUDA-core kernel below.
    const int impl = g_attn_impl.load(std::memory_order_relaxed);
    if (impl != 1) {
        const int e = launch_decode_umma_list(q, C, (const __half *) C_scales, sel, sel_stride, cnt, scale, o, part, T, H, R, splits,
                                              p.sm_count, (cudaStream_t) stream);
        if (e >= 0) return e;
    }
    if (impl == 2) return fail_invalid("gs_mla_attn: the tcgen05 kernel does not take this call (head count, alignment or scale)");
    p.q = q;
    p.q_is_f32 = true;
    p.cache = (const __half *) C;
    p.cache_scales = (const __half *) C_scales;  // non-null: int8 rows + f16 scale per 32 values (ops.cu:427)
    p.cache_rows = 0;
    p.seq_lens = cnt;
    p.sel = sel;
    p.sel_stride = sel_stride;
    p.page_rows = 1;
    p.scale = scale;
    p.tail_causal = 0;
    p.o = o;
    p.part_out = nullptr;
    // caller's `part`: T*H*splits*(R+2) floats (the size of ops.cu:578), used as [T*splits*H][R] accumulators then
    // [T*splits*H][2] (m, l).  With splits == 1 it is never touched and may be NULL (ops.cu:531-538).
    p.ws_acc = splits > 1 ? part : nullptr;
    p.ws_ml = splits > 1 ? part + (int64_t) T * splits * H * R : nullptr;
    p.max_segments = (int64_t) T * splits;
    p.n_seq = 1;
    p.T = T;
    p.H = H;
    p.d_qk = R;
    p.d_v = R;
    p.splits = splits;
    return launch_decode_simt(p, (cudaStream_t) stream);
}

GS_EXPORT int gs_mla_combine_parts(const float *parts, int n_parts, int64_t part_stride, int rows, int d_v, float *o,
                                   void *stream) {
    if (n_parts <= 0 || rows <= 0) return 0;
    if (!parts || !o || d_v <= 0 || d_v % 4 != 0) return fail_invalid("gs_mla_combine_parts: bad arguments");
    if (part_stride < (int64_t) rows * (d_v + 2) || part_stride % 4 != 0)
        return fail_invalid("gs_mla_combine_parts: part_stride must be >= rows*(d_v+2) and a multiple of 4");
    if (reinterpret_cast<uintptr_t>(parts) & 15 || reinterpret_cast<uintptr_t>(o) & 15)
        return fail_invalid("gs_mla_combine_parts: parts and o must be 16-byte aligned");
    // every block is one segment that holds all `rows` rows: a single group with H := rows
    CombinePlan c{};
    c.acc = parts;
    c.ml = parts + (int64_t) rows * d_v;
    c.desc = nullptr;
    c.regular_segments = n_parts;
    c.seg_stride_acc = part_stride;
    c.seg_stride_ml = part_stride;
    c.n_seq = 1;
    c.T = 1;
    c.H = rows;
    c.d_v = d_v;
    c.o = o;
    c.part_out = nullptr;
    return launch_combine(c, (cudaStream_t) stream);
}

static int prefill_attn(const char *who, const void *q, const void *k, const void *v, void *o, int o_f16, int S, int H, int d,
                        int p0, float scale, int impl, int32_t *status, void *stream) {
    if (S < 0 || H < 0 || p0 < 0) return fail_invalid("gs_prefill_attn: negative size");
    if (S == 0 || H == 0) return 0;
    if (!q || !k || !v || !o) return fail_invalid("gs_prefill_attn: null pointer");
    if (impl < 0 || impl > 2) return fail_invalid("gs_prefill_attn: impl must be 0, 1 or 2");
    const char *why = "";
    const bool umma_ok = prefill_umma_supported(S, H, d, p0, &why);
    if (impl == 2 && !umma_ok) {
        set_error("%s: tcgen05 kernel does not take this shape: %s", who, why);
        return (int) cudaErrorInvalidValue;
    }
    if (umma_ok && impl != 1)
        return launch_prefill_umma((const __half *) q, (const __half *) k, (const __half *) v, o, o_f16, S, H, d, p0,
                                   scale, status, (cudaStream_t) stream);
    return launch_prefill_simt((const __half *) q, (const __half *) k, (const __half *) v, o, o_f16, S, H, d, p0, scale,
                               (cudaStream_t) stream);
}

GS_EXPORT int gs_prefill_attn(const void *q, const void *k, const void *v, void *o, int o_f16, int S, int H, int d,
                              int p0, float scale, int impl, void *stream) {
    return prefill_attn("gs_prefill_attn", q, k, v, o, o_f16, S, H, d, p0, scale, impl, nullptr, stream);
}

GS_EXPORT int gs_prefill_attn_checked(const void *q, const void *k, const void *v, void *o, int o_f16, int S, int H, int d,
                                      int p0, float scale, int impl, int32_t *status, void *stream) {
    if (!status) return fail_invalid("gs_prefill_attn_checked: status (device) is required");
    return prefill_attn("gs_prefill_attn_checked", q, k, v, o, o_f16, S, H, d, p0, scale, impl, status, stream);
}

GS_EXPORT int gs_mla_decode_status(const void *workspace, int32_t *status_out, void *stream) {
    if (!workspace) return fail_invalid("gs_mla_decode_status: workspace == NULL");
    int32_t st = 0;
    GS_TRY(cudaStreamSynchronize((cudaStream_t) stream));
    GS_TRY(cudaMemcpy(&st, workspace, sizeof(st), cudaMemcpyDeviceToHost));
    if (status_out) *status_out = st;
    if (st != 0) {
        set_error("decode kernel gave up a bounded wait (status 0x%x)", st);
        return (int) cudaErrorLaunchTimeout;
    }
    return 0;
}

// ---- decode without caller-provided scratch -------------------------------------------------------
// The scratch array is part of the library image: every GPU that loads the library holds it until
// the process exits.  In host code `g_static_scratch` is only a handle for the symbol, not a device
// address; the address comes from cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[GS_MLA_DECODE_STATIC_SCRATCH_BYTES];
static std::atomic<void *> g_static_scratch_ptr[64];  // zero-initialised; racing first calls store the same address

// Device address of the built-in array on the current device (looked up once per device).
static int static_scratch_address(void **out, const char *who) {
    int dev = 0;
    GS_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("%s: device index beyond 63", who);
        return (int) cudaErrorInvalidValue;
    }
    void *scratch = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        // first call on this device (it is the current one): resolve the symbol to its device address
        GS_TRY(cudaGetSymbolAddress(&scratch, g_static_scratch));
        g_static_scratch_ptr[dev].store(scratch, std::memory_order_release);
    }
    *out = scratch;
    return 0;
}

GS_EXPORT int gs_mla_decode_static(const gs_mla_decode_args *a, void *stream) {
    if (!a) return fail_invalid("gs_mla_decode_static: args == NULL");
    if (a->n_seq < 0 || a->T < 0 || a->H < 0) return fail_invalid("gs_mla_decode_static: negative size");
    if (a->n_seq == 0 || a->T == 0 || a->H == 0) return 0;
    const int64_t need = gs_mla_decode_workspace_bytes(a->n_seq, a->T, a->H, a->d_v);
    if (need > (int64_t) GS_MLA_DECODE_STATIC_SCRATCH_BYTES) {
        set_error("gs_mla_decode_static: these sizes need %lld bytes of scratch, the built-in array holds %lld "
                  "(use gs_mla_decode with a caller-allocated workspace)",
                  (long long) need, (long long) GS_MLA_DECODE_STATIC_SCRATCH_BYTES);
        return (int) cudaErrorInvalidValue;
    }
    void *scratch = nullptr;
    if (int e = static_scratch_address(&scratch, "gs_mla_decode_static")) return e;
    // the status block must start at zero; the partial records are fully rewritten before they are read
    GS_TRY(cudaMemsetAsync(scratch, 0, kStatusBytes, (cudaStream_t) stream));
    gs_mla_decode_args b = *a;
    b.workspace = scratch;
    b.workspace_bytes = GS_MLA_DECODE_STATIC_SCRATCH_BYTES;
    return gs_mla_decode(&b, stream);
}

GS_EXPORT int gs_mla_decode_static_status(int32_t *status_out, void *stream) {
    void *scratch = nullptr;
    if (int e = static_scratch_address(&scratch, "gs_mla_decode_static_status")) return e;
    return gs_mla_decode_status(scratch, status_out, stream);
}
