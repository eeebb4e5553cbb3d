// C++ host-side mirror of the engine's wrappers and attention call site, on top of the C ABI.
//
// The reference's host code is Rust: RAII wrappers `Stream`, `Event`, `DeviceBuffer` with
// range-checked transfers (crates/cuda/src/lib.rs:201-366), `check()` turning a non-zero return
// code into an error (lib.rs:169-175), and `Engine::mla` (crates/engine/src/forward.rs:833-911),
// which appends the new latent rows and then attends with them visible.  This header restates
// those pieces in C++ with the same names and behaviour so that the call sequence can be exercised
// from compiled host code; errors are exceptions here where the reference returns `Result`.
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/glmssd_attn.h"

namespace glmssd {

// lib.rs:169-175: a non-zero code becomes an error carrying the library's message
inline void check(int code, const char *what) {
    if (code != 0) {
        std::string msg = std::string(what) + " failed with cudaError " + std::to_string(code) + ": ";
        const char *detail = gs_attn_last_error_string();
        msg += (detail && *detail) ? detail : cudaGetErrorString((cudaError_t) code);
        throw std::runtime_error(msg);
    }
}

// lib.rs:201-241: a stream that does not synchronise with the legacy default stream (runtime.cu:45-47)
class Stream {
  public:
    Stream() { check((int) cudaStreamCreateWithFlags(&s_, cudaStreamNonBlocking), "stream create"); }
    ~Stream() { cudaStreamDestroy(s_); }
    Stream(const Stream &) = delete;
    Stream &operator=(const Stream &) = delete;
    void sync() const { check((int) cudaStreamSynchronize(s_), "stream sync"); }
    void *raw() const { return (void *) s_; }

  private:
    cudaStream_t s_ = nullptr;
};

// lib.rs:281-287: `off..off+len` must lie inside a buffer of `cap` bytes (no overflow)
inline void check_range(size_t off, size_t len, size_t cap) {
    if (off + len < off || off + len > cap)
        throw std::out_of_range("device buffer access out of range: " + std::to_string(off) + " + " + std::to_string(len) +
                                " > " + std::to_string(cap) + " bytes");
}

// lib.rs:289-366: untyped device allocation, zero-initialised, with range-checked transfers
class DeviceBuffer {
  public:
    explicit DeviceBuffer(size_t len) : len_(len) {
        check((int) cudaMalloc(&ptr_, len ? len : 1), "device alloc");
        check((int) cudaMemset(ptr_, 0, len ? len : 1), "device memset");
    }
    ~DeviceBuffer() { cudaFree(ptr_); }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    void *ptr() const { return ptr_; }
    size_t len() const { return len_; }
    void upload(const void *src, size_t off, size_t n, const Stream &s) {
        check_range(off, n, len_);
        check((int) cudaMemcpyAsync((char *) ptr_ + off, src, n, cudaMemcpyHostToDevice, (cudaStream_t) s.raw()), "upload");
    }
    void download(void *dst, size_t off, size_t n, const Stream &s) const {
        check_range(off, n, len_);
        check((int) cudaMemcpyAsync(dst, (const char *) ptr_ + off, n, cudaMemcpyDeviceToHost, (cudaStream_t) s.raw()), "download");
    }

  private:
    void *ptr_ = nullptr;
    size_t len_ = 0;
};

// One MLA layer's latent cache and the attention part of Engine::mla for a dense cache:
//   forward.rs:839-841  bail when the context is full
//   forward.rs:849-860  append the rows of these positions to the f16 cache (here with the RoPE part)
//   forward.rs:900-906  attention over the cache with the new rows visible, scale 1/sqrt(mla_head_k)
//   forward.rs:1564-1575 a rejected MTP draft is undone by moving `pos` back; the cache needs no undo
class MlaLayer {
  public:
    MlaLayer(int ctx, int n_head, int t_max = 2, int d_qk = 576, int d_v = 512, int d_rope = 64)
        : ctx_(ctx), h_(n_head), t_max_(t_max), d_qk_(d_qk), d_v_(d_v), d_rope_(d_rope),
          latent_((size_t) ctx * d_qk * 2),
          ws_((size_t) gs_mla_decode_workspace_bytes(1, t_max, n_head, d_v)),
          q_((size_t) t_max * n_head * d_qk * 2), kv_((size_t) t_max * d_qk * 4),
          olat_((size_t) t_max * n_head * d_v * 4), seq_len_(sizeof(int32_t)) {}

    int pos() const { return pos_; }
    void rollback_to_first() { if (pos_ > 0) pos_ -= 1; }
    DeviceBuffer &latent() { return latent_; }

    // q: f16 bits [t][H][d_qk] (absorbed queries), kv: f32 [t][d_qk] (new latent rows), out: f32 [t][H][d_v]
    void mla(const uint16_t *q, const float *kv, float *out, int t, const Stream &s) {
        if (t < 1 || t > t_max_) throw std::invalid_argument("t out of range");
        if (pos_ + t > ctx_) throw std::runtime_error("context full (" + std::to_string(ctx_) + " tokens)");
        q_.upload(q, 0, (size_t) t * h_ * d_qk_ * 2, s);
        kv_.upload(kv, 0, (size_t) t * d_qk_ * 4, s);
        check(gs_rope_kv_append_at((const float *) kv_.ptr(), (char *) latent_.ptr() + (size_t) pos_ * d_qk_ * 2, pos_, t,
                                   d_qk_, d_rope_, 10000.0f, s.raw()),
              "gs_rope_kv_append_at");
        pos_ += t;
        const int32_t len = pos_;
        seq_len_.upload(&len, 0, sizeof(len), s);
        gs_mla_decode_args a{};
        a.q = q_.ptr();
        a.cache = latent_.ptr();
        a.cache_rows = ctx_;
        a.seq_lens = (const int32_t *) seq_len_.ptr();
        a.page_rows = 64;
        a.scale = 1.0f / std::sqrt(256.0f);
        a.tail_causal = 1;
        a.o = (float *) olat_.ptr();
        a.workspace = ws_.ptr();
        a.workspace_bytes = (int64_t) ws_.len();
        a.n_seq = 1;
        a.T = t;
        a.H = h_;
        a.d_qk = d_qk_;
        a.d_v = d_v_;
        a.max_seq_len = pos_;
        check(gs_mla_decode(&a, s.raw()), "gs_mla_decode");
        olat_.download(out, 0, (size_t) t * h_ * d_v_ * 4, s);
        s.sync();
        check(gs_mla_decode_status(ws_.ptr(), nullptr, s.raw()), "gs_mla_decode_status");
    }

  private:
    int ctx_, h_, t_max_, d_qk_, d_v_, d_rope_;
    int pos_ = 0;
    DeviceBuffer latent_, ws_, q_, kv_, olat_, seq_len_;
};

// Page-locked host memory the kernels of a replayed step read and write in place.
class PinnedBuffer {
  public:
    explicit PinnedBuffer(size_t len) : len_(len) { check((int) cudaHostAlloc(&ptr_, len ? len : 1, cudaHostAllocMapped), "pinned alloc"); }
    ~PinnedBuffer() { cudaFreeHost(ptr_); }
    PinnedBuffer(const PinnedBuffer &) = delete;
    PinnedBuffer &operator=(const PinnedBuffer &) = delete;
    void *ptr() const { return ptr_; }
    size_t len() const { return len_; }

  private:
    void *ptr_ = nullptr;
    size_t len_ = 0;
};

// The same layer with the whole step (stage inputs, append, attend, store the result) recorded once per T as
// a CUDA graph and replayed: the caller fills q() / kv(), calls mla(t), reads out().  The position is host
// state, as in the engine; moving it back (forward.rs:1564-1575) needs no device work.
class MlaLayerGraph {
  public:
    MlaLayerGraph(int ctx, int n_head, const Stream &s, int t_max = 2, int d_qk = 576, int d_v = 512, int d_rope = 64)
        : ctx_(ctx), h_(n_head), t_max_(t_max), d_qk_(d_qk), d_v_(d_v), d_rope_(d_rope), stream_(s),
          latent_((size_t) ctx * d_qk * 2), ws_((size_t) gs_mla_decode_workspace_bytes(1, t_max, n_head, d_v)),
          q_dev_((size_t) t_max * n_head * d_qk * 2), seq_len_(sizeof(int32_t)),
          q_((size_t) t_max * n_head * d_qk * 2), kv_((size_t) t_max * d_qk * 4), out_((size_t) t_max * n_head * d_v * 4) {
        for (auto &g : graphs_) g = nullptr;
    }
    ~MlaLayerGraph() {
        for (auto g : graphs_) gs_mla_layer_graph_destroy(g);
    }
    uint16_t *q() { return (uint16_t *) q_.ptr(); }
    float *kv() { return (float *) kv_.ptr(); }
    const float *out() const { return (const float *) out_.ptr(); }
    int pos() const { return pos_; }
    void set_pos(int p) { pos_ = p; }

    void mla(int t) {
        if (t < 1 || t > t_max_ || t > 4) throw std::invalid_argument("t out of range");
        if (pos_ + t > ctx_) throw std::runtime_error("context full (" + std::to_string(ctx_) + " tokens)");
        if (!graphs_[t]) {
            gs_mla_layer_step st{};
            st.q_host = q_.ptr();
            st.kv_host = (const float *) kv_.ptr();
            st.o_host = (float *) out_.ptr();
            st.q_dev = q_dev_.ptr();
            st.cache = latent_.ptr();
            st.cache_rows = ctx_;
            st.seq_len_dev = (int32_t *) seq_len_.ptr();
            st.workspace = ws_.ptr();
            st.workspace_bytes = (int64_t) ws_.len();
            st.T = t;
            st.H = h_;
            st.d_qk = d_qk_;
            st.d_v = d_v_;
            st.d_rope = d_rope_;
            st.rope_base = 10000.0f;
            st.scale = 1.0f / std::sqrt(256.0f);
            check((int) cudaDeviceSynchronize(), "device sync");
            check(gs_mla_layer_graph_create(&st, stream_.raw(), &graphs_[t]), "gs_mla_layer_graph_create");
        }
        check(gs_mla_layer_graph_step(graphs_[t], pos_, stream_.raw(), 1), "gs_mla_layer_graph_step");
        pos_ += t;
    }

  private:
    int ctx_, h_, t_max_, d_qk_, d_v_, d_rope_;
    int pos_ = 0;
    const Stream &stream_;
    DeviceBuffer latent_, ws_, q_dev_, seq_len_;
    PinnedBuffer q_, kv_, out_;
    gs_mla_layer_graph *graphs_[5];
};

}  // namespace glmssd
