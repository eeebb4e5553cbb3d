"""Host-side mirror of the engine's attention call sites, on top of the C ABI.

The reference's host code is Rust (``Engine::mla``, crates/engine/src/forward.rs:833-911, calling the
``ffi::gs_*`` declarations of crates/cuda/src/lib.rs:96-123).  This module keeps the same names and
argument meaning for the two reference entry points and adds the extended ones; torch is used only
to own device memory and streams.  Every function enqueues on the current CUDA stream and returns
without synchronising, like the reference's ``ck!(ffi::...)`` calls.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib

SCALE_256 = 1.0 / math.sqrt(256.0)  # 1/sqrt(mla_head_k), forward.rs:904


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


# ---- reference-compatible entry points -------------------------------------------------------------

def mla_attn(q, C_latent, C_scales, sel, sel_stride, cnt, scale, o, part, T, H, R, splits):
    """``gs_mla_attn`` with the reference's argument list (crates/cuda/src/lib.rs:97-100)."""
    L = _lib.load()
    _lib.check(L.gs_mla_attn(_ptr(q), _ptr(C_latent), _ptr(C_scales), _ptr(sel), sel_stride, _ptr(cnt), scale,
                             _ptr(o), _ptr(part), T, H, R, splits, _stream()), "gs_mla_attn")


def mla_attn_impl(impl: int) -> None:
    """Kernel choice of ``gs_mla_attn``: 0 automatic, 1 CUDA-core kernel (f32 queries stay f32), 2 tcgen05 kernel or error."""
    _lib.check(_lib.load().gs_mla_attn_set_impl(impl), "gs_mla_attn_set_impl")


def mla_attn_status() -> int:
    """Synchronises and returns the sticky status word of the tcgen05 path of ``gs_mla_attn`` (0 = ok)."""
    st = C.c_int32(0)
    _lib.load().gs_mla_attn_status(C.byref(st), _stream())
    return int(st.value)


def f32_to_f16(x, y, n):
    """``gs_f32_to_f16`` (crates/cuda/src/lib.rs:123): the reference's KV-append."""
    _lib.check(_lib.load().gs_f32_to_f16(_ptr(x), _ptr(y), n, _stream()), "gs_f32_to_f16")


def quant_q8_rows(x, q, d, n):
    """``gs_quant_q8_rows`` (crates/cuda/src/lib.rs:96): the KV-append of the Q8 latent cache.
    x f32 [n]; q int8 [n]; d f16 [n/32]."""
    _lib.check(_lib.load().gs_quant_q8_rows(_ptr(x), _ptr(q), _ptr(d), n, _stream()), "gs_quant_q8_rows")


# ---- extended entry points -------------------------------------------------------------------------

def decode_workspace_bytes(n_seq: int, T: int, H: int, d_v: int = 512) -> int:
    return int(_lib.load().gs_mla_decode_workspace_bytes(n_seq, T, H, d_v))


def new_workspace(n_seq: int, T: int, H: int, d_v: int = 512, device=None) -> torch.Tensor:
    nbytes = decode_workspace_bytes(n_seq, T, H, d_v)
    return torch.zeros(nbytes, dtype=torch.uint8, device=device or torch.cuda.current_device())


def mla_decode(q, cache, seq_lens, *, scale=SCALE_256, d_v=512, seq_base=None, page_table=None, page_rows=64,
               tail_causal=True, out=None, part_out=None, want_out=True, workspace=None, max_seq_len=0, impl=0,
               ev_after_main=None, no_combine=False, static_scratch=False, exchange=None):
    """Absorbed-MLA decode.  q f16 [n_seq,T,H,d_qk]; cache f16 [rows,d_qk]; seq_lens i32 [n_seq] (device).
    Returns ``out`` (f32 [n_seq,T,H,d_v]) or, with ``want_out=False``, ``part_out``."""
    L = _lib.load()
    _need(q, torch.float16, "q")
    _need(cache, torch.float16, "cache")
    _need(seq_lens, torch.int32, "seq_lens")
    n_seq, T, H, d_qk = q.shape
    if cache.dim() != 2 or cache.shape[1] != d_qk:
        raise ValueError("cache must be [rows, d_qk]")
    if workspace is None and not static_scratch:
        workspace = new_workspace(n_seq, T, H, d_v, q.device)
    if want_out and out is None:
        out = torch.empty((n_seq, T, H, d_v), dtype=torch.float32, device=q.device)
    a = _lib.DecodeArgs()
    a.q, a.cache, a.cache_rows = q.data_ptr(), cache.data_ptr(), cache.shape[0]
    a.seq_lens, a.seq_base = seq_lens.data_ptr(), _ptr(seq_base)
    a.page_table = _ptr(page_table)
    a.page_table_stride = 0 if page_table is None else page_table.shape[1]
    a.page_rows = page_rows
    a.scale = scale
    a.tail_causal = 1 if tail_causal else 0
    a.o = _ptr(out) if want_out else None
    a.part_out = _ptr(part_out)
    if not static_scratch:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.n_seq, a.T, a.H, a.d_qk, a.d_v = n_seq, T, H, d_qk, d_v
    a.max_seq_len = max_seq_len
    a.impl = impl
    a.ev_after_main = ev_after_main  # raw cudaEvent_t handle (int) or None
    a.flags = 1 if no_combine else 0
    if exchange is not None:  # a _lib.ShardExchange kept alive by the caller (see sharded.PeerExchange)
        a.exchange = C.pointer(exchange)
    if static_scratch:
        # the library's built-in scratch array instead of a workspace: nothing is allocated for the call
        _lib.check(L.gs_mla_decode_static(C.byref(a), _stream()), "gs_mla_decode_static")
    else:
        _lib.check(L.gs_mla_decode(C.byref(a), _stream()), "gs_mla_decode")
    return out if want_out else part_out


def decode_status(workspace) -> int:
    """Synchronises and returns the device status word of the last decode that used ``workspace``."""
    st = C.c_int32(0)
    _lib.load().gs_mla_decode_status(workspace.data_ptr(), C.byref(st), _stream())
    return int(st.value)


def part_floats(rows: int, d_v: int = 512) -> int:
    """Floats in one (acc, m, l) record block for ``rows`` query rows."""
    return rows * (d_v + 2)


def combine_parts(parts, n_parts, rows, d_v=512, out=None, part_stride=None):
    """Merge ``n_parts`` record blocks (f32, ``part_stride`` floats apart) into out f32 [rows, d_v]."""
    _need(parts, torch.float32, "parts")
    if part_stride is None:
        part_stride = parts.numel() // n_parts
    if out is None:
        out = torch.empty((rows, d_v), dtype=torch.float32, device=parts.device)
    _lib.check(_lib.load().gs_mla_combine_parts(parts.data_ptr(), n_parts, part_stride, rows, d_v, out.data_ptr(),
                                                _stream()), "gs_mla_combine_parts")
    return out


def prefill_attn(q, k, v, *, p0=0, scale=SCALE_256, out=None, out_f16=False, impl=0):
    """Causal prefill attention.  q f16 [S,H,d]; k, v f16 [p0+S,H,d] -> f32 or f16 [S,H,d]."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _need(t, torch.float16, n)
    S, H, d = q.shape
    if k.shape != (p0 + S, H, d) or v.shape != (p0 + S, H, d):
        raise ValueError("k and v must be [p0+S, H, d]")
    if out is None:
        out = torch.empty((S, H, d), dtype=torch.float16 if out_f16 else torch.float32, device=q.device)
    _lib.check(_lib.load().gs_prefill_attn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                           1 if out.dtype == torch.float16 else 0, S, H, d, p0, scale, impl,
                                           _stream()), "gs_prefill_attn")
    return out


def rope_kv_append_at(kv, cache, pos0, *, d_rope=64, rope_base=10000.0):
    """Append rows kv (f32 [T,d_row]) at positions pos0.. of a dense single-sequence cache [rows,d_row]."""
    _need(kv, torch.float32, "kv")
    _need(cache, torch.float16, "cache")
    T, d_row = kv.shape
    if pos0 + T > cache.shape[0]:
        raise ValueError(f"context full ({cache.shape[0]} rows)")  # forward.rs:839-841
    row0 = cache.data_ptr() + pos0 * d_row * 2
    _lib.check(_lib.load().gs_rope_kv_append_at(kv.data_ptr(), row0, pos0, T, d_row, d_rope, rope_base, _stream()),
               "gs_rope_kv_append_at")


def norm_rope_kv_append_at(kv, cache, pos0, *, weight=None, eps=1e-6, d_rope=64, rope_base=10000.0):
    """The same with the latent RMSNorm folded in (forward.rs:850): the first d_row - d_rope columns are normalised
    (``weight`` f32 [d_row - d_rope] or None), the rest rotated, all appended as f16."""
    _need(kv, torch.float32, "kv")
    _need(cache, torch.float16, "cache")
    T, d_row = kv.shape
    if pos0 + T > cache.shape[0]:
        raise ValueError(f"context full ({cache.shape[0]} rows)")
    if weight is not None:
        _need(weight, torch.float32, "weight")
    row0 = cache.data_ptr() + pos0 * d_row * 2
    _lib.check(_lib.load().gs_norm_rope_kv_append_at(kv.data_ptr(), _ptr(weight), eps, row0, pos0, T, d_row, d_rope,
                                                     rope_base, _stream()), "gs_norm_rope_kv_append_at")


def rope_kv_append(kv, cache, pos0, *, seq_base=None, page_table=None, page_rows=64, d_rope=64, rope_base=10000.0):
    """Batched append: kv f32 [n_seq,T,d_row]; pos0 i32 [n_seq] on the device."""
    _need(kv, torch.float32, "kv")
    _need(cache, torch.float16, "cache")
    _need(pos0, torch.int32, "pos0")
    n_seq, T, d_row = kv.shape
    _lib.check(_lib.load().gs_rope_kv_append(kv.data_ptr(), cache.data_ptr(), pos0.data_ptr(), _ptr(seq_base),
                                             _ptr(page_table), 0 if page_table is None else page_table.shape[1],
                                             page_rows, n_seq, T, d_row, d_rope, rope_base, _stream()),
               "gs_rope_kv_append")


def rope_f16_inplace(x, *, d_rope=64, pos0=0, rope_base=10000.0):
    """RoPE in place on x f16 [S,H,d] (last d_rope columns of each head at position pos0+s)."""
    _need(x, torch.float16, "x")
    S, H, d = x.shape
    _lib.check(_lib.load().gs_rope_f16_inplace(x.data_ptr(), S, H, d, d_rope, pos0, rope_base, _stream()),
               "gs_rope_f16_inplace")
    return x


# ---- the call-site mirror ----------------------------------------------------------------------------

class MlaDecodeLayer:
    """One MLA layer's latent cache plus the per-step sequence of ``Engine::mla``
    (forward.rs:849-860 then :900-906): append the new rows, then attend with the new rows visible.

    ``step`` is the end-to-end call a user of the library makes: host inputs in, host output back.
    The latent cache is persistent layer state in HBM (forward.rs:388-404), not a per-step input.
    """

    def __init__(self, ctx: int, H: int, *, d_qk=576, d_v=512, d_rope=64, T_max=2, device=None, use_graph=False):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.ctx, self.H, self.d_qk, self.d_v, self.d_rope, self.T_max = ctx, H, d_qk, d_v, d_rope, T_max
        self.cache = torch.zeros((ctx, d_qk), dtype=torch.float16, device=self.device)  # zero-initialised, forward.rs:390
        self.pos = 0
        self.workspace = new_workspace(1, T_max, H, d_v, self.device)
        self._seq_len = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._q_dev = torch.empty((1, T_max, H, d_qk), dtype=torch.float16, device=self.device)
        self._kv_dev = torch.empty((T_max, d_qk), dtype=torch.float32, device=self.device)
        self._o_dev = torch.empty((1, T_max, H, d_v), dtype=torch.float32, device=self.device)
        self._o_host = torch.empty((1, T_max, H, d_v), dtype=torch.float32).pin_memory()
        self._len_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        st = _lib.LayerStep()
        st.o_host = self._o_host.data_ptr()
        st.q_dev, st.kv_dev, st.o_dev = self._q_dev.data_ptr(), self._kv_dev.data_ptr(), self._o_dev.data_ptr()
        st.cache, st.cache_rows = self.cache.data_ptr(), ctx
        st.seq_len_dev = self._seq_len.data_ptr()
        st.workspace, st.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        st.H, st.d_qk, st.d_v, st.d_rope = H, d_qk, d_v, d_rope
        st.rope_base, st.scale = 10000.0, SCALE_256
        self._step = st
        # graph mode: the whole step (staging, append, attention) is one replayed CUDA graph of three kernels on a
        # stream of the layer's own; the kernels read and write the page-locked host tensors in place
        self.use_graph = bool(use_graph)
        self._graphs = {}
        self._fast = None  # (q_host, kv_host, T, graph handle, output view) of the last graph step
        self._graph_stream = None
        if self.use_graph:
            torch.cuda.synchronize(self.device)
            self._graph_stream = torch.cuda.Stream(device=self.device)
            self._graph_stream_handle = self._graph_stream.cuda_stream
            self._graph_step = _lib.load().gs_mla_layer_graph_step

    def __del__(self):
        try:
            L = _lib.load()
            for h in self._graphs.values():
                L.gs_mla_layer_graph_destroy(h)
        except Exception:
            pass

    def rollback(self, n: int = 1) -> None:
        """Drop the last n positions (rejected MTP draft): the rows are simply overwritten by the next
        append, as in forward.rs:1564-1575."""
        self.pos = max(0, self.pos - n)

    def _graph_for(self, q_host, kv_host, T):
        key = (q_host.data_ptr(), kv_host.data_ptr(), T)
        h = self._graphs.get(key)
        if h is None:
            s = self._step
            s.q_host, s.kv_host, s.T, s.pos0 = q_host.data_ptr(), kv_host.data_ptr(), T, 0
            out = C.c_void_p()
            _lib.check(_lib.load().gs_mla_layer_graph_create(C.byref(s), self._graph_stream.cuda_stream, C.byref(out)),
                       "gs_mla_layer_graph_create")
            h = self._graphs[key] = out.value
        return h

    def step(self, q_host: torch.Tensor, kv_host: torch.Tensor) -> torch.Tensor:
        """q_host f16 [T,H,d_qk], kv_host f32 [T,d_qk] in pinned host memory -> f32 [T,H,d_v] (host).
        One C call enqueues copy-in, append, attention and copy-out; then the stream is drained.  In graph
        mode the host buffers are part of the recorded graph: reuse the same two tensors every step."""
        fast = self._fast
        if fast is not None and q_host is fast[0] and kv_host is fast[1]:
            # the same two host tensors as in the step before (the graph names their memory): nothing to look up.
            # A step is tens of microseconds, so the interpreter's share of this method is measurable (2.5 us before).
            _, _, T, h, out = fast
            pos = self.pos
            if pos + T > self.ctx:
                raise RuntimeError(f"context full ({self.ctx} tokens)")
            rc = self._graph_step(h, pos, self._graph_stream_handle, 1)
            if rc:
                _lib.check(rc, "gs_mla_layer_graph_step")
            self.pos = pos + T
            return out
        T = q_host.shape[0]
        if T > self.T_max:
            raise ValueError("T exceeds T_max")
        if self.pos + T > self.ctx:
            raise RuntimeError(f"context full ({self.ctx} tokens)")
        if self.use_graph:
            h = self._graphs.get((q_host.data_ptr(), kv_host.data_ptr(), T))
            if h is None:
                if not (q_host.is_pinned() and kv_host.is_pinned()):
                    raise ValueError("graph mode needs page-locked host tensors")
                h = self._graph_for(q_host, kv_host, T)
            rc = self._graph_step(h, self.pos, self._graph_stream_handle, 1)
            if rc:
                _lib.check(rc, "gs_mla_layer_graph_step")
            self.pos += T
            out = self._o_host[0, :T]
            # remembered by identity; a tensor whose storage or shape was changed in place must not be passed again
            self._fast = (q_host, kv_host, T, h, out)
            return out
        s = self._step
        s.q_host, s.kv_host = q_host.data_ptr(), kv_host.data_ptr()
        s.pos0, s.T = self.pos, T
        _lib.check(_lib.load().gs_mla_layer_step_host(C.byref(s), _stream()), "gs_mla_layer_step_host")
        self.pos += T
        torch.cuda.current_stream().synchronize()
        return self._o_host[0, :T]
