"""ctypes/numpy front end of the CPU oracle (``oracle.c``).  Test infrastructure only: imported by
``tests/``, by ``__graft_entry__.smoke()`` as the checker and by ``bench.py`` for the timed CPU
baseline.  Nothing in the product package imports this module."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    so = _build.ORACLE_SO
    if not os.path.exists(so) or os.environ.get("GLMSSD_ORACLE_REBUILD"):
        so = _build.build_oracle()
    L = C.CDLL(so)
    i32, i64, f32, vp = C.c_int, C.c_int64, C.c_float, C.c_void_p
    L.oracle_f16_to_f32.restype = f32
    L.oracle_f16_to_f32.argtypes = [C.c_uint16]
    L.oracle_f32_to_f16.restype = C.c_uint16
    L.oracle_f32_to_f16.argtypes = [f32]
    L.oracle_f16_to_f32_array.argtypes = [vp, vp, i64]
    L.oracle_f32_to_f16_array.argtypes = [vp, vp, i64]
    L.oracle_host_cores.restype = i32
    L.oracle_mla_attn_ref.restype = i32
    L.oracle_mla_attn_ref.argtypes = [vp, vp, vp, i32, vp, f32, vp, i32, i32, i32, i32]
    L.oracle_combine.argtypes = [vp, i64, i32, i32, vp]
    L.oracle_mla_decode.restype = i32
    L.oracle_mla_decode.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, vp, i32, i32, i32, i32, i32, i32]
    L.oracle_mla_decode_split.restype = i32
    L.oracle_mla_decode_split.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, vp, i32, i32, i32, i32, i32, i32, vp, i32]
    L.oracle_mla_decode_partial.restype = i32
    L.oracle_mla_decode_partial.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, vp, i64, i64, i32, i32, i32, i32, i32,
                                            i32]
    L.oracle_prefill.restype = i32
    L.oracle_prefill.argtypes = [vp, vp, vp, f32, vp, i32, i32, i32, i32, i32, vp, i32, i32]
    L.oracle_quant_q8_rows.argtypes = [vp, vp, vp, i64]
    L.oracle_dequant_q8.argtypes = [vp, vp, vp, i64]
    L.oracle_rope_inv_freq.argtypes = [vp, i32, C.c_double]
    L.oracle_rope_append.argtypes = [vp, vp, i32, i32, i32, i64, C.c_double]
    L.oracle_norm_rope_append.argtypes = [vp, vp, f32, vp, i32, i32, i32, i64, C.c_double]
    L.oracle_rope_f16.argtypes = [vp, i32, i32, i32, i32, i64, C.c_double]
    L.oracle_mla_fused.restype = i32
    L.oracle_mla_fused.argtypes = [vp, vp, vp, vp, i32, f32, vp, i32, i32, i32, i32, i32, i32]
    L.oracle_idx_pool.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]
    L.oracle_idx_score.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, f32]
    L.oracle_idx_select.argtypes = [vp, i64, i32, i32, i32, i32, vp, i32, vp]
    _lib = L
    return L


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def host_cores() -> int:
    return int(lib().oracle_host_cores())


def f16_bits(a: np.ndarray) -> np.ndarray:
    """float16 array -> its uint16 bit pattern (no copy when contiguous)."""
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_f16_array(_p(x), _p(y), x.size)
    return y.view(np.float16)


def f16_to_f32(x: np.ndarray) -> np.ndarray:
    xb = f16_bits(x)
    y = np.empty(xb.shape, np.float32)
    lib().oracle_f16_to_f32_array(_p(xb), _p(y), xb.size)
    return y


def mla_attn_ref(q, cache, sel, cnt, scale, threads=0):
    """Reference-ABI attention. q f32 [T,H,R]; cache f16 [ctx,R]; sel i32 [T,stride]; cnt i32 [T]."""
    q = _c(q, np.float32)
    T, H, R = q.shape
    cb = f16_bits(cache)
    sel = _c(sel, np.int32)
    cnt = _c(cnt, np.int32)
    o = np.empty((T, H, R), np.float32)
    lib().oracle_mla_attn_ref(_p(q), _p(cb), _p(sel), sel.shape[1], _p(cnt), scale, _p(o), T, H, R, threads)
    return o


def combine(parts: np.ndarray) -> np.ndarray:
    """parts f32 [n_rows, n_parts, d_v + 2] (acc.., m, l) -> o f32 [n_rows, d_v]."""
    parts = _c(parts, np.float32)
    n_rows, n_parts, rec = parts.shape
    o = np.empty((n_rows, rec - 2), np.float32)
    lib().oracle_combine(_p(parts), n_rows, n_parts, rec - 2, _p(o))
    return o


def mla_decode(q, cache, seq_lens, scale, d_v=512, seq_base=None, page_table=None, page_rows=64, threads=0,
               part_range=None, return_threads=False, key_splits=0):
    """q f16 [n_seq,T,H,d_qk]; cache f16 [rows,d_qk].  Returns o f32 [n_seq,T,H,d_v], or with
    ``part_range=(lo, hi)`` the unnormalised records f32 [n_seq,T,H,d_v+2] over rows lo..hi.
    ``key_splits > 1`` cuts every row's attended range into that many work items (merged by the reference's
    combine arithmetic), so that all host cores work when n_seq*T*H is small."""
    qb = f16_bits(q)
    n_seq, T, H, d_qk = qb.shape
    cb = f16_bits(cache)
    seq_lens = _c(seq_lens, np.int32)
    sb = None if seq_base is None else _c(seq_base, np.int32)
    pt = None if page_table is None else _c(page_table, np.int32)
    pts = 0 if pt is None else pt.shape[1]
    if part_range is None and key_splits > 1:
        o = np.empty((n_seq, T, H, d_v), np.float32)
        scratch = np.empty((n_seq * T * H * key_splits, d_v + 2), np.float32)
        used = lib().oracle_mla_decode_split(_p(qb), _p(cb), _p(seq_lens), _p(sb), _p(pt), pts, page_rows, scale, _p(o),
                                             n_seq, T, H, d_qk, d_v, key_splits, _p(scratch), threads)
    elif part_range is None:
        o = np.empty((n_seq, T, H, d_v), np.float32)
        used = lib().oracle_mla_decode(_p(qb), _p(cb), _p(seq_lens), _p(sb), _p(pt), pts, page_rows, scale, _p(o),
                                       n_seq, T, H, d_qk, d_v, threads)
    else:
        o = np.empty((n_seq, T, H, d_v + 2), np.float32)
        used = lib().oracle_mla_decode_partial(_p(qb), _p(cb), _p(seq_lens), _p(sb), _p(pt), pts, page_rows, scale,
                                               _p(o), int(part_range[0]), int(part_range[1]), n_seq, T, H, d_qk, d_v,
                                               threads)
    return (o, used) if return_threads else o


def prefill(Q, K, V, scale, p0=0, rows=None, threads=0, return_threads=False):
    """Q f16 [S,H,d]; K f16 [p0+S,H,d]; V f16 [p0+S,H,dv] -> o f32 [S or len(rows),H,dv] (causal)."""
    Qb, Kb, Vb = f16_bits(Q), f16_bits(K), f16_bits(V)
    S, H, d = Qb.shape
    dv = Vb.shape[2]
    rs = None if rows is None else _c(rows, np.int32)
    n = S if rs is None else rs.size
    o = np.empty((n, H, dv), np.float32)
    used = lib().oracle_prefill(_p(Qb), _p(Kb), _p(Vb), scale, _p(o), S, H, d, dv, p0, _p(rs), 0 if rs is None else n,
                                threads)
    return (o, used) if return_threads else o


def rope_inv_freq(d_rope=64, base=10000.0) -> np.ndarray:
    f = np.empty(d_rope // 2, np.float32)
    lib().oracle_rope_inv_freq(_p(f), d_rope, base)
    return f


def rope_append(x, pos0, d_rope=64, base=10000.0) -> np.ndarray:
    """x f32 [T,d_row] -> f16 [T,d_row] with RoPE on the last d_rope columns at positions pos0+t."""
    x = _c(x, np.float32)
    T, d_row = x.shape
    y = np.empty((T, d_row), np.uint16)
    lib().oracle_rope_append(_p(x), _p(y), T, d_row, d_rope, pos0, base)
    return y.view(np.float16)


def norm_rope_append(x, pos0, weight=None, eps=1e-6, d_rope=64, base=10000.0) -> np.ndarray:
    """x f32 [T,d_row] -> f16 [T,d_row]: RMSNorm (weights ``weight`` or ones) on the first d_row - d_rope columns,
    RoPE on the rest at positions pos0+t."""
    x = _c(x, np.float32)
    T, d_row = x.shape
    w = None if weight is None else _c(weight, np.float32)
    y = np.empty((T, d_row), np.uint16)
    lib().oracle_norm_rope_append(_p(x), _p(w), eps, _p(y), T, d_row, d_rope, pos0, base)
    return y.view(np.float16)


def rope_f16(x, pos0=0, d_rope=64, base=10000.0) -> np.ndarray:
    """x f16 [S,H,d] -> rotated copy (last d_rope columns of each head at position pos0+s)."""
    xb = f16_bits(x).copy()
    S, H, d = xb.shape
    lib().oracle_rope_f16(_p(xb), S, H, d, d_rope, pos0, base)
    return xb.view(np.float16)


def quant_q8_rows(x):
    """x f32 [..., 32k] -> (q int8 same shape, d f16 [..., k]) : per block of 32, d = amax/127, q = rn(x/d)."""
    x = _c(x, np.float32)
    assert x.shape[-1] % 32 == 0
    q = np.empty(x.shape, np.int8)
    d = np.empty(x.shape[:-1] + (x.shape[-1] // 32,), np.uint16)
    lib().oracle_quant_q8_rows(_p(x), _p(q), _p(d), x.size // 32)
    return q, d.view(np.float16)


def dequant_q8(q, d):
    """The f16 tile the attention kernel rebuilds from a Q8 cache: half_rn(float(d) * q)."""
    q = _c(q, np.int8)
    db = f16_bits(d)
    out = np.empty(q.shape, np.uint16)
    lib().oracle_dequant_q8(_p(q), _p(db), _p(out), q.size // 32)
    return out.view(np.float16)


# ---- DSA k-pool indexer (crates/cuda/kernels/ops.cu:619-791) -------------------------------------------

def idx_pool(kc, gc, rk, rg, ape, P, p0, kpool):
    """In place on rk, rg (rings [kpool,Dk]) and P ([pools,Dk]); kc, gc f32 [T,Dk] are the chunk's rows."""
    kc, gc, ape = _c(kc, np.float32), _c(gc, np.float32), _c(ape, np.float32)
    assert rk.flags.c_contiguous and rg.flags.c_contiguous and P.flags.c_contiguous
    T, Dk = kc.shape
    lib().oracle_idx_pool(_p(kc), _p(gc), _p(rk), _p(rg), _p(ape), _p(P), int(p0), T, Dk, int(kpool))


def idx_score(q, w, P, score, pos0, kpool, scale):
    """q f32 [T,Hq,Dk], w f32 [T,Hq], P f32 [pools,Dk]; fills score f32 [T,stride] in place."""
    q, w, P = _c(q, np.float32), _c(w, np.float32), _c(P, np.float32)
    T, Hq, Dk = q.shape
    assert score.flags.c_contiguous and score.dtype == np.float32
    lib().oracle_idx_score(_p(q), _p(w), _p(P), _p(score), score.shape[1], int(pos0), T, int(kpool), Hq, Dk, float(scale))


def idx_select(score, pos0, kpool, top_k, sel_stride):
    """score f32 [T,stride] -> (sel i32 [T,sel_stride], cnt i32 [T]); pools in ascending index, ties to the lowest."""
    score = _c(score, np.float32)
    T = score.shape[0]
    sel = np.full((T, sel_stride), -1, np.int32)
    cnt = np.zeros(T, np.int32)
    lib().oracle_idx_select(_p(score), score.shape[1], int(pos0), T, int(kpool), int(top_k), _p(sel), sel_stride, _p(cnt))
    return sel, cnt


def mla_fused(q, k_b, v_b, cache, seq_len, scale, threads=0):
    """q f32 [T,H,d_q]; k_b f16 [H,R,d_q]; v_b f16 [H,d_out,R]; cache f16 [rows,R] -> ov f32 [T,H,d_out]
    (absorb, attend, expand: forward.rs:900-907)."""
    q = _c(q, np.float32)
    T, H, d_q = q.shape
    kb, vb, cb = f16_bits(k_b), f16_bits(v_b), f16_bits(cache)
    R, d_out = kb.shape[1], vb.shape[1]
    ov = np.empty((T, H, d_out), np.float32)
    lib().oracle_mla_fused(_p(q), _p(kb), _p(vb), _p(cb), int(seq_len), float(scale), _p(ov), T, H, d_q, R, d_out, threads)
    return ov
