"""ctypes binding of ``libglmssd_attn.so`` (the C ABI declared in ``include/glmssd_attn.h``).

There is no fallback: if the library is missing or an entry point is absent the import fails."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))

i32, i64, f32, vp = C.c_int, C.c_int64, C.c_float, C.c_void_p


class ShardExchange(C.Structure):
    """Mirror of ``struct gs_shard_exchange``."""
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("epoch", C.c_uint32), ("peer_bufs", C.POINTER(vp)),
                ("buf_bytes", i64), ("wait_limit_cycles", i64)]


class LayerStep(C.Structure):
    """Mirror of ``struct gs_mla_layer_step``."""
    _fields_ = [("q_host", vp), ("kv_host", vp), ("o_host", vp), ("q_dev", vp), ("kv_dev", vp), ("o_dev", vp),
                ("cache", vp), ("cache_rows", i64), ("seq_len_dev", vp), ("workspace", vp), ("workspace_bytes", i64),
                ("pos0", i64), ("T", C.c_int32), ("H", C.c_int32), ("d_qk", C.c_int32), ("d_v", C.c_int32),
                ("d_rope", C.c_int32), ("rope_base", f32), ("scale", f32)]


class DecodeArgs(C.Structure):
    """Mirror of ``struct gs_mla_decode_args``."""
    _fields_ = [
        ("q", vp), ("cache", vp), ("cache_rows", i64), ("seq_lens", vp), ("seq_base", vp), ("page_table", vp),
        ("page_table_stride", C.c_int32), ("page_rows", C.c_int32), ("scale", f32), ("tail_causal", C.c_int32),
        ("o", vp), ("part_out", vp), ("workspace", vp), ("workspace_bytes", i64),
        ("n_seq", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("d_qk", C.c_int32), ("d_v", C.c_int32),
        ("max_seq_len", C.c_int32), ("impl", C.c_int32), ("ev_after_main", vp), ("flags", C.c_int32), ("exchange", C.POINTER(ShardExchange)),
    ]


# name -> (restype, argtypes); every symbol include/glmssd_attn.h declares
class FusedArgs(C.Structure):
    """gs_mla_fused_args of include/glmssd_attn.h."""
    _fields_ = [("q", vp), ("k_b", vp), ("v_b", vp), ("cache", vp), ("cache_rows", i64), ("seq_len", vp), ("scale", f32),
                ("ov", vp), ("workspace", vp), ("workspace_bytes", i64), ("T", i32), ("H", i32), ("d_q", i32), ("d_lat", i32),
                ("d_out", i32)]


SIGNATURES = {
    "gs_mla_attn": (i32, [vp, vp, vp, vp, i32, vp, f32, vp, vp, i32, i32, i32, i32, vp]),
    "gs_f32_to_f16": (i32, [vp, vp, i64, vp]),
    "gs_quant_q8_rows": (i32, [vp, vp, vp, i64, vp]),
    "gs_idx_pool": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "gs_idx_score": (i32, [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, vp]),
    "gs_idx_select": (i32, [vp, i64, i32, i32, i32, i32, vp, i32, vp, vp]),
    "gs_cache_export_rows": (i32, [vp, i64, vp, i32, i32, i64, i64, i32, vp, vp, vp]),
    "gs_cache_import_rows": (i32, [vp, i64, vp, i32, i32, i64, i64, i32, vp, vp, vp]),
    "gs_mla_attn_set_impl": (i32, [i32]),
    "gs_mla_attn_status": (i32, [C.POINTER(C.c_int32), vp]),
    "gs_mla_decode_workspace_bytes": (i64, [i32, i32, i32, i32]),
    "gs_mla_decode": (i32, [C.POINTER(DecodeArgs), vp]),
    "gs_mla_decode_static": (i32, [C.POINTER(DecodeArgs), vp]),
    "gs_mla_fused_workspace_bytes": (i64, [i32, i32]),
    "gs_mla_decode_fused": (i32, [C.POINTER(FusedArgs), vp]),
    "gs_mla_decode_static_status": (i32, [C.POINTER(C.c_int32), vp]),
    "gs_mla_combine_parts": (i32, [vp, i32, i64, i32, i32, vp, vp]),
    "gs_shard_exchange_bytes": (i64, [i32, i32, i32]),
    "gs_peer_alloc": (i32, [C.POINTER(vp), i64]),
    "gs_peer_free": (i32, [vp]),
    "gs_peer_export": (i32, [vp, vp]),
    "gs_peer_open": (i32, [vp, C.POINTER(vp)]),
    "gs_peer_close": (i32, [vp]),
    "gs_prefill_attn": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp]),
    "gs_rope_kv_append_at": (i32, [vp, vp, i64, i32, i32, i32, f32, vp]),
    "gs_norm_rope_kv_append_at": (i32, [vp, vp, f32, vp, i64, i32, i32, i32, f32, vp]),
    "gs_rope_kv_append": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp]),
    "gs_prefill_attn_checked": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp, vp]),
    "gs_rope_kv_append_checked": (i32, [vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp]),
    "gs_rope_f16_inplace": (i32, [vp, i32, i32, i32, i32, i64, f32, vp]),
    "gs_mla_layer_step_host": (i32, [C.POINTER(LayerStep), vp]),
    "gs_mla_layer_graph_create": (i32, [C.POINTER(LayerStep), vp, C.POINTER(vp)]),
    "gs_mla_layer_graph_step": (i32, [vp, i64, vp, i32]),
    "gs_mla_layer_graph_destroy": (i32, [vp]),
    "gs_attn_last_error_string": (C.c_char_p, []),
    "gs_attn_version": (C.c_char_p, []),
    "gs_mla_decode_status": (i32, [vp, C.POINTER(C.c_int32), vp]),
}

_lib = None


def lib_path() -> str:
    return _build.LIB


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python {os.path.join(HERE, 'build.py')}` "
                          "(there is no fallback implementation)")
    L = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


class GsError(RuntimeError):
    def __init__(self, code: int, where: str):
        msg = load().gs_attn_last_error_string().decode(errors="replace")
        super().__init__(f"{where} failed with cudaError {code}: {msg}")
        self.code = code


def check(code: int, where: str) -> None:
    if code != 0:
        raise GsError(code, where)
