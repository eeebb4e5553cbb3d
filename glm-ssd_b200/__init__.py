"""B200 (sm_100a) attention hot path of the GLM-SSD engine: absorbed-MLA decode over the f16 latent
cache, causal prefill attention and the fused RoPE + KV-append, behind a C ABI.

The directory name carries a hyphen, so import it with
``importlib.import_module("glm-ssd_b200")``.  Importing loads ``libglmssd_attn.so`` and fails if it
is missing; there is no fallback implementation.
"""
from . import _lib

_lib.load()

from .attn import (  # noqa: E402
    SCALE_256, MlaDecodeLayer, combine_parts, decode_status, decode_workspace_bytes, f32_to_f16, mla_attn, mla_attn_impl, mla_attn_status, quant_q8_rows,
    mla_decode, new_workspace, part_floats, prefill_attn, rope_f16_inplace, rope_kv_append, rope_kv_append_at, norm_rope_kv_append_at,
)
from .sharded import PeerExchange, lpt_assign, shard_rows  # noqa: E402

__all__ = [
    "SCALE_256", "MlaDecodeLayer", "combine_parts", "decode_status", "decode_workspace_bytes", "f32_to_f16", "quant_q8_rows", "mla_attn_impl", "mla_attn_status",
    "mla_attn", "mla_decode", "new_workspace", "part_floats", "prefill_attn", "rope_f16_inplace",
    "rope_kv_append", "rope_kv_append_at", "norm_rope_kv_append_at", "lpt_assign", "shard_rows", "PeerExchange",
]
