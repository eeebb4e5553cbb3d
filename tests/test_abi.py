"""CPU tests of the boundary: the C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments with cudaErrorInvalidValue before touching the device."""
import ctypes as C
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_ERROR_INVALID_VALUE = 1


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "glmssd_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gs_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_reference_entry_points():
    names = _declared_functions()
    # the two names the engine's Rust FFI block binds for this path (crates/cuda/src/lib.rs:97-100, :123)
    assert "gs_mla_attn" in names and "gs_f32_to_f16" in names
    assert len(names) >= 10


def test_library_exports_every_declared_symbol(pkg):
    lib = C.CDLL(pkg._lib.lib_path())
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/glmssd_attn.h but not exported"
    assert set(_declared_functions()) == set(pkg._lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_error_string(pkg):
    L = pkg._lib.load()
    assert b"sm_100a" in L.gs_attn_version()
    assert isinstance(L.gs_attn_last_error_string(), bytes)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    m = importlib.import_module("glm-ssd_b200._lib")
    monkeypatch.setattr(m, "_lib", None)
    monkeypatch.setattr(m._build, "LIB", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        m.load()


@pytest.mark.parametrize("R,H,splits", [(256, 64, 4), (512, 40, 4), (512, 72, 4), (512, 64, 0)])
def test_reference_abi_rejections(pkg, R, H, splits):
    # same rejections as the reference launcher (ops.cu:581); the loader-level limits they mirror are
    # tested in the reference at crates/engine/src/validate.rs:493-497 (72 and 40 heads, rank 256)
    L = pkg._lib.load()
    rc = L.gs_mla_attn(None, None, None, None, 0, None, 0.0625, None, None, 1, H, R, splits, None)
    assert rc == CUDA_ERROR_INVALID_VALUE
    assert b"gs_mla_attn" in L.gs_attn_last_error_string()


def test_quant_q8_rows_rejects_ragged_length(pkg):
    L = pkg._lib.load()
    assert L.gs_quant_q8_rows(None, None, None, 33, None) == CUDA_ERROR_INVALID_VALUE  # ops.cu:612
    assert L.gs_quant_q8_rows(None, None, None, 0, None) == 0


def test_decode_argument_validation(pkg):
    L = pkg._lib.load()
    assert L.gs_mla_decode(None, None) == CUDA_ERROR_INVALID_VALUE
    a = pkg._lib.DecodeArgs()
    a.n_seq, a.T, a.H, a.d_qk, a.d_v = 1, 1, 20, 576, 512
    assert L.gs_mla_decode(C.byref(a), None) == CUDA_ERROR_INVALID_VALUE  # null pointers
    a.q = a.cache = a.seq_lens = a.o = 256
    a.cache_rows = 128
    a.d_v = 600
    assert L.gs_mla_decode(C.byref(a), None) == CUDA_ERROR_INVALID_VALUE  # d_v > d_qk
    a.d_v = 512
    a.page_table, a.page_rows, a.page_table_stride = 256, 32, 4
    assert L.gs_mla_decode(C.byref(a), None) == CUDA_ERROR_INVALID_VALUE  # page size
    a.page_table = None
    a.workspace, a.workspace_bytes = 256, 16
    assert L.gs_mla_decode(C.byref(a), None) == CUDA_ERROR_INVALID_VALUE  # workspace too small
    assert b"workspace" in L.gs_attn_last_error_string()
    # empty problems are a no-op success, like the reference's n <= 0 early return (gemm.cu:160)
    a.n_seq = 0
    assert L.gs_mla_decode(C.byref(a), None) == 0
    assert L.gs_f32_to_f16(None, None, 0, None) == 0


def test_workspace_query_is_monotone(pkg):
    w1 = pkg.decode_workspace_bytes(1, 1, 20)
    w2 = pkg.decode_workspace_bytes(1, 2, 20)
    w64 = pkg.decode_workspace_bytes(64, 1, 20)
    assert 0 < w1 <= w2 and w1 <= w64
    assert w1 % 256 == 0


def test_append_argument_validation(pkg):
    L = pkg._lib.load()
    assert L.gs_rope_kv_append_at(None, None, 0, 1, 575, 64, 10000.0, None) == CUDA_ERROR_INVALID_VALUE
    assert L.gs_rope_kv_append_at(None, None, 0, 1, 576, 63, 10000.0, None) == CUDA_ERROR_INVALID_VALUE
    assert L.gs_rope_kv_append_at(None, None, -1, 1, 576, 64, 10000.0, None) == CUDA_ERROR_INVALID_VALUE
    assert L.gs_rope_kv_append_at(None, None, 0, 0, 576, 64, 10000.0, None) == 0
    assert L.gs_prefill_attn(None, None, None, None, 0, 0, 20, 256, 0, 0.0625, 0, None) == 0
    assert L.gs_prefill_attn(None, None, None, None, 0, 8, 20, 256, 0, 0.0625, 0, None) == CUDA_ERROR_INVALID_VALUE
