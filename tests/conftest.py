import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# tolerance of the attention outputs (f16 inputs, fp32 accumulate)
MAX_ABS_TOL = 2e-3
MEAN_ABS_TOL = 2e-4


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle_py
    oracle_py.lib()
    return oracle_py


@pytest.fixture(scope="session")
def pkg():
    """The product package (loads libglmssd_attn.so; no fallback)."""
    return importlib.import_module("glm-ssd_b200")


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test collected on a machine without CUDA")
    torch.cuda.set_device(0)
    return torch


def check_close(got: np.ndarray, want: np.ndarray, what: str = "", max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    assert err.max() <= max_tol, f"{what}: max-abs error {err.max():.3e} > {max_tol}"
    assert err.mean() <= mean_tol, f"{what}: mean-abs error {err.mean():.3e} > {mean_tol}"


def check_not_degenerate(x: np.ndarray, what: str = ""):
    """Guard in the style of the reference's kernel cross-check (crates/engine/src/qtest.rs): the output
    must not be all zero or a handful of distinct values."""
    x = np.asarray(x)
    assert np.abs(x).max() > 0, f"{what}: all-zero output"
    assert np.unique(x.ravel()[:4096]).size > 16, f"{what}: degenerate output"


def make_decode_inputs(seed, n_seq, T, H, n_rows, d_qk=576, sigma=0.5):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n_seq, T, H, d_qk), dtype=np.float32).astype(np.float16)
    cache = (rng.standard_normal((n_rows, d_qk), dtype=np.float32) * np.float32(sigma)).astype(np.float16)
    return q, cache
