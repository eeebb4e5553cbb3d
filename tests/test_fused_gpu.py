"""GPU parity of the fused decode step (absorb k_b, attend, expand v_b: crates/engine/src/forward.rs:900-907) against
the fp32 oracle, through the C ABI."""
import ctypes as C

import numpy as np
import pytest

from conftest import check_close, check_not_degenerate
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _inputs(seed, T, H, n):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((T, H, 256), dtype=np.float32)
    # weights scaled so that the absorbed queries have unit-order entries, like the benchmark's queries
    k_b = (rng.standard_normal((H, 512, 256), dtype=np.float32) / np.float32(16.0)).astype(np.float16)
    v_b = (rng.standard_normal((H, 256, 512), dtype=np.float32) / np.float32(22.6)).astype(np.float16)
    cache = (rng.standard_normal((max(n, 1) + 3, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    return q, k_b, v_b, cache


def _run(pkg, torch, q, k_b, v_b, cache, n):
    L = pkg._lib.load()
    T, H, _ = q.shape
    a = pkg._lib.FusedArgs()
    qd, kd, vd, cd = to_dev(torch, q), to_dev(torch, k_b), to_dev(torch, v_b), to_dev(torch, cache)
    lens = to_dev(torch, np.array([n], np.int32))
    ov = torch.zeros((T, H, 256), dtype=torch.float32, device="cuda")
    nbytes = L.gs_mla_fused_workspace_bytes(T, H)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    a.q, a.k_b, a.v_b, a.cache, a.cache_rows = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), cd.data_ptr(), cache.shape[0]
    a.seq_len, a.scale, a.ov = lens.data_ptr(), 1 / 16, ov.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    a.T, a.H, a.d_q, a.d_lat, a.d_out = T, H, 256, 512, 256
    rc = L.gs_mla_decode_fused(C.byref(a), None)
    assert rc == 0, L.gs_attn_last_error_string()
    torch.cuda.synchronize()
    assert pkg.decode_status(ws) == 0
    return ov.cpu().numpy()


@pytest.mark.parametrize("T,H,n", [(1, 64, 4096), (2, 64, 2500), (1, 20, 1000), (2, 16, 70), (8, 16, 300), (1, 32, 1), (2, 16, 0)])
def test_fused_decode_step_vs_oracle(pkg, cuda, oracle, T, H, n):
    q, k_b, v_b, cache = _inputs(T * 100 + H + n, T, H, n)
    got = _run(pkg, cuda, q, k_b, v_b, cache, n)
    want = oracle.mla_fused(q, k_b, v_b, cache, n, 1 / 16)
    check_close(got, want, "fused decode step")  # the attention tolerance: the absorbed queries are rounded to f16
    if n > 8:
        check_not_degenerate(got, "fused decode step")


def test_fused_equals_the_three_separate_calls(pkg, cuda, oracle):
    """The same step as the caller would issue it without the fused entry point: products on the host in fp32 (as the
    oracle), gs_mla_decode in between.  Pins the glue (workspace carving, argument forwarding)."""
    torch = cuda
    T, H, n = 2, 32, 3000
    q, k_b, v_b, cache = _inputs(5, T, H, n)
    got = _run(pkg, torch, q, k_b, v_b, cache, n)
    qabs = np.einsum("hrk,thk->thr", k_b.astype(np.float32), q).astype(np.float16)
    olat = pkg.mla_decode(to_dev(torch, qabs[None]), to_dev(torch, cache), to_dev(torch, np.array([n], np.int32)), max_seq_len=n)
    torch.cuda.synchronize()
    ov = np.einsum("hjr,thr->thj", v_b.astype(np.float32), olat.cpu().numpy()[0])
    assert np.abs(got - ov).max() <= 5e-4  # the absorbed queries may round to a neighbouring f16 value on the two sides


def test_fused_rejects_what_it_does_not_take(pkg, cuda):
    L = pkg._lib.load()
    a = pkg._lib.FusedArgs()
    a.T, a.H, a.d_q, a.d_lat, a.d_out = 9, 16, 256, 512, 256
    assert L.gs_mla_decode_fused(C.byref(a), None) == 1
    a.T, a.d_q = 1, 192
    assert L.gs_mla_decode_fused(C.byref(a), None) == 1
