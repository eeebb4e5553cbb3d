"""GPU parity of the reference-compatible entry points (gs_mla_attn, gs_f32_to_f16) against the
oracle and, where the reference's own kernels were compiled (oracle/_ref), against those."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import ROOT, check_close, check_not_degenerate
from gpu_util import to_dev

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(ROOT, "oracle", "_ref", "libglmssd_ref.so")


def _legacy_inputs(seed, T, H, n, ctx, dense=True):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    Cc = (rng.standard_normal((ctx, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    stride = n + 4
    sel = np.zeros((T, stride), np.int32)
    cnt = np.zeros(T, np.int32)
    for t in range(T):
        k = max(0, n - (T - 1 - t))
        cnt[t] = k
        sel[t, :k] = np.arange(k) if dense else rng.permutation(ctx)[:k]
    return q, Cc, sel, cnt


def _call(torch, fn, q, Cc, sel, cnt, splits):
    T, H, R = q.shape
    qd, cd, sd, nd = to_dev(torch, q), to_dev(torch, Cc), to_dev(torch, sel), to_dev(torch, cnt)
    o = torch.zeros((T, H, R), dtype=torch.float32, device="cuda")
    part = torch.zeros(T * H * splits * (R + 2), dtype=torch.float32, device="cuda")
    rc = fn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel.shape[1], nd.data_ptr(), 1 / 16, o.data_ptr(),
            part.data_ptr(), T, H, R, splits, None)
    assert rc == 0
    torch.cuda.synchronize()
    return o.cpu().numpy()


@pytest.mark.parametrize("T,H,n,splits,dense", [
    (1, 64, 4096, 16, True), (2, 64, 5000, 4, True), (1, 32, 2052, 16, False), (9, 16, 300, 1, False),
    (1, 16, 0, 16, True), (3, 16, 1, 4, True), (2, 64, 33, 4, False), (1, 64, 7, 16, True),
])
def test_gs_mla_attn_vs_oracle(pkg, cuda, oracle, T, H, n, splits, dense):
    q, Cc, sel, cnt = _legacy_inputs(T * 1000 + n, T, H, n, max(n, 1) + 100, dense)
    got = _call(cuda, pkg._lib.load().gs_mla_attn, q, Cc, sel, cnt, splits)
    want = oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16)
    check_close(got, want, "gs_mla_attn")
    if n > 8:
        check_not_degenerate(got, "gs_mla_attn")


def test_gs_mla_attn_prefill_shape(pkg, cuda, oracle):
    # the reference's prefill launch: 256 queries, splits = 1, prior context p0 (forward.rs:898-901)
    T, H, p0 = 256, 16, 100
    rng = np.random.default_rng(1)
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    Cc = (rng.standard_normal((p0 + T, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    sel = np.tile(np.arange(p0 + T, dtype=np.int32), (T, 1))
    cnt = (p0 + 1 + np.arange(T)).astype(np.int32)
    got = _call(cuda, pkg._lib.load().gs_mla_attn, q, Cc, sel, cnt, 1)
    check_close(got, oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16), "prefill via gs_mla_attn")


def test_gs_f32_to_f16_bit_exact(pkg, cuda, oracle):
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.standard_normal(512 * 5 + 3).astype(np.float32) * s for s in (1e-7, 1.0, 1e3)])
    xd = to_dev(cuda, x)
    y = cuda.zeros(x.size, dtype=cuda.float16, device="cuda")
    pkg.f32_to_f16(xd, y, x.size)
    cuda.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy().view(np.uint16), oracle.f32_to_f16(x).view(np.uint16))
    # odd element offset (4-byte aligned source, 2-byte aligned destination)
    y2 = cuda.zeros(x.size, dtype=cuda.float16, device="cuda")
    L = pkg._lib.load()
    assert L.gs_f32_to_f16(xd.data_ptr() + 4, y2.data_ptr() + 2, x.size - 1, None) == 0
    cuda.cuda.synchronize()
    assert np.array_equal(y2.cpu().numpy().view(np.uint16)[1:], oracle.f32_to_f16(x[1:]).view(np.uint16))


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="reference kernels were not compiled (oracle/_ref absent)")
@pytest.mark.parametrize("T,H,n,splits,dense", [(1, 64, 4096, 16, True), (2, 32, 3000, 4, False), (20, 16, 500, 1, False),
                                                 (1, 16, 0, 16, True), (2, 64, 31, 4, True)])
def test_reference_kernel_pins_oracle_and_agrees_with_ours(pkg, cuda, oracle, T, H, n, splits, dense):
    ref = C.CDLL(REF_SO)
    ref.gs_mla_attn.restype = C.c_int
    ref.gs_mla_attn.argtypes = pkg._lib.SIGNATURES["gs_mla_attn"][1]
    q, Cc, sel, cnt = _legacy_inputs(7 * T + n, T, H, n, max(n, 1) + 64, dense)
    o_ref = _call(cuda, ref.gs_mla_attn, q, Cc, sel, cnt, splits)
    o_orc = oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16)
    o_new = _call(cuda, pkg._lib.load().gs_mla_attn, q, Cc, sel, cnt, splits)
    check_close(o_orc, o_ref, "oracle vs reference kernel", 2e-5, 2e-6)
    check_close(o_new, o_ref, "ours vs reference kernel", 2e-5, 2e-6)
