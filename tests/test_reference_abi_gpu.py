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


class _Impl:
    """gs_mla_attn_set_impl(impl) for the duration of a block; automatic choice afterwards."""

    def __init__(self, L, impl):
        self.L, self.impl = L, impl

    def __enter__(self):
        assert self.L.gs_mla_attn_set_impl(self.impl) == 0

    def __exit__(self, *exc):
        assert self.L.gs_mla_attn_set_impl(0) == 0


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


def _call(torch, fn, q, Cc, sel, cnt, splits, scales=None):
    T, H, R = q.shape
    qd, cd, sd, nd = to_dev(torch, q), to_dev(torch, Cc), to_dev(torch, sel), to_dev(torch, cnt)
    scd = None if scales is None else to_dev(torch, scales)
    o = torch.zeros((T, H, R), dtype=torch.float32, device="cuda")
    part = torch.zeros(T * H * splits * (R + 2), dtype=torch.float32, device="cuda")
    rc = fn(qd.data_ptr(), cd.data_ptr(), None if scd is None else scd.data_ptr(), sd.data_ptr(), sel.shape[1], nd.data_ptr(), 1 / 16, o.data_ptr(),
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


ENGINE_PART_FLOATS = 128 * (16 * 512 + 32)  # the engine's `part` allocation (crates/engine/src/forward.rs:498)


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("T,H,splits", [(256, 64, 1), (8, 64, 4), (1, 64, 16), (2, 64, 4)])
def test_gs_mla_attn_stays_inside_the_engines_part_buffer(pkg, cuda, oracle, T, H, splits, impl):
    """The engine passes one `part` buffer of 128 * (16*512 + 32) floats to every call: decode (T = 1, 16 splits),
    MTP verify (T = 2, 4 splits), chunks of up to 8 tokens with 4 splits, and prefill chunks of up to 256 tokens
    with splits = 1, where the reference never touches it (ops.cu:531-538).  A canary tail behind the usable part
    of the allocation must come back unchanged, and with splits = 1 the buffer itself too."""
    torch = cuda
    n = 300
    q, Cc, sel, cnt = _legacy_inputs(T + 31 * splits, T, H, n, n + 50, dense=False)
    qd, cd, sd, nd = to_dev(torch, q), to_dev(torch, Cc), to_dev(torch, sel), to_dev(torch, cnt)
    o = torch.zeros((T, H, 512), dtype=torch.float32, device="cuda")
    tail = 1 << 16
    part = torch.full((ENGINE_PART_FLOATS + tail,), -7.25, dtype=torch.float32, device="cuda")
    L = pkg._lib.load()
    with _Impl(L, impl):  # the automatic choice (tcgen05 kernel, records or none in `part`) and the CUDA-core kernel
        rc = L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel.shape[1], nd.data_ptr(), 1 / 16,
                           o.data_ptr(), part.data_ptr(), T, H, 512, splits, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool((part[ENGINE_PART_FLOATS:] == -7.25).all()), "gs_mla_attn wrote past the engine's part buffer"
    if splits == 1:
        assert bool((part == -7.25).all()), "part must not be touched when splits == 1"
    check_close(o.cpu().numpy(), oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16), "gs_mla_attn (engine part buffer)")


def test_gs_mla_attn_single_split_takes_null_part(pkg, cuda, oracle):
    torch = cuda
    T, H, n = 40, 16, 120
    q, Cc, sel, cnt = _legacy_inputs(3, T, H, n, n + 9, dense=True)
    qd, cd, sd, nd = to_dev(torch, q), to_dev(torch, Cc), to_dev(torch, sel), to_dev(torch, cnt)
    o = torch.zeros((T, H, 512), dtype=torch.float32, device="cuda")
    L = pkg._lib.load()
    assert L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel.shape[1], nd.data_ptr(), 1 / 16, o.data_ptr(),
                         None, T, H, 512, 1, None) == 0
    torch.cuda.synchronize()
    check_close(o.cpu().numpy(), oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16), "gs_mla_attn, part == NULL")
    # more than one split still needs the buffer
    assert L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel.shape[1], nd.data_ptr(), 1 / 16, o.data_ptr(),
                         None, T, H, 512, 4, None) == 1


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
    L = pkg._lib.load()
    with _Impl(L, 1):
        o_new = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
    o_auto = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
    check_close(o_orc, o_ref, "oracle vs reference kernel", 2e-5, 2e-6)
    check_close(o_new, o_ref, "ours (CUDA-core kernel, f32 queries) vs reference kernel", 2e-5, 2e-6)
    check_close(o_auto, o_ref, "ours (automatic choice: tcgen05 kernel, f16-rounded queries) vs reference kernel")


# ---- Q8 latent cache (int8 rows + one f16 scale per 32 values; crates/cuda/kernels/ops.cu:427, :461-477) ----

def _quant_gpu(torch, fn, x):
    xd = to_dev(torch, x)
    q = torch.zeros(x.size, dtype=torch.int8, device="cuda")
    d = torch.zeros(x.size // 32, dtype=torch.float16, device="cuda")
    assert fn(xd.data_ptr(), q.data_ptr(), d.data_ptr(), x.size, None) == 0
    torch.cuda.synchronize()
    return q.cpu().numpy().reshape(x.shape), d.cpu().numpy().reshape(x.shape[:-1] + (x.shape[-1] // 32,))


def test_gs_quant_q8_rows_bit_exact(pkg, cuda, oracle):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((301, 512)).astype(np.float32) * np.float32(2.0)
    x[7] = 0.0
    x[8, 32:64] *= np.float32(1e-4)
    q, d = _quant_gpu(cuda, pkg._lib.load().gs_quant_q8_rows, x)
    wq, wd = oracle.quant_q8_rows(x)
    assert np.array_equal(q, wq)
    assert np.array_equal(d.view(np.uint16), wd.view(np.uint16))


@pytest.mark.parametrize("T,H,n,splits,dense", [
    (1, 64, 4096, 16, True), (2, 64, 1500, 4, True), (1, 32, 2052, 16, False), (5, 16, 300, 1, False),
    (1, 16, 0, 16, True), (2, 64, 33, 4, False), (200, 64, 130, 1, False), (8, 48, 515, 4, False), (3, 96, 65, 2, False),
])
def test_gs_mla_attn_q8_cache_vs_oracle(pkg, cuda, oracle, T, H, n, splits, dense):
    q, Cc, sel, cnt = _legacy_inputs(T * 77 + n, T, H, n, max(n, 1) + 100, dense)
    cq, cs = oracle.quant_q8_rows(Cc.astype(np.float32))
    L = pkg._lib.load()
    got = _call(cuda, L.gs_mla_attn, q, cq, sel, cnt, splits, scales=cs)
    # the oracle attends over exactly the f16 rows the kernels rebuild from (q, scale)
    want = oracle.mla_attn_ref(q, oracle.dequant_q8(cq, cs), sel, cnt, 1 / 16)
    check_close(got, want, "gs_mla_attn q8")  # the automatic choice: the tcgen05 kernel, queries rounded to f16
    with _Impl(L, 1):
        slow = _call(cuda, L.gs_mla_attn, q, cq, sel, cnt, splits, scales=cs)
    check_close(slow, want, "gs_mla_attn q8, CUDA-core kernel", 2e-5, 2e-6)
    with _Impl(L, 2):
        fast = _call(cuda, L.gs_mla_attn, q, cq, sel, cnt, splits, scales=cs)
    assert np.array_equal(fast, got), "the automatic choice takes the tcgen05 kernel for a Q8 cache too"
    st = C.c_int32(-1)
    assert L.gs_mla_attn_status(C.byref(st), None) == 0 and st.value == 0
    if n > 8:
        check_not_degenerate(got[-1], "gs_mla_attn q8")


def test_q8_append_then_attend_round_trip(pkg, cuda, oracle):
    # Engine::mla with a Q8 cache (forward.rs:852-856): quantise the new f32 rows on the device, attend over them
    T, H, n = 1, 64, 1024
    q, Cc, sel, cnt = _legacy_inputs(5, T, H, n, n, True)
    L = pkg._lib.load()
    cq, cs = _quant_gpu(cuda, L.gs_quant_q8_rows, Cc.astype(np.float32))
    got = _call(cuda, L.gs_mla_attn, q, cq, sel, cnt, 16, scales=cs)
    want_q8 = oracle.mla_attn_ref(q, oracle.dequant_q8(cq, cs), sel, cnt, 1 / 16)
    check_close(got, want_q8, "q8 append + attend")
    # and the quantisation itself stays a small perturbation of the f16-cache result
    want_f16 = oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16)
    assert np.abs(got - want_f16).max() < 5e-2


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="reference kernels were not compiled (oracle/_ref absent)")
def test_reference_q8_kernels_pin_oracle(pkg, cuda, oracle):
    ref = C.CDLL(REF_SO)
    ref.gs_mla_attn.restype = C.c_int
    ref.gs_mla_attn.argtypes = pkg._lib.SIGNATURES["gs_mla_attn"][1]
    ref.gs_quant_q8_rows.restype = C.c_int
    ref.gs_quant_q8_rows.argtypes = pkg._lib.SIGNATURES["gs_quant_q8_rows"][1]
    rng = np.random.default_rng(31)
    x = rng.standard_normal((257, 512)).astype(np.float32)
    rq, rd = _quant_gpu(cuda, ref.gs_quant_q8_rows, x)
    oq, od = oracle.quant_q8_rows(x)
    # the reference is built with fast-math (approximate reciprocal and division): the scale may differ by one f16
    # ulp and a value that sits on a rounding boundary by one step; everything else must be identical
    assert np.abs(rq.astype(np.int32) - oq.astype(np.int32)).max() <= 1
    assert (rq != oq).mean() < 1e-3
    assert np.abs(rd.view(np.uint16).astype(np.int32) - od.view(np.uint16).astype(np.int32)).max() <= 1
    # attention over the same (q, scale) bytes: reference kernel, oracle and the new kernel agree
    T, H, n = 2, 32, 200
    q, _, sel, cnt = _legacy_inputs(9, T, H, n, 257, False)
    o_ref = _call(cuda, ref.gs_mla_attn, q, oq, sel, cnt, 4, scales=od)
    o_orc = oracle.mla_attn_ref(q, oracle.dequant_q8(oq, od), sel, cnt, 1 / 16)
    L = pkg._lib.load()
    with _Impl(L, 1):
        o_new = _call(cuda, L.gs_mla_attn, q, oq, sel, cnt, 4, scales=od)
    o_tc = _call(cuda, L.gs_mla_attn, q, oq, sel, cnt, 4, scales=od)
    check_close(o_orc, o_ref, "oracle vs reference kernel (q8)", 2e-5, 2e-6)
    check_close(o_new, o_ref, "CUDA-core kernel vs reference kernel (q8)", 2e-5, 2e-6)
    check_close(o_tc, o_ref, "tcgen05 kernel vs reference kernel (q8)")


# ---- kernel choice of gs_mla_attn: tcgen05 kernel by default for f16 caches, CUDA-core kernel as the second opinion ----

@pytest.mark.parametrize("T,H,n,dense,splits", [
    (1, 64, 2052, False, 16), (2, 64, 2052, False, 4), (1, 32, 700, False, 16), (4, 16, 33, False, 4),
    (1, 64, 0, True, 16), (2, 48, 1, True, 4), (3, 64, 1000, True, 4), (40, 64, 300, False, 4), (256, 16, 70, False, 1),
    (9, 80, 130, False, 1), (1, 16, 2052, False, 1), (8, 64, 515, False, 4), (2, 96, 64, True, 4), (5, 64, 63, False, 1),
    # 64 heads in one pass (64 query columns, two issuing warps): taken when it shortens the longest run of tiles
    (80, 64, 130, False, 1), (150, 64, 70, True, 1), (30, 64, 1000, False, 8), (256, 64, 200, False, 1),
])
def test_gs_mla_attn_tensor_kernel_vs_oracle_and_cuda_core_kernel(pkg, cuda, oracle, T, H, n, dense, splits):
    """The same call on both kernels: the CUDA-core kernel (f32 queries) and the tcgen05 kernel fed from the position
    lists by gather copies (queries rounded to f16 in the kernel).  splits > 1: records in `part`; splits == 1 or a
    `part` too small for enough records: one CTA per (token, head group) that stores o itself."""
    q, Cc, sel, cnt = _legacy_inputs(T * 31 + n + H, T, H, n, max(n, 1) + 3000, dense)
    L = pkg._lib.load()
    with _Impl(L, 1):
        slow = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
    with _Impl(L, 2):
        fast = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
    st = C.c_int32(-1)
    assert L.gs_mla_attn_status(C.byref(st), None) == 0 and st.value == 0
    auto = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
    want = oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16)
    check_close(slow, want, "CUDA-core kernel", 2e-5, 2e-6)
    check_close(fast, want, "tcgen05 kernel")  # f16-rounded queries: the tolerance of the f16-query entry points
    assert np.array_equal(auto, fast), "the automatic choice takes the tcgen05 kernel for an f16 cache"
    if n > 8:
        check_not_degenerate(fast[-1], "tcgen05 kernel")


def test_gs_mla_attn_lists_with_scattered_unsorted_and_repeated_rows(pkg, cuda, oracle):
    """Position lists are arbitrary: unsorted, with repeats, not in groups of four, different lengths per token."""
    rng = np.random.default_rng(5)
    T, H, ctx = 3, 32, 5000
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    Cc = (rng.standard_normal((ctx, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    cnt = np.array([777, 1, 130], np.int32)
    sel = rng.integers(0, ctx, size=(T, 800)).astype(np.int32)
    sel[0, 5:9] = sel[0, 4]  # one row named five times
    L = pkg._lib.load()
    for splits in (1, 4):
        with _Impl(L, 2):
            got = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, splits)
        check_close(got, oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16), f"lists with repeats, splits {splits}")


def test_gs_mla_attn_kernel_choice_limits(pkg, cuda, oracle):
    L = pkg._lib.load()
    # 128 heads (not cut into groups of 8..48) stay on the CUDA-core kernel: exact against the oracle
    q, Cc, sel, cnt = _legacy_inputs(3, 1, 128, 100, 150, False)
    got = _call(cuda, L.gs_mla_attn, q, Cc, sel, cnt, 4)
    check_close(got, oracle.mla_attn_ref(q, Cc, sel, cnt, 1 / 16), "128 heads", 2e-5, 2e-6)
    with _Impl(L, 2):
        T, H, R = q.shape
        o = cuda.zeros((T, H, R), dtype=cuda.float32, device="cuda")
        part = cuda.zeros(T * H * 4 * (R + 2), dtype=cuda.float32, device="cuda")
        qd, cd, sd, nd = to_dev(cuda, q), to_dev(cuda, Cc), to_dev(cuda, sel), to_dev(cuda, cnt)
        rc = L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel.shape[1],
                           nd.data_ptr(), 1 / 16, o.data_ptr(), part.data_ptr(), T, H, R, 4, None)
        assert rc == 1  # cudaErrorInvalidValue: the tcgen05 kernel was demanded and does not take 128 heads
    assert L.gs_mla_attn_set_impl(3) == 1
