"""GPU parity of causal prefill attention and of the fused RoPE + KV-append, through the C ABI."""
import numpy as np
import pytest

from conftest import check_close, check_not_degenerate
from gpu_util import paged_layout, to_dev

pytestmark = pytest.mark.gpu


def _qkv(seed, S, H, d, p0=0):
    rng = np.random.default_rng(seed)
    mk = lambda n: rng.standard_normal((n, H, d), dtype=np.float32).astype(np.float16)
    return mk(S), mk(p0 + S), mk(p0 + S)


@pytest.mark.parametrize("impl", [1, 0])
@pytest.mark.parametrize("S,H,p0", [(1, 2, 0), (31, 3, 0), (128, 2, 0), (129, 2, 0), (1024, 20, 0), (300, 4, 77), (256, 2, 256)])
def test_prefill_vs_oracle(pkg, cuda, oracle, impl, S, H, p0):
    Q, K, V = _qkv(S + p0, S, H, 256, p0)
    got = pkg.prefill_attn(to_dev(cuda, Q), to_dev(cuda, K), to_dev(cuda, V), p0=p0, impl=impl)
    cuda.cuda.synchronize()
    want = oracle.prefill(Q, K, V, 1 / 16, p0=p0)
    check_close(got.cpu().numpy(), want, f"prefill S={S} p0={p0} impl={impl}")
    if S > 8:
        check_not_degenerate(got.cpu().numpy())


def test_config4_prefill_8192_with_rope(pkg, cuda, oracle):
    # 8192-token chunk, 20 heads, d = 256 (192 nope + 64 rope), RoPE base 10000 on the last 64 dims
    S, H, d = 8192, 20, 256
    Q, K, V = _qkv(4, S, H, d)
    Qd, Kd, Vd = to_dev(cuda, Q), to_dev(cuda, K), to_dev(cuda, V)
    pkg.rope_f16_inplace(Qd)
    pkg.rope_f16_inplace(Kd)
    got = pkg.prefill_attn(Qd, Kd, Vd)
    cuda.cuda.synchronize()
    Qr, Kr = oracle.rope_f16(Q), oracle.rope_f16(K)
    # the device RoPE agrees with the oracle's to one f16 ulp on a few elements at most
    dq = np.abs(Qd.cpu().numpy().astype(np.float32) - Qr.astype(np.float32))
    assert dq.max() <= 4e-3 and (dq > 0).mean() < 1e-2
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([np.arange(128), np.arange(S - 128, S), rng.integers(0, S, 256)])).astype(np.int32)
    # score the oracle on the device-rotated inputs so only the attention is compared here
    want = oracle.prefill(Qd.cpu().numpy(), Kd.cpu().numpy(), V, 1 / 16, rows=rows)
    check_close(got.cpu().numpy()[rows], want, "config 4 (row subset)")
    # linearity in V: attention(V1 + V2) = attention(V1) + attention(V2), a size-independent property
    V2 = np.ascontiguousarray(V[::-1])
    o2 = pkg.prefill_attn(Qd, Kd, to_dev(cuda, V2))
    o12 = pkg.prefill_attn(Qd, Kd, to_dev(cuda, (V.astype(np.float32) + V2.astype(np.float32)).astype(np.float16)))
    cuda.cuda.synchronize()
    check_close(o12.cpu().numpy(), (got + o2).cpu().numpy(), "linearity in V", 4e-3, 4e-4)


def test_prefill_run_to_run_bit_stable(pkg, cuda):
    # many key tiles per query block: any unordered reuse of tensor memory shows up as run-to-run differences
    Q, K, V = _qkv(6, 4096, 8, 256)
    Qd, Kd, Vd = to_dev(cuda, Q), to_dev(cuda, K), to_dev(cuda, V)
    first = pkg.prefill_attn(Qd, Kd, Vd).clone()
    for _ in range(8):
        again = pkg.prefill_attn(Qd, Kd, Vd)
        cuda.cuda.synchronize()
        assert cuda.equal(first, again)


def test_prefill_f16_output(pkg, cuda, oracle):
    Q, K, V = _qkv(5, 200, 4, 256)
    got = pkg.prefill_attn(to_dev(cuda, Q), to_dev(cuda, K), to_dev(cuda, V), out_f16=True)
    cuda.cuda.synchronize()
    check_close(got.float().cpu().numpy(), oracle.prefill(Q, K, V, 1 / 16), "f16 out", 3e-3, 4e-4)


@pytest.mark.parametrize("pos0", [0, 1, 4095, 32766, 131070])
def test_rope_append_at(pkg, cuda, oracle, pos0):
    rng = np.random.default_rng(pos0)
    T = 2
    kv = rng.standard_normal((T, 576), dtype=np.float32)
    cache = cuda.zeros((pos0 + T + 1, 576), dtype=cuda.float16, device="cuda")
    pkg.rope_kv_append_at(to_dev(cuda, kv), cache, pos0)
    cuda.cuda.synchronize()
    got = cache.cpu().numpy()
    want = oracle.rope_append(kv, pos0)
    # the unrotated 512 columns are bit-exact; the rotated ones to one f16 ulp (device sincosf vs libm)
    assert np.array_equal(got[pos0:pos0 + T, :512].view(np.uint16), want[:, :512].view(np.uint16))
    d = np.abs(got[pos0:pos0 + T, 512:].astype(np.float32) - want[:, 512:].astype(np.float32))
    assert d.max() <= 4e-3 and (d > 0).mean() < 0.02
    assert (got[pos0 + T] == 0).all() and (pos0 == 0 or (got[pos0 - 1] == 0).all())


def test_plain_append_equals_reference_append(pkg, cuda, oracle):
    # d_rope = 0 is the reference's append: bit-exact half_rn
    rng = np.random.default_rng(3)
    kv = rng.standard_normal((3, 512), dtype=np.float32)
    cache = cuda.zeros((10, 512), dtype=cuda.float16, device="cuda")
    pkg.rope_kv_append_at(to_dev(cuda, kv), cache, 4, d_rope=0)
    cuda.cuda.synchronize()
    assert np.array_equal(cache.cpu().numpy()[4:7].view(np.uint16), oracle.f32_to_f16(kv).view(np.uint16))


def test_rope_append_batched_paged(pkg, cuda, oracle):
    rng = np.random.default_rng(12)
    lens = np.array([63, 64, 130, 0], np.int32)  # position of the first new row of each sequence
    T = 2
    pool, pt = paged_layout(rng, lens + T, spare_pages=1)
    pool[:] = 0
    kv = rng.standard_normal((len(lens), T, 576), dtype=np.float32)
    pd = to_dev(cuda, pool)
    pkg.rope_kv_append(to_dev(cuda, kv), pd, to_dev(cuda, lens), page_table=to_dev(cuda, pt))
    cuda.cuda.synchronize()
    got = pd.cpu().numpy()
    written = np.zeros(pool.shape[0], bool)
    for b, p0 in enumerate(lens):
        want = oracle.rope_append(kv[b], int(p0))
        for t in range(T):
            pos = int(p0) + t
            row = pt[b, pos // 64] * 64 + pos % 64
            written[row] = True
            assert np.array_equal(got[row, :512].view(np.uint16), want[t, :512].view(np.uint16))
            assert np.abs(got[row, 512:].astype(np.float32) - want[t, 512:].astype(np.float32)).max() <= 4e-3
    assert (got[~written] == 0).all()


def test_decode_layer_step_matches_oracle(pkg, cuda, oracle):
    """The call-site mirror: append then attend, host buffers in and out (the e2e path)."""
    rng = np.random.default_rng(21)
    H = 20
    layer = pkg.MlaDecodeLayer(ctx=600, H=H)
    ref_cache = np.zeros((600, 576), np.float16)
    pos = 0
    for T in (2, 1, 2, 2, 1):
        q = cuda.from_numpy(rng.standard_normal((T, H, 576), dtype=np.float32).astype(np.float16)).pin_memory()
        kv = cuda.from_numpy(rng.standard_normal((T, 576), dtype=np.float32) * np.float32(0.5)).pin_memory()
        o = layer.step(q, kv).numpy().copy()
        ref_cache[pos:pos + T] = oracle.rope_append(kv.numpy(), pos)
        pos += T
        want = oracle.mla_decode(q.numpy()[None], ref_cache, [pos], 1 / 16)[0]
        check_close(o, want, f"step pos={pos}", 4e-3, 4e-4)
    layer.rollback(1)
    assert layer.pos == pos - 1


def test_decode_layer_graph_step_matches_eager_and_oracle(pkg, cuda, oracle):
    """The same step replayed from a CUDA graph with the position kept on the device: equal to the eager
    step bit for bit, right against the oracle, and a moved-back position (rejected draft) is honoured."""
    rng = np.random.default_rng(22)
    H, ctx = 20, 700
    eager = pkg.MlaDecodeLayer(ctx=ctx, H=H)
    graph = pkg.MlaDecodeLayer(ctx=ctx, H=H, use_graph=True)
    bufs = {T: (cuda.empty((T, H, 576), dtype=cuda.float16).pin_memory(), cuda.empty((T, 576), dtype=cuda.float32).pin_memory())
            for T in (1, 2)}
    ref_cache = np.zeros((ctx, 576), np.float16)
    pos = 0
    for i, T in enumerate((2, 2, 1, 2, 1, 1, 2)):
        q = rng.standard_normal((T, H, 576), dtype=np.float32).astype(np.float16)
        kv = rng.standard_normal((T, 576), dtype=np.float32) * np.float32(0.5)
        qh, kvh = bufs[T]
        qh.copy_(cuda.from_numpy(q))
        kvh.copy_(cuda.from_numpy(kv))
        o_g = graph.step(qh, kvh).numpy().copy()
        o_e = eager.step(qh, kvh).numpy().copy()
        assert np.array_equal(o_g, o_e), f"graph and eager step differ at step {i}"
        ref_cache[pos:pos + T] = oracle.rope_append(kv, pos)
        pos += T
        check_close(o_g, oracle.mla_decode(q[None], ref_cache, [pos], 1 / 16)[0], f"graph step pos={pos}", 4e-3, 4e-4)
        if i == 3:  # the second token of this draft is rejected
            graph.rollback(1)
            eager.rollback(1)
            pos -= 1
    assert graph.pos == eager.pos == pos
    assert len(graph._graphs) == 2  # one graph per T
    assert pkg.decode_status(graph.workspace) == 0


def test_decode_layer_graph_refuses_to_run_past_the_cache(pkg, cuda):
    H, ctx = 20, 64
    layer = pkg.MlaDecodeLayer(ctx=ctx, H=H, T_max=2, use_graph=True)
    qh = cuda.zeros((2, H, 576), dtype=cuda.float16).pin_memory()
    kvh = cuda.ones((2, 576), dtype=cuda.float32).pin_memory()
    layer.pos = ctx - 2
    layer.step(qh, kvh)  # records the graph; the last two rows fit
    layer.pos = ctx - 1
    with pytest.raises(RuntimeError, match="context full"):
        layer.step(qh, kvh)
    h = next(iter(layer._graphs.values()))
    L = pkg._lib.load()
    assert L.gs_mla_layer_graph_step(h, ctx - 1, layer._graph_stream.cuda_stream, 1) != 0
    assert b"context full" in L.gs_attn_last_error_string()
    assert L.gs_mla_layer_graph_step(None, 0, layer._graph_stream.cuda_stream, 1) != 0


@pytest.mark.parametrize("d_row,d_rope,with_w", [(576, 64, True), (512, 0, True), (576, 64, False), (128, 32, True)])
def test_norm_rope_append_vs_oracle(pkg, cuda, oracle, d_row, d_rope, with_w):
    rng = np.random.default_rng(d_row + d_rope)
    T, pos0 = 3, 41
    x = rng.standard_normal((T, d_row)).astype(np.float32) * np.float32(3.0)
    w = (1.0 + 0.2 * rng.standard_normal(d_row - d_rope)).astype(np.float32) if with_w else None
    cache = cuda.zeros((pos0 + T + 2, d_row), dtype=cuda.float16, device="cuda")
    pkg.norm_rope_kv_append_at(cuda.from_numpy(x).cuda(), cache, pos0, weight=None if w is None else cuda.from_numpy(w).cuda(),
                               eps=1e-6, d_rope=d_rope)
    cuda.cuda.synchronize()
    got = cache.cpu().numpy()
    want = oracle.norm_rope_append(x, pos0, weight=w, eps=1e-6, d_rope=d_rope)
    assert (got[:pos0] == 0).all() and (got[pos0 + T:] == 0).all()
    g, v = got[pos0:pos0 + T].astype(np.float32), want.astype(np.float32)
    # the sum of squares is added up in another order than the oracle's: at most one f16 step apart
    ulp = np.maximum(np.abs(v), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(g - v) <= ulp + 4e-3 * (np.arange(d_row) >= d_row - d_rope))


def test_checked_append_skips_what_is_out_of_range_and_flags_it(pkg, cuda, oracle):
    """gs_rope_kv_append_checked: a position beyond the sequence's page-table row, a page id outside the pool and a
    negative position write nothing and set bit 17 of the status word; the other rows land as with the plain call."""
    import ctypes as C
    rng = np.random.default_rng(13)
    T, stride = 2, 3
    pos0 = np.array([10, 3 * 64 - 1, -1, 64], np.int32)  # ok | second row falls off the table row | negative | bad page id
    n_pages = 8
    pt = np.array([[0, 1, 2], [3, 4, 5], [6, 6, 6], [7, 9999, 7]], np.int32)
    pool = np.zeros((n_pages * 64, 576), np.float16)
    kv = rng.standard_normal((len(pos0), T, 576), dtype=np.float32)
    pd, st = to_dev(cuda, pool), cuda.zeros(1, dtype=cuda.int32, device="cuda")
    kvd, posd, ptd = to_dev(cuda, kv), to_dev(cuda, pos0), to_dev(cuda, pt)  # held until the call has run
    L = pkg._lib.load()
    rc = L.gs_rope_kv_append_checked(kvd.data_ptr(), pd.data_ptr(), pool.shape[0], posd.data_ptr(), None,
                                     ptd.data_ptr(), stride, 64, len(pos0), T, 576, 64, 10000.0, st.data_ptr(), None)
    assert rc == 0, L.gs_attn_last_error_string()
    cuda.cuda.synchronize()
    assert int(st.item()) == 1 << 17
    got = pd.cpu().numpy()
    written = np.zeros(pool.shape[0], bool)
    for b, t in ((0, 0), (0, 1), (1, 0), (2, 1)):  # the rows that are in range (sequence 2's second row is position 0)
        pos = int(pos0[b]) + t
        row = pt[b, pos // 64] * 64 + pos % 64
        written[row] = True
        want = oracle.rope_append(kv[b], int(pos0[b]))[t]
        assert np.array_equal(got[row, :512].view(np.uint16), want[:512].view(np.uint16))
    assert (got[~written] == 0).all()
    st2 = C.c_int32(0)
    assert L.gs_mla_decode_status(st.data_ptr(), C.byref(st2), None) != 0 and st2.value == 1 << 17


def test_prefill_checked_leaves_status_clear(pkg, cuda, oracle):
    Q, K, V = _qkv(5, 300, 2, 256)
    o = cuda.zeros((300, 2, 256), dtype=cuda.float32, device="cuda")
    st = cuda.zeros(1, dtype=cuda.int32, device="cuda")
    L = pkg._lib.load()
    Qd, Kd, Vd = to_dev(cuda, Q), to_dev(cuda, K), to_dev(cuda, V)  # held until the call has run
    rc = L.gs_prefill_attn_checked(Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), o.data_ptr(), 0,
                                   300, 2, 256, 0, 1 / 16, 2, st.data_ptr(), None)
    assert rc == 0, L.gs_attn_last_error_string()
    cuda.cuda.synchronize()
    assert int(st.item()) == 0
    check_close(o.cpu().numpy(), oracle.prefill(Q, K, V, 1 / 16), "prefill (checked entry)")
    assert L.gs_prefill_attn_checked(None, None, None, None, 0, 300, 2, 256, 0, 1 / 16, 2, None, None) == 1
