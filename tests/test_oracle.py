"""CPU tests of the oracle: the reference's own pin (f16 round trip), float64 numpy cross-checks,
split/combine algebra, RoPE, and the committed golden vectors."""
import glob
import os

import numpy as np
import pytest

from conftest import check_close

HERE = os.path.dirname(os.path.abspath(__file__))


def test_f16_roundtrip_all_values(oracle):
    # the reference's test: crates/quants/src/lib.rs:361-370
    h = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_to_f32(h.view(np.float16))
    keep = ~np.isnan(f)
    back = oracle.f32_to_f16(f[keep]).view(np.uint16)
    assert np.array_equal(back, h[keep])
    ref = h.view(np.float16).astype(np.float32)
    assert np.array_equal(f[keep], ref[keep])


def test_f32_to_f16_rne_matches_numpy(oracle):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * s for s in (1e-8, 1e-4, 1.0, 300.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 5.96e-8, 2.98e-8], np.float32)])
    assert np.array_equal(oracle.f32_to_f16(x).view(np.uint16), x.astype(np.float16).view(np.uint16))


def _numpy_attend(q, K, V, scale):
    s = (q.astype(np.float64) @ K.astype(np.float64).T) * scale
    if s.shape[-1] == 0:
        return np.zeros((q.shape[0], V.shape[1]))
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return p @ V.astype(np.float64)


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 63, 64, 65, 1000])
def test_ref_abi_attention_vs_numpy(oracle, n):
    rng = np.random.default_rng(n)
    T, H, R, ctx = 3, 16, 512, max(n, 1) + 40
    q = rng.standard_normal((T, H, R)).astype(np.float32)
    C = (rng.standard_normal((ctx, R)) * 0.5).astype(np.float16)
    stride = n + 5
    sel = np.zeros((T, stride), np.int32)
    cnt = np.zeros(T, np.int32)
    for t in range(T):
        k = max(0, n - t)
        cnt[t] = k
        sel[t, :k] = rng.permutation(ctx)[:k]
    o = oracle.mla_attn_ref(q, C, sel, cnt, 1 / 16)
    for t in range(T):
        want = _numpy_attend(q[t], C[sel[t, :cnt[t]]], C[sel[t, :cnt[t]]], 1 / 16)
        check_close(o[t], want, f"t={t}", 1e-5, 1e-6)


@pytest.mark.parametrize("T", [1, 2, 3])
def test_decode_dense_and_paged_agree(oracle, T):
    rng = np.random.default_rng(11 + T)
    H, n_seq = 5, 3
    lens = np.array([130, 64, 7], np.int32)
    q = rng.standard_normal((n_seq, T, H, 576)).astype(np.float16)
    n_pages = int(sum(-(-l // 64) for l in lens)) + 2
    pool = (rng.standard_normal((n_pages * 64, 576)) * 0.5).astype(np.float16)
    perm = rng.permutation(n_pages)
    pt = np.zeros((n_seq, 4), np.int32)
    k = 0
    dense = np.zeros((int(lens.sum()), 576), np.float16)
    base = np.zeros(n_seq, np.int32)
    off = 0
    for b in range(n_seq):
        base[b] = off
        for j in range(-(-int(lens[b]) // 64)):
            pt[b, j] = perm[k]
            k += 1
            rows = min(64, lens[b] - 64 * j)
            dense[off + 64 * j: off + 64 * j + rows] = pool[pt[b, j] * 64: pt[b, j] * 64 + rows]
        off += int(lens[b])
    o_paged = oracle.mla_decode(q, pool, lens, 1 / 16, page_table=pt)
    o_dense = oracle.mla_decode(q, dense, lens, 1 / 16, seq_base=base)
    assert np.array_equal(o_paged, o_dense)
    for b in range(n_seq):
        for t in range(T):
            n = max(0, lens[b] - (T - 1 - t))
            rows = dense[base[b]: base[b] + n]
            want = _numpy_attend(q[b, t], rows, rows[:, :512], 1 / 16)
            check_close(o_dense[b, t], want, f"b={b} t={t}", 1e-5, 1e-6)


def test_partials_combine_to_full(oracle):
    # the split/combine algebra of crates/cuda/kernels/ops.cu:539-574, with shards as splits
    rng = np.random.default_rng(5)
    n, H, T = 1000, 4, 2
    q = rng.standard_normal((1, T, H, 576)).astype(np.float16)
    cache = (rng.standard_normal((n, 576)) * 0.5).astype(np.float16)
    full = oracle.mla_decode(q, cache, [n], 1 / 16)
    for G in (1, 2, 3, 8, 16):
        per = -(-n // G)
        recs = [oracle.mla_decode(q, cache, [n], 1 / 16, part_range=(g * per, min(n, (g + 1) * per))) for g in range(G)]
        # an empty shard has m = -inf, l = 0 and must be ignored
        recs.append(oracle.mla_decode(q, cache, [n], 1 / 16, part_range=(n, n)))
        parts = np.stack([r.reshape(T * H, 514) for r in recs], axis=1)
        assert np.isneginf(parts[:, -1, 512]).all() and (parts[:, -1, 513] == 0).all()
        o = oracle.combine(parts).reshape(1, T, H, 512)
        check_close(o, full, f"G={G}", 1e-5, 1e-6)


def test_prefill_vs_numpy(oracle):
    rng = np.random.default_rng(8)
    S, H, d, p0 = 70, 3, 256, 9
    Q = rng.standard_normal((S, H, d)).astype(np.float16)
    K = rng.standard_normal((p0 + S, H, d)).astype(np.float16)
    V = rng.standard_normal((p0 + S, H, d)).astype(np.float16)
    o = oracle.prefill(Q, K, V, 1 / 16, p0=p0)
    for h in range(H):
        for i in (0, 1, 33, 69):
            want = _numpy_attend(Q[i:i + 1, h], K[:p0 + i + 1, h], V[:p0 + i + 1, h], 1 / 16)
            check_close(o[i, h][None], want, f"h={h} i={i}", 1e-5, 1e-6)
    sub = oracle.prefill(Q, K, V, 1 / 16, p0=p0, rows=[5, 69])
    assert np.array_equal(sub[0], o[5]) and np.array_equal(sub[1], o[69])


def test_rope_append_matches_float64(oracle):
    rng = np.random.default_rng(2)
    T, d_row, d_rope = 5, 576, 64
    x = rng.standard_normal((T, d_row)).astype(np.float32)
    for pos0 in (0, 1, 4097, 131000):
        y = oracle.rope_append(x, pos0).astype(np.float64)
        want = x.astype(np.float64).copy()
        i = np.arange(d_rope // 2)
        inv = 10000.0 ** (-2.0 * i / d_rope)
        for t in range(T):
            ang = (pos0 + t) * inv
            a, b = x[t, 512::2].astype(np.float64), x[t, 513::2].astype(np.float64)
            want[t, 512::2] = a * np.cos(ang) - b * np.sin(ang)
            want[t, 513::2] = a * np.sin(ang) + b * np.cos(ang)
        assert np.array_equal(y[:, :512], x[:, :512].astype(np.float16).astype(np.float64))
        # f32 angle at positions ~1e5 carries ~1e-2 * 2^-24 * 1e5 absolute angle error; allow f16-level slack
        assert np.abs(y - want).max() < 2e-2
    # position 0 is the identity rotation: bit-exact f16 rounding of the input
    assert np.array_equal(oracle.rope_append(x, 0)[0], x[0].astype(np.float16))


def test_rope_f16_norm_preserving(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((9, 2, 256)).astype(np.float16)
    y = oracle.rope_f16(x, pos0=100)
    assert np.array_equal(y[..., :192], x[..., :192])
    n0 = (x[..., 192:].astype(np.float64) ** 2).reshape(9, 2, 32, 2).sum(-1)
    n1 = (y[..., 192:].astype(np.float64) ** 2).reshape(9, 2, 32, 2).sum(-1)
    assert np.abs(n0 - n1).max() < 2e-2


def test_golden_vectors_from_reference_kernel(oracle):
    """Outputs of the reference's own CUDA kernel (gs_mla_attn / gs_f32_to_f16 compiled unmodified and
    run on a B200) pin the oracle.  The fixtures are made by tests/golden/make_golden_from_ref.py."""
    files = sorted(glob.glob(os.path.join(HERE, "golden", "ref_*.npz")))
    if not files:
        pytest.skip("no golden fixtures committed yet")
    for f in files:
        z = np.load(f)
        if "append_x" in z:
            assert np.array_equal(oracle.f32_to_f16(z["append_x"]).view(np.uint16), z["append_y"])
        o = oracle.mla_attn_ref(z["q"], z["C"].view(np.float16), z["sel"], z["cnt"], float(z["scale"]))
        # the reference kernel is built with fast-math (__expf) and sums in tiles of 32
        check_close(o, z["o"], os.path.basename(f), 2e-5, 2e-6)


def test_quant_q8_rows_matches_numpy_restatement(oracle):
    # crates/cuda/kernels/ops.cu:599-610: d = amax / 127 (kept as f16), q = round-to-nearest-even(x * (1 / d))
    rng = np.random.default_rng(11)
    x = rng.standard_normal((37, 512)).astype(np.float32) * np.float32(3.0)
    x[5] = 0.0                       # an all-zero block keeps q = 0, d = 0
    x[6, :32] = np.float32(1e-30)    # amax / 127 underflows towards a subnormal scale
    q, d = oracle.quant_q8_rows(x)
    xb = x.reshape(-1, 32)
    dd = (np.abs(xb).max(axis=1) / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
        inv = np.where(dd > 0, np.float32(1.0) / dd, np.float32(0.0)).astype(np.float32)
        want_q = np.clip(np.rint(xb * inv[:, None]), -128, 127).astype(np.int8)
    ok = np.isfinite(inv)
    assert np.array_equal(q.reshape(-1, 32)[ok], want_q[ok])
    assert np.array_equal(d.reshape(-1).view(np.uint16), dd.astype(np.float16).view(np.uint16))
    assert np.abs(q).max() == 127 and not q[5].any() and not d[5].any()


def test_dequant_q8_is_half_of_scale_times_q(oracle):
    rng = np.random.default_rng(12)
    q = rng.integers(-127, 128, size=(9, 512), dtype=np.int8)
    d = (rng.random((9, 16), dtype=np.float32) * np.float32(0.05)).astype(np.float16)
    got = oracle.dequant_q8(q, d)
    want = (np.repeat(d.astype(np.float32), 32, axis=1) * q.astype(np.float32)).astype(np.float16)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_q8_round_trip_error_is_half_a_step(oracle):
    rng = np.random.default_rng(13)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    q, d = oracle.quant_q8_rows(x)
    back = oracle.dequant_q8(q, d).astype(np.float32)
    step = np.repeat(d.astype(np.float32), 32, axis=1)
    assert np.all(np.abs(back - x) <= 0.5 * step * 1.01 + 2e-3 * np.abs(x))


def test_q8_golden_vectors_from_reference_kernels(oracle):
    """Outputs of the reference's own Q8 quantiser and Q8 attention branch (compiled unmodified, run on a B200) pin
    the oracle's Q8 functions.  The reference is built with fast-math: its scale may differ by one f16 ulp and a value
    on a rounding boundary by one step; the attention is compared over the reference's own (q8, scale) bytes."""
    path = os.path.join(HERE, "golden", "refq8_cache.npz")
    if not os.path.exists(path):
        pytest.skip("no Q8 golden fixture committed yet")
    g = np.load(path)
    oq, od = oracle.quant_q8_rows(g["x"])
    assert np.abs(oq.astype(np.int32) - g["q8"].astype(np.int32)).max() <= 1
    assert (oq != g["q8"]).mean() < 1e-3
    assert np.abs(od.view(np.uint16).astype(np.int32) - g["d"].astype(np.int32)).max() <= 1
    rows = oracle.dequant_q8(g["q8"], g["d"].view(np.float16))
    o = oracle.mla_attn_ref(g["q"], rows, g["sel"], g["cnt"], float(g["scale"]))
    check_close(o, g["o"], "oracle vs reference Q8 attention", 2e-5, 2e-6)


def test_norm_rope_append_matches_float64_numpy(oracle):
    rng = np.random.default_rng(41)
    x = rng.standard_normal((5, 576)).astype(np.float32) * np.float32(2.0)
    w = (1.0 + 0.1 * rng.standard_normal(512)).astype(np.float32)
    got = oracle.norm_rope_append(x, 100, weight=w, eps=1e-6).astype(np.float64)
    lat = x[:, :512].astype(np.float64)
    want_lat = lat / np.sqrt((lat ** 2).mean(1, keepdims=True) + 1e-6) * w
    assert np.abs(got[:, :512] - want_lat).max() <= 2e-3 * np.abs(want_lat).max()
    # the rotated columns are those of the plain RoPE append
    plain = oracle.rope_append(x, 100).astype(np.float64)
    assert np.array_equal(got[:, 512:], plain[:, 512:])


def test_decode_cut_into_key_ranges_equals_the_plain_decode(oracle):
    """oracle_mla_decode_split (every row's attended range cut by the reference's split rule, ops.cu:447-449, and
    merged by its combine arithmetic, ops.cu:558-573) against the single-pass decode: same result to rounding."""
    rng = np.random.default_rng(17)
    for n, T, ks in ((1000, 2, 7), (64, 1, 3), (5, 2, 8), (0, 1, 4)):
        q = rng.standard_normal((1, T, 3, 576), dtype=np.float32).astype(np.float16)
        cache = (rng.standard_normal((max(n, 1), 576), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
        a = oracle.mla_decode(q, cache, [n], 1 / 16)
        b = oracle.mla_decode(q, cache, [n], 1 / 16, key_splits=ks)
        assert np.abs(a - b).max() <= 2e-6, (n, T, ks, np.abs(a - b).max())


def test_key_range_decode_on_ragged_paged_batches_and_odd_row_counts(oracle):
    """The key-range form walks blocks of 32 keys with four query rows at a time: row counts that are no multiple of
    four, empty and short sequences, pages out of order and ranges that end inside a block must all agree with the
    single-pass decode, and with float64 numpy on the dense case."""
    rng = np.random.default_rng(23)
    lens = [100, 0, 777, 33]
    pt = np.array([[3, 1] + [0] * 11, [0] * 13, list(range(2, 15)), [15] + [0] * 12], np.int32)
    cache = (rng.standard_normal((16 * 64, 576), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    for T, Hh, ks in ((2, 4, 5), (3, 5, 2), (1, 1, 9), (2, 7, 1), (4, 3, 64)):
        q = rng.standard_normal((4, T, Hh, 576), dtype=np.float32).astype(np.float16)
        a = oracle.mla_decode(q, cache, lens, 1 / 16, page_table=pt)
        b = oracle.mla_decode(q, cache, lens, 1 / 16, page_table=pt, key_splits=ks)
        assert np.abs(a - b).max() <= 2e-6, (T, Hh, ks, np.abs(a - b).max())
        assert not b[1].any()  # the empty sequence
    n, T, Hh = 300, 2, 5
    q = rng.standard_normal((1, T, Hh, 576), dtype=np.float32).astype(np.float16)
    c = cache[:n]
    got = oracle.mla_decode(q, c, [n], 1 / 16, key_splits=3).astype(np.float64)
    for t in range(T):
        k = c[:n - (T - 1 - t)].astype(np.float64)
        sc = q[0, t].astype(np.float64) @ k.T / 16
        p = np.exp(sc - sc.max(1, keepdims=True))
        want = (p / p.sum(1, keepdims=True)) @ k[:, :512]
        assert np.abs(got[0, t] - want).max() <= 2e-6


# ---- DSA k-pool indexer (crates/cuda/kernels/ops.cu:619-791) ------------------------------------------------

def _np_pool(kc, gc, ape, kpool):
    """float64 pooled keys of all complete pools of a whole sequence (no chunking, no rings)."""
    n = kc.shape[0] // kpool
    k = kc[:n * kpool].reshape(n, kpool, -1).astype(np.float64)
    g = gc[:n * kpool].reshape(n, kpool, -1).astype(np.float64) + ape.astype(np.float64)[None]
    e = np.exp(g - g.max(axis=1, keepdims=True))
    return (e * k).sum(axis=1) / e.sum(axis=1)


def test_idx_pool_chunked_with_rings_equals_whole_sequence_pooling(oracle):
    rng = np.random.default_rng(31)
    Dk, kpool = 32, 4
    chunks = [5, 1, 1, 9, 3, 17, 2]  # pools straddle chunk boundaries: their older rows come back from the rings
    n = sum(chunks)
    kc = rng.standard_normal((n, Dk), dtype=np.float32)
    gc = rng.standard_normal((n, Dk), dtype=np.float32) * np.float32(2)
    ape = rng.standard_normal((kpool, Dk), dtype=np.float32)
    rk, rg = np.zeros((kpool, Dk), np.float32), np.zeros((kpool, Dk), np.float32)
    P = np.zeros((n // kpool + 1, Dk), np.float32)
    p0 = 0
    for T in chunks:
        oracle.idx_pool(kc[p0:p0 + T], gc[p0:p0 + T], rk, rg, ape, P, p0, kpool)
        p0 += T
    want = _np_pool(kc, gc, ape, kpool)
    assert np.abs(P[:n // kpool] - want).max() <= 1e-5
    assert (P[n // kpool:] == 0).all()  # the incomplete tail pool is not written
    tail = n - n % kpool
    for pos in range(tail, n):  # and its raw rows wait in the rings
        assert np.array_equal(rk[pos % kpool], kc[pos]) and np.array_equal(rg[pos % kpool], gc[pos])


def test_idx_score_and_select_against_numpy(oracle):
    rng = np.random.default_rng(32)
    T, pos0, kpool, Hq, Dk, top_k = 5, 203, 4, 3, 16, 10
    pools = (pos0 + T) // kpool + 1
    q = rng.standard_normal((T, Hq, Dk), dtype=np.float32)
    w = rng.standard_normal((T, Hq), dtype=np.float32)
    P = rng.standard_normal((pools, Dk), dtype=np.float32)
    score = np.full((T, pools), np.float32(7.5))
    oracle.idx_score(q, w, P, score, pos0, kpool, 0.25)
    sel, cnt = oracle.idx_select(score, pos0, kpool, top_k, (top_k + 1) * kpool)
    for t in range(T):
        n_pool = (pos0 + t + 1) // kpool
        d = np.einsum("hc,pc->hp", q[t].astype(np.float64), P[:n_pool].astype(np.float64)) * 0.25
        want = (w[t].astype(np.float64)[:, None] * np.maximum(d, 0)).sum(axis=0)
        assert np.abs(score[t, :n_pool] - want).max() <= 1e-5
        assert (score[t, n_pool:] == 7.5).all()  # pools not complete at this query's position are left alone
        top = np.sort(np.argsort(-score[t, :n_pool], kind="stable")[:top_k])
        lst = np.concatenate([np.arange(p * kpool, (p + 1) * kpool) for p in top] + [np.arange(n_pool * kpool, pos0 + t + 1)])
        assert cnt[t] == lst.size and np.array_equal(sel[t, :cnt[t]], lst)
    # below top_k pools every position is attended (ops.cu:728-731)
    sel, cnt = oracle.idx_select(score, 10, kpool, top_k, (top_k + 1) * kpool)
    assert cnt[0] == 11 and np.array_equal(sel[0, :11], np.arange(11))


def test_idx_select_ties_go_to_the_lowest_indices(oracle):
    score = np.array([[1.0, 2.0, 2.0, 2.0, 3.0, 2.0, -0.0, 0.0, 2.0]], np.float32)
    sel, cnt = oracle.idx_select(score, 8, 1, 3, 4)  # kpool 1: nine complete pools, three taken
    assert cnt[0] == 3 and sel[0, :3].tolist() == [1, 2, 4]  # 3.0 and the first two of the 2.0s
    sel, cnt = oracle.idx_select(score, 8, 1, 8, 9)
    assert sorted(sel[0, :8].tolist()) == [0, 1, 2, 3, 4, 5, 7, 8]  # -0.0 sorts below +0.0 (ops.cu:718-721)


def test_indexer_golden_vectors_from_reference_kernels(oracle):
    """Outputs of the reference's own gs_idx_pool / gs_idx_score / gs_idx_select (compiled unmodified, run on a B200)
    pin the oracle's indexer functions.  The fixture is made by tests/golden/make_golden_from_ref.py."""
    path = os.path.join(HERE, "golden", "refidx_pool_score_select.npz")
    if not os.path.exists(path):
        pytest.skip("no indexer golden fixture committed yet")
    g = np.load(path)
    kc, gc, ape, kpool, top_k = g["kc"], g["gc"], g["ape"], int(g["kpool"]), int(g["top_k"])
    Dk = kc.shape[1]
    rk, rg = np.zeros((kpool, Dk), np.float32), np.zeros((kpool, Dk), np.float32)
    P = np.zeros_like(g["P"])
    p0 = 0
    for T in g["chunks"]:
        oracle.idx_pool(kc[p0:p0 + T], gc[p0:p0 + T], rk, rg, ape, P, p0, kpool)
        p0 += int(T)
    assert np.abs(P - g["P"]).max() <= 1e-5
    assert np.array_equal(rk, g["rk"]) and np.array_equal(rg, g["rg"])
    score = np.zeros_like(g["score"])
    oracle.idx_score(g["q"], g["w"], g["P"], score, int(g["pos0"]), kpool, float(g["scale"]))
    assert np.abs(score - g["score"]).max() <= 1e-5
    sel, cnt = oracle.idx_select(g["score"], int(g["pos0"]), kpool, top_k, g["sel_sorted"].shape[1])
    assert np.array_equal(cnt, g["cnt"])
    for t in range(cnt.size):
        assert np.array_equal(np.sort(sel[t, :cnt[t]]), g["sel_sorted"][t, :cnt[t]])


def test_fused_step_oracle_against_float64(oracle):
    """absorb k_b, attend, expand v_b (crates/engine/src/forward.rs:900-907) against a float64 restatement."""
    rng = np.random.default_rng(33)
    T, H, n = 2, 3, 41
    q = rng.standard_normal((T, H, 256), dtype=np.float32)
    kb = (rng.standard_normal((H, 512, 256), dtype=np.float32) / 16).astype(np.float16)
    vb = (rng.standard_normal((H, 256, 512), dtype=np.float32) / 22.6).astype(np.float16)
    c = (rng.standard_normal((n, 512), dtype=np.float32) * 0.5).astype(np.float16)
    got = oracle.mla_fused(q, kb, vb, c, n, 1 / 16)
    qa = np.einsum("hrk,thk->thr", kb.astype(np.float64), q.astype(np.float64))
    want = np.zeros((T, H, 256))
    for t in range(T):
        nt = n - (T - 1 - t)  # the T new rows are causal among themselves
        for h in range(H):
            s = (c[:nt].astype(np.float64) @ qa[t, h]) / 16
            p = np.exp(s - s.max())
            want[t, h] = vb[h].astype(np.float64) @ ((p / p.sum()) @ c[:nt].astype(np.float64))
    assert np.abs(got - want).max() <= 2e-6
    assert np.abs(oracle.mla_fused(q, kb, vb, c, 0, 1 / 16)).max() == 0.0  # nothing attended: zeros (ops.cu:535)
