"""GPU parity of the DSA k-pool indexer entry points (gs_idx_pool, gs_idx_score, gs_idx_select) against the oracle
and, where the reference's own kernels were compiled (oracle/_ref), against those (crates/cuda/kernels/ops.cu:619-791)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import ROOT
from gpu_util import to_dev

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(ROOT, "oracle", "_ref", "libglmssd_ref.so")


def _ref_lib(pkg):
    ref = C.CDLL(REF_SO)
    for name in ("gs_idx_pool", "gs_idx_score", "gs_idx_select", "gs_mla_attn"):
        getattr(ref, name).restype = C.c_int
        getattr(ref, name).argtypes = pkg._lib.SIGNATURES[name][1]
    return ref


def _pool_chunks(torch, lib, kc, gc, ape, chunks, kpool, pools):
    Dk = kc.shape[1]
    rk, rg = torch.zeros((kpool, Dk), device="cuda"), torch.zeros((kpool, Dk), device="cuda")
    P = torch.zeros((pools, Dk), device="cuda")
    aped = to_dev(torch, ape)
    p0 = 0
    for T in chunks:
        kd, gd = to_dev(torch, kc[p0:p0 + T]), to_dev(torch, gc[p0:p0 + T])
        assert lib.gs_idx_pool(kd.data_ptr(), gd.data_ptr(), rk.data_ptr(), rg.data_ptr(), aped.data_ptr(), P.data_ptr(), p0, T, Dk,
                               kpool, None) == 0
        torch.cuda.synchronize()
        p0 += T
    return P.cpu().numpy(), rk.cpu().numpy(), rg.cpu().numpy()


@pytest.mark.parametrize("chunks,kpool,Dk", [
    ((5, 9, 17), 4, 128),          # pools straddling chunk boundaries: their older rows come from the rings
    ((1,) * 13, 4, 128),           # decode steps: a pool completes every fourth call
    ((256, 3, 1, 260), 4, 64),     # a prefill chunk, then ragged ones
    ((7, 2), 16, 96),              # no pool completes in the second call: hand-over only
    ((40,), 1, 128),               # kpool = 1: every position is a pool
])
def test_idx_pool_vs_oracle_and_reference(pkg, cuda, oracle, chunks, kpool, Dk):
    rng = np.random.default_rng(sum(chunks) + kpool)
    n_pos = sum(chunks)
    kc = rng.standard_normal((n_pos, Dk), dtype=np.float32)
    gc = rng.standard_normal((n_pos, Dk), dtype=np.float32) * np.float32(2.0)
    ape = rng.standard_normal((kpool, Dk), dtype=np.float32) * np.float32(0.3)
    pools = n_pos // kpool + 1
    got = _pool_chunks(cuda, pkg._lib.load(), kc, gc, ape, chunks, kpool, pools)
    rk, rg, P = np.zeros((kpool, Dk), np.float32), np.zeros((kpool, Dk), np.float32), np.zeros((pools, Dk), np.float32)
    p0 = 0
    for T in chunks:
        oracle.idx_pool(kc[p0:p0 + T], gc[p0:p0 + T], rk, rg, ape, P, p0, kpool)
        p0 += T
    assert np.abs(got[0] - P).max() <= 1e-5
    assert np.array_equal(got[1], rk) and np.array_equal(got[2], rg)  # the rings hold copies: bit-exact
    if os.path.exists(REF_SO):
        ref = _pool_chunks(cuda, _ref_lib(pkg), kc, gc, ape, chunks, kpool, pools)
        assert np.abs(got[0] - ref[0]).max() <= 1e-5
        assert np.array_equal(got[1], ref[1]) and np.array_equal(got[2], ref[2])


def _scores(torch, lib, q, w, P, pos0, kpool, stride, scale):
    T, Hq, Dk = q.shape
    score = torch.full((T, stride), -123.0, device="cuda")
    qd, wd, Pd = to_dev(torch, q), to_dev(torch, w), to_dev(torch, P)  # held until the call has run
    assert lib.gs_idx_score(qd.data_ptr(), wd.data_ptr(), Pd.data_ptr(), score.data_ptr(),
                            stride, pos0, T, kpool, Hq, Dk, scale, None) == 0
    torch.cuda.synchronize()
    return score.cpu().numpy()


@pytest.mark.parametrize("T,pos0,Hq,Dk,kpool", [(1, 4099, 32, 128, 4), (2, 700, 8, 128, 4), (256, 1000, 16, 64, 4), (3, 17, 4, 100, 8),
                                                 (1, 2, 8, 128, 4)])
def test_idx_score_vs_oracle_and_reference(pkg, cuda, oracle, T, pos0, Hq, Dk, kpool):
    rng = np.random.default_rng(T * 7 + pos0)
    pools = (pos0 + T) // kpool + 1
    q = rng.standard_normal((T, Hq, Dk), dtype=np.float32)
    w = rng.standard_normal((T, Hq), dtype=np.float32)
    P = rng.standard_normal((pools, Dk), dtype=np.float32)
    scale = float(1 / np.sqrt(Dk))
    got = _scores(cuda, pkg._lib.load(), q, w, P, pos0, kpool, pools, scale)
    want = np.full((T, pools), -123.0, np.float32)
    oracle.idx_score(q, w, P, want, pos0, kpool, scale)
    tol = 1e-5 * max(1.0, float(np.abs(want[want != -123.0]).max()) if (want != -123.0).any() else 1.0)
    assert np.abs(got - want).max() <= tol  # entries past a query's complete pools are left alone by both
    if os.path.exists(REF_SO):
        ref = _scores(cuda, _ref_lib(pkg), q, w, P, pos0, kpool, pools, scale)
        assert np.abs(got - ref).max() <= tol


def _select(torch, lib, score, pos0, kpool, top_k, sel_stride):
    T, stride = score.shape
    sel = torch.full((T, sel_stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(T, dtype=torch.int32, device="cuda")
    sd = to_dev(torch, score)  # held until the call has run
    assert lib.gs_idx_select(sd.data_ptr(), stride, pos0, T, kpool, top_k, sel.data_ptr(), sel_stride, cnt.data_ptr(),
                             None) == 0
    torch.cuda.synchronize()
    return sel.cpu().numpy(), cnt.cpu().numpy()


@pytest.mark.parametrize("T,pos0,kpool,top_k,ties", [
    (1, 8191, 4, 512, False),     # decode at 8K: 2048 pools, 512 taken
    (2, 32766, 4, 512, False),    # MTP verify at 32K
    (256, 3000, 4, 512, False),   # a prefill chunk that crosses from dense (n_pool <= top_k) to sparse lists
    (5, 2047, 4, 512, False),     # around n_pool == top_k: 2048 positions are still dense, 2052 no longer
    (3, 4097, 4, 512, True),      # many equal scores, also at the k-th largest: ties go to the lowest indices
    (4, 1000, 16, 7, True),
    (2, 131070, 4, 512, False),   # 128K context
    (3, 50, 4, 0, False),         # top_k = 0: only the incomplete tail is attended
    (1, 0, 4, 512, False),        # the very first position
])
def test_idx_select_bit_exact_vs_oracle(pkg, cuda, oracle, T, pos0, kpool, top_k, ties):
    rng = np.random.default_rng(pos0 + T)
    pools = (pos0 + T) // kpool + 1
    score = rng.standard_normal((T, pools), dtype=np.float32)
    if ties:
        score = np.round(score * 4) / 4  # a few dozen distinct values, negative zero included
        score[:, ::7] = -0.0
    sel_stride = (top_k + 1) * kpool
    got_sel, got_cnt = _select(cuda, pkg._lib.load(), score, pos0, kpool, top_k, sel_stride)
    want_sel, want_cnt = oracle.idx_select(score, pos0, kpool, top_k, sel_stride)
    assert np.array_equal(got_cnt, want_cnt)
    for t in range(T):
        assert np.array_equal(got_sel[t, :got_cnt[t]], want_sel[t, :want_cnt[t]]), f"query {t}"
    if os.path.exists(REF_SO):
        ref_sel, ref_cnt = _select(cuda, _ref_lib(pkg), score, pos0, kpool, top_k, sel_stride)
        assert np.array_equal(got_cnt, ref_cnt)
        for t in range(T):
            n = got_cnt[t]
            if not ties:  # a unique k-th largest score: the selected set is the reference's, only its order is ours
                assert np.array_equal(np.sort(ref_sel[t, :n]), got_sel[t, :n])  # ours is ascending already
            else:  # equal scores at the threshold: the reference takes whichever threads come first; the scores taken agree
                ord_of = lambda s: np.sort(score[t, (s[:top_k * kpool:kpool] // kpool)]) if (pos0 + t + 1) // kpool > top_k else np.zeros(0)
                assert np.array_equal(ord_of(ref_sel[t]), ord_of(got_sel[t]))


def test_select_then_attend_matches_reference_pipeline(pkg, cuda, oracle):
    """The engine's decode step beyond top_k positions (forward.rs:864-906): pooled keys -> scores -> position list ->
    gs_mla_attn over the listed rows, all through this library, against the oracle fed with the oracle's own list."""
    torch = cuda
    rng = np.random.default_rng(77)
    ctx, kpool, top_k, Hq, Dk, H = 4096, 4, 128, 8, 128, 16
    pos0, T = ctx - 2, 2
    pools = ctx // kpool + 1
    P = rng.standard_normal((pools, Dk), dtype=np.float32)
    qi = rng.standard_normal((T, Hq, Dk), dtype=np.float32)
    wi = rng.standard_normal((T, Hq), dtype=np.float32)
    L = pkg._lib.load()
    score = _scores(torch, L, qi, wi, P, pos0, kpool, pools, float(1 / np.sqrt(Dk)))
    sel_stride = (top_k + 1) * kpool
    sel, cnt = _select(torch, L, score, pos0, kpool, top_k, sel_stride)
    want_sel, want_cnt = oracle.idx_select(score, pos0, kpool, top_k, sel_stride)
    assert np.array_equal(cnt, want_cnt) and all(np.array_equal(sel[t, :cnt[t]], want_sel[t, :cnt[t]]) for t in range(T))
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    Cc = (rng.standard_normal((ctx, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    o = torch.zeros((T, H, 512), dtype=torch.float32, device="cuda")
    part = torch.zeros(T * H * 4 * 514, dtype=torch.float32, device="cuda")
    qd, cd, sd, nd = to_dev(torch, q), to_dev(torch, Cc), to_dev(torch, sel), to_dev(torch, cnt)  # held until the call has run
    assert L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), sel_stride,
                         nd.data_ptr(), 1 / 16, o.data_ptr(), part.data_ptr(), T, H, 512, 4, None) == 0
    torch.cuda.synchronize()
    want = oracle.mla_attn_ref(q, Cc, want_sel, want_cnt, 1 / 16)
    err = np.abs(o.cpu().numpy() - want)
    assert err.max() <= 2e-3 and err.mean() <= 2e-4  # the attention tolerance: f16 rows, fp32 accumulate
