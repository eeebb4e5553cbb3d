"""GPU parity of the absorbed-MLA decode against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import check_close, check_not_degenerate, make_decode_inputs
from gpu_util import paged_layout, to_dev

pytestmark = pytest.mark.gpu

IMPLS = [1, 0]  # 1 = CUDA-core kernel, 0 = automatic (tcgen05 where the shape allows)


def _run_decode(pkg, torch, q, cache, lens, impl, **kw):
    o = pkg.mla_decode(to_dev(torch, q), to_dev(torch, cache), to_dev(torch, np.asarray(lens, np.int32)), impl=impl,
                       **kw)
    torch.cuda.synchronize()
    return o.cpu().numpy()


@pytest.mark.parametrize("impl", IMPLS)
def test_config1_decode_4k(pkg, cuda, oracle, impl):
    # batch 1, 1 query token, 20 heads, 4096 positions
    q, cache = make_decode_inputs(1, 1, 1, 20, 4096)
    got = _run_decode(pkg, cuda, q, cache, [4096], impl)
    want = oracle.mla_decode(q, cache, [4096], 1 / 16)
    check_close(got, want, "config 1")
    check_not_degenerate(got, "config 1")


@pytest.mark.parametrize("impl", IMPLS)
def test_config2_mtp_verify_32k(pkg, cuda, oracle, impl):
    # 2 query tokens, causal between them: token 0 sees rows 0..32766, token 1 rows 0..32767
    q, cache = make_decode_inputs(2, 1, 2, 20, 32768)
    got = _run_decode(pkg, cuda, q, cache, [32768], impl)
    want = oracle.mla_decode(q, cache, [32768], 1 / 16)
    check_close(got, want, "config 2")
    check_not_degenerate(got, "config 2")
    # the two tokens must differ by exactly the last row's contribution: token 0 never sees row 32767
    cache2 = cache.copy()
    cache2[32767] = np.float16(30.0)
    got2 = _run_decode(pkg, cuda, q, cache2, [32768], impl)
    assert np.array_equal(got2[0, 0], got[0, 0])
    assert not np.array_equal(got2[0, 1], got[0, 1])


@pytest.mark.parametrize("impl", IMPLS)
def test_config3_decode_128k_single_gpu(pkg, cuda, oracle, impl):
    q, cache = make_decode_inputs(3, 1, 1, 20, 131072)
    got = _run_decode(pkg, cuda, q, cache, [131072], impl)
    want = oracle.mla_decode(q, cache, [131072], 1 / 16)
    check_close(got, want, "config 3 (1 GPU)")


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("T", [1, 2])
@pytest.mark.parametrize("n", [0, 1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 129, 1000, 2049])
def test_edge_lengths(pkg, cuda, oracle, impl, T, n):
    q, cache = make_decode_inputs(100 + n, 1, T, 20, max(n, 1) + 7)
    # rows past the attended range are NaN: they must not leak into the result
    cache[n:] = np.float16(np.nan)
    got = _run_decode(pkg, cuda, q, cache, [n], impl)
    want = oracle.mla_decode(q, cache, [n], 1 / 16)
    check_close(got, want, f"n={n} T={T}")
    if n == 0 or (T == 2 and n == 1):
        assert (got[0, 0] == 0).all()  # empty set -> zeros (ops.cu:535, :565)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("H", [1, 16, 20, 32, 33, 64])
def test_head_counts(pkg, cuda, oracle, impl, H):
    q, cache = make_decode_inputs(200 + H, 1, 1, H, 777)
    got = _run_decode(pkg, cuda, q, cache, [777], impl)
    check_close(got, oracle.mla_decode(q, cache, [777], 1 / 16), f"H={H}")


@pytest.mark.parametrize("impl", IMPLS)
def test_batched_dense_ragged(pkg, cuda, oracle, impl):
    rng = np.random.default_rng(9)
    lens = np.array([5, 0, 300, 64, 1, 4097, 129], np.int32)
    base = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    q, cache = make_decode_inputs(9, len(lens), 1, 20, int(lens.sum()) + 1)
    got = _run_decode(pkg, cuda, q, cache, lens, impl, seq_base=to_dev(cuda, base))
    want = oracle.mla_decode(q, cache, lens, 1 / 16, seq_base=base)
    check_close(got, want, "ragged dense batch")
    assert (got[1] == 0).all()


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("T", [1, 2])
def test_paged_batch(pkg, cuda, oracle, impl, T):
    rng = np.random.default_rng(10 + T)
    lens = np.array([64, 65, 1, 1000, 128, 63, 2500, 0, 700], np.int32)
    pool, pt = paged_layout(rng, lens)
    q = rng.standard_normal((len(lens), T, 20, 576), dtype=np.float32).astype(np.float16)
    got = _run_decode(pkg, cuda, q, pool, lens, impl, page_table=to_dev(cuda, pt))
    want = oracle.mla_decode(q, pool, lens, 1 / 16, page_table=pt)
    check_close(got, want, "paged batch")
    check_not_degenerate(got, "paged batch")


@pytest.mark.parametrize("impl", IMPLS)
def test_config5_paged_serving_batch(pkg, cuda, oracle, impl):
    # 64 sequences, lengths uniform in [1024, 65536], 64-row pages, random page table
    rng = np.random.default_rng(5)
    lens = rng.integers(1024, 65537, size=64).astype(np.int32)
    pool, pt = paged_layout(rng, lens)
    q = rng.standard_normal((64, 1, 20, 576), dtype=np.float32).astype(np.float16)
    got = _run_decode(pkg, cuda, q, pool, lens, impl, page_table=to_dev(cuda, pt), max_seq_len=int(lens.max()))
    want = oracle.mla_decode(q, pool, lens, 1 / 16, page_table=pt)
    check_close(got, want, "config 5")


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("G", [2, 4, 8])
def test_shard_partials_combine(pkg, cuda, oracle, impl, G):
    """Config 3's exchange on one GPU: G contiguous shards -> (acc, m, l) blocks -> combine."""
    n, H, T = 131072 // 8, 20, 1
    q, cache = make_decode_inputs(30 + G, 1, T, H, n)
    rows = T * H
    blocks = cuda.empty((G, pkg.part_floats(rows)), dtype=cuda.float32, device="cuda")
    qd = to_dev(cuda, q)
    for g in range(G):
        lo, hi = pkg.shard_rows(n, G, g, 16)
        shard = to_dev(cuda, cache[lo:hi].copy())
        lens = to_dev(cuda, np.array([hi - lo], np.int32))
        pkg.mla_decode(qd, shard, lens, tail_causal=(g == G - 1), want_out=False, part_out=blocks[g], impl=impl)
    o = pkg.combine_parts(blocks, G, rows)
    cuda.cuda.synchronize()
    want = oracle.mla_decode(q, cache, [n], 1 / 16)
    check_close(o.cpu().numpy().reshape(1, T, H, 512), want, f"G={G}")
    # the device records agree with the oracle's records after normalisation
    b0 = blocks[0].cpu().numpy()
    acc, ml = b0[:rows * 512].reshape(rows, 512), b0[rows * 512:].reshape(rows, 2)
    lo, hi = pkg.shard_rows(n, G, 0, 16)
    rec = oracle.mla_decode(q, cache, [n], 1 / 16, part_range=(lo, hi)).reshape(rows, 514)
    check_close(acc / ml[:, 1:2], rec[:, :512] / rec[:, 513:514], "shard 0 record")
    lse_dev = ml[:, 0] + np.log(ml[:, 1])
    lse_ref = rec[:, 512] + np.log(rec[:, 513])
    assert np.abs(lse_dev - lse_ref).max() < 1e-3


def test_run_to_run_bit_stable(pkg, cuda):
    q, cache = make_decode_inputs(4, 1, 2, 20, 9000)
    a = _run_decode(pkg, cuda, q, cache, [9000], 0)
    b = _run_decode(pkg, cuda, q, cache, [9000], 0)
    assert np.array_equal(a, b)


def test_large_scores_do_not_overflow(pkg, cuda, oracle):
    # scores of several hundred: the running maximum must keep exp() in range
    q, cache = make_decode_inputs(6, 1, 2, 20, 3000, sigma=4.0)
    q = (q.astype(np.float32) * 6).astype(np.float16)
    for impl in IMPLS:
        got = _run_decode(pkg, cuda, q, cache, [3000], impl)
        check_close(got, oracle.mla_decode(q, cache, [3000], 1 / 16), f"large scores impl={impl}", 8e-3, 1e-3)


def test_status_word_clean(pkg, cuda):
    q, cache = make_decode_inputs(7, 1, 1, 20, 500)
    ws = pkg.new_workspace(1, 1, 20)
    pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, np.array([500], np.int32)), workspace=ws)
    assert pkg.decode_status(ws) == 0
