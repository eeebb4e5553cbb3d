"""More GPU parity cases of the decode path: the largest batch the tcgen05 kernel takes, inputs that
change between back-to-back calls (the kernel builds its schedule once speculatively, before the inputs
of the call are final, and must not let anything from that pass reach a result), wider query blocks,
and the combine for every segment count around its register-resident limit."""
import numpy as np
import pytest

from conftest import check_close, check_not_degenerate, make_decode_inputs
from gpu_util import paged_layout, to_dev

pytestmark = pytest.mark.gpu


def test_batch_of_1024_sequences(pkg, cuda, oracle):
    rng = np.random.default_rng(31)
    lens = rng.integers(0, 200, size=1024).astype(np.int32)
    lens[[3, 500, 1023]] = 0
    base = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    q, cache = make_decode_inputs(31, 1024, 1, 20, int(lens.sum()) + 1)
    for impl in (2, 1):
        o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, lens), seq_base=to_dev(cuda, base), impl=impl)
        cuda.cuda.synchronize()
        got = o.cpu().numpy()
        check_close(got, oracle.mla_decode(q, cache, lens, 1 / 16, seq_base=base), f"1024 sequences impl={impl}")
        assert (got[lens == 0] == 0).all()
    with pytest.raises(Exception):
        pkg.mla_decode(to_dev(cuda, np.repeat(q, 2, 0)[:1025]), to_dev(cuda, cache), to_dev(cuda, np.zeros(1025, np.int32)), impl=2)


@pytest.mark.parametrize("T,H", [(3, 16), (4, 8), (4, 12), (1, 48), (2, 24)])
def test_wider_query_blocks(pkg, cuda, oracle, T, H):
    q, cache = make_decode_inputs(40 + T * H, 1, T, H, 1500)
    o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, np.array([1500], np.int32)), impl=2)
    cuda.cuda.synchronize()
    check_close(o.cpu().numpy(), oracle.mla_decode(q, cache, [1500], 1 / 16), f"T={T} H={H}")


def test_lengths_and_pages_that_change_between_calls(pkg, cuda, oracle):
    """Back-to-back launches on one stream, each with lengths / page table rewritten on the device just
    before it: the speculative schedule of every launch sees the previous call's values."""
    rng = np.random.default_rng(77)
    n_seq, H = 6, 20
    q = rng.standard_normal((n_seq, 1, H, 576), dtype=np.float32).astype(np.float16)
    cases = []
    for k in range(5):
        lens = rng.integers(0, 3000, size=n_seq).astype(np.int32)
        if k == 2:
            lens[:] = 0
        pool, pt = paged_layout(rng, np.maximum(lens, 1), spare_pages=2)
        cases.append((lens, pool, pt))
    rows = max(c[1].shape[0] for c in cases)
    stride = max(c[2].shape[1] for c in cases)
    pool_d = cuda.zeros((rows, 576), dtype=cuda.float16, device="cuda")
    pt_d = cuda.zeros((n_seq, stride), dtype=cuda.int32, device="cuda")
    lens_d = cuda.zeros(n_seq, dtype=cuda.int32, device="cuda")
    qd = to_dev(cuda, q)
    ws = pkg.new_workspace(n_seq, 1, H)
    outs = []
    staged = []
    for lens, pool, pt in cases:
        p = np.zeros((rows, 576), np.float16)
        p[:pool.shape[0]] = np.nan_to_num(pool, nan=0.0)
        t = np.zeros((n_seq, stride), np.int32)
        t[:, :pt.shape[1]] = pt
        staged.append((to_dev(cuda, lens), to_dev(cuda, p), to_dev(cuda, t), lens, p, t))
    cuda.cuda.synchronize()
    for ld, pd, td, *_ in staged:  # no host synchronisation inside this loop
        lens_d.copy_(ld, non_blocking=True)
        pool_d.copy_(pd, non_blocking=True)
        pt_d.copy_(td, non_blocking=True)
        outs.append(pkg.mla_decode(qd, pool_d, lens_d, page_table=pt_d, workspace=ws, impl=2).clone())
    cuda.cuda.synchronize()
    assert pkg.decode_status(ws) == 0
    for k, (o, (_, _, _, lens, p, t)) in enumerate(zip(outs, staged)):
        want = oracle.mla_decode(q, p, lens, 1 / 16, page_table=t)
        check_close(o.cpu().numpy(), want, f"call {k}")


def test_dense_length_growing_step_by_step_in_a_graph(pkg, cuda, oracle):
    """A decode loop: the length word is advanced on the device between replays of one captured call."""
    n0, steps, H = 700, 6, 20
    q, cache = make_decode_inputs(55, 1, 1, H, n0 + steps + 3)
    qd, cd = to_dev(cuda, q), to_dev(cuda, cache)
    lens_d = cuda.full((1,), n0, dtype=cuda.int32, device="cuda")
    ws = pkg.new_workspace(1, 1, H)
    out = cuda.empty((1, 1, H, 512), dtype=cuda.float32, device="cuda")
    keep = cuda.empty((steps, 1, 1, H, 512), dtype=cuda.float32, device="cuda")
    pkg.mla_decode(qd, cd, lens_d, workspace=ws, out=out, impl=2)
    cuda.cuda.synchronize()
    s = cuda.cuda.Stream()
    g = cuda.cuda.CUDAGraph()
    with cuda.cuda.stream(s):
        with cuda.cuda.graph(g, stream=s):
            pkg.mla_decode(qd, cd, lens_d, workspace=ws, out=out, impl=2)
            lens_d.add_(1)
        for k in range(steps):
            g.replay()
            keep[k].copy_(out, non_blocking=True)
    cuda.cuda.synchronize()
    for k in range(steps):
        check_close(keep[k].cpu().numpy(), oracle.mla_decode(q, cache, [n0 + k], 1 / 16), f"replay {k}")


@pytest.mark.parametrize("n_parts", [1, 2, 8, 159, 160, 161, 300, 1024])
def test_combine_parts_segment_counts(pkg, cuda, oracle, n_parts):
    rng = np.random.default_rng(n_parts)
    rows, d_v = 8, 512
    acc = rng.standard_normal((n_parts, rows, d_v), dtype=np.float32)
    m = rng.standard_normal((n_parts, rows), dtype=np.float32) * 3
    l = rng.random((n_parts, rows), dtype=np.float32) + 0.1
    if n_parts > 2:
        m[1] = -np.inf          # an empty segment: its accumulator (NaN here) must not enter the sum
        l[1] = 0
        acc[1] = np.nan
    blocks = np.concatenate([acc.reshape(n_parts, -1), np.stack([m, l], -1).reshape(n_parts, -1)], 1)
    got = pkg.combine_parts(to_dev(cuda, blocks.reshape(-1)), n_parts, rows, d_v)
    cuda.cuda.synchronize()
    recs = np.concatenate([acc, m[..., None], l[..., None]], -1).transpose(1, 0, 2)  # [rows][parts][d_v + 2]
    recs = np.nan_to_num(recs, nan=0.0, neginf=-np.inf)
    want = oracle.combine(np.ascontiguousarray(recs))
    check_close(got.cpu().numpy(), want, f"combine of {n_parts} parts", 1e-4, 1e-5)


@pytest.mark.parametrize("T,H", [(1, 64), (2, 64), (2, 48), (2, 32), (3, 32), (4, 16), (1, 56)])
def test_head_groups_beyond_48_query_rows(pkg, cuda, oracle, T, H):
    """The reference's models have up to 64 heads (validate.rs:52-54): blocks of more than 48 query rows run on the
    tcgen05 kernel as head groups, one launch per group, and must land in the right rows of the output."""
    rng = np.random.default_rng(T * 100 + H)
    lens = np.array([900, 0, 65, 2100], np.int32)
    pool, pt = paged_layout(rng, lens)
    q = rng.standard_normal((len(lens), T, H, 576), dtype=np.float32).astype(np.float16)
    o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, pool), to_dev(cuda, lens), page_table=to_dev(cuda, pt), impl=2)
    cuda.cuda.synchronize()
    got = o.cpu().numpy()
    check_close(got, oracle.mla_decode(q, pool, lens, 1 / 16, page_table=pt), f"T={T} H={H} paged")
    check_not_degenerate(got[0], "head groups")
    # dense single sequence, and the merged records instead of the normalised output
    q1, cache = make_decode_inputs(T + H, 1, T, H, 3000)
    part = cuda.zeros(pkg.part_floats(T * H), dtype=cuda.float32, device="cuda")
    o1 = pkg.mla_decode(to_dev(cuda, q1), to_dev(cuda, cache), to_dev(cuda, np.array([3000], np.int32)), impl=2, part_out=part)
    cuda.cuda.synchronize()
    want = oracle.mla_decode(q1, cache, [3000], 1 / 16)
    check_close(o1.cpu().numpy(), want, f"T={T} H={H} dense")
    pr = part.cpu().numpy()
    acc, ml = pr[:T * H * 512].reshape(T * H, 512), pr[T * H * 512:].reshape(T * H, 2)
    check_close((acc / ml[:, 1:2]).reshape(1, T, H, 512), want, "records of the head groups")


def test_reference_twin_shape_64_heads_runs_on_the_tensor_core_kernel(pkg, cuda, oracle):
    # R = 512 rows (V = all columns), 64 heads: the shape of the reference's own models
    q, cache = make_decode_inputs(64, 1, 1, 64, 4096, d_qk=512)
    o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, np.array([4096], np.int32)), impl=2, d_v=512)
    cuda.cuda.synchronize()
    check_close(o.cpu().numpy(), oracle.mla_decode(q, cache, [4096], 1 / 16, d_v=512), "R=512 H=64")


@pytest.mark.parametrize("n_seq,T,H,paged", [(1, 2, 32, False), (3, 1, 56, False), (5, 1, 64, True), (2, 4, 16, False), (1, 1, 80, False)])
def test_512_column_rows_with_49_to_64_query_rows_in_one_pass(pkg, cuda, oracle, n_seq, T, H, paged):
    """Over 512-column rows up to 64 query rows (tokens x heads) ride in one pass of the tcgen05 kernel (64 query
    columns, two issuing warps); 80 heads still run as head groups.  Ragged lengths, dense with bases and paged."""
    rng = np.random.default_rng(n_seq * 100 + T * 10 + H)
    lens = rng.integers(1, 700, size=n_seq).astype(np.int32)
    lens[0] = 643
    q = rng.standard_normal((n_seq, T, H, 512), dtype=np.float32).astype(np.float16)
    if paged:
        pages_per = -(-lens // 64)
        n_pages = int(pages_per.sum()) + 3
        cache = (rng.standard_normal((n_pages * 64, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
        perm = rng.permutation(n_pages)
        pt = np.zeros((n_seq, int(pages_per.max())), np.int32)
        k = 0
        for b in range(n_seq):
            pt[b, :pages_per[b]] = perm[k:k + pages_per[b]]
            k += int(pages_per[b])
        o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, lens), page_table=to_dev(cuda, pt), impl=2, d_v=512)
        want = oracle.mla_decode(q, cache, lens, 1 / 16, d_v=512, page_table=pt)
    else:
        base = (np.arange(n_seq) * 704).astype(np.int32)
        cache = (rng.standard_normal((n_seq * 704, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
        o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, lens), seq_base=to_dev(cuda, base), impl=2, d_v=512)
        want = oracle.mla_decode(q, cache, lens, 1 / 16, d_v=512, seq_base=base)
    cuda.cuda.synchronize()
    check_close(o.cpu().numpy(), want, f"R=512, {T}x{H} query rows")


@pytest.mark.parametrize("T", [1, 2])
def test_length_beyond_the_cache_is_taken_as_the_cache_size(pkg, cuda, oracle, T):
    """Input hardening: a length word larger than the cache allocation (or negative) must not be followed past the
    cache.  The tcgen05 kernel takes it as cache_rows (or 0)."""
    q, cache = make_decode_inputs(90 + T, 3, T, 20, 3 * 500)
    base = np.array([0, 500, 1000], np.int32)
    lens = np.array([2**31 - 1, -5, 400], np.int32)
    o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, lens), seq_base=to_dev(cuda, base), impl=2)
    cuda.cuda.synchronize()
    got = o.cpu().numpy()
    # sequence 0: base 0, length clamped to the 1500 rows of the allocation; sequence 1: empty
    want = oracle.mla_decode(q, cache, np.array([1500, 0, 400], np.int32), 1 / 16, seq_base=base)
    check_close(got, want, "clamped lengths")
    assert (got[1] == 0).all()
