"""Seeded random shapes through the decode entry points against the CPU oracle: head counts, token counts, ragged
and degenerate lengths, dense with bases / paged / position lists, record and single-split forms - the shapes nobody
thought of listing by hand.  Every case is small; the seeds are fixed."""
import ctypes as C

import numpy as np
import pytest

from conftest import check_close
from gpu_util import paged_layout, to_dev

pytestmark = pytest.mark.gpu

EDGE_LENS = (0, 1, 63, 64, 65, 127, 128, 129)


def _tcgen05_takes(d_qk, T, H):
    """The shapes gs_mla_decode's tensor-core kernel takes (others are asked of the CUDA-core kernel)."""
    rows = T * H
    if rows <= 48 or (d_qk == 512 and rows <= 64):
        return True
    return T <= 4 and H % 8 == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_decode_shapes(pkg, cuda, oracle, seed):
    rng = np.random.default_rng(1000 + seed)
    for it in range(12):
        d_qk = int(rng.choice([576, 512]))
        T = int(rng.integers(1, 5))
        H = int(rng.choice([8, 16, 20, 24, 32, 40, 48, 56, 64, 80, 96]))
        n_seq = int(rng.integers(1, 7))
        lens = rng.integers(0, 900, size=n_seq).astype(np.int32)
        if rng.random() < 0.4:
            lens[rng.integers(0, n_seq)] = int(rng.choice(EDGE_LENS + (T, max(T - 1, 0))))
        q = rng.standard_normal((n_seq, T, H, d_qk), dtype=np.float32).astype(np.float16)
        impl = 2 if _tcgen05_takes(d_qk, T, H) else 0
        what = f"seed {seed} case {it}: d_qk={d_qk} T={T} H={H} lens={lens.tolist()}"
        if rng.random() < 0.5:
            base = (np.arange(n_seq) * 960).astype(np.int32)
            cache = (rng.standard_normal((n_seq * 960, d_qk), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
            o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, lens), seq_base=to_dev(cuda, base), impl=impl)
            want = oracle.mla_decode(q, cache, lens, 1 / 16, seq_base=base)
        else:
            pool, pt = paged_layout(rng, lens, d_qk=d_qk)
            o = pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, pool), to_dev(cuda, lens), page_table=to_dev(cuda, pt), impl=impl)
            want = oracle.mla_decode(q, np.nan_to_num(pool, nan=0.0), lens, 1 / 16, page_table=pt)
        cuda.cuda.synchronize()
        check_close(o.cpu().numpy(), want, what)


@pytest.mark.parametrize("seed", range(4))
def test_random_position_lists_through_the_reference_entry_point(pkg, cuda, oracle, seed):
    rng = np.random.default_rng(2000 + seed)
    L = pkg._lib.load()
    for it in range(10):
        T = int(rng.choice([1, 2, 3, 8, 40, 90, 160]))
        H = int(rng.choice([16, 32, 48, 64, 96]))
        n = int(rng.integers(0, 400))
        splits = int(rng.choice([1, 2, 4, 16]))
        ctx = 3000
        q = rng.standard_normal((T, H, 512), dtype=np.float32)
        cache = (rng.standard_normal((ctx, 512), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
        stride = n + int(rng.integers(0, 9)) + 1
        sel = rng.integers(0, ctx, size=(T, stride)).astype(np.int32)
        cnt = rng.integers(max(0, n - 70), n + 1, size=T).astype(np.int32)
        qd, cd, sd, nd = to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, sel), to_dev(cuda, cnt)
        scd, attended = None, cache
        if rng.random() < 0.5:  # the Q8 cache: int8 rows + f16 scales; the oracle attends over the rows rebuilt from them
            cq, cs = oracle.quant_q8_rows(cache.astype(np.float32))
            cd, scd = to_dev(cuda, cq), to_dev(cuda, cs)
            attended = oracle.dequant_q8(cq, cs)
        o = cuda.zeros((T, H, 512), dtype=cuda.float32, device="cuda")
        part_floats = T * H * splits * 514  # crates/cuda/kernels/ops.cu:578
        part = cuda.zeros(part_floats + 64, dtype=cuda.float32, device="cuda")
        part[part_floats:] = 7.0
        rc = L.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None if scd is None else scd.data_ptr(), sd.data_ptr(), stride, nd.data_ptr(),
                           1 / 16, o.data_ptr(), part.data_ptr(), T, H, 512, splits, None)
        cuda.cuda.synchronize()
        what = f"seed {seed} case {it}: T={T} H={H} n={n} splits={splits} q8={scd is not None}"
        assert rc == 0, what
        assert bool((part[part_floats:] == 7.0).all()), what + ": wrote past the caller's part buffer"
        check_close(o.cpu().numpy(), oracle.mla_attn_ref(q, attended, sel, cnt, 1 / 16), what)
    st = C.c_int32(-1)
    assert L.gs_mla_attn_status(C.byref(st), None) == 0 and st.value == 0
