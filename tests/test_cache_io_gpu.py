"""Cache persistence for paged caches: gs_cache_export_rows / gs_cache_import_rows move a sequence between a paged
pool and the position-major byte layout the reference saves and restores (crates/engine/src/forward.rs:654-695,
crates/engine/src/session.rs:152-204).  Byte work: everything here is compared bit for bit."""
import numpy as np
import pytest

from conftest import check_close
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _pages(rng, n_pages_total, need):
    return rng.permutation(n_pages_total)[:need].astype(np.int32)


def _export(torch, L, pool, pages, page_rows, row0, upto, unit, host=False):
    dst = torch.zeros(max(upto, 1) * unit, dtype=torch.uint8, device="cuda") if not host else torch.zeros(max(upto, 1) * unit, dtype=torch.uint8).pin_memory()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.gs_cache_export_rows(pool.data_ptr(), pool.shape[0], None if pages is None else pages.data_ptr(), 0 if pages is None else pages.numel(),
                                page_rows, row0, upto, unit, dst.data_ptr(), st.data_ptr(), None)
    assert rc == 0, L.gs_attn_last_error_string()
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return dst


@pytest.mark.parametrize("unit,upto", [(1152, 1000), (1024, 64), (512, 777), (32, 777), (1152, 1), (6, 130), (1152, 0)])
def test_dense_export_import_into_permuted_pool_round_trip(pkg, cuda, unit, upto):
    """dense cache -> export -> import into a paged pool with a random page order -> re-export: byte-identical, and a
    differently permuted second pool gives the same bytes again."""
    torch = cuda
    L = pkg._lib.load()
    rng = np.random.default_rng(unit + upto)
    ctx = max(upto, 1) + 70
    dense = torch.from_numpy(rng.integers(0, 256, size=(ctx, unit), dtype=np.uint8)).cuda()
    flat = _export(torch, L, dense, None, 0, 0, upto, unit)
    assert np.array_equal(flat.cpu().numpy()[:upto * unit], dense.cpu().numpy()[:upto].ravel())  # save_state's bytes (forward.rs:675-679)
    page_rows = 64
    need = -(-max(upto, 1) // page_rows)
    for seed in (1, 2):
        n_total = need + 5
        pages = to_dev(torch, _pages(np.random.default_rng(seed), n_total, need))
        pool = torch.full((n_total * page_rows, unit), 0xEE, dtype=torch.uint8, device="cuda")
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert L.gs_cache_import_rows(pool.data_ptr(), pool.shape[0], pages.data_ptr(), need, page_rows, 0, upto, unit, flat.data_ptr(),
                                      st.data_ptr(), None) == 0
        again = _export(torch, L, pool, pages, page_rows, 0, upto, unit, host=(seed == 2))  # second time into page-locked host memory
        assert np.array_equal(again.cpu().numpy()[:upto * unit], flat.cpu().numpy()[:upto * unit])
        # rows the import did not name are untouched
        ph, pg = pool.cpu().numpy(), pages.cpu().numpy()
        named = np.zeros(n_total * page_rows, bool)
        for i in range(upto):
            named[pg[i // page_rows] * page_rows + i % page_rows] = True
        assert (ph[~named] == 0xEE).all()


def test_attention_is_the_same_after_a_save_and_a_load_into_other_pages(pkg, cuda, oracle):
    """A 3000-position sequence in a dense cache is exported and imported into a paged pool; the paged decode over the
    pool then reads the same rows as the dense decode, through other addresses: both are checked against the oracle
    (attention tolerance) and against each other (2e-5: the dense call cuts the rows into 16-row units, the paged one
    into pages, so the partial sums are merged in another order)."""
    torch = cuda
    L = pkg._lib.load()
    rng = np.random.default_rng(9)
    n, T, H = 3000, 1, 20
    q = rng.standard_normal((1, T, H, 576), dtype=np.float32).astype(np.float16)
    cache = (rng.standard_normal((n + 8, 576), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    cd = to_dev(torch, cache)
    flat = _export(torch, L, cd.view(torch.uint8).view(n + 8, 1152), None, 0, 0, n, 1152)
    need = -(-n // 64)
    pages = to_dev(torch, _pages(rng, need + 3, need))
    pool = torch.zeros(((need + 3) * 64, 576), dtype=torch.float16, device="cuda")
    assert L.gs_cache_import_rows(pool.data_ptr(), pool.shape[0], pages.data_ptr(), need, 64, 0, n, 1152, flat.data_ptr(), None, None) == 0
    lens = to_dev(torch, np.array([n], np.int32))
    o_dense = pkg.mla_decode(to_dev(torch, q), cd, lens, max_seq_len=n)
    o_paged = pkg.mla_decode(to_dev(torch, q), pool, lens, page_table=pages.view(1, -1), max_seq_len=n)
    torch.cuda.synchronize()
    a, b = o_dense.cpu().numpy(), o_paged.cpu().numpy()
    check_close(a, oracle.mla_decode(q, cache, [n], 1 / 16), "dense decode")
    assert np.abs(a - b).max() <= 2e-5


def test_q8_cache_rows_and_scales_round_trip(pkg, cuda, oracle):
    """A Q8 cache is two per-position buffers (int8 rows, f16 scales: forward.rs:659-663): each goes through the same
    calls with its own unit."""
    torch = cuda
    L = pkg._lib.load()
    rng = np.random.default_rng(10)
    n = 500
    x = rng.standard_normal((n, 512), dtype=np.float32)
    q8, d = oracle.quant_q8_rows(x)
    need = -(-n // 64)
    pages = to_dev(torch, _pages(rng, need + 2, need))
    for arr, unit in ((q8.view(np.uint8), 512), (d.view(np.uint8).reshape(n, 32), 32)):
        src = to_dev(torch, arr.reshape(-1))
        pool = torch.zeros(((need + 2) * 64, unit), dtype=torch.uint8, device="cuda")
        assert L.gs_cache_import_rows(pool.data_ptr(), pool.shape[0], pages.data_ptr(), need, 64, 0, n, unit, src.data_ptr(), None, None) == 0
        back = _export(torch, L, pool, pages, 64, 0, n, unit)
        assert np.array_equal(back.cpu().numpy(), arr.reshape(-1))


def test_bad_page_ids_are_skipped_and_flagged_and_bad_arguments_rejected(pkg, cuda):
    torch = cuda
    L = pkg._lib.load()
    pool = torch.zeros((4 * 64, 16), dtype=torch.uint8, device="cuda")
    pages = to_dev(torch, np.array([1, 99, -3], np.int32))
    dst = torch.full((192 * 16,), 7, dtype=torch.uint8, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.gs_cache_export_rows(pool.data_ptr(), pool.shape[0], pages.data_ptr(), 3, 64, 0, 192, 16, dst.data_ptr(), st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 1 << 19
    h = dst.cpu().numpy().reshape(192, 16)
    assert (h[:64] == 0).all() and (h[64:] == 7).all()
    assert L.gs_cache_export_rows(pool.data_ptr(), pool.shape[0], pages.data_ptr(), 2, 64, 0, 192, 16, dst.data_ptr(), None, None) == 1  # list too short
    assert L.gs_cache_export_rows(pool.data_ptr(), pool.shape[0], None, 0, 0, 200, 100, 16, dst.data_ptr(), None, None) == 1  # dense rows outside
