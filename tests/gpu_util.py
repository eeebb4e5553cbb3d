"""Helpers shared by the GPU parity tests."""
import numpy as np


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def paged_layout(rng, lens, d_qk=576, page_rows=64, sigma=0.5, spare_pages=3):
    """Random page pool + page table for sequences of the given lengths.  Rows past a sequence's length
    inside its last page are filled with NaN to prove the kernels never let them contribute."""
    lens = np.asarray(lens, np.int64)
    pages_per = -(-lens // page_rows)
    n_pages = int(pages_per.sum()) + spare_pages
    pool = (rng.standard_normal((n_pages * page_rows, d_qk), dtype=np.float32) * np.float32(sigma)).astype(np.float16)
    perm = rng.permutation(n_pages)
    stride = max(1, int(pages_per.max()))
    pt = np.zeros((len(lens), stride), np.int32)
    k = 0
    for b, L in enumerate(lens):
        for j in range(int(pages_per[b])):
            pt[b, j] = perm[k]
            k += 1
        if L % page_rows and L > 0:
            last = pt[b, int(pages_per[b]) - 1]
            pool[last * page_rows + int(L % page_rows): (last + 1) * page_rows] = np.float16(np.nan)
    return pool, pt
