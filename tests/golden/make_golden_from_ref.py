"""Generate the golden fixtures that pin the CPU oracle: outputs of the reference engine's own CUDA
kernels (gs_mla_attn, gs_f32_to_f16, gs_quant_q8_rows, gs_idx_pool / gs_idx_score / gs_idx_select), compiled unmodified into oracle/_ref/libglmssd_ref.so by
oracle/build.py and run on a GPU.

    python tests/golden/make_golden_from_ref.py <out_dir>

writes ref_*.npz, refq8_cache.npz and refidx_pool_score_select.npz into <out_dir>; the committed copies live beside this script.  Inputs are seeded
(numpy default_rng) so the run is reproducible.  Needs a CUDA device; not used at test time.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libglmssd_ref.so")

CASES = [  # name, seed, T, H, n, ctx, splits, dense
    ("decode_dense", 101, 1, 16, 200, 256, 16, True),
    ("mtp_verify", 102, 2, 32, 129, 160, 4, True),
    ("sparse_list", 103, 3, 16, 100, 300, 4, False),
    ("prefill_block", 104, 12, 16, 40, 64, 1, True),
    ("empty_and_one", 105, 2, 16, 1, 32, 16, True),
]


def main(out_dir: str) -> None:
    os.makedirs(out_dir, exist_ok=True)
    ref = C.CDLL(REF_SO)
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    ref.gs_mla_attn.restype = i32
    ref.gs_mla_attn.argtypes = [vp, vp, vp, vp, i32, vp, f32, vp, vp, i32, i32, i32, i32, vp]
    ref.gs_f32_to_f16.restype = i32
    ref.gs_f32_to_f16.argtypes = [vp, vp, C.c_int64, vp]
    for name, seed, T, H, n, ctx, splits, dense in CASES:
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
        qd, cd = torch.from_numpy(q).cuda(), torch.from_numpy(Cc).cuda()
        sd, nd = torch.from_numpy(sel).cuda(), torch.from_numpy(cnt).cuda()
        o = torch.zeros((T, H, 512), dtype=torch.float32, device="cuda")
        part = torch.zeros(T * (H // 16) * splits * (16 * 512 + 32), dtype=torch.float32, device="cuda")
        rc = ref.gs_mla_attn(qd.data_ptr(), cd.data_ptr(), None, sd.data_ptr(), stride, nd.data_ptr(), 1 / 16,
                             o.data_ptr(), part.data_ptr(), T, H, 512, splits, None)
        assert rc == 0, rc
        x = rng.standard_normal(2048, dtype=np.float32) * np.float32(10.0 ** rng.integers(-6, 4))
        xd = torch.from_numpy(x).cuda()
        yd = torch.zeros(2048, dtype=torch.float16, device="cuda")
        assert ref.gs_f32_to_f16(xd.data_ptr(), yd.data_ptr(), 2048, None) == 0
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), q=q, C=Cc.view(np.uint16), sel=sel, cnt=cnt,
                            scale=np.float32(1 / 16), o=o.cpu().numpy(), splits=np.int32(splits), append_x=x,
                            append_y=yd.cpu().numpy().view(np.uint16))
        print("wrote", name)
    # Q8 latent cache: the reference's quantiser and its attention over (int8 rows, f16 scales)
    ref.gs_quant_q8_rows.restype = i32
    ref.gs_quant_q8_rows.argtypes = [vp, vp, vp, C.c_int64, vp]
    rng = np.random.default_rng(201)
    T, H, n, ctx, splits = 2, 16, 90, 128, 4
    x = rng.standard_normal((ctx, 512), dtype=np.float32) * np.float32(0.5)
    x[3] = 0.0
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    sel = np.zeros((T, n + 4), np.int32)
    cnt = np.array([n - 1, n], np.int32)
    for t in range(T):
        sel[t, :cnt[t]] = rng.permutation(ctx)[:cnt[t]]
    xd = torch.from_numpy(x).cuda()
    c8 = torch.zeros((ctx, 512), dtype=torch.int8, device="cuda")
    cs = torch.zeros((ctx, 16), dtype=torch.float16, device="cuda")
    assert ref.gs_quant_q8_rows(xd.data_ptr(), c8.data_ptr(), cs.data_ptr(), ctx * 512, None) == 0
    qd, sd, nd = torch.from_numpy(q).cuda(), torch.from_numpy(sel).cuda(), torch.from_numpy(cnt).cuda()
    o = torch.zeros((T, H, 512), dtype=torch.float32, device="cuda")
    part = torch.zeros(T * (H // 16) * splits * (16 * 512 + 32), dtype=torch.float32, device="cuda")
    assert ref.gs_mla_attn(qd.data_ptr(), c8.data_ptr(), cs.data_ptr(), sd.data_ptr(), n + 4, nd.data_ptr(), 1 / 16,
                           o.data_ptr(), part.data_ptr(), T, H, 512, splits, None) == 0
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "refq8_cache.npz"), x=x, q8=c8.cpu().numpy(),
                        d=cs.cpu().numpy().view(np.uint16), q=q, sel=sel, cnt=cnt, scale=np.float32(1 / 16),
                        o=o.cpu().numpy())
    print("wrote q8_cache")
    make_indexer(ref, out_dir)


def make_indexer(ref, out_dir: str) -> None:
    """DSA k-pool indexer: the reference's gs_idx_pool over three consecutive chunks (a pool straddling a chunk
    boundary goes through the rings), gs_idx_score and gs_idx_select on the result (ops.cu:619-791).  Scores are
    continuous random values, so the k-th largest is unique and the selected set is well defined; the order inside
    sel is not fixed in the reference (slots are handed out by an atomic counter), so the fixture keeps each list
    sorted."""
    vp, i32, f32, i64 = C.c_void_p, C.c_int, C.c_float, C.c_int64
    for fn, args in (("gs_idx_pool", [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
                     ("gs_idx_score", [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, vp]),
                     ("gs_idx_select", [vp, i64, i32, i32, i32, i32, vp, i32, vp, vp])):
        getattr(ref, fn).restype = i32
        getattr(ref, fn).argtypes = args
    rng = np.random.default_rng(301)
    Dk, kpool, Hq, top_k = 128, 4, 8, 6  # top_k counts pools
    chunks = [5, 9, 17]                   # tokens per chunk: 31 positions, 7 complete pools
    n_pos = sum(chunks)
    kc = rng.standard_normal((n_pos, Dk), dtype=np.float32)
    gc = rng.standard_normal((n_pos, Dk), dtype=np.float32)
    ape = rng.standard_normal((kpool, Dk), dtype=np.float32) * np.float32(0.3)
    pools = n_pos // kpool + 1
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rk, rg = torch.zeros((kpool, Dk), device="cuda"), torch.zeros((kpool, Dk), device="cuda")
    P = torch.zeros((pools, Dk), device="cuda")
    aped = dev(ape)
    p0 = 0
    for T in chunks:
        kd, gd = dev(kc[p0:p0 + T]), dev(gc[p0:p0 + T])
        assert ref.gs_idx_pool(kd.data_ptr(), gd.data_ptr(), rk.data_ptr(), rg.data_ptr(), aped.data_ptr(), P.data_ptr(), p0, T,
                               Dk, kpool, None) == 0
        torch.cuda.synchronize()
        p0 += T
    # queries at the last chunk's positions
    T, pos0 = chunks[-1], n_pos - chunks[-1]
    q = rng.standard_normal((T, Hq, Dk), dtype=np.float32)
    w = rng.standard_normal((T, Hq), dtype=np.float32)
    stride = pools
    score = torch.zeros((T, stride), device="cuda")
    assert ref.gs_idx_score(dev(q).data_ptr(), dev(w).data_ptr(), P.data_ptr(), score.data_ptr(), stride, pos0, T, kpool, Hq, Dk,
                            1 / np.sqrt(Dk), None) == 0
    sel_stride = (top_k + 1) * kpool
    sel = torch.full((T, sel_stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(T, dtype=torch.int32, device="cuda")
    assert ref.gs_idx_select(score.data_ptr(), stride, pos0, T, kpool, top_k, sel.data_ptr(), sel_stride, cnt.data_ptr(), None) == 0
    torch.cuda.synchronize()
    sel_h, cnt_h = sel.cpu().numpy(), cnt.cpu().numpy()
    for t in range(T):
        sel_h[t, :cnt_h[t]] = np.sort(sel_h[t, :cnt_h[t]])
        sel_h[t, cnt_h[t]:] = -1
    np.savez_compressed(os.path.join(out_dir, "refidx_pool_score_select.npz"), kc=kc, gc=gc, ape=ape, chunks=np.array(chunks, np.int32),
                        kpool=np.int32(kpool), top_k=np.int32(top_k), P=P.cpu().numpy(), rk=rk.cpu().numpy(), rg=rg.cpu().numpy(),
                        q=q, w=w, pos0=np.int32(pos0), scale=np.float32(1 / np.sqrt(Dk)), score=score.cpu().numpy(),
                        sel_sorted=sel_h, cnt=cnt_h)
    print("wrote indexer")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out"))
