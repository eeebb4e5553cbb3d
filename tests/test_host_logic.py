"""CPU tests of the host-side multi-GPU logic: shard ranges, longest-first assignment, and a
world-size-2 gloo run of the sharded decode (records from the oracle, exchange by all-gather)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_cover_exactly(pkg):
    for n in (0, 1, 15, 16, 17, 4096, 131072, 131071):
        for world in (1, 2, 4, 8):
            for align in (1, 16, 64):
                got = [pkg.shard_rows(n, world, r, align) for r in range(world)]
                assert got[0][0] == 0 and got[-1][1] == n
                for (a, b), (c, d) in zip(got, got[1:]):
                    assert b == c and a <= b
                for lo, hi in got[:-1]:
                    assert hi == n or (hi - lo) % align == 0


def test_lpt_assign_balances(pkg):
    rng = np.random.default_rng(0)
    lens = rng.integers(1024, 65537, size=64).tolist()
    for world in (1, 2, 4, 8):
        owners, load = pkg.lpt_assign(lens, world)
        assert sorted(i for o in owners for i in o) == list(range(64))
        assert sum(load) == sum(lens)
        assert max(load) <= sum(lens) / world + max(lens)
        assert max(load) / (sum(load) / world) < 1.05
    owners, load = pkg.lpt_assign([], 4)
    assert owners == [[], [], [], []] and load == [0, 0, 0, 0]


def _gloo_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib

    import torch
    import torch.distributed as dist
    from oracle import oracle_py as O
    sharded = importlib.import_module("glm-ssd_b200.sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(77)
    n, H, T = 1500, 4, 2
    q = rng.standard_normal((1, T, H, 576)).astype(np.float16)
    cache = (rng.standard_normal((n, 576)) * 0.5).astype(np.float16)
    lo, hi = sharded.shard_rows(n, world, rank, 16)

    def local_partial():
        # a rank holds only its rows; only the last non-empty shard applies the causal tail
        rec = O.mla_decode(q, cache, [n], 1 / 16, part_range=(lo, hi)).reshape(T * H, 514)
        block = np.concatenate([rec[:, :512].ravel(), rec[:, 512:].ravel()])
        return torch.from_numpy(block)

    def combine(blocks, world_):
        b = blocks.numpy().reshape(world_, -1)
        acc = b[:, :T * H * 512].reshape(world_, T * H, 512)
        ml = b[:, T * H * 512:].reshape(world_, T * H, 2)
        parts = np.concatenate([acc, ml], axis=2).transpose(1, 0, 2)
        return torch.from_numpy(O.combine(parts))

    o = sharded.sharded_decode(local_partial, combine).numpy().reshape(1, T, H, 512)
    full = O.mla_decode(q, cache, [n], 1 / 16)
    np.save(os.path.join(out_dir, f"err{rank}.npy"), np.abs(o - full).max())
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_decode_world2_gloo(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_gloo_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 1e-5
