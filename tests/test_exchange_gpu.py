"""Cross-GPU merge of a sequence-sharded decode (gs_shard_exchange): the protocol on one GPU, with the
ranks played one after the other, and the real thing on two GPUs in child processes."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, check_close, make_decode_inputs
from gpu_util import to_dev

pytestmark = pytest.mark.gpu
ST_EXCHANGE = 1 << 16


def _exchange(pkg, bufs, rank, epoch, nbytes, limit=0):
    x = pkg._lib.ShardExchange()
    arr = (C.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
    x.world, x.rank, x.epoch = len(bufs), rank, epoch
    x.peer_bufs = C.cast(arr, C.POINTER(C.c_void_p))
    x.buf_bytes = nbytes
    x.wait_limit_cycles = limit
    x._keep = arr
    return x


@pytest.mark.parametrize("T", [1, 2])
def test_protocol_with_ranks_played_in_turn(pkg, cuda, oracle, T):
    """Two ranks on one GPU cannot wait for each other, so rank 1 runs first with a short bound: it
    delivers its record and flags, then gives up waiting (status bit set, context intact).  Rank 0
    then finds everything it needs; rank 1 repeated completes as well."""
    n, H, world = 6000, 20, 2
    q, cache = make_decode_inputs(60 + T, 1, T, H, n)
    rows = T * H
    nbytes = int(pkg._lib.load().gs_shard_exchange_bytes(world, rows, 512))
    bufs = [cuda.zeros(nbytes, dtype=cuda.uint8, device="cuda") for _ in range(world)]
    qd = to_dev(cuda, q)
    shards, lens, ws, outs = [], [], [], []
    for r in range(world):
        lo, hi = pkg.shard_rows(n, world, r, 16)
        shards.append(to_dev(cuda, cache[lo:hi].copy()))
        lens.append(to_dev(cuda, np.array([hi - lo], np.int32)))
        ws.append(pkg.new_workspace(1, T, H))
        outs.append(cuda.zeros((1, T, H, 512), dtype=cuda.float32, device="cuda"))

    def run(r, epoch, limit):
        x = _exchange(pkg, bufs, r, epoch, nbytes, limit)
        pkg.mla_decode(qd, shards[r], lens[r], tail_causal=(r == world - 1), out=outs[r], workspace=ws[r], exchange=x)
        cuda.cuda.synchronize()
        return pkg.decode_status(ws[r])

    want = oracle.mla_decode(q, cache, [n], 1 / 16)
    # consecutive epochs (the record slots alternate with the epoch's parity); every epoch begins with a wait that runs
    # out on rank 1, after which both ranks complete that epoch and carry on with the next one: resynchronising after
    # a timed-out step needs nothing but the next consecutive epoch
    for epoch in (1, 2, 3):
        for w in ws:
            w[:8].zero_()
        assert run(1, epoch, 2_000_000) & ST_EXCHANGE      # nothing has set rank 0's flags yet
        assert run(0, epoch, 0) == 0
        check_close(outs[0].cpu().numpy(), want, f"rank 0, epoch {epoch}")
        ws[1][:8].zero_()
        assert run(1, epoch, 0) == 0
        check_close(outs[1].cpu().numpy(), want, f"rank 1, epoch {epoch}")


def test_exchange_argument_validation(pkg, cuda):
    q, cache = make_decode_inputs(70, 1, 1, 20, 100)
    bufs = [cuda.zeros(1024, dtype=cuda.uint8, device="cuda") for _ in range(2)]
    x = _exchange(pkg, bufs, 0, 1, 1024)
    with pytest.raises(RuntimeError, match="exchange"):
        pkg.mla_decode(to_dev(cuda, q), to_dev(cuda, cache), to_dev(cuda, np.array([100], np.int32)), exchange=x)


WORKER = r'''
import importlib, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["GS_ROOT"]); sys.path.insert(0, os.path.join(os.environ["GS_ROOT"], "tests"))
pkg = importlib.import_module("glm-ssd_b200")
from oracle import oracle_py as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rng = np.random.default_rng(123)
n, T, H = 20000, 2, 20
q = rng.standard_normal((1, T, H, 576), dtype=np.float32).astype(np.float16)
cache = (rng.standard_normal((n, 576), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
lo, hi = pkg.shard_rows(n, world, rank, 16)
ex = pkg.PeerExchange(T * H)
qd = torch.from_numpy(q).cuda(); shard = torch.from_numpy(cache[lo:hi].copy()).cuda()
lens = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
ws = pkg.new_workspace(1, T, H); out = torch.zeros((1, T, H, 512), dtype=torch.float32, device="cuda")
want = O.mla_decode(q, cache, [n], 1 / 16)
worst = 0.0
for step in range(6):
    x = ex.next(device_epoch=True)
    pkg.mla_decode(qd, shard, lens, tail_causal=(rank == world - 1), out=out, workspace=ws, exchange=x)
    torch.cuda.synchronize()
    assert pkg.decode_status(ws) == 0
    worst = max(worst, float(np.abs(out.cpu().numpy() - want).max()))
dist.barrier()
ex.close()
dist.destroy_process_group()
print(f"rank {rank} worst {worst:.3e}", flush=True)
assert worst <= 2e-3
'''


def test_two_gpus_peer_exchange(cuda, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, GS_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29547", str(script)],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("worst") == 2
