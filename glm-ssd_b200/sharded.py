"""Multi-GPU forms of the decode path (one process per GPU, ``torch.distributed``).

* One long context sharded by contiguous sequence ranges: every rank attends its own rows and
  produces one (acc, m, l) record per query row; the records are exchanged and merged with the same
  arithmetic the reference uses between its intra-GPU splits (crates/cuda/kernels/ops.cu:539-574,
  "split" = rank).  Nothing else is partitioned.
* Many sequences: whole sequences are assigned to ranks by longest-processing-time-first on their
  KV length; there is no exchange.

The host-side logic here is backend-neutral so it runs under ``gloo`` on CPU in the tests; the
device work is injected by the caller.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    """Contiguous row range [lo, hi) of ``rank``: ceil(n/world) rows each, rounded up to ``align``,
    the last ranks possibly empty (the split rule of ops.cu:447-449 applied across GPUs)."""
    per = -(-n_rows // world)
    per = -(-per // align) * align
    lo = min(n_rows, rank * per)
    hi = min(n_rows, lo + per)
    return lo, hi


def lpt_assign(lengths: Sequence[int], world: int) -> tuple[list[list[int]], list[int]]:
    """Greedy longest-first assignment of sequences to ranks.  Returns (indices per rank, load per rank)."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    owners: list[list[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        owners[r].append(i)
        load[r] += int(lengths[i])
    for o in owners:
        o.sort()
    return owners, load


def exchange_parts(part: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one record block per rank -> [world, block] (every rank can then combine locally)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
    # views of one buffer, so the gathered blocks are contiguous for the combine kernel
    dist.all_gather([out[r] for r in range(world)], part.contiguous(), group=group)
    return out


def sharded_decode(local_partial: Callable[[], torch.Tensor], combine: Callable[[torch.Tensor, int], torch.Tensor],
                   group=None) -> torch.Tensor:
    """Run one sharded decode: ``local_partial()`` returns this rank's record block, the blocks are
    all-gathered, and ``combine(blocks, world)`` merges them."""
    part = local_partial()
    blocks = exchange_parts(part, group)
    return combine(blocks, dist.get_world_size(group))


class PeerExchange:
    """Exchange buffers for the peer-to-peer merge of a sequence-sharded decode (one per rank, mapped
    into every rank's process).  ``next()`` returns the ``gs_shard_exchange`` argument of the next call;
    every rank must call it in step.  Allocation and mapping happen here, once; the decode calls
    themselves allocate nothing."""

    def __init__(self, rows: int, d_v: int = 512, group=None, wait_limit_cycles: int = 0, world=None, rank=None,
                 handles=None):
        import ctypes as C

        from . import _lib
        self._C, self._lib = C, _lib
        L = _lib.load()
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        self.bytes = int(L.gs_shard_exchange_bytes(self.world, rows, d_v))
        self.wait_limit_cycles = wait_limit_cycles
        self.epoch = 0
        self._opened = []
        local = C.c_void_p()
        _lib.check(L.gs_peer_alloc(C.byref(local), self.bytes), "gs_peer_alloc")
        self.local = local.value
        handle = (C.c_ubyte * 64)()
        _lib.check(L.gs_peer_export(self.local, handle), "gs_peer_export")
        self.handle = bytes(handle)
        if handles is None:
            handles = [None] * self.world
            dist.all_gather_object(handles, self.handle, group=group)
        self.ptrs = (C.c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                self.ptrs[r] = self.local
            else:
                p = C.c_void_p()
                buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                _lib.check(L.gs_peer_open(buf, C.byref(p)), "gs_peer_open")
                self.ptrs[r] = p.value
                self._opened.append(p.value)

    def next(self, device_epoch: bool = False):
        """``device_epoch=True`` (on every call of every rank) keeps the epoch in the buffers: graph-capturable."""
        self.epoch += 1
        x = self._lib.ShardExchange()
        x.world, x.rank, x.epoch = self.world, self.rank, 0 if device_epoch else self.epoch
        x.peer_bufs = self._C.cast(self.ptrs, self._C.POINTER(self._C.c_void_p))
        x.buf_bytes = self.bytes
        x.wait_limit_cycles = self.wait_limit_cycles
        return x

    def close(self):
        L = self._lib.load()
        for p in self._opened:
            L.gs_peer_close(p)
        self._opened = []
        if self.local:
            L.gs_peer_free(self.local)
            self.local = None
