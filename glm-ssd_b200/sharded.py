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
