"""Partitioning of one separation job over the GPUs of a node, one process per GPU.

The ops have no cross-sample coupling, and every output except gF2 is indexed by an image-1 pixel.
So a job of B samples with H1 image-1 rows is split into ``G_batch x G_rows`` shards:

* batch shards need no data exchange at all;
* row shards of the same sample each see all of F2 and produce a PARTIAL gF2 (a sum over their own
  image-1 pixels) that has to be summed over the row group;
* the parameters of the two attention Conv3d modules are shared by everything, so their gradients
  are summed over all ranks (what DistributedDataParallel does in the reference, train.py:397).

Only these two reductions use the process group (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rank: int
    world_size: int
    g_batch: int          # number of batch groups
    g_rows: int           # ranks sharing one batch group, each owning a block of image-1 rows
    b0: int
    b1: int               # samples [b0, b1)
    r0: int
    r1: int               # image-1 rows [r0, r1)

    @property
    def row_group_ranks(self) -> List[int]:
        first = (self.rank // self.g_rows) * self.g_rows
        return list(range(first, first + self.g_rows))


def split_range(n: int, parts: int, index: int):
    """Contiguous near-equal split: the first ``n % parts`` parts get one extra element."""
    base, extra = divmod(n, parts)
    start = index * base + min(index, extra)
    return start, start + base + (1 if index < extra else 0)


def make_shard(B: int, H1: int, world_size: int, rank: int) -> Shard:
    """Batch first, rows for what is left: G_batch = gcd(B, world_size), G_rows = world_size / G_batch."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    g_batch = math.gcd(B, world_size)
    g_rows = world_size // g_batch
    if g_rows > H1:
        raise ValueError(f"{g_rows} row shards for {H1} image-1 rows")
    bi, ri = divmod(rank, g_rows)
    b0, b1 = split_range(B, g_batch, bi)
    r0, r1 = split_range(H1, g_rows, ri)
    return Shard(rank, world_size, g_batch, g_rows, b0, b1, r0, r1)


def new_row_groups(world_size: int, g_rows: int):
    """One process group per set of ranks that share samples; every rank must call this with the same
    arguments (torch.distributed.new_group is collective).  Returns this rank's group, or None when
    rows are not sharded."""
    if g_rows == 1:
        return None
    mine = None
    rank = dist.get_rank()
    for first in range(0, world_size, g_rows):
        ranks = list(range(first, first + g_rows))
        grp = dist.new_group(ranks)
        if rank in ranks:
            mine = grp
    return mine


def reduce_row_partial(gF2: torch.Tensor, row_group) -> torch.Tensor:
    """Sum the partial image-2 feature gradients of the ranks that share a sample."""
    if row_group is not None:
        dist.all_reduce(gF2, op=dist.ReduceOp.SUM, group=row_group)
    return gF2


def reduce_parameter_grads(params: Iterable[torch.nn.Parameter], group=None) -> Optional[torch.Tensor]:
    """Sum the gradients of the shared attention parameters over all ranks with ONE flat all-reduce
    (a few hundred floats: latency-bound, so one message).  Returns the flat buffer."""
    params = [p for p in params if p.grad is not None]
    if not params:
        return None
    flat = torch.cat([p.grad.reshape(-1) for p in params])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for p in params:
        n = p.grad.numel()
        p.grad.copy_(flat[off:off + n].view_as(p.grad))
        off += n
    return flat
