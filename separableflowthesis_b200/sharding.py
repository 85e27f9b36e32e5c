"""Partitioning of one separation job over the GPUs of a node, one process per GPU.

The ops have no cross-sample coupling, and every output except gF2 is indexed by an image-1 pixel.
So a job of B samples with H1 image-1 rows is split into ``G_batch x G_rows`` shards:

* batch shards need no data exchange at all;
* row shards of the same sample each see all of F2 and produce a PARTIAL gF2 (a sum over their own
  image-1 pixels) that has to be summed over the row group;
* the parameters of the two attention Conv3d modules are shared by everything, so their gradients
  are summed over all ranks (what DistributedDataParallel does in the reference, train.py:397).

* the attention modules are 3x3x3 convolutions over (displacement, h1, w1), so a row shard needs the max/avg
  channels of one image-1 row above and below its block.  They are recomputed, not exchanged: a row shard runs
  on its block extended by one halo row per side (``halo_range``) and keeps the interior of the outputs; in the
  backward the halo rows of its feature gradient belong to the neighbouring shards and are handed over
  (``exchange_halo_grads``).

Only these reductions / exchanges use the process group (NCCL on GPUs, gloo in the CPU tests).
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


def make_shard(B: int, H1: int, world_size: int, rank: int, prefer: str = "batch") -> Shard:
    """``prefer="batch"``: batch first, rows for what is left (G_batch = gcd(B, world_size), G_rows = world_size /
    G_batch) -- no exchange on the data path when B is a multiple of the world size.  ``prefer="rows"``: every rank
    gets all samples and a block of image-1 rows (G_rows = world_size), the partition for batches smaller than the
    machine; it costs a halo row per side, a sum of gF2 over the ranks and F2 replicated on every rank."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    if prefer not in ("batch", "rows"):
        raise ValueError(f"prefer must be 'batch' or 'rows', got {prefer!r}")
    g_batch = math.gcd(B, world_size) if prefer == "batch" else 1
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


def allgather_batch(part: torch.Tensor, group) -> torch.Tensor:
    """Image-2 features of all samples from the slices the ranks of a row group hold (sample-major, equal slices):
    every rank copies 1/G of the samples from the host and the rest crosses NVLink once, instead of every rank
    copying all of F2 from the host."""
    world = dist.get_world_size(group)
    full = torch.empty((part.shape[0] * world,) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(full, part.contiguous(), group=group)
    return full


def reduce_scatter_batch(gF2: torch.Tensor, group) -> torch.Tensor:
    """The adjoint of ``allgather_batch``: sums the partial image-2 feature gradients over the row group and leaves
    every rank with the gradient of its own slice of the samples (half the traffic of an all-reduce, and the shard the
    producer of that slice's features needs)."""
    world = dist.get_world_size(group)
    if gF2.shape[0] % world != 0:
        raise ValueError(f"{gF2.shape[0]} samples do not split over {world} ranks")
    out = torch.empty((gF2.shape[0] // world,) + tuple(gF2.shape[1:]), dtype=gF2.dtype, device=gF2.device)
    if dist.get_backend(group) == "gloo":   # gloo has no reduce-scatter: all-reduce and keep the own slice
        full = gF2.contiguous().clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        out.copy_(full[r * out.shape[0]:(r + 1) * out.shape[0]])
        return out
    dist.reduce_scatter_tensor(out, gF2.contiguous(), op=dist.ReduceOp.SUM, group=group)
    return out


def reduce_parameter_grads(params: Iterable[torch.nn.Parameter], group=None) -> Optional[torch.Tensor]:
    """Sum the gradients of the shared attention parameters over all ranks with ONE flat all-reduce
    (a few hundred floats: latency-bound, so one message).  Returns the flat buffer.

    Every rank passes the same parameters in the same order, and the flat buffer always covers all of them: a
    parameter that got no gradient on this rank (a shard whose outputs did not reach the loss) contributes zeros
    and receives the sum of the others, so the ranks never all-reduce buffers of different lengths."""
    params = list(params)
    if not params:
        return None
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in params])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for p in params:
        n = p.numel()
        piece = flat[off:off + n].view_as(p)
        if p.grad is None:
            p.grad = piece.clone()
        else:
            p.grad.copy_(piece)
        off += n
    return flat


def halo_range(shard: Shard, H1: int):
    """Image-1 rows a row shard computes on: its block plus one row per side (inside the image), so that the
    attention stencil sees true neighbours at the shard borders.  Returns (e0, e1, i0, i1): rows [e0, e1) of the
    image, and the shard's own rows as [i0, i1) inside that extended block.  Without row sharding nothing is added."""
    if shard.g_rows == 1:
        return shard.r0, shard.r1, 0, shard.r1 - shard.r0
    e0, e1 = max(shard.r0 - 1, 0), min(shard.r1 + 1, H1)
    return e0, e1, shard.r0 - e0, shard.r1 - e0


def interior(t: torch.Tensor, shard: Shard, H1: int, dim: int) -> torch.Tensor:
    """The shard's own image-1 rows of a tensor computed on the extended block (rows along ``dim``)."""
    _, _, i0, i1 = halo_range(shard, H1)
    return t.narrow(dim, i0, i1 - i0)


def exchange_halo_grads(g_ext: torch.Tensor, shard: Shard, H1: int, row_group, dim: int = 2) -> torch.Tensor:
    """Feature gradient of the shard's own rows from the gradient on its extended block ``g_ext`` (image-1 rows
    along ``dim``): the interior, plus what the neighbouring shards computed for this shard's first and last row in
    their halos.  One small all-gather (two rows per rank) inside the row group."""
    e0, e1, i0, i1 = halo_range(shard, H1)
    own = g_ext.narrow(dim, i0, i1 - i0).clone()
    if shard.g_rows == 1:
        return own
    zero_row = torch.zeros_like(g_ext.narrow(dim, 0, 1))
    top = g_ext.narrow(dim, 0, 1) if i0 > 0 else zero_row                       # belongs to the shard above
    bottom = g_ext.narrow(dim, g_ext.shape[dim] - 1, 1) if e1 > shard.r1 else zero_row   # ... below
    mine = torch.cat((top, bottom), dim=dim).contiguous()
    gathered = [torch.empty_like(mine) for _ in range(shard.g_rows)]
    dist.all_gather(gathered, mine, group=row_group)
    ri = shard.rank % shard.g_rows
    if ri > 0:             # the shard above sent its bottom halo row = my first row
        own.narrow(dim, 0, 1).add_(gathered[ri - 1].narrow(dim, 1, 1))
    if ri < shard.g_rows - 1:   # the shard below sent its top halo row = my last row
        own.narrow(dim, own.shape[dim] - 1, 1).add_(gathered[ri + 1].narrow(dim, 0, 1))
    return own
