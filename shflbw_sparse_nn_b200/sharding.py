"""Multi-GPU use of the path: shard the dense dimension, replicate the sparse operand.

An output column of the SpMM (a token) and an output image of the SpConv depend only on
the same column / image of the dense input and on the (small) sparse weights.  So N GPUs
need no exchange to compute: every rank uploads the same Shfl-BW matrix and owns a
contiguous slice of the dense columns (SpMM) or of the batch (SpConv).  A collective is
needed only if the caller wants the full output on every rank; `gather_output` does that
with one all-gather (NCCL over NVLink on GPUs, gloo on CPU for tests).

One process per GPU (`torch.distributed`), as launched by `torchrun`.
"""
from __future__ import annotations

from typing import List, Tuple


def shard_range(total: int, rank: int, world: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous [begin, end) slice of `total` units for `rank`, sizes multiples of `multiple`.

    Units are dense columns (multiple=8: 16-byte rows of fp16) or images (multiple=1).
    The first ranks get the larger shards; trailing ranks may get an empty shard when
    total < world * multiple.
    """
    if total < 0 or world <= 0 or not (0 <= rank < world) or multiple <= 0:
        raise ValueError("bad shard arguments")
    if total % multiple:
        raise ValueError(f"total={total} is not a multiple of {multiple}")
    groups = total // multiple
    base, extra = divmod(groups, world)
    begin = rank * base + min(rank, extra)
    size = base + (1 if rank < extra else 0)
    return begin * multiple, (begin + size) * multiple


def shard_plan(total: int, world: int, multiple: int = 1) -> List[Tuple[int, int]]:
    return [shard_range(total, r, world, multiple) for r in range(world)]


def gather_output(local, dim: int, group=None):
    """All-gather equally-shaped local outputs along `dim` (0 = batch for NHWC SpConv,
    1 = dense columns for SpMM) and return the full tensor on every rank."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
