"""Context-parallel read: the compressed history is split by token range over
the ranks of one NVSwitch box; every rank attends its shard for all queries
and heads, the (O, lse) partials are all-gathered and merged by log-sum-exp.

The reference has no history-sharded mode (its only multi-GPU mode is
head-sharding by all-to-all); the merge arithmetic is its two-way merge
(MGC/core.py:33-42) folded over the shards.  Encoding needs no exchange: the
rank that owns a token range encodes it.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


def shard_bounds(units: int, world: int) -> list[tuple[int, int]]:
    """Contiguous, balanced [start, stop) ranges of ``units`` (frames / segments) per rank;
    the first ``units % world`` ranks take one extra."""
    if world <= 0 or units < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(units, world)
    bounds, start = [], 0
    for rank in range(world):
        stop = start + base + (1 if rank < extra else 0)
        bounds.append((start, stop))
        start = stop
    return bounds


def gather_partials(out: torch.Tensor, lse: torch.Tensor, group=None):
    """All-gather (O [Q,H,D], lse [Q,H]) over the group -> per-rank lists, rank order."""
    world = dist.get_world_size(group)
    outs = torch.empty((world, *out.shape), dtype=out.dtype, device=out.device)
    lses = torch.empty((world, *lse.shape), dtype=lse.dtype, device=lse.device)
    if out.is_cuda:
        dist.all_gather_into_tensor(outs, out.contiguous(), group=group)
        dist.all_gather_into_tensor(lses, lse.contiguous(), group=group)
    else:  # gloo (host-logic tests): list form
        dist.all_gather(list(outs.unbind(0)), out.contiguous(), group=group)
        dist.all_gather(list(lses.unbind(0)), lse.contiguous(), group=group)
    return [(outs[r], lses[r]) for r in range(world)]


def merge_partials(partials):
    """P-way LSE merge on the device (an empty shard contributes (0, -inf))."""
    return ops.lse_merge(partials)


def gather_and_merge(out: torch.Tensor, lse: torch.Tensor, group=None):
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out, lse
    return merge_partials(gather_partials(out, lse, group))
