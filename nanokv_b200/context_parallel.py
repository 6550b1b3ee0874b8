"""Context-parallel read: the compressed history is split by token range over
the ranks of one NVSwitch box; every rank attends its shard for all queries
and heads, and the (O, lse) partials are merged by log-sum-exp.  Two exchanges:
``PeerExchange`` (the default on GPUs) -- every rank merges its slice of the
rows straight out of the peers' partial buffers over NVLink and stores the
merged rows into every rank's result buffer, one kernel for merge and
all-gather; and ``gather_and_merge`` -- NCCL all-gather of whole partials,
then a P-way merge on every rank (the plain form, P times the NVLink traffic).

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


def _aligned(nbytes: int) -> int:
    return (nbytes + 255) // 256 * 256


class PeerExchange:
    """Fused merge + all-gather of context-parallel partials over peer memory.

    Every rank owns one peer-visible block holding its partial (O, lse), its
    merged result and a few flag words; ``partial_out`` / ``partial_lse`` are the
    buffers the read kernel fills.  ``merge()`` is ONE launch per rank
    (nkv_cp_exchange_peer): the kernel tells every rank that this rank's partial
    is complete, waits until every rank has said so, loads its row slice of all P
    partials (P-1 of them over NVLink), stores the merged rows into all P result
    buffers, tells every rank that its slice has landed and waits for all slices
    to land here.  No collective, no host synchronisation; each rank moves
    2 x (P-1)/P of one partial instead of receiving P-1 whole ones.
    The same buffers serve every layer: the kernel's last wait also means that
    nobody still reads this rank's partial when the next read overwrites it.
    ``ordering="nccl"`` keeps the earlier form (nkv_cp_merge_peer between two
    four-byte all-reduces) for comparison.
    """

    def __init__(self, queries: int, heads: int, width: int, dtype: torch.dtype, device, group=None,
                 ordering: str = "flags"):
        if not dist.is_initialized():
            raise RuntimeError("PeerExchange needs an initialised process group")
        if ordering not in ("flags", "nccl"):
            raise ValueError("ordering is 'flags' or 'nccl'")
        self.group, self.device, self.ordering = group, torch.device(device), ordering
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shape, self.dtype = (queries, heads, width), dtype
        self.rows = queries * heads
        itemsize = torch.empty((), dtype=dtype).element_size()
        out_bytes, lse_bytes = _aligned(self.rows * width * itemsize), _aligned(self.rows * 4)
        flag_bytes = _aligned(ops.PEER_FLAG_WORDS * 4)
        self._offsets = {"part_out": 0, "part_lse": out_bytes, "out": out_bytes + lse_bytes,
                         "lse": 2 * out_bytes + lse_bytes, "flags": 2 * (out_bytes + lse_bytes)}
        self.nbytes = 2 * (out_bytes + lse_bytes) + flag_bytes
        self.block = ops.PeerBuffer.allocate(self.nbytes, self.device)
        self.flags = self.block.tensor(self._offsets["flags"], (ops.PEER_FLAG_WORDS,), torch.int32)
        self.flags.zero_()
        torch.cuda.synchronize(self.device)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.block.handle, group=group)
        self.blocks = [self.block if r == self.rank else
                       ops.PeerBuffer.open(handles[r], self.nbytes, self.device)
                       for r in range(self.world)]
        self.partial_out = self.block.tensor(self._offsets["part_out"], self.shape, dtype)
        self.partial_lse = self.block.tensor(self._offsets["part_lse"], (queries, heads), torch.float32)
        self.out = self.block.tensor(self._offsets["out"], self.shape, dtype)
        self.lse = self.block.tensor(self._offsets["lse"], (queries, heads), torch.float32)
        self.row_begin, self.row_end = shard_bounds(self.rows, self.world)[self.rank]
        self.epoch = 0
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._fence()   # every rank has mapped every block (and cleared its flags) before anyone uses one

    def _fence(self) -> None:
        dist.all_reduce(self._token, group=self.group)

    def merge(self, status: torch.Tensor | None = None):
        """Partials in ``partial_out`` / ``partial_lse`` on every rank -> merged (out, lse),
        identical on every rank.  Stream-ordered; no host synchronisation."""
        pointers = {name: [blk.pointer + off for blk in self.blocks]
                    for name, off in self._offsets.items()}
        if self.ordering == "nccl":
            self._fence()
            ops.cp_merge_peer(pointers["part_out"], pointers["part_lse"], pointers["out"], pointers["lse"],
                              rows=self.rows, width=self.shape[2], row_begin=self.row_begin,
                              row_end=self.row_end, dtype=self.dtype, device=self.device)
            self._fence()
            return self.out, self.lse
        self.epoch += 1
        ops.cp_exchange_peer(pointers["part_out"], pointers["part_lse"], pointers["out"], pointers["lse"],
                             pointers["flags"], rank=self.rank, rows=self.rows, width=self.shape[2],
                             row_begin=self.row_begin, row_end=self.row_end, dtype=self.dtype,
                             epoch=self.epoch, device=self.device, status=status)
        return self.out, self.lse

    def close(self) -> None:
        """Collective: unmap the peers' blocks, then free this rank's."""
        torch.cuda.synchronize(self.device)
        self.partial_out = self.partial_lse = self.out = self.lse = self.flags = None
        for r, blk in enumerate(self.blocks):
            if r != self.rank:
                blk.release()
        dist.barrier(group=self.group)
        self.block.release()
