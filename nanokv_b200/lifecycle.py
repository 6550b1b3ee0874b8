"""Segment lifecycle of a rolling compressed cache: sink + recent window, pruning, windowed read.

The policy is the reference's (LingBot): of the ``committed_end`` tokens written so far the
attention sees the first ``sink_tokens`` and the most recent ``capacity - sink`` ones
(LB/lingbot_v2_cache_runtime.py:132-137); a segment is kept while it intersects either interval
(_prune_segments :194-204); a segment cut by the window contributes only the tokens inside it,
each with its absolute position (_decode_active_history :139-163).

Here nothing is decoded to apply the policy: a cut is a token sub-range of the struct-of-arrays
history (``CompressedHistory.view_tokens``), pruning moves the surviving segments' codes, scales,
ids and centre rows down in place, and the read attends each contiguous run of kept tokens with
the fused kernel and merges the runs by log-sum-exp.
"""
from __future__ import annotations

import torch

from . import attention, ops
from .cache import CompressedHistory
from .codec import Operator, QuantSpec, encode_append


def active_intervals(committed_end: int, capacity: int, sink_tokens: int) -> list[tuple[int, int]]:
    """[start, stop) runs of absolute positions the attention sees: the sink, then the recent tail."""
    if committed_end <= 0:
        return []
    sink_stop = min(sink_tokens, committed_end)
    recent_start = max(sink_stop, committed_end - max(capacity - sink_stop, 0))
    runs = [(0, sink_stop)] if sink_stop > 0 else []
    if recent_start < committed_end:
        runs.append((recent_start, committed_end))
    return runs


def kept_segments(ranges: list[tuple[int, int]], *, committed_end: int, capacity: int,
                  sink_tokens: int) -> list[int]:
    """Indices of the segments (given as absolute [start, stop) ranges) that survive a prune."""
    sink_stop = min(sink_tokens, committed_end)
    recent_start = max(sink_stop, committed_end - max(capacity - sink_stop, 0))
    return [i for i, (start, stop) in enumerate(ranges) if start < sink_stop or stop > recent_start]


def active_pieces(ranges: list[tuple[int, int]], *, committed_end: int, capacity: int,
                  sink_tokens: int) -> list[tuple[int, int, int]]:
    """(segment index, absolute start, absolute stop) of every piece of a segment inside the window,
    in cache order (segment by segment, sink piece before recent piece)."""
    pieces = []
    runs = active_intervals(committed_end, capacity, sink_tokens)
    for index, (start, stop) in enumerate(ranges):
        for left, right in runs:
            begin, end = max(start, left), min(stop, right)
            if begin < end:
                pieces.append((index, begin, end))
    return pieces


class RollingHistory:
    """K and V histories of one layer under the sink + recent policy.

    ``commit`` encodes one chunk as a new segment and records its absolute token range;
    ``prune`` drops the segments the window has left; ``read`` attends what the window shows.
    """

    def __init__(self, *, joint: int, rank: int, capacity_tokens: int, max_segments: int,
                 clusters: int = 64, quant: QuantSpec = QuantSpec(), device="cuda"):
        common = dict(joint=joint, rank=rank, capacity=capacity_tokens, max_segments=max_segments,
                      centers_per_segment=clusters, group=quant.group, scale_dtype=quant.scale_dtype,
                      device=device)
        self.k = CompressedHistory(**common)
        self.v = CompressedHistory(**common)
        self.quant, self.clusters = quant, clusters
        self.ranges: list[tuple[int, int]] = []       # absolute [start, stop) of every segment
        self.committed_end = 0

    def commit(self, rows_k: torch.Tensor, rows_v: torch.Tensor, op_k: Operator, op_v: Operator, *,
               global_start: int | None = None, iters: int = 2, seed_k: int = 0, seed_v: int = 0) -> None:
        start = self.committed_end if global_start is None else int(global_start)
        if start < self.committed_end:
            raise ValueError("segments are committed in increasing position order")
        count = rows_k.shape[0]
        if rows_v.shape[0] != count:
            raise ValueError("K and V chunks differ in length")
        encode_append(self.k, rows_k, op_k, self.quant, clusters=self.clusters, iters=iters, seed=seed_k)
        encode_append(self.v, rows_v, op_v, self.quant, clusters=self.clusters, iters=iters, seed=seed_v)
        self.ranges.append((start, start + count))
        self.committed_end = start + count

    def prune(self, *, capacity: int, sink_tokens: int) -> int:
        """Drop the segments outside the window; returns how many were dropped."""
        keep = kept_segments(self.ranges, committed_end=self.committed_end, capacity=capacity,
                             sink_tokens=sink_tokens)
        dropped = len(self.ranges) - len(keep)
        if dropped:
            self.k.retain(keep)
            self.v.retain(keep)
            self.ranges = [self.ranges[i] for i in keep]
        return dropped

    def window(self, *, capacity: int, sink_tokens: int):
        """Contiguous runs of kept tokens: [(cache token start, cache token stop, positions i32)]."""
        pieces = active_pieces(self.ranges, committed_end=self.committed_end, capacity=capacity,
                               sink_tokens=sink_tokens)
        offsets, total = [], 0
        for start, stop in self.ranges:
            offsets.append(total)
            total += stop - start
        runs: list[list] = []
        for index, begin, end in pieces:
            a = offsets[index] + begin - self.ranges[index][0]
            b = a + end - begin
            if runs and runs[-1][1] == a:
                runs[-1][1] = b
                runs[-1][2].append((begin, end))
            else:
                runs.append([a, b, [(begin, end)]])
        device = self.k.device
        return [(a, b, torch.cat([torch.arange(s, e, dtype=torch.int32, device=device) for s, e in spans]))
                for a, b, spans in runs]

    def read(self, q: torch.Tensor, op_k: Operator, op_v: Operator, *, capacity: int, sink_tokens: int,
             rope: "attention.RopeTable | None" = None, scale: float | None = None,
             status: torch.Tensor | None = None):
        """Attention of q over the windowed history -> (O, lse, positions)."""
        runs = self.window(capacity=capacity, sink_tokens=sink_tokens)
        if not runs:
            Q, H, D = q.shape
            return (torch.zeros_like(q), torch.full((Q, H), float("-inf"), device=q.device),
                    torch.empty(0, dtype=torch.int32, device=q.device))
        partials = []
        for a, b, positions in runs:
            partials.append(attention.codec_attention(
                q, self.k.view_tokens(a, b), self.v.view_tokens(a, b), op_k, op_v, scale=scale,
                status=status, rope=rope, positions=positions if rope is not None else None))
        out, lse = partials[0] if len(partials) == 1 else ops.lse_merge(partials)
        return out, lse, torch.cat([p for _, _, p in runs])
