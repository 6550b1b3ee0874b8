"""Pre-allocated compressed history cache (one K or V tensor of one layer).

Struct-of-arrays in HBM, grown in place by appends:
  codes   u8  [capacity, rank/2]      two INT4 per byte
  scales  16b [capacity, rank/group]  bf16 (reference) or fp16
  ids     u8 / i16 [capacity]         centre id inside the token's segment
  centers bf16 [center_capacity, J]   every segment's centre table, stacked
  seg_start / seg_center_row  i32     segment table (device copy + host mirror)
A segment is one encoded chunk; it owns a token range and a centre table, as
the reference's immutable per-chunk payloads do (MGM/nanokv_codec.py:352-365,
concat_values :600-609; LB/lingbot_v2_kv_codec.py:288-297).
"""
from __future__ import annotations

import torch

from . import ops
from .ops import HistoryView


class CompressedHistory:
    def __init__(self, *, joint: int, rank: int, capacity: int, max_segments: int,
                 centers_per_segment: int, group: int | None = None,
                 scale_dtype: torch.dtype = torch.bfloat16, device="cuda",
                 center_width: int | None = None, shared_centers: bool = False):
        if rank % 2:
            raise ValueError("rank must be even")
        self.joint, self.rank = int(joint), int(rank)
        self.group = self.rank if group is None else int(group)
        if self.rank % self.group:
            raise ValueError(f"group {self.group} must divide rank {self.rank}")
        self.capacity, self.max_segments = int(capacity), int(max_segments)
        self.centers_per_segment = int(centers_per_segment)
        device = torch.device(device)
        self.device = device
        width = self.joint if center_width is None else int(center_width)
        self.codes = torch.zeros(self.capacity, self.rank // 2, dtype=torch.uint8, device=device)
        self.scales = torch.zeros(self.capacity, self.rank // self.group, dtype=scale_dtype,
                                  device=device)
        self.ids = torch.zeros(self.capacity, dtype=ops.id_dtype(self.centers_per_segment),
                               device=device)
        # shared_centers: one externally supplied table serves every segment (fixed-centre form)
        self.shared_centers = bool(shared_centers)
        table_segments = 1 if self.shared_centers else self.max_segments
        self.centers = torch.zeros(table_segments * self.centers_per_segment, width,
                                   dtype=torch.bfloat16, device=device)
        self.seg_start = torch.zeros(self.max_segments + 1, dtype=torch.int32, device=device)
        self.seg_center_row = torch.zeros(self.max_segments, dtype=torch.int32, device=device)
        self._starts = [0]
        self._center_rows: list[int] = []
        self._center_used = 0

    # ------------------------------------------------------------------ bookkeeping
    @property
    def tokens(self) -> int:
        return self._starts[-1]

    @property
    def segments(self) -> int:
        return len(self._center_rows)

    def reserve_segment(self, count: int, clusters: int):
        """Claim the next token range and centre rows; returns (offset, centre rows view)."""
        if count <= 0:
            raise ValueError("a segment needs at least one token")
        if self.tokens + count > self.capacity:
            raise ValueError(f"history capacity {self.capacity} exceeded")
        if self.segments + 1 > self.max_segments:
            raise ValueError(f"segment capacity {self.max_segments} exceeded")
        if self.shared_centers:
            if clusters > self.centers.shape[0]:
                raise ValueError("centre table capacity exceeded")
            offset, row = self.tokens, 0
            self._center_used = max(self._center_used, clusters)
        else:
            if self._center_used + clusters > self.centers.shape[0]:
                raise ValueError("centre table capacity exceeded")
            offset, row = self.tokens, self._center_used
            self._center_used += clusters
        self._starts.append(offset + count)
        self._center_rows.append(row)
        index = self.segments - 1
        # two tiny async H2D-free updates of the device segment table
        self.seg_start[index + 1].fill_(offset + count)
        self.seg_center_row[index].fill_(row)
        return offset, self.centers[row:row + clusters]

    def view(self, start_segment: int = 0, stop_segment: int | None = None) -> HistoryView:
        """ABI view of a run of whole segments (default: everything)."""
        stop_segment = self.segments if stop_segment is None else stop_segment
        if not 0 <= start_segment <= stop_segment <= self.segments:
            raise ValueError("bad segment range")
        t0, t1 = self._starts[start_segment], self._starts[stop_segment]
        if start_segment == 0:
            seg_start = self.seg_start
        else:  # token offsets relative to the sliced arrays
            seg_start = (self.seg_start[start_segment:stop_segment + 1] - t0).to(torch.int32)
        return HistoryView(
            codes=self.codes[t0:], scales=self.scales[t0:], ids=self.ids[t0:],
            centers=self.centers, seg_start=seg_start,
            seg_center_row=self.seg_center_row[start_segment:],
            tokens=t1 - t0, segments=stop_segment - start_segment, rank=self.rank,
            group=self.group)

    def view_tokens(self, start: int, stop: int) -> HistoryView:
        """ABI view of the token range [start, stop), which may cut segments: the arrays are
        offset to ``start`` and the segment table is shifted and clipped to the range, so a cut
        segment simply starts at 0 or ends at ``stop - start``."""
        if not 0 <= start <= stop <= self.tokens:
            raise ValueError("bad token range")
        if start == stop:
            return HistoryView(codes=self.codes[start:], scales=self.scales[start:], ids=self.ids[start:],
                               centers=self.centers, seg_start=self.seg_start,
                               seg_center_row=self.seg_center_row, tokens=0, segments=0,
                               rank=self.rank, group=self.group)
        first = max(i for i in range(self.segments) if self._starts[i] <= start)
        last = min(i for i in range(self.segments) if self._starts[i + 1] >= stop)
        seg_start = (self.seg_start[first:last + 2] - start).clamp_(0, stop - start).to(torch.int32)
        return HistoryView(
            codes=self.codes[start:], scales=self.scales[start:], ids=self.ids[start:],
            centers=self.centers, seg_start=seg_start, seg_center_row=self.seg_center_row[first:],
            tokens=stop - start, segments=last - first + 1, rank=self.rank, group=self.group)

    def retain(self, keep: list[int]) -> None:
        """Keep only the listed segments (increasing order), moving their codes, scales, ids and
        centre rows down in place and rebuilding the segment table.  Device copies only: one per
        array and run of consecutive kept segments."""
        keep = [int(i) for i in keep]
        if keep != sorted(set(keep)) or any(not 0 <= i < self.segments for i in keep):
            raise ValueError("segments to keep must be distinct, increasing and in range")
        starts, rows, token_cursor, row_cursor = [0], [], 0, 0

        def move(array, dst, src, count):
            """array[dst:dst+count] = array[src:src+count] with dst < src; staged when they overlap."""
            source = array[src:src + count]
            array[dst:dst + count].copy_(source.clone() if dst + count > src else source)

        runs, position = [], 0                     # runs of consecutive kept segments move as one block
        while position < len(keep):
            end = position
            while end + 1 < len(keep) and keep[end + 1] == keep[end] + 1:
                end += 1
            runs.append((keep[position], keep[end]))
            position = end + 1
        for first, last in runs:
            src, count = self._starts[first], self._starts[last + 1] - self._starts[first]
            if src != token_cursor and count:
                for array in (self.codes, self.scales, self.ids):
                    move(array, token_cursor, src, count)
            if not self.shared_centers:
                src_row = self._center_rows[first]
                next_row = self._center_rows[last + 1] if last + 1 < self.segments else self._center_used
                if src_row != row_cursor and next_row > src_row:
                    move(self.centers, row_cursor, src_row, next_row - src_row)
            for index in range(first, last + 1):
                rows.append(0 if self.shared_centers else self._center_rows[index] - src_row + row_cursor)
                starts.append(token_cursor + self._starts[index + 1] - src)
            token_cursor += count
            if not self.shared_centers:
                row_cursor += next_row - src_row
        self._starts, self._center_rows = starts, rows
        if not self.shared_centers:
            self._center_used = row_cursor
        table = torch.zeros(self.max_segments + 1, dtype=torch.int32)
        table[:len(starts)] = torch.tensor(starts, dtype=torch.int32)
        self.seg_start.copy_(table.to(self.device), non_blocking=True)
        row_table = torch.zeros(self.max_segments, dtype=torch.int32)
        row_table[:len(rows)] = torch.tensor(rows, dtype=torch.int32) if rows else row_table[:0]
        self.seg_center_row.copy_(row_table.to(self.device), non_blocking=True)

    def resident_bytes(self) -> int:
        """Bytes of payload actually in use (codes, scales, ids, centre tables)."""
        per_token = self.rank // 2 + 2 * (self.rank // self.group) + self.ids.element_size()
        return self.tokens * per_token + self._center_used * self.centers.shape[1] * 2


class PackedRows:
    """Rows of one payload segment as the kernels read them (codes, scales, centre ids and table in
    the payload's packed form) with the operator mean f32 [J]; after a token selection ``visible``
    lists the kept rows.  It stands where the reference hands a dequantised latent tensor to its
    readers (MGM/nanokv_codec.py direct_latent_pair_segments): here no latent row exists in HBM."""

    def __init__(self, history: CompressedHistory, mean: torch.Tensor, visible: torch.Tensor | None = None):
        self.history, self.mean, self.visible = history, mean, visible

    @property
    def tokens(self) -> int:
        return self.history.tokens if self.visible is None else int(self.visible.numel())
