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

    def resident_bytes(self) -> int:
        """Bytes of payload actually in use (codes, scales, ids, centre tables)."""
        per_token = self.rank // 2 + 2 * (self.rank // self.group) + self.ids.element_size()
        return self.tokens * per_token + self._center_used * self.centers.shape[1] * 2
