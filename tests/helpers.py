"""Shared helpers of the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

from nanokv_b200.cache import CompressedHistory
from nanokv_b200.codec import Operator
from oracle import nkv_oracle as oracle

BF16_REL_TOL = 2e-2   # attention outputs, bf16 path (relative to the largest reference magnitude)
F32_REL_TOL = 1e-3    # attention outputs, fp32 path


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-20))


def history_from_segments(segments, *, joint, rank, group=None, scale_dtype=torch.bfloat16,
                          capacity=None, device="cuda") -> CompressedHistory:
    """Load oracle-encoded segments into a device cache (read-path tests start from here)."""
    total = sum(int(s["shape"][1]) for s in segments)
    clusters = max([int(s["centers"].shape[1]) for s in segments] or [1])
    hist = CompressedHistory(joint=joint, rank=rank, capacity=capacity or max(total, 1),
                             max_segments=max(len(segments), 1), centers_per_segment=clusters,
                             group=group, scale_dtype=scale_dtype, device=device)
    for seg in segments:
        n = int(seg["shape"][1])
        c = int(seg["centers"].shape[1])
        offset, rows = hist.reserve_segment(n, c)
        rows.copy_(seg["centers"][0].to(torch.bfloat16))
        hist.codes[offset:offset + n].copy_(seg["packed"].reshape(n, rank // 2))
        hist.scales[offset:offset + n].copy_(seg["scale"].reshape(n, -1))
        ids = seg["ids"].reshape(-1)
        hist.ids[offset:offset + n].copy_(ids.to(torch.int16) if hist.ids.dtype == torch.int16 else ids)
    return hist


def device_operator(op: dict) -> Operator:
    return Operator(op["mean"], op["encoder"], op["decoder"], device="cuda")


def unpack_device_codes(codes: torch.Tensor, rank: int) -> torch.Tensor:
    flat = codes.cpu().reshape(-1)
    return oracle.unpack_int4(flat, flat.numel() * 2, (-1, rank))


def code_flip_report(got_codes: torch.Tensor, want_codes: torch.Tensor) -> dict:
    """Count differing INT4 codes and check that every flip is by one step."""
    diff = (got_codes.to(torch.int16) - want_codes.to(torch.int16)).abs()
    return {"total": int(diff.numel()), "flips": int((diff > 0).sum()),
            "max_step": int(diff.max()) if diff.numel() else 0,
            "rows_touched": int((diff > 0).any(-1).sum())}


def oracle_segments_of(hist: CompressedHistory, joint: int) -> list[dict]:
    """Device cache -> the oracle's segment dicts (what ``oracle.encode_rows`` returns, minus the
    encoder-side extras), so that a history encoded on the GPU can be read by the CPU oracle."""
    starts = list(hist._starts)
    segments = []
    for index in range(hist.segments):
        a, b = starts[index], starts[index + 1]
        first = 0 if hist.shared_centers else hist._center_rows[index]
        table = hist.centers[first:first + hist.centers_per_segment].cpu()
        codes = hist.codes[a:b].cpu()
        segments.append({
            "shape": (1, b - a, joint), "rank": hist.rank,
            "packed": codes.reshape(-1), "count": (b - a) * hist.rank,
            "codes": oracle.unpack_int4(codes.reshape(-1), (b - a) * hist.rank, (b - a, hist.rank)),
            "scale": hist.scales[a:b].cpu(), "centers": table[None],
            "ids": hist.ids[a:b].cpu().to(torch.int64).bitwise_and(0xFFFF)[None],
        })
    return segments
