"""LingBot rolling-cache attention on the B200 kernels.

Two entry points over the same cache dictionary the reference keeps per layer
(LB/lingbot_v2_cache_runtime.py:337-352, ``configure_cache``):

* ``codec_cache_attention_inputs`` has the reference's name, argument list, return value and side
  effects (LB/lingbot_v2_cache_runtime.py:263-334): windowed history K / V / positions with the
  current chunk appended, cut to ``max_attention_size``; commit + prune when the cache asks for it.
  It is the import-swap form: the caller still runs its own RoPE and attention on the returned
  rows, so K and V of the window are written to HBM once by the decode kernel.
* ``codec_cache_attention`` does the whole step and returns the attention output: the window is
  read straight from the packed payloads by the fused kernel (keys rotated in-kernel by their
  absolute positions), the current chunk is attended as plain rows, and the partial results are
  merged by log-sum-exp.  No history row is materialised.  Same cache side effects.

* ``attend`` is the NanoKV-Fast step with the reference's name, argument list and
  None-means-native-fallback contract (LB/codec_native_attention.py:588-817): protected tokens (sink
  frames, recent frames, anchor frames) at full width, the rest of the window through the layer's
  low-width readers, one global softmax.  Readers are registered (``register_reader``) with their
  policy instead of being read from a manifest directory.

The window policy (sink + recent, pruning, pieces of a cut segment) is ``lifecycle``'s.
"""
from __future__ import annotations

import os
from typing import Any

import torch

from . import attention, lifecycle, ops
from .lingbot_codec import decode_segments, encode_pair, history_from_payloads, operator_of


def configure_cache(cache: dict[str, Any], *, layer: int, sp_rank: int, options: dict[str, Any]) -> None:
    """Attach the run's options and the empty per-layer codec state."""
    cache.update(options)
    cache.update({"codec_layer": int(layer), "codec_sp_rank": int(sp_rank), "codec_segments": [],
                  "codec_committed_end": 0, "codec_commit": False, "codec_chunk_id": 0})


def _ranges(segments: list[dict]) -> list[tuple[int, int]]:
    return [(int(s["global_start"]), int(s["global_end"])) for s in segments]


def _prune_segments(segments: list[dict], *, committed_end: int, capacity: int, sink_tokens: int) -> list[dict]:
    keep = lifecycle.kept_segments(_ranges(segments), committed_end=committed_end, capacity=capacity,
                                   sink_tokens=sink_tokens)
    return [segments[i] for i in keep]


def _window(segments: list[dict], *, committed_end: int, capacity: int, sink_tokens: int):
    """(active segments, [(row start, row stop, position start)] over their stacked rows)."""
    if not segments or committed_end <= 0:
        return [], []
    ranges = _ranges(segments)
    pieces = lifecycle.active_pieces(ranges, committed_end=committed_end, capacity=capacity,
                                     sink_tokens=sink_tokens)
    used = sorted({index for index, _, _ in pieces})
    base, total = {}, 0
    for index in used:
        base[index] = total
        total += ranges[index][1] - ranges[index][0]
    runs = [(base[i] + begin - ranges[i][0], base[i] + end - ranges[i][0], begin) for i, begin, end in pieces]
    return [segments[i] for i in used], runs


def _positions(runs, device, dtype=torch.long) -> torch.Tensor:
    return torch.cat([torch.arange(p, p + (b - a), device=device, dtype=dtype) for a, b, p in runs])


def _decode_active_history(segments: list[dict], *, committed_end: int, capacity: int, sink_tokens: int,
                           dtype: torch.dtype, device, cache: dict | None = None):
    """(K [1,N,H,D], V [1,N,H,D], positions [N]) of the window, or None when it is empty: one
    decode launch per target over the rows the window shows (LB/lingbot_v2_cache_runtime.py:122-191)."""
    if cache is not None and cache.get("a1_controller") is not None:
        raise NotImplementedError("the A1 training controller is not part of the inference path")
    active, runs = _window(segments, committed_end=committed_end, capacity=capacity, sink_tokens=sink_tokens)
    if not runs:
        return None
    rows = torch.cat([torch.arange(a, b, device=device, dtype=torch.int32) for a, b, _ in runs])
    key, value = decode_segments(active, dtype=dtype, device=device, rows=rows)
    return key, value, _positions(runs, device)


def _cut(runs, current: int, *, protected: int, limit: int):
    """The reference's overflow rule on the concatenation [window rows..., current chunk]: keep the
    first ``protected`` rows and the newest ``limit - protected`` ones
    (LB/lingbot_v2_cache_runtime.py:301-314).  ``protected`` never exceeds the sink rows the window
    starts with, so the prefix lies in the history.  Returns (history runs, rows cut from the front
    of the current chunk)."""
    total = sum(b - a for a, b, _ in runs) + current
    if total <= limit:
        return runs, 0
    keep = ((0, protected), (max(protected, total - (limit - protected)), total))
    out, cursor = [], 0
    for a, b, p in runs:
        for low, high in keep:
            begin, end = max(cursor, low), min(cursor + b - a, high)
            if begin < end:
                out.append((a + begin - cursor, a + end - cursor, p + begin - cursor))
        cursor += b - a
    return out, min(current, max(0, keep[1][0] - cursor))


def _commit(cache: dict, key: torch.Tensor, value: torch.Tensor, *, current_start: int, capacity: int,
            sink_tokens: int) -> None:
    committed_end = int(cache.get("codec_committed_end", 0))
    current_end = current_start + int(key.shape[1])
    if cache.get("codec_commit", False):
        if current_start != committed_end:
            raise RuntimeError(f"non-causal codec commit: start={current_start}, committed={committed_end}")
        cache["codec_commit_start"] = current_start
        segments = cache.setdefault("codec_segments", [])
        segments.append(encode_pair(key, value, cache=cache))
        cache["codec_committed_end"] = current_end
        cache["codec_segments"] = _prune_segments(segments, committed_end=current_end, capacity=capacity,
                                                  sink_tokens=sink_tokens)
    for name, end in (("global_end_index", current_end), ("local_end_index", min(current_end, capacity))):
        if torch.is_tensor(cache.get(name)):
            cache[name].fill_(end)


@torch.no_grad()
def codec_cache_attention_inputs(cache: dict[str, Any], key: torch.Tensor, value: torch.Tensor, *,
                                 current_start: int, capacity: int, sink_tokens: int,
                                 max_attention_size: int):
    """history + current K / V [1,N,H,D] and positions [N]; commits the chunk when
    ``cache["codec_commit"]``.  ``key`` is pre-RoPE, ``value`` the raw projection."""
    segments = cache.setdefault("codec_segments", [])
    committed_end = int(cache.get("codec_committed_end", 0))
    device, current = key.device, int(key.shape[1])
    active, runs = _window(segments, committed_end=committed_end, capacity=capacity, sink_tokens=sink_tokens)
    protected = min(sink_tokens, committed_end, max_attention_size)
    kept, lead = _cut(runs, current, protected=protected, limit=max_attention_size)
    stop = current
    now = torch.arange(current_start + lead, current_start + stop, device=device)
    if kept:
        rows = torch.cat([torch.arange(a, b, device=device, dtype=torch.int32) for a, b, _ in kept])
        hist_k, hist_v = decode_segments(active, dtype=value.dtype, device=device, rows=rows)
        key_cache = torch.cat((hist_k, key[:, lead:stop]), dim=1)
        value_cache = torch.cat((hist_v, value[:, lead:stop]), dim=1)
        positions = torch.cat((_positions(kept, device), now))
    else:
        key_cache, value_cache, positions = key[:, lead:stop], value[:, lead:stop], now
    _commit(cache, key, value, current_start=current_start, capacity=capacity, sink_tokens=sink_tokens)
    return key_cache, value_cache, positions


@torch.no_grad()
def codec_cache_attention(cache: dict[str, Any], query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *,
                          current_start: int, capacity: int, sink_tokens: int, max_attention_size: int,
                          rope: "attention.RopeTable | None" = None, scale: float | None = None,
                          status: torch.Tensor | None = None):
    """Attention output [1,S,H,D] (and lse f32 [S,H]) of ``query`` over the window and the current chunk.

    ``query`` arrives rotated; ``key`` is pre-RoPE and is rotated here by ``rope`` at positions
    ``current_start + i``; the history's keys are rotated inside the fused kernel.  Replaces
    codec_cache_attention_inputs + rope_pre_key_by_positions + flash attention at the reference's
    call site (LB/model_fast.py:170-195) without writing a history row to HBM."""
    if query.ndim != 4 or query.shape[0] != 1:
        raise ValueError(f"expected [1,S,H,D], got {tuple(query.shape)}")
    segments = cache.setdefault("codec_segments", [])
    committed_end = int(cache.get("codec_committed_end", 0))
    device, current = key.device, int(key.shape[1])
    head_dim = int(query.shape[-1])
    scale = head_dim ** -0.5 if scale is None else scale
    active, runs = _window(segments, committed_end=committed_end, capacity=capacity, sink_tokens=sink_tokens)
    protected = min(sink_tokens, committed_end, max_attention_size)
    kept, lead = _cut(runs, current, protected=protected, limit=max_attention_size)
    stop = current
    q = query[0]
    partials = []
    if kept:
        hist_k = history_from_payloads([s["k"] for s in active], device=device)
        hist_v = history_from_payloads([s["v"] for s in active], device=device)
        op_k, op_v = operator_of(active[0]["k"], device), operator_of(active[0]["v"], device)
        merged: list[list[int]] = []
        for a, b, p in kept:                       # adjacent pieces become one launch
            if merged and merged[-1][1] == a:
                merged[-1][1] = b
                merged[-1][2].append((p, p + b - a))
            else:
                merged.append([a, b, [(p, p + b - a)]])
        for a, b, spans in merged:
            positions = None
            if rope is not None:
                positions = torch.cat([torch.arange(s, e, device=device, dtype=torch.int32) for s, e in spans])
            partials.append(attention.codec_attention(
                q, hist_k.view_tokens(a, b), hist_v.view_tokens(a, b), op_k, op_v, scale=scale,
                status=status, rope=rope, positions=positions))
    if stop > lead:
        rows_k = key[0, lead:stop]
        if rope is not None:
            now = torch.arange(current_start + lead, current_start + stop, device=device, dtype=torch.int32)
            rows_k = rope.rotate(rows_k, now)
        partials.append(ops.attention_lse(q, rows_k, value[0, lead:stop], scale=scale))
    if not partials:
        raise ValueError("nothing to attend to")
    out, lse = partials[0] if len(partials) == 1 else ops.lse_merge(partials)
    _commit(cache, key, value, current_start=current_start, capacity=capacity, sink_tokens=sink_tokens)
    return out[None], lse


# ------------------------------------------------------------------ NanoKV-Fast step
_READERS: dict[tuple[int, int], tuple["attention.Reader", dict]] = {}
_ROPE_TABLES: dict[tuple, "attention.RopeTable"] = {}


def register_reader(layer: int, payload: dict, *, sp_rank: int = 0, policy: dict | None = None,
                    dtype: torch.dtype = torch.bfloat16, device="cuda") -> "attention.Reader":
    """Make the reader groups of (sp_rank, layer) resident, with the layer's protection policy
    (``recent_native_frames``, ``sink_native_frames``, ``anchor_stride``, ``native_prefix_chunks``,
    ``native_denoise_calls``, ``native_commit``: the manifest's "policy" merged with its
    "layer_policy" entry, LB/codec_native_attention.py:404-407).  A layer without a reader makes
    ``attend`` return None, which the caller answers with its native path."""
    reader = attention.Reader(payload, dtype=dtype, device=device)
    _READERS[(int(sp_rank), int(layer))] = (reader, dict(policy or {}))
    return reader


def _rope_table(freqs: torch.Tensor, frame_seqlen: int, width: int, device) -> "attention.RopeTable":
    key = (freqs.data_ptr(), tuple(freqs.shape), int(frame_seqlen), int(width), str(device))
    if key not in _ROPE_TABLES:
        _ROPE_TABLES[key] = attention.RopeTable(freqs, frame_seqlen=frame_seqlen, width=width, device=device)
    return _ROPE_TABLES[key]


@torch.no_grad()
def attend(q_pre: torch.Tensor, q_native: torch.Tensor, key_current: torch.Tensor, value_current: torch.Tensor,
           cache: dict[str, Any], *, current_start: int, capacity: int, sink_tokens: int,
           max_attention_size: int, grid_sizes: torch.Tensor, freqs: torch.Tensor, frame_seqlen: int):
    """[1,S,H,D], or None when this layer (or this call) is a native fallback.  ``q_pre`` and
    ``key_current`` are pre-RoPE, ``q_native`` is rotated; ``freqs`` is the complex 3-D table."""
    layer, sp_rank = int(cache["codec_layer"]), int(cache.get("codec_sp_rank", 0))
    entry = _READERS.get((sp_rank, layer))
    if entry is None:
        return None
    reader, policy = entry
    if reader.heads != int(q_pre.shape[2]) or reader.native_dim != int(q_pre.shape[3]):
        raise ValueError("reader does not match this sequence-parallel head shard")
    if cache.get("a1_controller") is not None:
        raise RuntimeError("codec-native deployment cannot share the legacy A1 training cache")
    if 0 < int(policy.get("native_prefix_chunks", 0)) >= int(cache.get("codec_chunk_id", 0)):
        return None
    native_calls = policy.get("native_denoise_calls", [])
    if native_calls:       # the call index restarts whenever a new chunk (a new current_start) begins
        repeat = cache.get("_codec_native_schedule_start") == int(current_start)
        index = int(cache.get("_codec_native_schedule_index", -1)) + 1 if repeat else 0
        cache["_codec_native_schedule_start"], cache["_codec_native_schedule_index"] = int(current_start), index
        if not cache.get("codec_commit", False) and index in native_calls:
            return None
    if policy.get("native_commit", False) and cache.get("codec_commit", False):
        return None
    device = q_pre.device
    current = int(key_current.shape[1])
    frame_seqlen = int(frame_seqlen)
    recent_tokens = int(policy.get("recent_native_frames", 0)) * frame_seqlen
    anchor_stride = int(policy.get("anchor_stride", 0))
    native_sink = min(int(sink_tokens),
                      int(policy.get("sink_native_frames", int(sink_tokens) // frame_seqlen)) * frame_seqlen)
    committed = int(cache.get("codec_committed_end", 0))
    budget = min(int(capacity), max(0, int(max_attention_size) - current))
    active, runs = _window(cache.get("codec_segments", []), committed_end=committed, capacity=budget,
                           sink_tokens=min(int(sink_tokens), budget))
    # protected / low split on host integers: rows of the stacked active segments and their positions
    rows = torch.cat([torch.arange(a, b) for a, b, _ in runs]) if runs else torch.empty(0, dtype=torch.long)
    where = torch.cat([torch.arange(p, p + b - a) for a, b, p in runs]) if runs else rows
    protect = where < native_sink
    if recent_tokens:
        protect |= where >= max(0, committed - recent_tokens)
    if anchor_stride:
        protect |= torch.div(where, frame_seqlen, rounding_mode="floor").remainder(anchor_stride) == 0
    if bool(protect.all()):
        return None                      # seed / all-protected: the caller's exact native path
    hist_k = history_from_payloads([s["k"] for s in active], device=device)
    hist_v = history_from_payloads([s["v"] for s in active], device=device)
    op_k, op_v = operator_of(active[0]["k"], device), operator_of(active[0]["v"], device)
    heads, dim = int(q_pre.shape[2]), int(q_pre.shape[3])
    table = _rope_table(freqs, frame_seqlen, int(grid_sizes[0][2]), device)
    now = torch.arange(current_start, current_start + current, device=device, dtype=torch.int32)
    key_rows, value_rows = [table.rotate(key_current[0], now)], [value_current[0]]
    if bool(protect.any()):
        index = rows[protect].to(device=device, dtype=torch.int32)
        spots = where[protect].to(device=device, dtype=torch.int32)
        decoded_k = ops.decode_rows(hist_k.view(), op_k.decoder, op_k.mean, rows=index, dtype=q_pre.dtype)
        decoded_v = ops.decode_rows(hist_v.view(), op_v.decoder, op_v.mean, rows=index, dtype=q_pre.dtype)
        key_rows.insert(0, table.rotate(decoded_k.view(-1, heads, dim), spots))
        value_rows.insert(0, decoded_v.view(-1, heads, dim))
    native = [(torch.cat(key_rows).to(q_native.dtype), torch.cat(value_rows))]
    visible = rows[~protect].to(device)
    positions = torch.zeros(hist_k.tokens, dtype=torch.int32, device=device)
    positions[visible] = where[~protect].to(device=device, dtype=torch.int32)
    low = [{"k": hist_k, "v": hist_v, "k_mean": op_k.mean, "v_mean": op_v.mean, "v_decoder": op_v.decoder,
            "positions": positions, "visible": visible}]
    out = attention.hybrid_attention(
        q_pre[0], q_native[0], native, low, reader, rope=table, q_positions=now,
        value_mean_residual=os.environ.get("LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL", "0") == "1")
    if cache.get("codec_commit", False) and current_start != committed:
        raise RuntimeError("non-causal codec-native commit")
    _commit(cache, key_current, value_current, current_start=current_start, capacity=capacity,
            sink_tokens=sink_tokens)
    return out[None]
