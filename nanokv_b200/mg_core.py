"""Matrix-Game codec-native attention interface on the B200 kernels.

Same function names, argument order and [B, H, tokens, D] layout as the reference's
model-independent module MGC/core.py (merge :33, attention_lse :45, rope_selected :75,
attention_grouped_mask :94, camera_selected :111, protected_tokens :140, ReaderGroup :155,
ReaderLayer :207, hybrid_attention :278), so the Matrix-Game call site (MGC/mg35.py:192-347) can
import this module instead.  Batch is 1, as at that call site.

What differs, and why: a low segment's ``"k"`` / ``"v"`` entry is a ``PackedRows`` (packed INT4 codes,
scales, centre ids and table still in the payload's form, plus the operator mean) and not a
dequantised latent tensor -- ``mg_codec.direct_latent_pair_segments`` produces it -- because the
fused read expands codes on chip and no latent row exists in HBM.

Positional hooks.  ``query_position(query, group)`` and ``output_position(out, group)`` are called
as given: reduced queries and low-width outputs are real tensors.  ``kv_position(kk, vv, segment,
group)`` is where the fused read has nothing to hand over: low-width K and V only exist tile by tile
inside the kernel.  When the three hooks are the bound methods of one ``PositionHooks`` object (the
rotation multipliers and camera matrices as data) the read stays fused and the kernel rotates /
transforms the tiles itself.  Any other callable still works: K and V of the segment are then
written at the group's width by the decode kernel, handed to the callable, and attended as plain
rows -- every step on this library's kernels, but unfused.
"""
from __future__ import annotations

import math
from typing import Any, Callable

import torch

from . import attention, ops
from .cache import PackedRows


# ------------------------------------------------------------------ layout helpers
def _rows(x: torch.Tensor) -> torch.Tensor:
    """[1,H,S,D] -> [S,H,D] view."""
    if x.dim() != 4 or x.shape[0] != 1:
        raise ValueError(f"expected [1,H,S,D], got {tuple(x.shape)}")
    return x[0].permute(1, 0, 2)


def _heads_first(x: torch.Tensor) -> torch.Tensor:
    """[S,H,D] -> [1,H,S,D] view."""
    return x.permute(1, 0, 2)[None]


def _visibility(mask: torch.Tensor | None, queries: int):
    """bool mask [..., Q or 1, S] -> (rows [G, S], query_groups i64 [Q] or None): queries with the
    same visible keys share a group, so that a masked read is one unmasked read per group."""
    if mask is None:
        return None, None
    if mask.dtype != torch.bool:
        raise ValueError("Only boolean visibility masks are supported")
    flat = mask.reshape(-1, mask.shape[-2], mask.shape[-1])
    if flat.shape[0] != 1:
        raise ValueError("visibility is shared by batch and heads: mask [1,1,Q,S] or [1,1,1,S]")
    flat = flat[0]
    if flat.shape[0] == 1:
        return flat, None
    if flat.shape[0] != queries:
        raise ValueError("mask rows must match the queries")
    rows, groups = torch.unique(flat, dim=0, return_inverse=True)
    return (rows, None) if rows.shape[0] == 1 else (rows, groups)


def _joint_visibility(masks, lengths, queries: int, device):
    """Per-segment masks ([1,1,Q or 1,S] or None) -> ([bool [G, S] per segment], query_groups i64 [Q] or
    None): one grouping of the queries over all segments, by their visible keys across the whole read."""
    if all(mask is None for mask in masks):
        return None, None
    flat = []
    for mask, tokens in zip(masks, lengths):
        if mask is None:
            flat.append(torch.ones(1, tokens, dtype=torch.bool, device=device))
            continue
        if mask.dtype != torch.bool:
            raise ValueError("Only boolean visibility masks are supported")
        rows = mask.reshape(-1, mask.shape[-2], mask.shape[-1])
        if rows.shape[0] != 1 or rows.shape[1] not in (1, queries) or rows.shape[2] != tokens:
            raise ValueError("visibility is shared by batch and heads: mask [1,1,Q,S] or [1,1,1,S]")
        flat.append(rows[0])
    groups = None
    if all(rows.shape[0] == 1 for rows in flat):
        joined = torch.cat(flat, 1)
    else:
        joined, groups = torch.unique(torch.cat([rows.expand(queries, -1) for rows in flat], 1), dim=0,
                                      return_inverse=True)
        if joined.shape[0] == 1:
            groups = None
    return list(joined.split(lengths, dim=1)), groups


# ------------------------------------------------------------------ MGC/core.py functions
def merge(out_a, lse_a, out_b, lse_b):
    """Exact global-softmax merge of two partitions; a row empty in both gives zero and -inf."""
    return ops.lse_merge([(out_a.contiguous(), lse_a.contiguous()), (out_b.contiguous(), lse_b.contiguous())])


def attention_lse(q, k, v, mask=None, *, scale=None, q_tile=128, k_tile=1024):
    """q [1,H,Q,D], k [1,H,S,D], v [1,H,S,Dv], mask True = visible -> (O [1,H,Q,Dv], lse f32 [1,H,Q]).
    ``q_tile`` / ``k_tile`` are accepted for signature parity; the kernel tiles by itself."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if k.shape[-2] == 0:
        return (q.new_zeros(*q.shape[:-1], v.shape[-1]),
                torch.full(q.shape[:-1], -math.inf, device=q.device, dtype=torch.float32))
    rows, groups = _visibility(mask, q.shape[-2])
    if rows is not None and groups is None:
        index = torch.nonzero(rows[0]).flatten()
        k, v, rows = k.index_select(2, index), v.index_select(2, index), None
        if index.numel() == 0:
            return attention_lse(q, k, v, scale=scale)
    if rows is not None:
        return attention_grouped_mask(q, k, v, rows[groups][None, None], groups, scale=scale)
    out, lse = ops.attention_lse(_rows(q).contiguous(), _rows(k).contiguous(), _rows(v).contiguous(), scale=scale)
    return _heads_first(out), lse.t()[None]


def attention_grouped_mask(q, k, v, mask, query_groups, *, scale):
    """Queries of one group share their visible keys: per group, gather the keys the group's first
    query sees and attend them unmasked."""
    out = torch.zeros(*q.shape[:-1], v.shape[-1], dtype=q.dtype, device=q.device)
    lse = torch.full(q.shape[:-1], -math.inf, device=q.device, dtype=torch.float32)
    for group in torch.unique(query_groups):
        qi = torch.nonzero(query_groups == group).flatten()
        row = mask[0, 0, qi[0] if mask.shape[-2] > 1 else 0]
        ki = torch.nonzero(row).flatten()
        oo, ll = attention_lse(q.index_select(2, qi), k.index_select(2, ki), v.index_select(2, ki), scale=scale)
        out.index_copy_(2, qi, oo.to(out.dtype))
        lse.index_copy_(2, qi, ll)
    return out, lse


def _pair_index(indices: torch.Tensor) -> torch.Tensor:
    if not torch.equal(indices[:, 1::2], indices[:, ::2] + 1) or bool((indices[:, ::2] % 2).any()):
        raise ValueError("RoPE mapping must retain complete original pairs")
    return (indices[:, ::2] // 2).to(torch.int32).contiguous()


def rope_selected(x, multiplier, indices):
    """x [1,H,S,d] rotated with the ORIGINAL frequencies of the native pairs it retains:
    multiplier complex [S, D/2] or [S,1,D/2] (one row per token), indices [H, d]."""
    if multiplier.ndim == 3:
        multiplier = multiplier[:, 0]
    table = attention.RopeTable.per_token(multiplier, device=x.device)
    positions = torch.arange(x.shape[-2], device=x.device, dtype=torch.int32)
    return _heads_first(table.rotate(_rows(x), positions, _pair_index(indices).to(x.device)))


def camera_selected(x, matrix, indices, *, layout="full"):
    """PRoPE block transform of low-width rows that keep whole 8-wide (j, r) blocks of the native
    (p=4, c=4, j=4, r=2) layout: x [1,H,S,d], matrix [1,F,4,4,4] as the caller selected it
    (Q: P^T, K / V: P^-1, output: P), indices [H, d]."""
    if layout != "full" or x.shape[-1] % 8:
        raise ValueError("MG low PRoPE currently requires full layout and whole 8D blocks")
    if x.shape[-2] % int(matrix.shape[1]):
        raise ValueError("PRoPE frame count must divide the token sequence")
    view = attention.camera_view(matrix, indices, x.shape[-2], device=x.device)
    return _heads_first(ops.camera_rows(_rows(x), view))


def protected_tokens(frame_ids, recent, stride, sink=0):
    """bool [tokens]: tokens of the newest ``recent`` frame runs, of the first ``sink`` runs, and of
    every ``stride``-th older run counted back from the newest old one.  A run is a stretch of equal
    consecutive frame ids, so repeated ids far apart stay distinct frames."""
    if min(recent, stride, sink) < 0:
        raise ValueError("Negative protection policy")
    if frame_ids.numel() == 0:
        return torch.zeros(0, dtype=torch.bool, device=frame_ids.device)
    starts = torch.ones_like(frame_ids, dtype=torch.bool)
    starts[1:] = frame_ids[1:] != frame_ids[:-1]
    run = torch.cumsum(starts, 0) - 1
    count = int(run[-1]) + 1
    old = max(0, count - recent)
    index = torch.arange(count, device=frame_ids.device)
    keep = (index >= old) | (index < sink)
    if stride and old:
        keep |= (index < old) & ((old - 1 - index) % stride == 0)
    return keep[run]


# ------------------------------------------------------------------ readers
class ReaderGroup(attention.ReaderGroup):
    """attention.ReaderGroup with the reference's methods in its [1,h,S,d] layout."""

    def __init__(self, state: dict, *, dtype, device, native_dim: int):
        super().__init__(state, dtype=dtype, device=device, native_dim=native_dim)
        self.indices = state["indices"].long().to(device)
        self.v_indices = state.get("v_indices", state["indices"]).long().to(device)

    def query(self, q):
        """q [1,h,Q,D] of this group's heads -> [1,h,Q,d]."""
        return _heads_first(ops.head_linear(_rows(q), self.q_reduce))

    def lift_output(self, x):
        """[1,h,Q,d] -> [1,h,Q,D]."""
        return _heads_first(ops.head_linear(_rows(x), self.lift, din=self.value_width))

    def read(self, rows: PackedRows, *, target: str, dtype=None):
        """K or V of the segment at this group's width, [1,h,S,d]: the decode kernel with the read
        weights as its decoder, the projected mean as its bias and the projected centre table."""
        view = self.projected_centers(rows.history, target)
        weight = self.k_read if target == "k" else self.v_read
        out = ops.decode_rows(view, weight.reshape(-1, self.rank), self.bias(rows.mean, target).reshape(-1),
                              rows=None if rows.visible is None else rows.visible.to(torch.int32),
                              dtype=dtype or self.dtype)
        out = out.view(-1, self.heads.numel(), self.padded)[..., :self.width]
        return _heads_first(out)


class ReaderLayer(attention.Reader):
    """All groups of one layer.  ``to(device=, dtype=)`` returns the reader rebuilt there, which is
    how the reference's loader places it (MGC/core.py:258)."""
    group_class = ReaderGroup

    def __init__(self, payload: dict, *, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        self._payload = payload
        super().__init__(payload, dtype=dtype, device=device)

    def to(self, device=None, dtype=None):
        return ReaderLayer(self._payload, dtype=dtype or self.groups[0].dtype,
                           device=device or self.groups[0].heads.device)


# ------------------------------------------------------------------ positional hooks as data
class PositionHooks:
    """The positional glue of the Matrix-Game call site (MGC/mg35.py:318-347) as data.

    q_multiplier   complex [Q, D/2] (or [Q,1,D/2]): rotation of the reduced query, or None
    kv_multiplier  segment -> complex [S, D/2]: rotation of a low segment's keys (default: its "freqs")
    q_camera, out_camera   [1,F,4,4,4]: P^T for the query, P for the low-width output, or None
    kv_camera      segment -> [1,F',4,4,4]: P^-1 over the segment's tokens (default: its "camera")

    Pass ``hooks.query_position``, ``hooks.kv_position``, ``hooks.output_position`` to
    ``hybrid_attention``: it recognises them and keeps the read fused.  The same methods are ordinary
    callables on tensors, so they also serve any other implementation of the interface."""

    def __init__(self, *, q_multiplier=None, kv_multiplier: Callable | None = None, q_camera=None,
                 out_camera=None, kv_camera: Callable | None = None):
        self.q_multiplier, self.q_camera, self.out_camera = q_multiplier, q_camera, out_camera
        self.rotates = q_multiplier is not None
        self.transforms = q_camera is not None
        if self.transforms != (out_camera is not None):
            raise ValueError("the camera transform needs both the query and the output matrices")
        self.kv_multiplier = kv_multiplier or (lambda segment: segment["freqs"])
        self.kv_camera = kv_camera or (lambda segment: segment["camera"])

    def query_position(self, value, group):
        if self.rotates:
            value = rope_selected(value, self.q_multiplier, group.indices)
        if self.transforms:
            value = camera_selected(value, self.q_camera, group.indices)
        return value

    def kv_position(self, kk, vv, segment, group):
        if self.rotates:
            kk = rope_selected(kk, self.kv_multiplier(segment), group.indices)
        if self.transforms:
            matrix = self.kv_camera(segment)
            kk = camera_selected(kk, matrix, group.indices)
            vv = camera_selected(vv, matrix, group.v_indices)
        return kk, vv

    def output_position(self, value, group):
        return camera_selected(value, self.out_camera, group.v_indices) if self.transforms else value


def identity_query(value, group):
    return value


def identity_kv(kk, vv, segment, group):
    return kk, vv


def _hooks_object(query_position, kv_position, output_position):
    """The PositionHooks all three hooks belong to, None-object for the identity, else False."""
    owner = getattr(kv_position, "__self__", None)
    if isinstance(owner, PositionHooks):
        if getattr(query_position, "__self__", None) is not owner:
            return False
        if owner.transforms and getattr(output_position, "__self__", None) is not owner:
            return False
        return owner
    if kv_position is identity_kv and query_position is identity_query and output_position is identity_query:
        return PositionHooks()
    return False


def _low_entry(segment: dict) -> dict:
    k, v = segment["k"], segment["v"]
    if not isinstance(k, PackedRows) or not isinstance(v, PackedRows):
        raise TypeError("low segments carry PackedRows (mg_codec.direct_latent_pair_segments), not "
                        "dequantised latents: the fused read expands the packed codes on chip")
    entry = {"k": k.history, "v": v.history, "k_mean": k.mean, "v_mean": v.mean}
    if k.visible is not None:
        entry["visible"] = k.visible
    return entry


@torch.no_grad()
def hybrid_attention(q_pre, q_native, native_segments, low_segments, reader, *,
                     query_position=identity_query, kv_position=identity_kv,
                     output_position=identity_query):
    """Mixed-dimensional read with one global softmax.  q_pre / q_native [1,H,Q,D]; native segments
    (K [1,H,S,D], V, bool mask or None); low segments {"k": PackedRows, "v": PackedRows, "mask",
    position metadata for the hooks}.  Returns [1,H,Q,D]."""
    hooks = _hooks_object(query_position, kv_position, output_position)
    if hooks is False:
        return _hybrid_unfused(q_pre, q_native, native_segments, low_segments, reader,
                               query_position, kv_position, output_position)
    queries = q_native.shape[-2]
    native = [[_rows(key).contiguous(), _rows(value).contiguous()] for key, value, *_ in native_segments]
    low = [_low_entry(segment) for segment in low_segments]
    masks = [rest[0] if rest else None for _, _, *rest in native_segments]
    masks += [segment.get("mask") for segment in low_segments]
    lengths = [n[0].shape[0] for n in native] + [segment["k"].tokens for segment in low_segments]
    rows, groups = _joint_visibility(masks, lengths, queries, q_native.device)
    if rows is not None:
        if hooks.transforms or any("visible" in entry for entry in low):
            # the in-kernel camera transform and a token_keep selection index tokens by their place
            # in the segment, which a gather of the visible keys changes
            return _hybrid_unfused(q_pre, q_native, native_segments, low_segments, reader,
                                   hooks.query_position, hooks.kv_position, hooks.output_position)
        for target, mask in zip(native + low, rows):
            if isinstance(target, list):
                target.append(mask)
            else:
                target["mask"] = mask
    native = [tuple(n) for n in native]
    rope = q_positions = camera = None
    if hooks.rotates:
        tables, offset = [hooks.q_multiplier.reshape(queries, -1)], queries
        q_positions = torch.arange(queries, device=q_native.device, dtype=torch.int32)
        for entry, segment in zip(low, low_segments):
            multiplier = hooks.kv_multiplier(segment)
            multiplier = multiplier.reshape(multiplier.shape[0], -1)
            positions = torch.arange(offset, offset + multiplier.shape[0], device=q_native.device,
                                     dtype=torch.int32)
            if "visible" in entry:       # multipliers come per kept token; the read indexes the segment
                full = torch.zeros(entry["k"].tokens, dtype=torch.int32, device=q_native.device)
                full[entry["visible"]] = positions
                positions = full
            entry["positions"] = positions
            offset += multiplier.shape[0]
            tables.append(multiplier)
        rope = attention.RopeTable.per_token(torch.cat([t.to(q_native.device) for t in tables]),
                                             device=q_native.device)
    if hooks.transforms:
        camera = {"q": hooks.q_camera, "out": hooks.out_camera}
        for entry, segment in zip(low, low_segments):
            entry["camera"] = hooks.kv_camera(segment)
    out = attention.hybrid_attention(_rows(q_pre).contiguous(), _rows(q_native).contiguous(), native, low, reader, rope=rope,
                                     q_positions=q_positions, camera=camera, query_groups=groups)
    return _heads_first(out)


def _hybrid_unfused(q_pre, q_native, native_segments, low_segments, reader, query_position, kv_position,
                    output_position):
    """hybrid_attention with arbitrary callables as hooks: the loop of MGC/core.py:286-310 with every
    tensor operation on this library's kernels; K / V of each low segment are written at the group's
    width so that ``kv_position`` has rows to work on."""
    scale = reader.native_dim ** -0.5
    native_out = torch.zeros_like(q_native)
    native_lse = torch.full(q_native.shape[:-1], -math.inf, device=q_native.device, dtype=torch.float32)
    for key, value, *rest in native_segments:
        out, lse = attention_lse(q_native, key, value, rest[0] if rest else None, scale=scale)
        native_out, native_lse = merge(native_out, native_lse, out, lse)
    result = torch.zeros_like(q_native)
    for group in reader.groups:
        head = group.heads
        query = query_position(group.query(q_pre.index_select(1, head)), group)
        out = native_out.index_select(1, head).contiguous()
        lse = native_lse.index_select(1, head).contiguous()
        for segment in low_segments:
            kk = group.read(segment["k"], target="k", dtype=q_native.dtype)
            vv = group.read(segment["v"], target="v", dtype=q_native.dtype)
            kk, vv = kv_position(kk, vv, segment, group)
            oo, ll = attention_lse(query, kk, vv, segment.get("mask"), scale=scale)
            oo = output_position(oo, group)
            out, lse = merge(out, lse, group.lift_output(oo).contiguous(), ll.contiguous())
        result.index_copy_(1, head, out)
    return result
