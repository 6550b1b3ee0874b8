"""Read path: fused codec-attention, NanoKV-Fast hybrid attention, LSE merge."""
from __future__ import annotations

import math

import torch

from . import ops
from .cache import CompressedHistory
from .codec import Operator
from .ops import HistoryView


def _view(hist) -> HistoryView:
    return hist.view() if isinstance(hist, CompressedHistory) else hist


def codec_attention(q: torch.Tensor, hist_k, hist_v, op_k: Operator, op_v: Operator, *,
                    scale: float | None = None, status: torch.Tensor | None = None,
                    splits: int | None = None, out: torch.Tensor | None = None,
                    lse: torch.Tensor | None = None, rope: "RopeTable | None" = None,
                    positions: torch.Tensor | None = None):
    """Full-dimensional read: q [Q,H,D] -> (O [Q,H,D], lse f32 [Q,H]).

    K and V of every history token are rebuilt on chip from codes, scales, the
    decoder slice of each head and the token's centre; nothing full-width is
    written to HBM.  Replaces decode + attention of the reference
    (MGM/nanokv_codec.py:393-455 + MGC/core.py:45-72).  With ``rope`` and the history tokens'
    absolute ``positions`` the rebuilt keys are rotated inside the kernel, which also replaces
    rope_pre_key_by_positions (LB/lingbot_v2_cache_runtime.py:19-76); q arrives rotated.
    """
    Q, H, D = q.shape
    if H * D != op_k.joint:
        raise ValueError("query heads do not match the operator's joint width")
    scale = D ** -0.5 if scale is None else scale
    prepared = (ops.tensor_core_read(q.dtype, D, D, op_k.rank) and op_k.decoder_tc is not None
                and op_v.decoder_tc is not None)
    wk = (op_k.decoder_tc if prepared else op_k.decoder).view(H, D, op_k.rank)
    wv = (op_v.decoder_tc if prepared else op_v.decoder).view(H, D, op_v.rank)
    rope_view = None
    if rope is not None:
        if positions is None:
            raise ValueError("RoPE needs the absolute positions of the history tokens")
        if positions.dim() != 1 or positions.numel() != _view(hist_k).tokens:
            raise ValueError("RoPE position/K length mismatch")
        rope_view = rope.view(positions)
    return ops.attn_codec(q, _view(hist_k), _view(hist_v), wk, op_k.bias.view(H, D), wv,
                          op_v.bias.view(H, D), scale=scale, status=status, splits=splits,
                          out=out, lse=lse, rope=rope_view, prepared=prepared)


class RopeTable:
    """Device-resident rotation table of the 3-D RoPE: (cos, sin) in fp32 of the reference's
    complex128 ``freqs`` [rows, head_dim/2] (LB/model.py:29-36, :426-430), with the frame grid
    that maps a token position to (frame, row, column)."""

    def __init__(self, freqs: torch.Tensor, *, frame_seqlen: int, width: int, device="cuda"):
        if not freqs.is_complex() or freqs.dim() != 2:
            raise ValueError("freqs must be a complex [rows, head_dim/2] tensor")
        if frame_seqlen != 0 and (frame_seqlen < 0 or width <= 0 or frame_seqlen % width):
            raise ValueError(f"frame_seqlen mismatch: width {width} does not divide {frame_seqlen}")
        self.cos_sin = torch.view_as_real(freqs).to(device=device, dtype=torch.float32).contiguous()
        self.frame_seqlen, self.width = int(frame_seqlen), int(width)

    @classmethod
    def per_token(cls, multiplier: torch.Tensor, device="cuda") -> "RopeTable":
        """Table with one row per token: ``multiplier`` complex [S, native half] as Matrix-Game
        passes it (MGC/core.py:75-91); ``positions`` then index its rows."""
        return cls(multiplier, frame_seqlen=0, width=0, device=device)

    def view(self, positions: torch.Tensor, pair_index: torch.Tensor | None = None) -> "ops.RopeView":
        """``pair_index`` i32 [heads, d/2]: the native pair every pair of a low-width row retains."""
        positions = positions.to(device=self.cos_sin.device, dtype=torch.int32).contiguous()
        return ops.RopeView(positions, self.cos_sin, self.frame_seqlen, self.width, pair_index)

    def rotate(self, rows: torch.Tensor, positions: torch.Tensor,
               pair_index: torch.Tensor | None = None) -> torch.Tensor:
        """rows [S,H,d] (queries, the current chunk's keys) rotated by their positions."""
        return ops.rope_rows(rows, self.view(positions, pair_index))


def camera_index(indices: torch.Tensor, device="cuda") -> torch.Tensor:
    """reader indices [h, e] that retain whole 8-wide native blocks -> camera of every block,
    i32 [h, e/8]: native block id modulo 4 (MGC/core.py:119-127)."""
    blocks = indices.long().reshape(indices.shape[0], -1, 8)
    if (not torch.equal(blocks, blocks[..., :1] + torch.arange(8, device=blocks.device))
            or bool((blocks[..., 0] % 8).any())):
        raise ValueError("Invalid MG camera blocks")
    return ((blocks[..., 0] // 8) % 4).to(device=device, dtype=torch.int32).contiguous()


def camera_view(matrix: torch.Tensor, indices: torch.Tensor, tokens: int, device="cuda") -> "ops.CameraView":
    """matrix [1, frames, 4, 4, 4] (already the role's: P^T for queries, P^-1 for keys and values,
    P for outputs) over ``tokens`` rows split evenly over its frames."""
    if matrix.dim() != 5 or matrix.shape[0] != 1 or tuple(matrix.shape[2:]) != (4, 4, 4):
        raise ValueError("camera matrix must be [1, frames, 4, 4, 4]")
    frames = int(matrix.shape[1])
    if tokens % frames:
        raise ValueError("PRoPE frame count must divide the token sequence")
    return ops.CameraView(matrix[0].to(device=device, dtype=torch.float32).contiguous(),
                          camera_index(indices, device), tokens // frames)


def _camera(matrix: torch.Tensor, cam_index: torch.Tensor, tokens: int) -> "ops.CameraView":
    if matrix.dim() != 5 or matrix.shape[0] != 1 or tuple(matrix.shape[2:]) != (4, 4, 4):
        raise ValueError("camera matrix must be [1, frames, 4, 4, 4]")
    if tokens % int(matrix.shape[1]):
        raise ValueError("PRoPE frame count must divide the token sequence")
    return ops.CameraView(matrix[0].to(device=cam_index.device, dtype=torch.float32).contiguous(),
                          cam_index, tokens // int(matrix.shape[1]))


def merge(out_a, lse_a, out_b, lse_b):
    """Two-partition softmax merge (MGC/core.py:33-42)."""
    return ops.lse_merge([(out_a.contiguous(), lse_a.contiguous()),
                          (out_b.contiguous(), lse_b.contiguous())])


# ------------------------------------------------------------------ NanoKV-Fast
class ReaderGroup:
    """Device-resident reader of one head-width group (MGC/core.py:155-204)."""

    def __init__(self, state: dict, *, dtype: torch.dtype, device, native_dim: int):
        self.heads = state["heads"].long().to(device)
        self.width = int(state["k_read"].shape[1])
        self.value_width = int(state["v_read"].shape[1])
        if self.width != self.value_width:
            raise ValueError("reader groups with different K and V widths are not built")
        self.dtype, self.native_dim = dtype, native_dim
        to = dict(device=device, dtype=dtype)
        self.q_reduce = state["q_reduce"].to(**to)
        self.k_affine = state["k_affine"].to(**to)
        self.v_affine = state["v_affine"].to(**to)
        self.lift = state["lift"].to(**to)
        # bf16 tensor-core tiles are at least 64 wide: narrower readers are zero-padded
        pad_to = 64 if (dtype == torch.bfloat16 and self.width < 64) else self.width
        self.padded = pad_to

        def pad_rows(weight):  # [h, d, r] -> [h, pad, r]
            out = torch.zeros(weight.shape[0], pad_to, weight.shape[2], **to)
            out[:, :weight.shape[1]] = weight.to(**to)
            return out.contiguous()
        self.k_read = pad_rows(state["k_read"])
        self.v_read = pad_rows(state["v_read"])
        # the same rows in the order the tensor-core read expands code words
        self.rank = int(self.k_read.shape[2])
        self.prepared = (dtype == torch.bfloat16 and pad_to in (64, 128) and self.rank % 64 == 0
                         and self.k_read.is_cuda)
        self.k_read_tc = ops.prepare_decoder(self.k_read) if self.prepared else None
        self.v_read_tc = ops.prepare_decoder(self.v_read) if self.prepared else None
        self._tables: dict = {}
        self._biases: dict = {}
        # native pair retained by every pair of the (padded) low-width row, for the selected RoPE
        # (LB/codec_native_attention.py:111, :271-272: indices keep native complex pairs together)
        self.pair_index = None
        if state.get("indices") is not None:
            indices = state["indices"].long()
            if (not torch.equal(indices[:, 1::2], indices[:, ::2] + 1)
                    or bool((indices[:, ::2] % 2).any())):
                raise ValueError("low-dimensional RoPE indices must preserve native complex pairs")
            pairs = torch.zeros(indices.shape[0], pad_to // 2, dtype=torch.int32)
            pairs[:, :indices.shape[1] // 2] = (indices[:, ::2] // 2).to(torch.int32)
            self.pair_index = pairs.to(device).contiguous()
        # camera of every 8-wide block of the (padded) row, for the PRoPE transform (K / Q and V / output)
        self.cam_index_k = self.cam_index_v = None
        if state.get("indices") is not None and self.width % 8 == 0:
            def cams(indices):
                try:
                    index = camera_index(indices, "cpu")
                except ValueError:
                    return None   # this reader does not keep whole native blocks: no camera transform
                padded = torch.zeros(index.shape[0], pad_to // 8, dtype=torch.int32)
                padded[:, :index.shape[1]] = index
                return padded.to(device).contiguous()
            self.cam_index_k = cams(state["indices"])
            self.cam_index_v = cams(state.get("v_indices", state["indices"]))

    def _pad_last(self, tensor):
        if tensor.shape[-1] == self.padded:
            return tensor.contiguous()
        out = tensor.new_zeros(*tensor.shape[:-1], self.padded)
        out[..., :tensor.shape[-1]] = tensor
        return out

    def bias(self, mean: torch.Tensor, target: str) -> torch.Tensor:
        """(mean_h @ affine) in the working dtype, as float [h, pad] (MGC/core.py:179-180)."""
        key = (id(mean), mean._version, target)
        cached = self._biases.get(target)
        if cached is not None and cached[0] == key:
            return cached[1]
        affine = self.k_affine if target == "k" else self.v_affine
        mean_heads = mean.reshape(-1, self.native_dim).index_select(0, self.heads).to(self.dtype)
        value = self._pad_last(torch.einsum("hd,hde->he", mean_heads, affine).float())
        self._biases[target] = (key, value, mean)     # the mean is kept so that its id cannot be reused
        return value

    def projected_centers(self, hist: CompressedHistory, target: str) -> HistoryView:
        """History view whose centre table is projected to this group's heads and width
        (MGC/core.py:194-195); cached per (history, segments) as derived state."""
        key = (id(hist), target, hist.segments)
        if key not in self._tables:
            affine = self.k_affine if target == "k" else self.v_affine
            table = hist.centers.view(hist.centers.shape[0], -1, self.native_dim)
            table = table.index_select(1, self.heads).to(self.dtype)
            projected = self._pad_last(torch.einsum("chd,hde->che", table, affine))
            self._tables = {k: v for k, v in self._tables.items() if k[0] != id(hist) or k[1] != target}
            # stored like every centre table: bf16
            self._tables[key] = projected.reshape(projected.shape[0], -1).to(torch.bfloat16).contiguous()
        view = hist.view()
        view.centers = self._tables[key]
        return view


class Reader:
    """All groups of one layer; groups partition the heads (MGC/core.py:207-224)."""
    group_class = ReaderGroup

    def __init__(self, payload: dict, *, dtype: torch.dtype, device="cuda"):
        self.heads, self.native_dim = int(payload["heads"]), int(payload["native_dim"])
        self.rank = int(payload["rank"])
        self.groups = [self.group_class(s, dtype=dtype, device=device, native_dim=self.native_dim)
                       for s in payload["groups"]]
        listed = sorted(int(h) for g in self.groups for h in g.heads.tolist())
        if listed != list(range(self.heads)):
            raise ValueError("Reader groups must partition heads exactly once")


def history_moments(low_segments):
    """[(latent_sum f32 [r], centre counts f32 [rows], tokens)] of every low segment's V history."""
    moments = []
    for segment in low_segments:
        view = _view(segment["v"])
        if segment.get("visible") is not None:
            view = ops.gather_view(view, segment["visible"])
        latent_sum, counts = ops.history_moments(view)
        moments.append((latent_sum, counts.float(), view.tokens))
    return moments


def compressed_value_mean(low_segments, moments, *, heads: int, native_dim: int) -> torch.Tensor:
    """Mean decoded V over the low history, f32 [heads, native_dim], from the latent sums and centre
    counts (never from decoded rows): decoder (sum latent / n) + bf16(mean) + (counts^T centres) / n
    (LB/codec_native_attention.py:465-501)."""
    first = low_segments[0]
    total = sum(n for _, _, n in moments)
    latent_sum = sum(ls for ls, _, _ in moments)
    center_sum = sum(counts @ _view(seg["v"]).centers.float() for seg, (_, counts, _) in zip(low_segments, moments))
    value = (torch.mv(first["v_decoder"].float(), latent_sum / total)
             + first["v_mean"].to(torch.bfloat16).float() + center_sum / total)
    return value.view(heads, native_dim)


def hybrid_attention(q_pre: torch.Tensor, q_native: torch.Tensor, native_segments,
                     low_segments, reader: Reader, *, rope: "RopeTable | None" = None,
                     q_positions: torch.Tensor | None = None, value_mean_residual: bool = False,
                     camera: dict | None = None, query_groups: torch.Tensor | None = None):
    """Mixed-dimensional read (MGC/core.py:278-310).  Positional hooks are the identity unless
    ``rope`` is given: then the reduced query is rotated by ``q_positions`` and every low-width
    key read by its segment's ``"positions"``, with the native pairs the group retains
    (LB/codec_native_attention.py:757, :779); native keys and q_native arrive rotated.
    ``value_mean_residual`` adds, for groups narrower than the head, the mean decoded V of the low
    history minus the lifted mean of its low-width read (a first-moment correction, :726, :793-796);
    every low segment then also carries ``"v_decoder"`` [J, r].  The low-width mean follows from the
    same moments by linearity rather than from materialised rows.
    ``camera`` = {"q": P^T, "out": P} ([1, frames, 4, 4, 4] over the query rows) with a ``"camera"``
    entry (P^-1 over the segment's tokens) in every low segment switches on Matrix-Game's PRoPE: the
    reduced query, the low-width keys and values (inside the kernel) and the low-width output are
    transformed block-wise (MGC/mg35.py:318-347).

    Visibility (Matrix-Game's boolean masks, MGC/core.py:55-65, :94-108, :290-291, :303): a native
    segment may be (K, V, mask) and a low segment may carry ``"mask"``, bool [G, tokens]; query row n
    sees the keys ``mask[query_groups[n]]`` (G = 1 without ``query_groups``).  Queries of one group
    share their visible keys, so each group attends the gathered keys (codes, scales and ids of a
    compressed segment are gathered, not decoded) with the unmasked kernels.

    q_pre / q_native [Q,H,D]; native_segments [(K [n,H,D], V [n,H,D])] full
    width (protected history, current chunk), or {"k", "v": compressed histories, "op_k", "op_v":
    operators} for protected tokens that stay compressed and are rebuilt at full width inside the
    fused kernel instead of being decoded to rows first (_decode_active_history
    LB/lingbot_v2_cache_runtime.py:139-163 followed by the native attention); low_segments [{"k": history,
    "v": history, "k_mean": f32 [J], "v_mean": f32 [J]}] read through the
    reader projections.  Returns O [Q,H,D].
    """
    if any(not isinstance(segment, dict) and len(segment) > 2 and segment[2] is not None
           for segment in native_segments) or \
            any(segment.get("mask") is not None for segment in low_segments):
        return _hybrid_visible(q_pre, q_native, native_segments, low_segments, reader, rope=rope,
                               q_positions=q_positions, value_mean_residual=value_mean_residual,
                               camera=camera, query_groups=query_groups)
    Q, H, D = q_native.shape
    scale = reader.native_dim ** -0.5
    native_out = native_lse = None
    for segment in native_segments:
        if isinstance(segment, dict):      # protected tokens kept compressed: rebuilt inside the kernel
            out, lse = codec_attention(q_native.contiguous(), segment["k"], segment["v"], segment["op_k"],
                                       segment["op_v"], scale=scale)
        else:
            key, value = segment[0], segment[1]
            out, lse = ops.attention_lse(q_native.contiguous(), key.contiguous(), value.contiguous(),
                                         scale=scale)
        # merging into the empty partition (0, -inf) returns the partial unchanged
        native_out, native_lse = (out, lse) if native_out is None else \
            ops.lse_merge([(native_out, native_lse), (out, lse)])
    if native_out is None:
        native_out = torch.zeros_like(q_native)
        native_lse = torch.full((Q, H), -math.inf, device=q_native.device)
    result = torch.empty_like(q_native)
    running_lse = torch.empty_like(native_lse)
    moments = value_mean = None
    if value_mean_residual and low_segments:
        moments = history_moments(low_segments)
        value_mean = compressed_value_mean(low_segments, moments, heads=H, native_dim=reader.native_dim)
    for group in reader.groups:
        head = group.heads
        # reduced query of the group's heads, zero-padded to the kernel's tile width (own kernel)
        query = ops.head_linear(q_pre, group.q_reduce, heads=head, pad_to=group.padded)
        if rope is not None:
            if group.pair_index is None or q_positions is None:
                raise ValueError("the selected RoPE needs the group's indices and the query positions")
            query = rope.rotate(query, q_positions, group.pair_index)
        if camera is not None:
            if group.cam_index_k is None:
                raise ValueError("the camera transform needs reader indices that keep whole 8-wide blocks")
            query = ops.camera_rows(query, _camera(camera["q"], group.cam_index_k, Q))
        mean_rows = projected = None
        if value_mean is not None and group.width < reader.native_dim:
            # mean over the low tokens of the group's low-width V read, by linearity
            total = sum(n for _, _, n in moments)
            mean_low = torch.zeros(head.numel(), group.padded, device=q_native.device)
            for segment, (latent_sum, counts, n) in zip(low_segments, moments):
                table = group.projected_centers(segment["v"], "v").centers.float()
                mean_low += (torch.einsum("her,r->he", group.v_read.float(), latent_sum)
                             + n * group.bias(segment["v_mean"], "v")
                             + (counts @ table).view(head.numel(), group.padded))
            mean_low = (mean_low / total)[:, :group.width]
            projected = torch.einsum("he,hed->hd", mean_low, group.lift.float())
            mean_rows = value_mean
        partials = []
        for segment in low_segments:
            view_k = group.projected_centers(segment["k"], "k")
            view_v = group.projected_centers(segment["v"], "v")
            positions = segment.get("positions")
            if segment.get("visible") is not None:
                view_k = ops.gather_view(view_k, segment["visible"])
                view_v = ops.gather_view(view_v, segment["visible"])
                if positions is not None:
                    positions = positions.index_select(0, segment["visible"])
            rope_view = rope.view(positions, group.pair_index) if rope is not None else None
            cam_k = cam_v = None
            if camera is not None:
                cam_k = _camera(segment["camera"], group.cam_index_k, view_k.tokens)
                cam_v = _camera(segment["camera"], group.cam_index_v, view_v.tokens)
            prepared = group.prepared and ops.tensor_core_read(query.dtype, group.padded, group.padded,
                                                               group.rank)
            oo, ll = ops.attn_codec(
                query, view_k, view_v, group.k_read_tc if prepared else group.k_read,
                group.bias(segment["k_mean"], "k"), group.v_read_tc if prepared else group.v_read,
                group.bias(segment["v_mean"], "v"), scale=scale, rope=rope_view,
                camera_k=cam_k, camera_v=cam_v, prepared=prepared)
            if camera is not None:
                oo = ops.camera_rows(oo, _camera(camera["out"], group.cam_index_v, Q))
            partials.append((oo, ll))
        if value_mean is not None and len(partials) > 1:
            # LingBot's form attends the joined low history once: one low partial per group
            partials = [ops.lse_merge(partials)]
        # value-mean correction, log-sum-exp merge and head scatter in one launch per partial;
        # the running (O, lse) of the group's heads lives in ``result`` / ``running_lse``
        source, source_lse = native_out, native_lse
        for oo, ll in partials:
            lifted = ops.head_linear(oo, group.lift, din=group.width)   # [Q, h, D]
            ops.fast_finish(source, source_lse, lifted, ll, head, result, value_mean=mean_rows,
                            projected_mean=projected, out_lse=running_lse)
            source, source_lse = result, running_lse
        if not partials:
            result.index_copy_(1, head, native_out.index_select(1, head))
    return result


def _hybrid_visible(q_pre, q_native, native_segments, low_segments, reader, *, rope, q_positions,
                    value_mean_residual, camera, query_groups):
    """hybrid_attention under boolean visibility: one unmasked read per query group over the keys
    the group sees (attention_grouped_mask MGC/core.py:94-108, applied to every segment)."""
    if camera is not None or value_mean_residual:
        raise ValueError("visibility masks combine with the rotation only: the camera transform and "
                         "the value-mean residual index tokens by their place in the segment")
    masks = [segment[2] for segment in native_segments
             if not isinstance(segment, dict) and len(segment) > 2 and segment[2] is not None]
    masks += [segment["mask"] for segment in low_segments if segment.get("mask") is not None]
    groups = masks[0].shape[0]
    if any(mask.dtype != torch.bool or mask.dim() != 2 or mask.shape[0] != groups for mask in masks):
        raise ValueError("Only boolean visibility masks [groups, tokens] are supported")
    if query_groups is None and groups != 1:
        raise ValueError("several visibility rows need query_groups")
    if query_groups is not None and (query_groups.numel() != q_native.shape[0] or
                                     int(query_groups.min()) < 0 or int(query_groups.max()) >= groups):
        raise ValueError("query_groups holds one visibility row index per query")
    result = torch.empty_like(q_native)
    for g in range(groups):
        rows = None
        if query_groups is not None:
            rows = torch.nonzero(query_groups == g).flatten()
            if rows.numel() == 0:
                continue
        native = []
        for segment in native_segments:
            if isinstance(segment, dict):          # compressed protected tokens carry no mask
                native.append(segment)
                continue
            key, value, *visible = segment
            if visible and visible[0] is not None:
                index = torch.nonzero(visible[0][g]).flatten()
                if index.numel() == 0:
                    continue
                key, value = key.index_select(0, index), value.index_select(0, index)
            native.append((key, value))
        low = []
        for segment in low_segments:
            entry = {name: item for name, item in segment.items() if name != "mask"}
            if segment.get("mask") is not None:
                entry["visible"] = torch.nonzero(segment["mask"][g]).flatten()
                if entry["visible"].numel() == 0:
                    continue
            low.append(entry)
        pick = (lambda t: t) if rows is None else (lambda t: t.index_select(0, rows).contiguous())
        part = hybrid_attention(pick(q_pre), pick(q_native), native, low, reader, rope=rope,
                                q_positions=None if q_positions is None else pick(q_positions))
        if rows is None:
            return part
        result.index_copy_(0, rows, part)
    return result
