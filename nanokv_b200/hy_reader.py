"""HY-WorldPlay's two-branch dictionary reader on the B200 kernels.

``attend_dictionary_lowkv`` has the name-sake's argument list and return value
(HY/direct_codec_latent_attention.py:4165-4247, `_attend_dictionary_lowkv`; the public `attend` :4251
dispatches to it for the dictionary low-KV runtime): the model evaluates two attention branches over
all heads, stacked on the batch axis -- a Main branch whose low-width keys carry the selected 3-D
RoPE pairs, and a PRoPE branch whose low-width keys and values are transformed quartet by quartet
with the camera projection of each token's frame -- both reading the same packed INT4 history
through their own read matrices and their own pre-projected centre tables, merged by log-sum-exp
with the native attention over the text and current tokens.

Here each branch is one launch of the fused read: codes are expanded on chip, the branch's read
matrix is the decode operand, the rotation / camera transform runs on the rebuilt tile, and no
positioned low-width history (the reference's cached ``_direct_codec_positioned_history``) is ever
written to HBM.  What the reference computes in fp32 between kernels (the PRoPE query path, the
quartet lift, the final combine) stays fp32 here.

The PRoPE branch's low-width channels are stored permuted inside the prepared state so that two
neighbouring quartets form one 8-wide (component, quartet) block, the layout the kernel's camera
transform works on; queries, read matrices, centre tables and the lift are permuted alike, so the
permutation cancels in every product.  ``recent_native_frames > 0`` (a second, full-width history
partition) is not built: the call raises.
"""
from __future__ import annotations

import math

import torch

from . import attention, ops

_PREPARED: dict = {}


def projection_matrices(viewmats: torch.Tensor, Ks: torch.Tensor | None):
    """(P, P^T, P^-1) [1, cameras, 4, 4] f32 of world-to-camera transforms and optional intrinsics:
    P = lift(K with zero principal point) @ viewmat, P^-1 = inverse rigid transform @ lift(K^-1)
    (HY/../prope/camera_rope.py:196-222)."""
    view = viewmats.float()
    rotation_t = view[..., :3, :3].transpose(-1, -2)
    inverse = torch.zeros_like(view)
    inverse[..., :3, :3] = rotation_t
    inverse[..., :3, 3] = -(rotation_t @ view[..., :3, 3:4])[..., 0]
    inverse[..., 3, 3] = 1.0
    if Ks is None:
        return view, view.transpose(-1, -2), inverse
    fx, fy = Ks[..., 0, 0].float(), Ks[..., 1, 1].float()
    lift = torch.zeros_like(view)
    lift[..., 0, 0], lift[..., 1, 1], lift[..., 2, 2], lift[..., 3, 3] = fx, fy, 1.0, 1.0
    lift_inverse = torch.zeros_like(view)
    lift_inverse[..., 0, 0], lift_inverse[..., 1, 1] = 1.0 / fx, 1.0 / fy
    lift_inverse[..., 2, 2], lift_inverse[..., 3, 3] = 1.0, 1.0
    P = lift @ view
    return P, P.transpose(-1, -2), inverse @ lift_inverse


def _block_order(width: int, device) -> torch.Tensor:
    """old channel of every new channel: new[b*8 + j*2 + q] = old[(2b + q)*4 + j]."""
    new = torch.arange(width, device=device)
    block, inside = new // 8, new % 8
    return (2 * block + inside % 2) * 4 + inside // 2


def _prepare(state: dict, device, dtype):
    """Device-resident operands of both branches in the kernels' layouts, cached per state dict."""
    key = (id(state), str(device), dtype)
    if key in _PREPARED:
        return _PREPARED[key]
    to = dict(device=device, dtype=dtype)
    heads, main_width, native = state["q_main_reduce"].shape
    quartets = state["q_prope_mix"].shape[1]
    prope_width = 4 * quartets
    if prope_width % 8 or native % 4:
        raise ValueError("the PRoPE branch needs an even number of quartets")
    order = _block_order(prope_width, device)
    eye = torch.eye(4, device=device)
    # quartet mixes as dense per-head matrices: reduce [H, native, 4q], lift [H, 4q, native]
    reduce = torch.einsum("hro,cd->hocrd", state["q_prope_mix"].to(device).float(), eye)
    reduce = reduce.reshape(heads, native, prope_width).index_select(2, order)
    lift = torch.einsum("hro,cd->hrcod", state["v_prope_mix"].to(device).float(), eye)
    lift = lift.reshape(heads, prope_width, native).index_select(1, order)
    indices = state["main_indices"].long().cpu()
    if not torch.equal(indices[:, 1::2], indices[:, ::2] + 1) or bool((indices[:, ::2] % 2).any()):
        raise ValueError("RoPE mapping must retain complete original pairs")
    prepared = {
        "heads": heads, "main_width": main_width, "prope_width": prope_width, "native": native,
        "order": order, "indices": state["main_indices"].long().to(device),
        "pair_index": (indices[:, ::2] // 2).to(torch.int32).to(device).contiguous(),
        "q_main": state["q_main_reduce"].to(**to).transpose(1, 2).contiguous(),
        "q_prope": reduce.contiguous(),
        "k_main": state["k_main_read"].to(**to).contiguous(),
        "v_main": state["v_main_read"].to(**to).contiguous(),
        "k_prope": state["k_prope_read"].to(**to).index_select(1, order).contiguous(),
        "v_prope": state["v_prope_read"].to(**to).index_select(1, order).contiguous(),
        "lift_main": state["v_main_lift"].to(**to).contiguous(),
        "lift_prope": lift.contiguous(),
        "scale_main": state["log_residual_scale_main"].to(device).float().exp(),
        "scale_prope": state["log_residual_scale_prope"].to(device).float().exp(),
        "zero_main": torch.zeros(heads, main_width, device=device),
        "zero_prope": torch.zeros(heads, prope_width, device=device),
        "cam_index": torch.zeros(heads, prope_width // 8, dtype=torch.int32, device=device),
    }
    _PREPARED[key] = prepared
    return prepared


def _history_views(payload: dict, prepared: dict, device):
    """(Main view, PRoPE view) of one packed payload: same codes, scales and ids, the branch's own
    centre table; derived state, cached on the payload."""
    cached = payload.get("_nkv_views")
    if cached is not None and cached[0] == (str(device), id(prepared)):
        return cached[1]
    batch, tokens, rank = (int(v) for v in payload["latent_shape"])
    if batch != 1:
        raise ValueError("only batch 1 histories are supported")
    codes = payload["latent_int4"].to(device).reshape(tokens, rank // 2).contiguous()
    scales = payload["latent_scale"].to(device=device, dtype=torch.bfloat16).reshape(tokens, 1).contiguous()
    centres = int(payload["centre_main"].shape[2])
    ids = payload["semantic_ids"].to(device).reshape(tokens).to(ops.id_dtype(centres)).contiguous()
    seg_start = torch.tensor([0, tokens], dtype=torch.int32, device=device)
    seg_row = torch.zeros(1, dtype=torch.int32, device=device)

    def view(table):
        rows = table.to(device=device, dtype=torch.bfloat16)[0].permute(1, 0, 2)      # [C, H, d]
        return ops.HistoryView(codes=codes, scales=scales, ids=ids,
                               centers=rows.reshape(centres, -1).contiguous(), seg_start=seg_start,
                               seg_center_row=seg_row, tokens=tokens, segments=1, rank=rank, group=rank)

    prope_table = payload["centre_prope"].to(device).index_select(3, prepared["order"])
    views = (view(payload["centre_main"]), view(prope_table))
    payload["_nkv_views"] = ((str(device), id(prepared)), views)
    return views


def _multiplier(freqs_cis, device) -> "attention.RopeTable":
    """Rotation table with one row per token from the model's (cos, sin) [tokens, D] pair (or a
    complex [tokens, D/2] tensor); both channels of a pair must share their angle."""
    if isinstance(freqs_cis, tuple):
        cos, sin = (item.to(device).float() for item in freqs_cis)
        if not torch.equal(cos[:, ::2], cos[:, 1::2]) or not torch.equal(sin[:, ::2], sin[:, 1::2]):
            raise ValueError("cos / sin tables must repeat every angle over its channel pair")
        freqs_cis = torch.complex(cos[:, ::2].double(), sin[:, ::2].double())
    return attention.RopeTable.per_token(freqs_cis, device=device)


def _camera(matrix: torch.Tensor, prepared: dict, tokens: int) -> "ops.CameraView":
    cameras = int(matrix.shape[1])
    if tokens % cameras:
        raise ValueError("PRoPE frame count must divide the token sequence")
    slots = torch.zeros(cameras, 4, 4, 4, device=matrix.device)
    slots[:, 0] = matrix[0].float()
    return ops.CameraView(slots.contiguous(), prepared["cam_index"], tokens // cameras)


def _rows(x: torch.Tensor) -> torch.Tensor:
    return x.permute(1, 0, 2)          # [H,S,D] -> [S,H,D]


@torch.no_grad()
def attend_dictionary_lowkv(layer_idx, q_pre_bshd, query_bhsd, current_key_bhsd, current_value_bhsd,
                            encoder_key_bhsd, encoder_value_bhsd, layer_cache, current_freqs_cis,
                            current_viewmats, current_Ks, runtime):
    """(Main output, PRoPE output), each [1, S, H*D].  q_pre [1,S,H,D] pre-RoPE; query / current /
    encoder tensors [2,H,*,D] with the Main branch first; ``layer_cache`` holds the packed
    "k_vision" / "v_vision" payloads, "vision_freqs_cis", "vision_viewmats" and optional "vision_Ks";
    ``runtime["attention"]`` is the reader state of the layer."""
    if runtime.get("recent_native_frames", 0) > 0:
        raise NotImplementedError("the recent-native partition of the two-branch reader is not built")
    if q_pre_bshd.shape[0] != 1 or query_bhsd.shape[0] != 2:
        raise ValueError("expected batch 1: q_pre [1,S,H,D] and branch-stacked tensors [2,H,*,D]")
    device, dtype = query_bhsd.device, query_bhsd.dtype
    prepared = _prepare(runtime["attention"], device, dtype)
    queries, heads = int(q_pre_bshd.shape[1]), prepared["heads"]
    scale = 1.0 / math.sqrt(128.0)
    q_pre = q_pre_bshd[0]
    now = torch.arange(queries, device=device, dtype=torch.int32)
    # ---- Main query: learned reduction + selected RoPE, or the rotated native query's channels
    if runtime["main_k_mode"] == "learned_rope":
        q_main = ops.head_linear(q_pre, prepared["q_main"])
        q_main = _multiplier(current_freqs_cis, device).rotate(q_main, now, prepared["pair_index"])
    else:
        q_main = torch.gather(_rows(query_bhsd[0]), -1, prepared["indices"][None].expand(queries, -1, -1))
    q_main = (q_main * prepared["scale_main"][None, :, None]).to(dtype)
    # ---- PRoPE query: quartet reduction and P^T in fp32, as the reference keeps them
    _, p_transpose, _ = projection_matrices(current_viewmats.to(device), None if current_Ks is None
                                            else current_Ks.to(device))
    q_prope = ops.head_linear(q_pre.float(), prepared["q_prope"])
    q_prope = ops.camera_rows(q_prope, _camera(p_transpose, prepared, queries)).to(dtype)
    q_prope = (q_prope * prepared["scale_prope"][None, :, None]).to(dtype)
    # ---- the packed history through both branches' readers
    main_k, prope_k = _history_views(layer_cache["k_vision"], prepared, device)
    main_v, prope_v = _history_views(layer_cache["v_vision"], prepared, device)
    tokens = main_k.tokens
    past = torch.arange(tokens, device=device, dtype=torch.int32)
    rope = _multiplier(layer_cache["vision_freqs_cis"], device).view(past, prepared["pair_index"])
    vision_Ks = layer_cache.get("vision_Ks")
    _, _, p_inverse = projection_matrices(layer_cache["vision_viewmats"].to(device),
                                          None if vision_Ks is None else vision_Ks.to(device))
    camera = _camera(p_inverse, prepared, tokens)
    main_low, main_lse = ops.attn_codec(q_main.contiguous(), main_k, main_v, prepared["k_main"],
                                        prepared["zero_main"], prepared["v_main"], prepared["zero_main"],
                                        scale=scale, rope=rope)
    prope_low, prope_lse = ops.attn_codec(q_prope.contiguous(), prope_k, prope_v, prepared["k_prope"],
                                          prepared["zero_prope"], prepared["v_prope"], prepared["zero_prope"],
                                          scale=scale, camera_k=camera, camera_v=camera)
    # ---- native attention over text + current tokens, lift, one global softmax per branch
    outputs = []
    for branch, (low, low_lse) in enumerate(((main_low, main_lse), (prope_low, prope_lse))):
        native_k = torch.cat((_rows(encoder_key_bhsd[branch]), _rows(current_key_bhsd[branch]))).contiguous()
        native_v = torch.cat((_rows(encoder_value_bhsd[branch]), _rows(current_value_bhsd[branch]))).contiguous()
        native, native_lse = ops.attention_lse(_rows(query_bhsd[branch]).contiguous(), native_k, native_v,
                                               scale=scale)
        if branch == 0:
            lifted = ops.head_linear(low, prepared["lift_main"]).float()
        else:
            lifted = ops.head_linear(low.float(), prepared["lift_prope"])
        merged, _ = ops.lse_merge([(native.float(), native_lse), (lifted, low_lse)])
        outputs.append(merged.to(dtype).reshape(1, queries, heads * prepared["native"]))
    return outputs[0], outputs[1]
