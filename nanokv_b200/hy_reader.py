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
transform works on (branches narrower than the kernel's 64 columns -- HY's deployed heads are 32 wide -- are
padded with zero channels first); queries, read matrices, centre tables and the lift are permuted alike, so the
permutation cancels in every product.  ``recent_native_frames > 0`` (a second, full-width history
partition) is not built: the call raises.

``compress_layer_cache`` is the write side (`compress_layer_cache` :1657-1675 with `_compress_one`
:1457-1596 for the dictionary low-KV payload): the layer cache's raw `k_vision` / `v_vision` tensors
become the packed payloads the reader takes.  The per-layer runtime the reference builds from its
manifest (`_device_layer`) is handed over with ``register_runtime``.
"""
from __future__ import annotations

import math
import os

import torch

from . import attention, ops
from .codec import kmeans_init_rows

_PREPARED: dict = {}
_RUNTIMES: dict = {}


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


def _kernel_width(width: int) -> int:
    """The fused read is built for head widths 64 and 128: a narrower branch (HY's deployed heads are 32
    wide) is padded with zero channels, which add nothing to a score and give zero output columns."""
    if width <= 64:
        return 64
    if width <= 128:
        return 128
    raise ValueError(f"branch width {width} exceeds 128")


def _pad_rows(tensor: torch.Tensor, width: int) -> torch.Tensor:      # [H, d, X] -> [H, width, X]
    return torch.nn.functional.pad(tensor, (0, 0, 0, width - tensor.shape[1]))


def _pad_cols(tensor: torch.Tensor, width: int) -> torch.Tensor:      # [..., d] -> [..., width]
    return torch.nn.functional.pad(tensor, (0, width - tensor.shape[-1]))


def _prepare(state: dict, device, dtype):
    """Device-resident operands of both branches in the kernels' layouts, cached per state dict."""
    key = (id(state), str(device), dtype)
    if key in _PREPARED:
        return _PREPARED[key]
    to = dict(device=device, dtype=dtype)
    heads, main_width, native = state["q_main_reduce"].shape
    quartets = state["q_prope_mix"].shape[1]
    prope_width = 4 * quartets
    if native % 4 or main_width % 2:
        raise ValueError("branch widths must hold whole pairs and quartets")
    main_pad, prope_pad = _kernel_width(main_width), _kernel_width(prope_width)
    order = _block_order(prope_pad, device)      # over the padded width: the added quartets are zero
    eye = torch.eye(4, device=device)
    # quartet mixes as dense per-head matrices: reduce [H, native, 4q], lift [H, 4q, native]
    reduce = torch.einsum("hro,cd->hocrd", state["q_prope_mix"].to(device).float(), eye)
    reduce = _pad_cols(reduce.reshape(heads, native, prope_width), prope_pad).index_select(2, order)
    lift = torch.einsum("hro,cd->hrcod", state["v_prope_mix"].to(device).float(), eye)
    lift = _pad_rows(lift.reshape(heads, prope_width, native), prope_pad).index_select(1, order)
    indices = state["main_indices"].long().cpu()
    if not torch.equal(indices[:, 1::2], indices[:, ::2] + 1) or bool((indices[:, ::2] % 2).any()):
        raise ValueError("RoPE mapping must retain complete original pairs")
    prepared = {
        "heads": heads, "main_width": main_width, "prope_width": prope_width, "native": native,
        "main_pad": main_pad, "prope_pad": prope_pad,
        "order": order, "indices": state["main_indices"].long().to(device),
        # the padded pairs rotate zeros: any table column will do
        "pair_index": _pad_cols((indices[:, ::2] // 2).to(torch.int32), main_pad // 2).to(device).contiguous(),
        "q_main": _pad_cols(state["q_main_reduce"].to(**to).transpose(1, 2), main_pad).contiguous(),
        "q_prope": reduce.contiguous(),
        "k_main": _pad_rows(state["k_main_read"].to(**to), main_pad).contiguous(),
        "v_main": _pad_rows(state["v_main_read"].to(**to), main_pad).contiguous(),
        "k_prope": _pad_rows(state["k_prope_read"].to(**to), prope_pad).index_select(1, order).contiguous(),
        "v_prope": _pad_rows(state["v_prope_read"].to(**to), prope_pad).index_select(1, order).contiguous(),
        "lift_main": _pad_rows(state["v_main_lift"].to(**to), main_pad).contiguous(),
        "lift_prope": lift.contiguous(),
        "scale_main": state["log_residual_scale_main"].to(device).float().exp(),
        "scale_prope": state["log_residual_scale_prope"].to(device).float().exp(),
        "zero_main": torch.zeros(heads, main_pad, device=device),
        "zero_prope": torch.zeros(heads, prope_pad, device=device),
        "cam_index": torch.zeros(heads, prope_pad // 8, dtype=torch.int32, device=device),
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

    prope_table = _pad_cols(payload["centre_prope"].to(device), prepared["prope_pad"]).index_select(3, prepared["order"])
    views = (view(_pad_cols(payload["centre_main"].to(device), prepared["main_pad"])), view(prope_table))
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
        q_main = _pad_cols(q_main, prepared["main_pad"])
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


# --------------------------------------------------------------------------------- write side
def register_runtime(layer_idx: int, runtime: dict) -> None:
    """The runtime of one layer as the reference's `_device_layer` returns it: ``operators`` (per
    target ``mean`` f32 [2048] and ``encoder`` bf16 [r, 2048]), ``attention`` (the reader state with
    `k_main_anchor_reduce` / `main_indices`, `q_prope_mix` or `k_prope_anchor_mix`,
    `v_main_anchor_reduce`, `v_prope_anchor_mix`), ``main_k_mode``, ``shape``
    (k_heads, k_dim, v_heads, v_dim), ``payload_mode`` = "dictionary_lowkv"."""
    if runtime.get("payload_mode", "dictionary_lowkv") != "dictionary_lowkv":
        raise NotImplementedError("only the dictionary low-KV payload is built")
    if runtime.get("grouped_attention") is not None:
        raise NotImplementedError("grouped head widths are not built")
    _RUNTIMES[int(layer_idx)] = runtime


def _quartet_reduce(native: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """[B, H, n, 128] -> [B, H, n, 4 * quartets]: the 32 quartets of a head row mixed per component
    (`_quartet_reduce_runtime` :1191-1193)."""
    quartets = native.float().reshape(*native.shape[:-1], 32, 4)
    return torch.einsum("hro,bhnoc->bhnrc", mix.float(), quartets).flatten(-2)


@torch.no_grad()
def _compress_one(x: torch.Tensor, layer_idx: int, target: str, runtime: dict) -> dict:
    """x [1, 16, S, 128] -> the dictionary low-KV payload of one tensor (:1457-1596): online joint-head
    C-means (HY/kv_codecs.py:116-208, residual rounded to the input dtype), encoder in bf16, INT4
    codes against an fp32 scale with floor 1e-12, and the centre table projected once into the two
    branches' low widths (centres + mean, per head: the Main reduce resp. the quartet mix)."""
    if x.ndim != 4 or x.shape[0] != 1 or x.shape[1] * x.shape[3] != 2048 or x.shape[1] != 16:
        raise ValueError(f"expected [1,16,S,128], got {tuple(x.shape)}")
    batch, heads, sequence, dim = x.shape
    op = runtime["operators"][target]
    state = runtime["attention"]
    mean = op["mean"].to(device=x.device, dtype=torch.float32).contiguous()
    encoder = op["encoder"].to(device=x.device, dtype=torch.bfloat16).contiguous()
    clusters = int(os.environ.get("HY_KV_CODEC_SEMANTIC_CLUSTERS", "64"))
    iters = int(os.environ.get("HY_KV_CODEC_SEMANTIC_ITERS", "2"))
    if clusters <= 0 or clusters > sequence or clusters > 256:
        raise ValueError(f"semantic clusters must be in [1,min(S,256)], got {clusters}")
    rows = x.permute(0, 2, 1, 3).reshape(sequence, heads * dim).contiguous()
    init = kmeans_init_rows(sequence, clusters, 20260804 + int(layer_idx)).to(x.device)
    centers, ids = ops.kmeans(rows, clusters, iters, init)
    residual = (rows.float() - centers.float().index_select(0, ids.long())).to(x.dtype)
    zero_center = torch.zeros(1, heads * dim, dtype=torch.bfloat16, device=x.device)
    zero_ids = torch.zeros(sequence, dtype=torch.uint8, device=x.device)
    coeff = ops.project(residual, zero_center, zero_ids, mean, encoder)          # bf16 [S, r]
    packed, _ = ops.quant_pack(coeff, eps=1e-12, in_coeff_dtype=False)
    amax = coeff.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-12)
    scale = (amax / torch.full_like(amax, 7.0)).reshape(batch, sequence, 1)      # the fp32 scale the codes used
    native = (centers.float() + mean[None]).reshape(batch, clusters, heads, dim).permute(0, 2, 1, 3)
    to = lambda name: state[name].to(x.device)
    if target == "k":
        if runtime.get("main_k_mode", "learned_rope") == "learned_rope":
            centre_main = torch.einsum("bhnr,hdr->bhnd", native, to("k_main_anchor_reduce").float())
        else:
            index = to("main_indices")
            centre_main = torch.gather(native, -1, index[None, :, None].expand(batch, -1, native.shape[2], -1))
        mix = to("k_prope_anchor_mix") if "k_prope_anchor_mix" in state else to("q_prope_mix")
        centre_prope = _quartet_reduce(native, mix)
    else:
        centre_main = torch.einsum("bhco,hdo->bhcd", native, to("v_main_anchor_reduce").float())
        centre_prope = _quartet_reduce(native, to("v_prope_anchor_mix"))
    k_heads, k_dim, v_heads, v_dim = runtime["shape"]
    kv_heads, head_dim = (k_heads, k_dim) if target == "k" else (v_heads, v_dim)
    return {
        "direct_codec_latent": True, "layer_idx": int(layer_idx), "tensor_name": target,
        "shape": tuple(int(v) for v in x.shape),
        "latent_int4": packed.reshape(-1), "latent_shape": (batch, sequence, int(encoder.shape[0])),
        "latent_numel": batch * sequence * int(encoder.shape[0]), "latent_scale": scale,
        "centre_latent": None, "centre_main": centre_main.to(torch.bfloat16),
        "centre_prope": centre_prope.to(torch.bfloat16), "semantic_ids": ids[None].to(torch.uint8),
        "kv_heads": kv_heads, "head_dim": head_dim, "payload_mode": "dictionary_lowkv",
    }


def compress_layer_cache(layer_cache: dict, layer_idx: int) -> dict:
    """Replace the raw `k_vision` / `v_vision` history of a layer cache by packed payloads (:1657-1675).
    A layer without a registered runtime is left alone, as a layer outside the manifest is there."""
    runtime = _RUNTIMES.get(int(layer_idx))
    if runtime is None:
        return layer_cache
    if int(runtime.get("recent_native_frames", 0)) > 0:
        raise NotImplementedError("the recent-native history partition is not built")
    first, second = layer_cache.get("k_vision"), layer_cache.get("v_vision")
    if not isinstance(first, torch.Tensor):
        raise RuntimeError("direct codec-latent compression must run before the formal codec")
    if not isinstance(second, torch.Tensor):
        raise RuntimeError("direct codec-latent compression requires raw V history")
    layer_cache.pop("_direct_codec_positioned_history", None)
    layer_cache.pop("_direct_codec_recent_native_pre", None)
    layer_cache["k_vision"] = _compress_one(first, layer_idx, "k", runtime)
    layer_cache["v_vision"] = _compress_one(second, layer_idx, "v", runtime)
    layer_cache["direct_codec_latent"] = True
    return layer_cache


def attend(layer_idx: int, q_pre_bshd, query_bhsd, current_key_bhsd, current_value_bhsd, encoder_key_bhsd,
           encoder_value_bhsd, layer_cache: dict, current_freqs_cis, current_viewmats, current_Ks):
    """The reference's public entry point (`attend` :4251-4279) for the dictionary low-KV runtime: the
    layer's registered runtime, the same two checks, then `attend_dictionary_lowkv`."""
    if not layer_cache.get("direct_codec_latent"):
        raise RuntimeError("selected direct layer is missing a direct latent payload")
    if query_bhsd.shape[0] != 2 * q_pre_bshd.shape[0]:
        raise RuntimeError("direct codec attention expects stacked main/PRoPE batches")
    runtime = _RUNTIMES.get(int(layer_idx))
    if runtime is None:
        raise KeyError(f"no runtime registered for layer {int(layer_idx)}")
    return attend_dictionary_lowkv(layer_idx, q_pre_bshd, query_bhsd, current_key_bhsd, current_value_bhsd,
                                   encoder_key_bhsd, encoder_value_bhsd, layer_cache, current_freqs_cis,
                                   current_viewmats, current_Ks, runtime)

