"""LingBot codec interface on the B200 kernels.

Same function names, argument lists, payload dictionaries and error classes as the reference
module LB/lingbot_v2_kv_codec.py (encode_tensor :256-297, decode_tensor :301-326,
direct_latent_rows :330-362, direct_latent_slice :365-401, decode_tensor_slice :404-417,
decode_tensor_rows :420-437, encode_pair :441-462, decode_segments :465-476, preload_operators
:55-78, tensor_bytes :81-88), so the backbone's call sites (LB/model_fast.py:170-195,
LB/lingbot_v2_cache_runtime.py:139-163,263-337) can import this module instead.

Operators: `register_operator` makes (mean, encoder, decoder) resident for a (target, layer,
sp_rank); `preload_operators` / the `basis_root` arguments read the reference's artefact files
(`global_head_pca.pt` with "mean" and ascending-eigenvalue "components", optionally a V-QAT or K-A1
checkpoint under `linear_root`, or the prepacked INT8 file named by
LINGBOT_V2_KV_CODEC_PREPACKED_OPERATOR_PATH) when nothing is registered for the key.
Every arithmetic step runs on the kernels of libnanokv_b200; there is no CPU path.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Any

import torch

from . import ops
from .cache import CompressedHistory
from .codec import LINGBOT_QUANT, Operator, kmeans_init_rows

FORMAT = "lingbot_v2_semantic_residual_int4_v1"
OPERATOR_FORMAT = "lingbot_v2_operator_int8_v1"

_OPERATORS: dict[tuple, Operator] = {}
_PREPACKED: dict[str, dict] = {}


def register_operator(target: str, layer: int, *, mean, encoder, decoder, sp_rank: int = 0,
                      device="cuda") -> Operator:
    """Make (mean [J], encoder [r,J], decoder [J,r]) resident for (target, layer, sp_rank); LingBot's
    operators are bf16 (LB/lingbot_v2_kv_codec.py:202-206)."""
    if target not in {"k", "v"}:
        raise ValueError(target)
    op = Operator(mean, encoder.to(torch.bfloat16), decoder.to(torch.bfloat16), device=device)
    _OPERATORS[(target, int(layer), int(sp_rank), torch.device(device).type)] = op
    return op


def _artifact_path(root, sp_rank: int, layer: int) -> Path:
    root = Path(root)
    ranked = root / f"rank_{sp_rank:02d}" / f"layer_{layer:02d}" / "global_head_pca.pt"
    legacy = root / f"layer_{layer:02d}" / "global_head_pca.pt"
    return ranked if ranked.exists() or not legacy.exists() else legacy


def _load_operator(root, *, target: str, sp_rank: int, layer: int, joint_dim: int, rank: int,
                   device, linear_root=None) -> Operator:
    """Registered operator, else the reference's artefact files (LB/lingbot_v2_kv_codec.py:108-207)."""
    device = torch.device(device)
    key = (target, int(layer), int(sp_rank), device.type)
    if key in _OPERATORS:
        op = _OPERATORS[key]
        if op.joint != joint_dim or op.rank != rank:
            raise RuntimeError(f"operator cannot serve dim/rank={joint_dim}/{rank}: {op.joint}/{op.rank}")
        return op
    prepacked_path = os.environ.get("LINGBOT_V2_KV_CODEC_PREPACKED_OPERATOR_PATH", "").strip()
    if prepacked_path:
        resolved = str(Path(prepacked_path).resolve())
        if resolved not in _PREPACKED:
            packed = torch.load(resolved, map_location="cpu", weights_only=False)
            if packed.get("format") != OPERATOR_FORMAT:
                raise RuntimeError(f"bad prepacked operator: {resolved}")
            _PREPACKED[resolved] = packed
        packed = _PREPACKED[resolved]
        entry_key = f"rank{sp_rank:02d}:{target}:{layer:02d}"
        entry = packed["entries"].get(entry_key)
        if entry is None:
            raise KeyError(f"prepacked operator missing {entry_key}")
        if int(packed.get("rank", -1)) != rank:
            raise RuntimeError(f"prepacked rank mismatch: {packed.get('rank')} != {rank}")
        op = Operator.from_int8(entry["mean"].float(), entry["encoder"], entry["decoder"], device=device)
        _OPERATORS[key] = op
        return op
    path = _artifact_path(root, sp_rank, layer)
    if not path.exists():
        raise KeyError(f"no operator registered for {target}:{int(layer):02d} (sp_rank {sp_rank}) on "
                       f"{device} and no artefact at {path}")
    item = torch.load(path, map_location="cpu", weights_only=False)
    if item.get("target", item.get("tensor_name")) != target:
        raise RuntimeError(f"operator target mismatch: {path}")
    if int(item.get("sp_rank", sp_rank)) != sp_rank:
        raise RuntimeError(f"operator SP-rank mismatch: {path}")
    mean, components = item["mean"].float(), item["components"].float()
    if tuple(mean.shape) != (joint_dim,) or components.ndim != 2:
        raise RuntimeError(f"operator shape mismatch: {path}")
    if components.shape[1] != joint_dim or components.shape[0] < rank:
        raise RuntimeError(f"operator cannot serve dim/rank={joint_dim}/{rank}: {tuple(components.shape)}")
    encoder = components[-rank:].contiguous()       # highest-variance subspace: the suffix
    decoder = encoder.T.contiguous()
    if linear_root is not None:
        checkpoint = Path(linear_root)
        if checkpoint.is_dir():
            checkpoint = checkpoint / f"rank_{sp_rank:02d}" / f"layer_{layer:02d}" / "checkpoint_best.pt"
        trained = torch.load(checkpoint, map_location="cpu", weights_only=False)
        if target == "v":
            if trained.get("format") != "lingbot_v2_c64_int4_qat_v1":
                raise RuntimeError(f"bad V-QAT checkpoint: {checkpoint}")
            state = trained["model"]
            encoder = state["basis"].float() + state["encoder_delta"].float()
            decoder = state["basis"].float().T + state["decoder_delta"].float()
            mean = state["mean"].float()
        else:
            if trained.get("format") != "lingbot_v2_k_a1_decoder_delta_v1":
                raise RuntimeError(f"bad K-A1 checkpoint: {checkpoint}")
            saved = trained["decoder_delta"].get(str(layer))
            if saved is not None:
                decoder = decoder + saved.float()
    op = Operator(mean, encoder.to(torch.bfloat16), decoder.contiguous().to(torch.bfloat16), device=device)
    _OPERATORS[key] = op
    return op


@torch.no_grad()
def preload_operators(*, basis_root_k, basis_root_v, linear_root_k, linear_root_v, rank: int,
                      layers: int, joint_dim: int, sp_rank: int, device) -> None:
    """Make every layer's operators resident before the timed interval."""
    for layer in range(int(layers)):
        _load_operator(basis_root_k, target="k", sp_rank=int(sp_rank), layer=layer, joint_dim=int(joint_dim),
                       rank=int(rank), device=device, linear_root=linear_root_k)
        _load_operator(basis_root_v, target="v", sp_rank=int(sp_rank), layer=layer, joint_dim=int(joint_dim),
                       rank=int(rank), device=device, linear_root=linear_root_v)


def tensor_bytes(value: Any) -> int:
    if torch.is_tensor(value):
        return value.numel() * value.element_size()
    if isinstance(value, dict):
        return sum(tensor_bytes(v) for k, v in value.items() if not str(k).startswith("_"))
    if isinstance(value, (list, tuple)):
        return sum(tensor_bytes(v) for v in value)
    return 0


def _seed(layer: int, sp_rank: int, target: str) -> int:
    return 20260826 + int(layer) * 17 + int(sp_rank) * 1009 + (target == "v")


@torch.no_grad()
def encode_tensor(value: torch.Tensor, *, target: str, layer: int, sp_rank: int, basis_root, rank: int,
                  clusters: int = 64, iters: int = 2, linear_root=None) -> dict[str, Any]:
    """value [1,S,H,D] on the GPU -> the reference's payload dictionary (online C-means over the
    joint H*D axis, residual projection, per-token INT4)."""
    if value.ndim != 4 or value.shape[0] != 1:
        raise ValueError(f"expected [1,S,H,D], got {tuple(value.shape)}")
    batch, sequence, heads, head_dim = map(int, value.shape)
    if not 0 < clusters <= min(sequence, 256):
        raise ValueError(f"invalid C={clusters} for S={sequence}")
    joint_dim = heads * head_dim
    op = _load_operator(basis_root, target=target, sp_rank=sp_rank, layer=layer, joint_dim=joint_dim,
                        rank=rank, device=value.device, linear_root=linear_root)
    rows = value.reshape(sequence, joint_dim).contiguous()
    init = kmeans_init_rows(sequence, clusters, _seed(layer, sp_rank, target)).to(value.device)
    centers, ids = ops.kmeans(rows, clusters, iters, init)
    packed, scale = ops.project_quant(rows, centers, ids, op.mean, op.encoder, eps=LINGBOT_QUANT.eps,
                                      in_coeff_dtype=False)
    return {
        "format": FORMAT, "target": target, "layer": layer, "sp_rank": sp_rank,
        "shape": (batch, sequence, heads, head_dim), "rank": rank,
        "clusters": clusters, "centers": centers[None], "ids": ids[None],
        "latent_packed": packed.reshape(-1), "latent_count": sequence * rank,
        "latent_shape": (batch, sequence, rank),
        "latent_scale": scale.reshape(batch, sequence, 1),
        "basis_root": str(Path(basis_root).resolve()),
        "linear_root": "" if linear_root is None else str(Path(linear_root).resolve()),
    }


def _check(payload: dict) -> None:
    if payload.get("format") != FORMAT:
        raise RuntimeError(f"bad codec payload: {payload.get('format')}")


def history_from_payloads(parts: list[dict], *, device) -> CompressedHistory:
    """Same-layer payloads of one target stacked into one struct-of-arrays history (the form the
    kernels read); derived state, cached on the first payload when the list is reused unchanged."""
    first = parts[0]
    target, layer = str(first["target"]), int(first["layer"])
    batch, _, heads, head_dim = map(int, first["shape"])
    joint, rank = heads * head_dim, int(first["rank"])
    for part in parts:
        _check(part)
        if (str(part["target"]) != target or int(part["layer"]) != layer
                or tuple(map(int, part["shape"][::3])) != (batch, head_dim)
                or int(part["shape"][2]) != heads or int(part["rank"]) != rank):
            raise ValueError("incompatible LingBot codec segments")
    if batch != 1:
        raise ValueError("only batch 1 payloads are supported")
    key = tuple(id(part) for part in parts) + (str(torch.device(device)),)
    cached = first.get("_nkv_history")
    if cached is not None and cached[0] == key:
        return cached[1]
    total = sum(int(part["shape"][1]) for part in parts)
    clusters = max(int(part["centers"].shape[1]) for part in parts)
    hist = CompressedHistory(joint=joint, rank=rank, capacity=total, max_segments=len(parts),
                             centers_per_segment=clusters, device=device)
    for part in parts:
        count = int(part["shape"][1])
        offset, rows = hist.reserve_segment(count, int(part["centers"].shape[1]))
        rows.copy_(part["centers"][0].to(device=device, dtype=torch.bfloat16))
        hist.codes[offset:offset + count].copy_(part["latent_packed"].to(device).reshape(count, -1))
        hist.scales[offset:offset + count].copy_(
            part["latent_scale"].to(device=device, dtype=torch.bfloat16).reshape(count, -1))
        hist.ids[offset:offset + count].copy_(part["ids"].to(device).reshape(-1))
    first["_nkv_history"] = (key, hist)
    return hist


def operator_of(payload: dict, device) -> Operator:
    batch, _, heads, head_dim = map(int, payload["shape"])
    return _load_operator(payload["basis_root"], target=str(payload["target"]), sp_rank=int(payload["sp_rank"]),
                          layer=int(payload["layer"]), joint_dim=heads * head_dim, rank=int(payload["rank"]),
                          device=device, linear_root=payload.get("linear_root") or None)


def _decode(parts: list[dict], rows, *, dtype, device) -> torch.Tensor:
    hist = history_from_payloads(parts, device=device)
    op = operator_of(parts[0], device)
    out = ops.decode_rows(hist.view(), op.decoder, op.mean, rows=rows, dtype=dtype)
    _, _, heads, head_dim = map(int, parts[0]["shape"])
    return out.reshape(1, -1, heads, head_dim)


@torch.no_grad()
def decode_tensor(payload: dict, *, dtype: torch.dtype, device) -> torch.Tensor:
    """payload -> [1,S,H,D]: bf16(code * scale) @ decoder^T + bf16(mean), rounded, plus the bf16 centre."""
    _check(payload)
    return _decode([payload], None, dtype=dtype, device=device)


@torch.no_grad()
def decode_tensor_rows(payload: dict, row_index: torch.Tensor, *, dtype: torch.dtype, device) -> torch.Tensor:
    """Decode only the listed rows (policy-protected tokens) to native head width."""
    _check(payload)
    index = row_index.to(device=device, dtype=torch.int32).contiguous()
    return _decode([payload], index, dtype=dtype, device=device)


@torch.no_grad()
def decode_tensor_slice(payload: dict, start: int, stop: int, *, dtype: torch.dtype, device) -> torch.Tensor:
    _check(payload)
    sequence = int(payload["latent_shape"][1])
    start, stop = int(start), int(stop)
    if not 0 <= start <= stop <= sequence:
        raise ValueError(f"invalid latent interval [{start}:{stop}] for {tuple(payload['latent_shape'])}")
    index = torch.arange(start, stop, dtype=torch.int32, device=device)
    return _decode([payload], index, dtype=dtype, device=device)


def _latent(payload: dict, device) -> torch.Tensor:
    """bf16(code * scale) of every row, [1,S,r]: the accessor form of the latent (bit operations and
    one multiply; the kernels never need it -- they read the packed codes)."""
    shape = tuple(map(int, payload["latent_shape"]))
    packed = payload["latent_packed"].to(device)
    nibbles = torch.stack((packed & 15, (packed >> 4) & 15), dim=1).reshape(-1)[:int(payload["latent_count"])]
    codes = nibbles.to(torch.int16).sub_(7).reshape(shape)
    return codes.to(torch.bfloat16) * payload["latent_scale"].to(device=device, dtype=torch.bfloat16)


@torch.no_grad()
def direct_latent_rows(payload: dict, row_index: torch.Tensor, *, device):
    """(latent [1,n,r], (centers [1,C,J], ids [1,n]), mean f32 [J]) of the selected rows."""
    if payload.get("format") != FORMAT:
        raise RuntimeError("codec-native attention accepts only the frozen codec payload")
    index = row_index.to(device=device, dtype=torch.long)
    latent = _latent(payload, device).index_select(1, index)
    centers = payload["centers"].to(device=device, dtype=torch.bfloat16)
    ids = payload["ids"].to(device=device, dtype=torch.long).index_select(1, index)
    return latent, (centers, ids), operator_of(payload, device).mean


@torch.no_grad()
def direct_latent_slice(payload: dict, start: int, stop: int, *, device):
    if payload.get("format") != FORMAT:
        raise RuntimeError("codec-native attention accepts only the frozen codec payload")
    shape = tuple(map(int, payload["latent_shape"]))
    start, stop = int(start), int(stop)
    if not 0 <= start <= stop <= shape[1]:
        raise ValueError(f"invalid latent interval [{start}:{stop}] for {shape}")
    latent = _latent(payload, device)[:, start:stop]
    centers = payload["centers"].to(device=device, dtype=torch.bfloat16)
    ids = payload["ids"].to(device=device, dtype=torch.long)[:, start:stop]
    return latent, (centers, ids), operator_of(payload, device).mean


@torch.no_grad()
def encode_pair(key: torch.Tensor, value: torch.Tensor, *, cache: dict[str, Any]) -> dict[str, Any]:
    common = {
        "layer": int(cache["codec_layer"]), "sp_rank": int(cache.get("codec_sp_rank", 0)),
        "rank": int(cache["codec_rank"]), "clusters": int(cache.get("codec_clusters", 64)),
        "iters": int(cache.get("codec_iters", 2)),
    }
    result = {
        "format": FORMAT,
        "global_start": int(cache["codec_commit_start"]),
        "global_end": int(cache["codec_commit_start"] + key.shape[1]),
        "k": encode_tensor(key, target="k", basis_root=cache["codec_basis_root_k"],
                           linear_root=cache.get("codec_linear_root_k"), **common),
        "v": encode_tensor(value, target="v", basis_root=cache["codec_basis_root_v"],
                           linear_root=cache.get("codec_linear_root_v"), **common),
    }
    result["resident_bytes"] = tensor_bytes(result)
    return result


@torch.no_grad()
def decode_segments(segments: list[dict[str, Any]], *, dtype: torch.dtype, device, rows=None):
    """[{"k": payload, "v": payload}, ...] -> (K [1,N,H,D], V [1,N,H,D]), or None for an empty list.
    ``rows`` (i32, an addition to the reference's signature) limits the decode to those rows of the
    stacked segments, so that a window cut costs no decode of the rows outside it."""
    if not segments:
        return None
    return tuple(_decode([segment[target] for segment in segments], rows, dtype=dtype, device=device)
                 for target in ("k", "v"))
