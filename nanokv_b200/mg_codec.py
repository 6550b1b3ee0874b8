"""Matrix-Game codec interface on the B200 kernels.

Same function names, argument meaning, payload dictionaries and error classes
as the reference module MGM/nanokv_codec.py (encode_tensor :334-365,
decode_tensor :369-390, decode_value :516-539, concat_values :600-609,
value_shape :489-513, payload_bytes :697-704, preload_operator_weights :258-279), so its call sites in the
backbone (MGM/wan_video_dit.py:493-500,710-795) can import this module
instead.  Operators come from `register_operator`, or -- when nothing is
registered for a (kind, layer) -- from the reference's artefact files named by
its environment variables (`_from_artifacts`).
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Any

import torch

from . import ops
from .cache import CompressedHistory, PackedRows
from .codec import F32_EPS, Operator, kmeans_init_rows

CODEC = "worldplay_c64_pca_int4_v1"
SEGMENTS = "worldplay_segments_v1"
RAW = "worldplay_raw_v1"

_OPERATORS: dict[tuple[str, int, str], Operator] = {}


def register_operator(kind: str, layer: int, *, mean, encoder, decoder, device="cuda") -> Operator:
    """Make (mean [J], encoder [r,J], decoder [J,r]) resident for (kind, layer).
    fp32 or bf16 weights select the arithmetic, as the reference's operator storage does."""
    if kind not in {"k", "v"}:
        raise ValueError(kind)
    op = Operator(mean, encoder, decoder, device=device)
    _OPERATORS[(kind, int(layer), str(torch.device(device)))] = op
    return op


def _pack_int8(weight: torch.Tensor) -> dict:
    """The reference's INT8 operator packing (per row, or per MG35_KVCODEC_INT8_WEIGHT_GROUP_SIZE
    input columns): symmetric, scale = amax / 127 kept in bf16 (MGM/nanokv_codec.py:108-131)."""
    weight = weight.detach().float().cpu().contiguous()
    group = int(os.environ.get("MG35_KVCODEC_INT8_WEIGHT_GROUP_SIZE", "0") or 0) or int(weight.shape[1])
    if group > weight.shape[1] or weight.shape[1] % group:
        raise ValueError(f"INT8 group size {group} must divide {weight.shape[1]}")
    grouped = weight.reshape(weight.shape[0], -1, group)
    scale = grouped.abs().amax(dim=2).clamp_min(1e-12) / 127.0
    quantised = (grouped / scale[:, :, None]).round().clamp(-127, 127).to(torch.int8)
    return {"qweight": quantised.reshape_as(weight), "scale": scale.to(torch.bfloat16), "group_size": group}


def _from_artifacts(kind: str, layer: int, device) -> Operator | None:
    """Operator of (kind, layer) from the reference's artefact files, as its `_operator` reads them
    (MGM/nanokv_codec.py:151-249): the prepacked INT8 file named by
    MG35_KVCODEC_PREPACKED_OPERATOR_PATH, else the K basis under MG35_KVCODEC_BASIS_DIR/k_c64 with an
    optional trained decoder under MG35_KVCODEC_DECODER_DIR_K, resp. the V-QAT checkpoint under
    MG35_KVCODEC_DECODER_DIR_V; stored per MG35_KVCODEC_OPERATOR_WEIGHT_MODE (int8 | bf16 | fp32).
    None when no such variable is set.  Provenance bookkeeping (centre storage mode, directory
    hashes) stays with the caller."""
    prepacked = os.environ.get("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", "").strip()
    if prepacked:
        packed = torch.load(prepacked, map_location="cpu", weights_only=True)
        if packed.get("format") != "mg35_worldplay_operator_int8_v1":
            raise RuntimeError(f"bad prepacked WorldPlay operator: {prepacked}")
        entry = packed["entries"][f"{kind}:{int(layer):02d}"]
        return Operator.from_int8(entry["mean"].float(), entry["encoder"], entry["decoder"], device=device)
    if kind == "k":
        root = os.environ.get("MG35_KVCODEC_BASIS_DIR", "").strip()
        if not root:
            return None
        basis = torch.load(Path(root) / "k_c64" / f"layer_{int(layer):02d}.pt", map_location="cpu",
                           weights_only=True)
        mean, encoder = basis["mean"].float(), basis["components"].float()
        decoder = encoder.t().contiguous()
        trained = os.environ.get("MG35_KVCODEC_DECODER_DIR_K", "").strip()
        if trained:
            checkpoint = torch.load(Path(trained) / f"layer_{int(layer):02d}.pt", map_location="cpu",
                                    weights_only=True)
            if checkpoint.get("target") != "k_c64":
                raise RuntimeError(f"bad WorldPlay K decoder L{layer}: {trained}")
            decoder = checkpoint["decoder"].float()
    else:
        root = os.environ.get("MG35_KVCODEC_DECODER_DIR_V", "").strip()
        if not root:
            return None
        checkpoint = torch.load(Path(root) / f"layer_{int(layer):02d}.pt", map_location="cpu", weights_only=True)
        if checkpoint.get("format") != "mg35_worldplay_v_c64_int4_qat_v1":
            raise RuntimeError(f"bad WorldPlay V-QAT checkpoint L{layer}: {root}")
        mean, encoder, decoder = (checkpoint[name].float() for name in ("mean", "encoder", "decoder"))
    mode = os.environ.get("MG35_KVCODEC_OPERATOR_WEIGHT_MODE", "int8").strip().lower()
    if mode == "fp32":
        return Operator(mean, encoder, decoder, device=device)
    if mode == "bf16":
        return Operator(mean, encoder.to(torch.bfloat16), decoder.to(torch.bfloat16), device=device)
    if mode != "int8":
        raise ValueError(f"unsupported MG35 operator mode={mode}")
    return Operator.from_int8(mean, _pack_int8(encoder), _pack_int8(decoder), device=device)


def _operator(kind: str, layer: int, device) -> Operator:
    device = torch.device(device)
    for key in ((kind, int(layer), str(device)), (kind, int(layer), device.type)):
        if key in _OPERATORS:
            return _OPERATORS[key]
    loaded = _from_artifacts(kind, layer, device)
    if loaded is None:
        raise KeyError(f"no operator registered for {kind}:{int(layer):02d} on {device} and none of "
                       "MG35_KVCODEC_PREPACKED_OPERATOR_PATH / MG35_KVCODEC_BASIS_DIR / "
                       "MG35_KVCODEC_DECODER_DIR_V names its artefacts")
    _OPERATORS[(kind, int(layer), str(device))] = loaded
    return loaded


@torch.no_grad()
def preload_operator_weights(device) -> None:
    """Make every operator of the prepacked file resident before the timed rollout
    (MGM/nanokv_codec.py:258-279): the file named by MG35_KVCODEC_PREPACKED_OPERATOR_PATH is read
    once and each entry expanded to its bf16 form on `device`.  Same errors as there for a missing
    variable or a file of another format; the provenance checks stay with the caller."""
    path = os.environ.get("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", "").strip()
    if not path:
        raise RuntimeError("formal worldplay_method requires MG35_KVCODEC_PREPACKED_OPERATOR_PATH")
    payload = torch.load(path, map_location="cpu", weights_only=True)
    if payload.get("format") != "mg35_worldplay_operator_int8_v1":
        raise RuntimeError(f"bad prepacked WorldPlay operator: {path}")
    device = torch.device(device)
    for name in sorted(payload["entries"]):
        kind, layer = name.split(":", 1)
        entry = payload["entries"][name]
        _OPERATORS[(kind, int(layer), str(device))] = Operator.from_int8(
            entry["mean"].float(), entry["encoder"], entry["decoder"], device=device)


def _clusters() -> int:
    return int(os.environ.get("MG35_KVCODEC_C64_CLUSTERS", "64"))


def _iterations() -> int:
    return int(os.environ.get("MG35_KVCODEC_C64_ITERS", "2"))


@torch.no_grad()
def encode_tensor(kind: str, layer: int, value: torch.Tensor) -> dict:
    """value [1,S,J] on the GPU -> the reference's payload dictionary."""
    if kind not in {"k", "v"}:
        raise ValueError(kind)
    if value.dim() != 3 or value.shape[0] != 1:
        raise ValueError(f"expected [1,S,J], got {tuple(value.shape)}")
    _, sequence, dim = value.shape
    clusters = _clusters()
    if clusters <= 0 or clusters > sequence or clusters > 256:
        raise ValueError(f"C64 clusters must be in [1,min(S,256)], got {clusters}")
    op = _operator(kind, layer, value.device)
    rows = value[0].contiguous()
    init = kmeans_init_rows(sequence, clusters, 20260804 + int(layer)).to(value.device)
    centers, ids = ops.kmeans(rows, clusters, _iterations(), init)
    packed, scale = ops.project_quant(rows, centers, ids, op.mean, op.encoder, eps=F32_EPS,
                                      in_coeff_dtype=op.dtype == torch.bfloat16)
    return {
        "codec": CODEC, "kind": kind, "layer": int(layer),
        "shape": tuple(int(v) for v in value.shape),
        "latent_shape": (sequence, op.rank), "latent_numel": sequence * op.rank,
        "packed_codes": packed.reshape(-1), "scale": scale,
        "centers": centers[None], "ids": ids[None], "semantic": True,
        "source_dtype": str(value.dtype).replace("torch.", ""),
    }


def is_payload(value: Any) -> bool:
    return isinstance(value, dict) and value.get("codec") in {RAW, CODEC, SEGMENTS}


def _parts(value: dict) -> list[dict]:
    return list(value["segments"]) if value.get("codec") == SEGMENTS else [value]


def concat_values(left: Any, right: Any) -> Any:
    if left is None:
        return right
    if right is None:
        return left
    if not is_payload(left) or not is_payload(right):
        raise RuntimeError("WorldPlay packed-cache concat received a raw/payload mixture")
    return {"codec": SEGMENTS, "segments": _parts(left) + _parts(right)}


def value_shape(value: Any):
    if value is None:
        return None
    if torch.is_tensor(value):
        return tuple(int(v) for v in value.shape)
    if value.get("codec") == RAW:
        return tuple(int(v) for v in value["tensor"].shape)
    if value.get("codec") == CODEC:
        return tuple(int(v) for v in value["shape"])
    if value.get("codec") == SEGMENTS:
        shapes = [value_shape(item) for item in value["segments"]]
        if not shapes:
            return None
        return (shapes[0][0], sum(shape[1] for shape in shapes), shapes[0][2])
    raise RuntimeError(f"unsupported cache value {value.get('codec')}")


def encode_raw_tensor(tensor: torch.Tensor) -> dict:
    """Uncompressed payload segment (the reference keeps protected frames this way)."""
    return {"codec": RAW, "tensor": tensor.contiguous(), "shape": tuple(int(v) for v in tensor.shape)}


def select_value(value: Any, token_idx: torch.Tensor, *, kind: str, layer: int, dtype: torch.dtype,
                 device) -> Any:
    """Keep the tokens listed in ``token_idx`` (sorted positions along the sequence).

    Same contract as the reference's select_value (MGM/nanokv_codec.py:612-694): a segment that
    is selected whole is reused as it is (immutable payload, no copy); a segment the selection
    cuts is decoded, its selected rows are gathered and encoded again as a new segment; a
    selection that takes nothing returns None.  Decode and re-encode run on the GPU kernels.
    """
    if torch.is_tensor(value):
        return value.index_select(1, token_idx).contiguous()
    parts = _parts(value)
    lengths = [int(value_shape(part)[1]) for part in parts]
    bounds = torch.tensor([0] + lengths).cumsum(0)
    wanted = token_idx.detach().to(device="cpu", dtype=torch.long)
    if wanted.numel() and (bool((wanted[1:] < wanted[:-1]).any()) or int(wanted[0]) < 0
                           or int(wanted[-1]) >= int(bounds[-1])):
        raise RuntimeError("segmented cache selection expects sorted in-range token indices")
    owner = torch.bucketize(wanted, bounds[1:], right=True)      # segment of every wanted token
    result = []
    for index, part in enumerate(parts):
        local = wanted[owner == index] - int(bounds[index])
        if local.numel() == 0:
            continue
        if local.numel() == lengths[index] and bool((local == torch.arange(lengths[index])).all()):
            result.append(part)                                   # whole segment: reuse
            continue
        rows = decode_value(part, dtype=dtype, device=device)
        chosen = rows.index_select(1, local.to(rows.device)).contiguous()
        result.append(encode_raw_tensor(chosen) if part.get("codec") == RAW
                      else encode_tensor(kind, layer, chosen))
    if not result:
        return None
    return result[0] if len(result) == 1 else {"codec": SEGMENTS, "segments": result}


def payload_bytes(value: Any) -> int:
    if torch.is_tensor(value):
        return value.numel() * value.element_size()
    if isinstance(value, dict):
        return sum(payload_bytes(v) for k, v in value.items() if not str(k).startswith("_"))
    if isinstance(value, (list, tuple)):
        return sum(payload_bytes(v) for v in value)
    return 0


def history_from_payloads(parts: list[dict], *, device) -> CompressedHistory:
    """Stack same-layer payload segments into one struct-of-arrays history."""
    first = parts[0]
    kind, layer = str(first["kind"]), int(first["layer"])
    batch, _, dim = (int(v) for v in first["shape"])
    rank = int(first["latent_shape"][-1])
    for part in parts:
        if (part.get("codec") != CODEC or str(part["kind"]) != kind or int(part["layer"]) != layer
                or int(part["shape"][0]) != batch or int(part["shape"][2]) != dim):
            raise ValueError("incompatible WorldPlay method segments")
    if batch != 1:
        raise ValueError("only batch 1 payloads are supported")
    total = sum(int(part["shape"][1]) for part in parts)
    clusters = max(int(part["centers"].shape[1]) for part in parts)
    hist = CompressedHistory(joint=dim, rank=rank, capacity=total, max_segments=len(parts),
                             centers_per_segment=clusters, device=device)
    for part in parts:
        count = int(part["shape"][1])
        offset, rows = hist.reserve_segment(count, int(part["centers"].shape[1]))
        rows.copy_(part["centers"][0].to(device=device, dtype=torch.bfloat16))
        hist.codes[offset:offset + count].copy_(part["packed_codes"].to(device).reshape(count, -1))
        hist.scales[offset:offset + count].copy_(part["scale"].to(device).reshape(count, -1))
        hist.ids[offset:offset + count].copy_(part["ids"].to(device).reshape(-1))
    return hist


@torch.no_grad()
def decode_tensor(payload: dict, *, dtype: torch.dtype, device) -> torch.Tensor:
    if payload.get("codec") == RAW:
        return payload["tensor"].to(device=device, dtype=dtype)
    if payload.get("codec") != CODEC:
        raise RuntimeError(f"unsupported WorldPlay payload {payload.get('codec')}")
    return _decode_parts([payload], dtype=dtype, device=device)


def _decode_parts(parts: list[dict], *, dtype, device) -> torch.Tensor:
    hist = history_from_payloads(parts, device=device)
    op = _operator(str(parts[0]["kind"]), int(parts[0]["layer"]), device)
    rows = ops.decode_rows(hist.view(), op.decoder, op.mean, dtype=dtype)
    return rows.reshape(1, hist.tokens, hist.joint)


@torch.no_grad()
def decode_value(value: Any, *, dtype: torch.dtype, device):
    if value is None:
        return None
    if torch.is_tensor(value):
        return value.to(device=device, dtype=dtype)
    if value.get("codec") == SEGMENTS:
        parts = value["segments"]
        if not parts:
            return None
        if all(part.get("codec") == CODEC for part in parts):
            return _decode_parts(parts, dtype=dtype, device=device)
        return torch.cat([decode_value(p, dtype=dtype, device=device) for p in parts], dim=1)
    return decode_tensor(value, dtype=dtype, device=device)


def decode_pair_values(key: Any, value: Any, *, dtype: torch.dtype, device):
    return (decode_value(key, dtype=dtype, device=device),
            decode_value(value, dtype=dtype, device=device))


@torch.no_grad()
def direct_latent_pair_segments(key: Any, value: Any, *, device, token_keep: torch.Tensor | None = None):
    """Paired K / V payload segments exposed for the low-width readers without reconstructing joint
    K / V (MGF/nanokv_codec.py:708-797): one dictionary per segment with "k" / "v" (``PackedRows``:
    the packed rows as stored, never dequantised to a latent tensor), "length" and
    "logical_indices".  ``token_keep`` (bool over the whole history) keeps a subset; a segment it
    empties is left out.  The stacked form of a payload is derived state cached on the payload."""
    key_parts, value_parts = _parts(key), _parts(value)
    if len(key_parts) != len(value_parts):
        raise ValueError("paired codec segment count mismatch")
    wanted = None
    if token_keep is not None:
        wanted = token_keep.to(device="cpu", dtype=torch.bool).reshape(-1)
        if wanted.numel() != sum(int(value_shape(part)[1]) for part in key_parts):
            raise ValueError("direct latent token mask/cache length mismatch")
    result, offset = [], 0
    for k_part, v_part in zip(key_parts, value_parts):
        if (k_part.get("codec") != CODEC or v_part.get("codec") != CODEC or k_part.get("kind") != "k"
                or v_part.get("kind") != "v" or tuple(k_part["shape"]) != tuple(v_part["shape"])
                or int(k_part["layer"]) != int(v_part["layer"])):
            raise RuntimeError("codec-native attention requires paired formal method payloads")
        length = int(k_part["shape"][1])
        local = None if wanted is None else wanted[offset:offset + length]
        offset += length
        if local is not None and not bool(local.any()):
            continue
        index = None if local is None else torch.nonzero(local).flatten().to(device)
        rows = {}
        for name, part in (("k", k_part), ("v", v_part)):
            cached = part.get("_nkv_history")
            if cached is None or cached.device.type != torch.device(device).type:
                cached = part["_nkv_history"] = history_from_payloads([part], device=device)
            rows[name] = PackedRows(cached, _operator(name, int(part["layer"]), device).mean, index)
        logical = torch.arange(offset - length, offset, device=device)
        if index is not None:
            logical = logical.index_select(0, index)
        result.append({"k": rows["k"], "v": rows["v"], "length": int(logical.numel()),
                       "logical_indices": logical})
    return result


@torch.no_grad()
def decode_pair_selected(key: Any, value: Any, token_keep: torch.Tensor, *, dtype: torch.dtype, device):
    """Decode only the rows ``token_keep`` (bool over the whole history) marks -- protected recent /
    sink / anchor tokens -- to native width: (K [1,n,J], V [1,n,J]) (MGF/nanokv_codec.py:801-861).
    One decode launch per target over the stacked segments, rows chosen by index."""
    key_parts, value_parts = _parts(key), _parts(value)
    keep = token_keep.to(device="cpu", dtype=torch.bool).reshape(-1)
    if keep.numel() != sum(int(value_shape(part)[1]) for part in key_parts):
        raise ValueError("selected decode mask/cache length mismatch")
    index = torch.nonzero(keep).flatten()
    if index.numel() == 0:
        shape = value_shape(key)
        empty = torch.empty((shape[0], 0, shape[2]), device=device, dtype=dtype)
        return empty, empty.clone()
    rows = index.to(device=device, dtype=torch.int32)
    out = []
    for kind, parts in (("k", key_parts), ("v", value_parts)):
        hist = history_from_payloads(parts, device=device)
        op = _operator(kind, int(parts[0]["layer"]), device)
        out.append(ops.decode_rows(hist.view(), op.decoder, op.mean, rows=rows, dtype=dtype)[None])
    return out[0], out[1]
