"""HY-WorldPlay codec interface on the B200 kernels.

Same function names, argument meaning, payload dictionaries and error classes as the reference
module HY/kv_codecs.py for its deployed form -- HY_KV_CODEC_MODE=global_pca with INT4 coefficients
(HY_KV_CODEC_COEFF_QUANT=int4) and the online joint-head C-means (HY_KV_CODEC_SEMANTIC_SMOOTH_K / _V):
compress_kv_tensor :1224-1253 -> global_pca_compress_v :1000-1146, decompress_kv_tensor :1256-1437,
apply_codec_to_layer_cache :1638-1732, quantize_kv_tensor :237-255, pack_quantized_codes :266-314,
unpack_quantized_codes :317-344.  Tensors are [B, H, S, D] with H * D = 2048 as there; B = 1.

What differs from the Matrix-Game form of the same algorithm, and is kept: the C-means residual is
rounded to the input dtype before the mean is taken off and the encoder applied (:190-208, :1078-1081),
the coefficients are quantised in fp32 whatever dtype the encoder produced them in (:237-255), the
scale may be stored as bf16 or fp16 (HY_KV_CODEC_SCALE_DTYPE), and payloads and results keep the
[B, H, S, D] layout; asked for fp32 rows from bf16 operators, the centre is added in fp32 as there
(:1391-1404).  Operators come from `register_operator` (the reference reads them from
artefact files through _global_device_operator_weights :834-912).  The other modes of that module
(uniform INT2/3/8, per-head PCA, block sketches, residual MLP) are research baselines and raise
NotImplementedError here.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Tuple

import torch

from . import ops
from .cache import CompressedHistory
from .codec import F32_EPS, Operator, kmeans_init_rows

JOINT = 2048
_OPERATORS: dict[tuple[str, int, str], Operator] = {}


def _env_flag(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).strip().lower() in {"1", "true", "yes", "on"}


def enabled() -> bool:
    return _env_flag("HY_KV_CODEC_ENABLE", "0") and mode() != "none"


def mode() -> str:
    value = os.environ.get("HY_KV_CODEC_MODE", "none").strip().lower()
    if value not in {"none", "int8", "int4", "int3", "int2", "pca", "global_pca"}:
        raise ValueError(f"unsupported HY_KV_CODEC_MODE={value}")
    return value


def _target_enabled(tensor_name: str) -> bool:
    target = os.environ.get("HY_KV_CODEC_TARGET", "both").strip().lower()
    if target not in {"k", "v", "both"}:
        raise ValueError(f"unsupported HY_KV_CODEC_TARGET={target}")
    return target == "both" or target == tensor_name


def _semantic_smooth_enabled(layer_idx: int, tensor_name: str) -> bool:
    if tensor_name not in {"k", "v"}:
        return False
    if not _env_flag(f"HY_KV_CODEC_SEMANTIC_SMOOTH_{tensor_name.upper()}", "0"):
        return False
    value = os.environ.get("HY_KV_CODEC_SEMANTIC_SMOOTH_LAYERS", "").strip()
    if not value or value.lower() == "all":
        return True
    return int(layer_idx) in {int(item.strip()) for item in value.split(",") if item.strip()}


def _scale_storage_dtype() -> torch.dtype:
    value = os.environ.get("HY_KV_CODEC_SCALE_DTYPE", "bf16").strip().lower()
    if value in {"bf16", "bfloat16"}:
        return torch.bfloat16
    if value in {"fp16", "float16"}:
        return torch.float16
    if value in {"fp32", "float32"}:
        raise NotImplementedError("fp32 scale storage is not built; use bf16 or fp16")
    raise ValueError(f"unsupported HY_KV_CODEC_SCALE_DTYPE={value}")


def register_operator(tensor_name: str, layer_idx: int, *, mean, encoder, decoder, device="cuda") -> Operator:
    """Make (mean [2048], encoder [r, 2048], decoder [2048, r]) resident for (tensor, layer).  bf16
    weights are the reference's bf16_fused / int8 operator modes (INT8 storage is expanded to bf16
    per call there), fp32 weights its fp32_fused mode (:627-701)."""
    if tensor_name not in {"k", "v"}:
        raise ValueError(tensor_name)
    op = Operator(mean, encoder, decoder, device=device)
    if op.joint != JOINT:
        raise ValueError(f"global PCA expects H*D={JOINT}, got {op.joint}")
    _OPERATORS[(tensor_name, int(layer_idx), str(torch.device(device)))] = op
    return op


def _operator(tensor_name: str, layer_idx: int, device) -> Operator:
    device = torch.device(device)
    for key in ((tensor_name, int(layer_idx), str(device)), (tensor_name, int(layer_idx), device.type)):
        if key in _OPERATORS:
            return _OPERATORS[key]
    if device.type == "cuda":
        for (name, layer, where), op in _OPERATORS.items():
            if name == tensor_name and layer == int(layer_idx) and torch.device(where).type == "cuda" and (
                    torch.device(where).index in (None, device.index)):
                return op
    raise KeyError(f"no HY codec operator registered for {tensor_name}:{int(layer_idx):02d}")


# ------------------------------------------------------------------ quantiser and nibble packing
@torch.no_grad()
def quantize_kv_tensor(x: torch.Tensor, num_bits: int, granularity: str):
    """Symmetric INT4 per token: (codes int8, scale fp32 [..., 1]) (:237-255)."""
    if num_bits not in {2, 3, 4, 8}:
        raise ValueError(f"supported KV quantization bits are 2,3,4,8; got {num_bits}")
    granularity = granularity.replace("-", "_")
    if granularity not in {"per_token", "per_channel", "per_tensor"}:
        raise ValueError(f"unsupported quantization granularity={granularity}")
    if num_bits != 4 or granularity != "per_token":
        raise NotImplementedError("only INT4 per-token quantisation is built")
    rows = x.reshape(-1, x.shape[-1]).contiguous()
    if rows.dtype not in (torch.float32, torch.bfloat16):
        rows = rows.float()
    packed, _ = ops.quant_pack(rows, eps=F32_EPS, in_coeff_dtype=False)
    codes = unpack_quantized_codes(packed, 4, rows.numel(), tuple(x.shape))
    # the fp32 scale the codes were formed with (the kernel stores it rounded to 16 bits)
    amax = rows.float().abs().amax(dim=-1, keepdim=True).clamp_min(F32_EPS)
    scale = amax / torch.full_like(amax, 7.0)   # an IEEE division (a scalar divisor becomes a reciprocal on the GPU)
    return codes, scale.reshape(*x.shape[:-1], 1)


def pack_quantized_codes(codes: torch.Tensor, num_bits: int) -> torch.Tensor:
    """Signed INT4 codes -> bytes, two per byte, the even index in the low nibble (:266-314)."""
    if num_bits != 4:
        raise NotImplementedError("only INT4 packing is built")
    flat = codes.reshape(-1).to(torch.int16) + 7
    if torch.any(flat < 0) or torch.any(flat >= 16):
        raise ValueError("codes are outside the representable INT4 range")
    if flat.numel() % 2:
        flat = torch.cat([flat, flat.new_zeros(1)])
    pairs = flat.reshape(-1, 2).to(torch.uint8)
    return (pairs[:, 0] | (pairs[:, 1] << 4)).contiguous()


def unpack_quantized_codes(packed: torch.Tensor, num_bits: int, numel: int, shape=None) -> torch.Tensor:
    """Bytes -> signed int8 codes (:317-344)."""
    if num_bits != 4:
        raise NotImplementedError("only INT4 unpacking is built")
    packed = packed.reshape(-1).to(torch.uint8)
    unsigned = torch.stack([packed & 15, packed >> 4], dim=1).reshape(-1)
    codes = unsigned[: int(numel)].to(torch.int16).sub_(7).to(torch.int8)
    return codes.reshape(shape).contiguous() if shape is not None else codes


def _payload_tensor_bytes(value: Any) -> int:
    if isinstance(value, torch.Tensor):
        return value.numel() * value.element_size()
    if isinstance(value, dict):
        return sum(_payload_tensor_bytes(item) for item in value.values())
    if isinstance(value, (list, tuple)):
        return sum(_payload_tensor_bytes(item) for item in value)
    return 0


# ------------------------------------------------------------------------------------- encoder
@torch.no_grad()
def global_pca_compress_v(x: torch.Tensor, layer_idx: int, tensor_name: str = "v") -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """x [1, H, S, D] on the GPU -> (payload, statistics) of the reference (:1000-1146)."""
    if x.ndim != 4:
        raise ValueError(f"global PCA expects [B,H,S,D], got {tuple(x.shape)}")
    batch, heads, sequence, dim = x.shape
    if heads * dim != JOINT:
        raise ValueError(f"global PCA expects H*D={JOINT}, got {heads}*{dim}")
    if batch != 1:
        raise ValueError("only batch 1 tensors are supported")
    if not _semantic_smooth_enabled(layer_idx, tensor_name):
        raise NotImplementedError("the form without joint-head C-means is not built "
                                  f"(set HY_KV_CODEC_SEMANTIC_SMOOTH_{tensor_name.upper()}=1)")
    coeff_quant = os.environ.get(f"HY_KV_CODEC_COEFF_QUANT_{tensor_name.upper()}",
                                 os.environ.get("HY_KV_CODEC_COEFF_QUANT", "none")).strip().lower()
    if coeff_quant not in {"none", "int8", "int4"}:
        raise ValueError(f"global PCA supports coefficient quantization none|int8|int4, got {coeff_quant}")
    if coeff_quant != "int4":
        raise NotImplementedError("only INT4 coefficients are built")
    op = _operator(tensor_name, layer_idx, x.device)
    rank = int(os.environ.get("HY_KV_CODEC_GLOBAL_PCA_RANK", str(op.rank)))
    if rank != op.rank:
        raise ValueError(f"global PCA rank must be the registered operator's {op.rank}, got {rank}")
    clusters = int(os.environ.get("HY_KV_CODEC_SEMANTIC_CLUSTERS", "64"))
    iters = int(os.environ.get("HY_KV_CODEC_SEMANTIC_ITERS", "2"))
    if clusters <= 0 or clusters > sequence or clusters > 256:
        raise ValueError(f"semantic clusters must be in [1,min(S,256)], got {clusters}")
    scale_dtype = _scale_storage_dtype()
    rows = x.permute(0, 2, 1, 3).reshape(sequence, JOINT).contiguous()
    init = kmeans_init_rows(sequence, clusters, 20260804 + int(layer_idx)).to(x.device)
    centers, ids = ops.kmeans(rows, clusters, iters, init)
    # the residual against the STORED (bf16) centres, rounded to the input dtype as the reference
    # hands it on (:190-208); the projection then takes the mean off in fp32
    residual = (rows.float() - centers.float().index_select(0, ids.long())).to(x.dtype)
    zero_center = torch.zeros(1, JOINT, dtype=torch.bfloat16, device=x.device)
    zero_ids = torch.zeros(sequence, dtype=torch.uint8, device=x.device)
    packed, scale = ops.project_quant(residual, zero_center, zero_ids, op.mean, op.encoder, eps=F32_EPS,
                                      in_coeff_dtype=False, scale_dtype=scale_dtype)
    payload = {
        "kv_codec": True, "codec": "global_pca", "coeff_quant": coeff_quant, "rank": rank,
        "shape": tuple(int(v) for v in x.shape), "layer_idx": int(layer_idx), "tensor_name": tensor_name,
        "basis_root": os.environ.get(f"HY_KV_CODEC_SEMANTIC_BASIS_DIR_{tensor_name.upper()}", "").strip(),
        "source_dtype": str(x.dtype).replace("torch.", ""), "semantic_smooth": True,
        "semantic_centers": centers[None], "semantic_ids": ids[None], "semantic_clusters": clusters,
        "semantic_linear_root": os.environ.get(
            f"HY_KV_CODEC_SEMANTIC_LINEAR_DIR_{tensor_name.upper()}", "").strip(),
        "latent_int8": packed.reshape(-1), "latent_scale": scale.reshape(batch, sequence, 1),
        "latent_shape": (batch, sequence, rank), "latent_numel": batch * sequence * rank,
    }
    actual = _payload_tensor_bytes(payload)
    return payload, {"rank": rank, "coeff_quant": coeff_quant, "estimated_bytes": actual, "actual_bytes": actual,
                     "basis_file": ""}


def compress_kv_tensor(x: torch.Tensor, layer_idx: int, tensor_name: str) -> Tuple[Any, Dict[str, Any]]:
    codec_mode = mode()
    if codec_mode == "global_pca":
        return global_pca_compress_v(x, layer_idx, tensor_name)
    if codec_mode == "none":
        return x, {"estimated_bytes": x.numel() * x.element_size()}
    raise NotImplementedError(f"HY_KV_CODEC_MODE={codec_mode} is a baseline of the reference and is not built")


# ------------------------------------------------------------------------------------- decoder
def history_from_payload(payload: dict, *, device) -> CompressedHistory:
    """One payload as a one-segment struct-of-arrays history (what the fused reads take)."""
    batch, heads, sequence, dim = (int(v) for v in payload["shape"])
    rank = int(payload["rank"])
    if batch != 1:
        raise ValueError("only batch 1 payloads are supported")
    centers = payload["semantic_centers"]
    scale = payload["latent_scale"]
    hist = CompressedHistory(joint=heads * dim, rank=rank, capacity=sequence, max_segments=1,
                             centers_per_segment=int(centers.shape[1]), device=device,
                             scale_dtype=scale.dtype)
    offset, rows = hist.reserve_segment(sequence, int(centers.shape[1]))
    rows.copy_(centers[0].to(device=device, dtype=torch.bfloat16))
    hist.codes[offset:offset + sequence].copy_(payload["latent_int8"].to(device).reshape(sequence, -1))
    hist.scales[offset:offset + sequence].copy_(scale.to(device).reshape(sequence, -1))
    hist.ids[offset:offset + sequence].copy_(payload["semantic_ids"].to(device).reshape(-1))
    return hist


@torch.no_grad()
def decompress_kv_tensor(obj_or_tensor: Any, dtype: torch.dtype = torch.float32, device=None) -> Any:
    """Payload -> [B, H, S, D] in `dtype`; tensors pass through (:1256-1437)."""
    if not (isinstance(obj_or_tensor, dict) and obj_or_tensor.get("kv_codec")):
        return obj_or_tensor
    payload = obj_or_tensor
    if payload.get("codec") != "global_pca":
        raise ValueError(f"unsupported resident KV codec={payload.get('codec')}")
    if payload.get("coeff_quant", "none") != "int4" or not payload.get("semantic_smooth"):
        raise NotImplementedError("only INT4 coefficients with joint-head C-means are built")
    if payload.get("kv_sketch") is not None:
        raise NotImplementedError("block sketches are not built")
    batch, heads, sequence, dim = (int(v) for v in payload["shape"])
    if int(payload["latent_shape"][-1]) != int(payload["rank"]):
        raise ValueError("global PCA payload rank mismatch")
    device = payload["latent_int8"].device if device is None else torch.device(device)
    op = _operator(str(payload.get("tensor_name", "v")), int(payload["layer_idx"]), device)
    hist = history_from_payload(payload, device=device)
    if dtype == torch.float32 and op.dtype == torch.bfloat16:
        # the reference adds the centre to the bf16 decoder output in fp32 and returns that sum
        # (:1391-1404); the decode kernel's centre add rounds to bf16, so the centres are taken out of
        # the kernel's sight (a zero table) and added here
        table = hist.centers.clone()
        hist.centers.zero_()
        rows = ops.decode_rows(hist.view(), op.decoder, op.mean, dtype=torch.bfloat16).float()
        rows += table.float().index_select(0, hist.ids[:sequence].long())
    else:
        rows = ops.decode_rows(hist.view(), op.decoder, op.mean, dtype=dtype)
    return rows.reshape(batch, sequence, heads, dim).permute(0, 2, 1, 3).contiguous()


def apply_codec_to_layer_cache(layer_cache: Dict[str, Any], layer_idx: int) -> Dict[str, Any]:
    """Replace the layer cache's `k_vision` / `v_vision` tensors by payloads (:1638-1732).  A tensor
    the codec cannot take stays as it is unless HY_KV_CODEC_STRICT is set."""
    if not enabled():
        return layer_cache
    strict = _env_flag("HY_KV_CODEC_STRICT", "0")
    for cache_name, short_name in (("k_vision", "k"), ("v_vision", "v")):
        tensor = layer_cache.get(cache_name)
        if not isinstance(tensor, torch.Tensor) or not _target_enabled(short_name):
            continue
        try:
            layer_cache[cache_name], _ = compress_kv_tensor(tensor, layer_idx, short_name)
        except Exception:
            if strict:
                raise
    return layer_cache
