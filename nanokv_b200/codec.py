"""Codec encoder / decoder over the compressed history cache.

Host-side orchestration only: every arithmetic step is a kernel of
libnanokv_b200 (see ops.py).  The quantiser flavours are the reference's:
Matrix-Game computes scale and codes in the coefficient dtype
(MGM/nanokv_codec.py:349-351), LingBot and HY upcast to fp32 first
(LB/lingbot_v2_kv_codec.py:285-287, HY/kv_codecs.py:237-255).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, ops
from .cache import CompressedHistory

F32_EPS = 1.1920928955078125e-07


@dataclass(frozen=True)
class QuantSpec:
    group: int | None = None            # None: one scale per token (the reference)
    eps: float = F32_EPS
    in_coeff_dtype: bool = False
    scale_dtype: torch.dtype = torch.bfloat16


MG_QUANT = QuantSpec(eps=F32_EPS, in_coeff_dtype=True)
LINGBOT_QUANT = QuantSpec(eps=1e-12, in_coeff_dtype=False)
GROUP32_FP16 = QuantSpec(group=32, eps=F32_EPS, in_coeff_dtype=False, scale_dtype=torch.float16)


class Operator:
    """Encoder / decoder / mean of one (kind, layer), resident on the device."""

    def __init__(self, mean: torch.Tensor, encoder: torch.Tensor, decoder: torch.Tensor,
                 device="cuda"):
        if encoder.dtype != decoder.dtype or encoder.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("operator weights must both be fp32 or both bf16")
        rank, joint = encoder.shape
        if tuple(decoder.shape) != (joint, rank) or tuple(mean.shape) != (joint,):
            raise ValueError("operator shapes do not match [r,J] / [J,r] / [J]")
        self.rank, self.joint, self.dtype = int(rank), int(joint), encoder.dtype
        self.mean = mean.to(device=device, dtype=torch.float32).contiguous()
        self.encoder = encoder.to(device=device).contiguous()
        self.decoder = decoder.to(device=device).contiguous()
        # bias as the decoder GEMM sees it: the bf16 path rounds the mean to bf16 first
        self.bias = (self.mean.to(torch.bfloat16).float() if self.dtype == torch.bfloat16
                     else self.mean).contiguous()
        # decoder rows in the order the tensor-core read expands code words (one-time copy)
        self.decoder_tc = (ops.prepare_decoder(self.decoder)
                           if self.dtype == torch.bfloat16 and self.decoder.is_cuda and self.rank % 8 == 0
                           else None)


    @classmethod
    def from_int8(cls, mean: torch.Tensor, encoder: dict, decoder: dict, device="cuda") -> "Operator":
        """Operator stored as INT8 (``{"qweight", "scale", "group_size"}`` per matrix: the reference's
        deployed format, MGM/nanokv_codec.py:108-131, LB/lingbot_v2_kv_codec.py:98-108).  The weights
        are expanded to bf16 once, here, with the reference's per-call expression; every kernel then
        reads the resident bf16 copy."""
        def unpack(packed):
            q = packed["qweight"].to(device=device).contiguous()
            scale = packed["scale"].to(device=device)
            return ops.unpack_int8_weight(q, scale, packed.get("group_size"))
        return cls(mean, unpack(encoder), unpack(decoder), device=device)


def kmeans_init_rows(sequence: int, clusters: int, seed: int) -> torch.Tensor:
    """Seeded CPU permutation prefix, as the reference draws it
    (MGM/nanokv_codec.py:310-311, LB/lingbot_v2_kv_codec.py:220-221)."""
    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randperm(sequence, generator=generator)[:clusters].to(torch.int32)


def encode_append(hist: CompressedHistory, rows: torch.Tensor, op: Operator,
                  quant: QuantSpec = QuantSpec(), *, centers: torch.Tensor | None = None,
                  clusters: int = 64, iters: int = 2, seed: int = 0) -> int:
    """Encode rows [S,J] as one new segment of ``hist``; returns its token offset.

    centers=None runs the online C-means (the reference's semantic_residual);
    a tensor [C,J] is stored and used as given; "resident" uses the table already
    in a shared-centre history (``hist.centers``) without copying it again.
    """
    if rows.dim() != 2 or rows.shape[1] != hist.joint:
        raise ValueError(f"expected rows [S,{hist.joint}], got {tuple(rows.shape)}")
    if (quant.group or op.rank) != hist.group or quant.scale_dtype != hist.scales.dtype:
        raise ValueError("quantiser spec does not match the history cache")
    rows = rows.contiguous()
    S = rows.shape[0]
    resident = isinstance(centers, str)
    if resident and (centers != "resident" or not hist.shared_centers):
        raise ValueError('centers="resident" needs a history built with shared_centers=True')
    if resident:
        clusters = hist.centers_per_segment
    else:
        clusters = int(centers.shape[0]) if centers is not None else int(clusters)
    if clusters > hist.centers_per_segment:
        raise ValueError("more centres than the cache reserves per segment")
    offset, center_rows = hist.reserve_segment(S, clusters)
    ids = hist.ids[offset:offset + S]
    codes = hist.codes[offset:offset + S]
    scales = hist.scales[offset:offset + S]
    if centers is None:
        init = kmeans_init_rows(S, clusters, seed).to(rows.device)
        ops.kmeans(rows, clusters, iters, init, centers=center_rows, ids=ids)
        ops.project_quant(rows, center_rows, ids, op.mean, op.encoder, group=hist.group, eps=quant.eps,
                          in_coeff_dtype=quant.in_coeff_dtype and op.dtype == torch.bfloat16,
                          codes=codes, scales=scales)
        return offset
    if not resident:
        center_rows.copy_(centers.to(torch.bfloat16))
    workspace = torch.empty(S, op.rank, dtype=op.dtype, device=rows.device)
    lib = _lib.library()
    in_bf16 = quant.in_coeff_dtype and op.dtype == torch.bfloat16
    _lib.check(lib.nkv_encode_append(
        ctypes.c_void_p(rows.data_ptr()), ops.dtype_code(rows.dtype),
        ctypes.c_void_p(center_rows.data_ptr()), clusters, ctypes.c_void_p(op.mean.data_ptr()),
        ctypes.c_void_p(op.encoder.data_ptr()), ops.dtype_code(op.dtype), S, hist.joint, op.rank,
        hist.group, float(quant.eps), _lib.NKV_QUANT_IN_BF16 if in_bf16 else _lib.NKV_QUANT_F32,
        ops.dtype_code(hist.scales.dtype), hist.ids.element_size(), offset,
        ctypes.c_void_p(hist.codes.data_ptr()), ctypes.c_void_p(hist.scales.data_ptr()),
        ctypes.c_void_p(hist.ids.data_ptr()), ctypes.c_void_p(workspace.data_ptr()),
        workspace.numel() * workspace.element_size(),
        ctypes.c_void_p(torch.cuda.current_stream(rows.device).cuda_stream)))
    return offset


def decode(hist: CompressedHistory, op: Operator, *, rows: torch.Tensor | None = None,
           dtype: torch.dtype | None = None) -> torch.Tensor:
    """Reconstruct history rows [n,J] (all, or the listed token indices)."""
    return ops.decode_rows(hist.view(), op.decoder, op.mean, rows=rows, dtype=dtype)
