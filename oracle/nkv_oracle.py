"""CPU restatement of NanoKV's compressed-KV hot path (TEST INFRASTRUCTURE ONLY).

This module is the checker that the CUDA path is compared against.  It is not
part of the product: only the test-suite, the smoke entry and the benchmark's
CPU-baseline leg may import it.  Nothing under ``nanokv_b200/`` imports it.

Every function restates, in plain CPU PyTorch, one function of the reference
implementation and cites the reference file:line it follows.  Paths are given
relative to the reference project root with these shorthands:

  MGM/  = models/Matrix-Game-3.5/fast/diffsynth/models/
  MGC/  = models/Matrix-Game-3.5/fast/codec_native/
  LB/   = models/LingBot-World-2.0/fast/wan/modules/
  HY/   = models/HY-WorldPlay/fast/hyvideo/models/transformers/modules/

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the unmodified
reference modules (MG codec, LingBot codec, MGC core) on seeded inputs and
stores their outputs; ``tests/test_oracle_golden.py`` checks this restatement
against those stored outputs bit for bit (integers) / to float equality.
The three generalisations that the reference has no code for (quantisation
groups smaller than the rank, externally supplied centres, more than 256
centres) are restated from the reference's own formulas and are pinned only
through the cases where they coincide with the reference (group == rank,
centres taken from the reference's k-means, <= 256 centres).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

F32_EPS = float(torch.finfo(torch.float32).eps)

# --------------------------------------------------------------------------- #
# INT4 nibble packing
# --------------------------------------------------------------------------- #


def pack_int4(codes: torch.Tensor) -> tuple[torch.Tensor, int]:
    """codes int8 in [-7, 7] -> bytes; even element in the low nibble.

    MGM/nanokv_codec.py:282-292, LB/lingbot_v2_kv_codec.py:242-247.  The two
    differ only in the pad nibble of an odd-length stream (0 vs 7); ranks here
    are even so no pad nibble is ever produced.
    """
    flat = codes.reshape(-1).to(torch.int16) + 7
    if bool((flat < 0).any()) or bool((flat > 14).any()):
        raise RuntimeError("INT4 codes outside the symmetric range [-7, 7]")
    count = flat.numel()
    if count % 2:
        flat = torch.cat((flat, torch.zeros(1, dtype=flat.dtype)))
    pairs = flat.reshape(-1, 2)
    return (pairs[:, 0] | (pairs[:, 1] << 4)).to(torch.uint8).contiguous(), count


def unpack_int4(packed: torch.Tensor, count: int, shape) -> torch.Tensor:
    """MGM/nanokv_codec.py:295-298, LB/lingbot_v2_kv_codec.py:250-252."""
    packed = packed.reshape(-1).to(torch.uint8)
    nibbles = torch.stack((packed & 0x0F, (packed >> 4) & 0x0F), dim=1).reshape(-1)
    return nibbles[:count].to(torch.int16).sub_(7).to(torch.int8).reshape(shape)


# --------------------------------------------------------------------------- #
# Centre assignment / online C-means
# --------------------------------------------------------------------------- #


def squared_distances(rows: torch.Tensor, centers: torch.Tensor) -> torch.Tensor:
    """rows [B,S,J] f32, centers [B,C,J] f32 -> [B,S,C] f32.

    The expanded form ||x||^2 + ||c||^2 - 2 x.c in fp32, exactly as
    MGM/nanokv_codec.py:313-320 and LB/lingbot_v2_kv_codec.py:224-229.
    """
    row_norm = rows.square().sum(-1, keepdim=True)
    return row_norm + centers.square().sum(-1).unsqueeze(1) - 2.0 * torch.bmm(
        rows, centers.transpose(1, 2)
    )


def assign_labels(rows: torch.Tensor, centers: torch.Tensor) -> torch.Tensor:
    """argmin over centres, first index wins ties (torch.argmin on CPU).

    MGM/nanokv_codec.py:321, LB/lingbot_v2_kv_codec.py:230.
    """
    return squared_distances(rows.float(), centers.float()).argmin(-1)


def kmeans_init_rows(sequence: int, clusters: int, seed: int) -> torch.Tensor:
    """Initial centre rows: first C entries of a seeded CPU permutation.

    MGM/nanokv_codec.py:310-311 (seed 20260804 + layer),
    LB/lingbot_v2_kv_codec.py:220-221 (seed 20260826 + 17*layer + 1009*sp + [v]).
    """
    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randperm(sequence, generator=generator)[:clusters]


def kmeans(rows: torch.Tensor, clusters: int, iters: int, seed: int):
    """Deterministic Lloyd iterations -> (centres f32 [B,C,J], labels long [B,S]).

    Labels come from the LAST assignment step, i.e. against the centres as they
    were before the last update; empty clusters keep their previous centre.
    MGM/nanokv_codec.py:312-325, LB/lingbot_v2_kv_codec.py:222-234.
    """
    batch, sequence, _ = rows.shape
    rows = rows.float()
    if not 0 < clusters <= sequence:
        raise ValueError(f"clusters must be in [1, S]; got {clusters} for S={sequence}")
    centers = rows.index_select(1, kmeans_init_rows(sequence, clusters, seed)).clone()
    labels = torch.zeros((batch, sequence), dtype=torch.long)
    for _ in range(int(iters)):
        labels = assign_labels(rows, centers)
        assignment = F.one_hot(labels, num_classes=clusters).transpose(1, 2).float()
        counts = assignment.sum(-1)
        updated = torch.bmm(assignment, rows) / counts.clamp_min(1.0).unsqueeze(-1)
        centers = torch.where((counts > 0).unsqueeze(-1), updated, centers)
    return centers, labels


def id_dtype(clusters: int) -> torch.dtype:
    """uint8 ids as the reference stores them (MGM/nanokv_codec.py:330); the
    >256-centre generalisation widens to int32 holding a 16-bit value."""
    return torch.uint8 if clusters <= 256 else torch.int32


def semantic_residual(rows: torch.Tensor, clusters: int, iters: int, seed: int):
    """residual f32, stored centres bf16, ids.

    The STORED (bf16-rounded) centres are what is subtracted.
    MGM/nanokv_codec.py:326-330, LB/lingbot_v2_kv_codec.py:235-239.
    """
    rows = rows.float()
    centers, labels = kmeans(rows, clusters, iters, seed)
    stored = centers.to(torch.bfloat16)
    assigned = torch.gather(stored.float(), 1, labels[..., None].expand(-1, -1, rows.shape[-1]))
    return rows - assigned, stored, labels.to(id_dtype(clusters))


def residual_given_centers(rows: torch.Tensor, stored_centers: torch.Tensor):
    """Fixed-centre form: nearest stored centre, residual against it.

    Restatement (the reference always derives centres online): the assignment
    formula of MGM/nanokv_codec.py:316-321 evaluated against the given bf16
    centres, residual per MGM/nanokv_codec.py:326-330.
    """
    rows = rows.float()
    table = stored_centers.float()
    labels = assign_labels(rows, table)
    assigned = torch.gather(table, 1, labels[..., None].expand(-1, -1, rows.shape[-1]))
    return rows - assigned, labels.to(id_dtype(stored_centers.shape[1]))


# --------------------------------------------------------------------------- #
# Operator GEMMs
# --------------------------------------------------------------------------- #


def operator_linear(rows: torch.Tensor, weight: torch.Tensor, bias=None) -> torch.Tensor:
    """y = rows @ weight.T + bias in the weight's arithmetic.

    fp32 weight -> fp32 GEMM (MGM/nanokv_codec.py:136-137); bf16 weight -> the
    input and the bias are rounded to bf16, the GEMM accumulates in fp32 and
    the output is rounded once to bf16 (MGM/nanokv_codec.py:138-141,
    LB/lingbot_v2_kv_codec.py:102-106).
    """
    if weight.dtype == torch.float32:
        return F.linear(rows.float(), weight, None if bias is None else bias.float())
    if weight.dtype != torch.bfloat16:
        raise ValueError(f"unsupported operator dtype {weight.dtype}")
    return F.linear(
        rows.to(torch.bfloat16), weight, None if bias is None else bias.to(torch.bfloat16)
    )


# --------------------------------------------------------------------------- #
# INT4 symmetric quantisation
# --------------------------------------------------------------------------- #


def quantize_rows(
    coeff: torch.Tensor,
    *,
    group: int | None = None,
    eps: float = F32_EPS,
    in_coeff_dtype: bool = False,
    scale_dtype: torch.dtype = torch.bfloat16,
):
    """coeff [S, r] -> (codes int8 [S, r], stored scale [S, r/group]).

    ``in_coeff_dtype=True`` is Matrix-Game's form, where amax, the divide by 7
    and coeff/scale all run in the coefficient dtype (bf16 when the operator is
    bf16) -- MGM/nanokv_codec.py:349-351.  ``False`` upcasts to fp32 first:
    LB/lingbot_v2_kv_codec.py:285-287 (eps 1e-12) and HY/kv_codecs.py:237-255
    (eps = fp32 machine epsilon).  Codes always divide by the UNROUNDED scale;
    only the stored copy is rounded to ``scale_dtype``.  torch.round is
    round-half-to-even.  ``group`` < r is the grouped generalisation: the same
    arithmetic applied to each contiguous block of ``group`` coefficients.
    """
    rows, rank = coeff.shape
    group = rank if group is None else int(group)
    if rank % group:
        raise ValueError(f"group {group} must divide rank {rank}")
    work = coeff if in_coeff_dtype else coeff.float()
    work = work.reshape(rows, rank // group, group)
    scale = work.abs().amax(-1, keepdim=True).clamp_min(eps) / 7.0
    codes = (work / scale).round().clamp(-7, 7).to(torch.int8).reshape(rows, rank)
    return codes, scale.reshape(rows, rank // group).to(scale_dtype)


def dequantize_rows(codes, stored_scale, *, out_dtype=torch.bfloat16):
    """latent = code * stored_scale, rounded once to ``out_dtype``.

    bf16: LB/lingbot_v2_kv_codec.py:317-319 and the fused unpack at
    MGM/nanokv_codec_kernels.py:11-27; fp32: MGM/nanokv_codec.py:381.
    """
    rows, rank = codes.shape
    groups = stored_scale.shape[-1]
    product = codes.float().reshape(rows, groups, rank // groups) * stored_scale.float().reshape(
        rows, groups, 1
    )
    return product.reshape(rows, rank).to(out_dtype)


# --------------------------------------------------------------------------- #
# Whole encode / decode of one tensor (K or V) of one chunk
# --------------------------------------------------------------------------- #


def encode_rows(
    rows: torch.Tensor,
    *,
    encoder: torch.Tensor,
    mean: torch.Tensor,
    centers: torch.Tensor | None = None,
    clusters: int = 64,
    iters: int = 2,
    seed: int = 0,
    group: int | None = None,
    eps: float = F32_EPS,
    in_coeff_dtype: bool = False,
    scale_dtype: torch.dtype = torch.bfloat16,
) -> dict:
    """rows [1,S,J] -> compressed segment.

    centers=None -> online C-means (the reference), else the fixed-centre form.
    MGM/nanokv_codec.py:334-365, LB/lingbot_v2_kv_codec.py:256-297.
    """
    if centers is None:
        residual, stored, ids = semantic_residual(rows, clusters, iters, seed)
    else:
        stored = centers.to(torch.bfloat16)
        residual, ids = residual_given_centers(rows, stored)
    flat = residual.reshape(-1, residual.shape[-1]) - mean.float()
    coeff = operator_linear(flat, encoder)
    codes, scale = quantize_rows(
        coeff, group=group, eps=eps, in_coeff_dtype=in_coeff_dtype, scale_dtype=scale_dtype
    )
    packed, count = pack_int4(codes)
    return {
        "shape": tuple(rows.shape), "rank": int(encoder.shape[0]),
        "packed": packed, "count": count, "codes": codes, "coeff": coeff,
        "scale": scale, "centers": stored, "ids": ids,
    }


def decode_rows(segment: dict, *, decoder: torch.Tensor, mean: torch.Tensor,
                dtype: torch.dtype) -> torch.Tensor:
    """segment -> [1,S,J] in ``dtype``.

    bf16 decoder: latent bf16, GEMM with the bf16 mean as bias, bf16 output,
    centre added in bf16 (LB/lingbot_v2_kv_codec.py:313-326; the segment form
    MGM/nanokv_codec.py:438-455 rounds identically).  fp32 decoder: everything
    fp32 (MGM/nanokv_codec.py:376-390).
    """
    batch, sequence, dim = segment["shape"]
    rank = segment["rank"]
    codes = unpack_int4(segment["packed"], segment["count"], (batch * sequence, rank))
    ids = segment["ids"].to(torch.long)
    if decoder.dtype == torch.float32:
        latent = dequantize_rows(codes, segment["scale"], out_dtype=torch.float32)
        rows = operator_linear(latent, decoder, mean).reshape(batch, sequence, dim)
        table = segment["centers"].float()
        rows = rows + torch.gather(table, 1, ids[..., None].expand(-1, -1, dim))
        return rows.to(dtype)
    latent = dequantize_rows(codes, segment["scale"], out_dtype=torch.bfloat16)
    rows = operator_linear(latent, decoder, mean).reshape(batch, sequence, dim)
    table = segment["centers"].to(torch.bfloat16)
    rows += torch.gather(table, 1, ids[..., None].expand(-1, -1, dim))
    return rows.to(dtype)


def hy_compress(x: torch.Tensor, *, encoder: torch.Tensor, mean: torch.Tensor, clusters: int, iters: int,
                layer: int, scale_dtype: torch.dtype = torch.bfloat16) -> dict:
    """HY-WorldPlay's form of the encoder on x [1, H, S, D] (HY/kv_codecs.py:1000-1146 with
    _joint_semantic_smooth :116-208).  The same algorithm as encode_rows with three differences that
    change bits: the C-means residual is rounded to the input dtype before anything else happens to
    it (:207), the coefficients are quantised in fp32 whatever the encoder produced (:237-255), and
    the seed of the start rows is 20260804 + layer (:139).
    """
    batch, heads, sequence, dim = x.shape
    rows = x.permute(0, 2, 1, 3).reshape(batch, sequence, heads * dim)
    residual, stored, ids = semantic_residual(rows, clusters, iters, 20260804 + int(layer))
    residual = residual.to(x.dtype)
    flat = residual.reshape(-1, heads * dim).float() - mean.float()
    coeff = operator_linear(flat, encoder)
    codes, scale = quantize_rows(coeff, eps=F32_EPS, in_coeff_dtype=False, scale_dtype=scale_dtype)
    packed, count = pack_int4(codes)
    return {"shape": (batch, sequence, heads * dim), "rank": int(encoder.shape[0]), "packed": packed,
            "count": count, "codes": codes, "scale": scale, "centers": stored, "ids": ids}


def hy_decompress(segment: dict, *, decoder: torch.Tensor, mean: torch.Tensor, heads: int,
                  dtype: torch.dtype) -> torch.Tensor:
    """segment -> [1, H, S, D] in `dtype` as HY decodes it (HY/kv_codecs.py:1264-1437): latent =
    code * scale in fp32, the decoder GEMM in the operator's arithmetic with the mean as bias, the
    centre added in FP32 (:1391-1404), one cast to `dtype`, layout [B, H, S, D]."""
    batch, sequence, joint = segment["shape"]
    codes = unpack_int4(segment["packed"], segment["count"], (batch * sequence, segment["rank"]))
    latent = codes.float() * segment["scale"].float().reshape(-1, 1)
    rows = operator_linear(latent, decoder, mean)
    table = segment["centers"].float()
    ids = segment["ids"].to(torch.long)
    assigned = torch.gather(table, 1, ids[..., None].expand(-1, -1, joint)).reshape(-1, joint)
    rows = rows + assigned
    return rows.reshape(batch, sequence, heads, joint // heads).permute(0, 2, 1, 3).contiguous().to(dtype)


# --------------------------------------------------------------------------- #
# Attention with log-sum-exp, and the LSE merge
# --------------------------------------------------------------------------- #


def merge(out_a, lse_a, out_b, lse_b):
    """Exact two-partition softmax merge; an empty partition is (0, -inf).

    MGC/core.py:33-42 (same arithmetic as LB/codec_native_attention.py:43-50):
    fp32 logaddexp, weights exp(lse_x - lse) with a zero origin where the
    total is not finite, fp32 blend, one cast to the dtype of ``out_a``.
    """
    lse = torch.logaddexp(lse_a, lse_b)
    origin = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    wa, wb = (lse_a - origin).exp(), (lse_b - origin).exp()
    out = out_a.float() * wa[..., None] + out_b.float() * wb[..., None]
    return out.to(out_a.dtype), lse


def attention_lse(q, k, v, mask=None, *, scale=None, q_tile=128, k_tile=1024):
    """[B,H,Q,D] x [B,H,N,D] -> (O [B,H,Q,Dv] in q.dtype, lse f32 [B,H,Q]).

    The reference's own CPU arithmetic statement (tiled fp32, tiles merged by
    ``merge``): MGC/core.py:45-72.
    """
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if k.shape[-2] == 0:
        return (q.new_zeros(*q.shape[:-1], v.shape[-1]),
                torch.full(q.shape[:-1], -math.inf))
    outs, lses = [], []
    for qi in range(0, q.shape[-2], q_tile):
        qq = q[..., qi:qi + q_tile, :]
        out = qq.new_zeros(*qq.shape[:-1], v.shape[-1])
        lse = torch.full(qq.shape[:-1], -math.inf)
        for ki in range(0, k.shape[-2], k_tile):
            logits = (qq.float() @ k[..., ki:ki + k_tile, :].float().transpose(-1, -2)) * scale
            if mask is not None:
                m = mask if mask.shape[-2] == 1 else mask[..., qi:qi + q_tile, :]
                logits = logits.masked_fill(~m[..., ki:ki + k_tile], -math.inf)
            ll = torch.logsumexp(logits, -1)
            origin = torch.where(torch.isfinite(ll), ll, torch.zeros_like(ll))
            probabilities = (logits - origin[..., None]).exp()
            oo = (probabilities @ v[..., ki:ki + k_tile, :].float()).to(q.dtype)
            out, lse = merge(out, lse, oo, ll)
        outs.append(out)
        lses.append(lse)
    return torch.cat(outs, -2), torch.cat(lses, -1)


def merge_many(partials):
    """Left fold of ``merge`` over [(O, lse), ...]: the context-parallel merge.

    The reference has no history-sharded mode; its two-way merge
    (MGC/core.py:33-42) folded over the shards is the arithmetic statement.
    """
    out, lse = partials[0]
    for other_out, other_lse in partials[1:]:
        out, lse = merge(out, lse, other_out, other_lse)
    return out, lse


def codec_attention(q, k_segments, v_segments, *, k_decoder, k_mean, v_decoder, v_mean,
                    heads: int, dtype: torch.dtype, scale=None, rope=None):
    """Full-dimensional read: decode every segment, concatenate, (rotate the keys,) attend.

    ``rope`` = dict(positions, freqs, frame_seqlen, width): the decoded keys are rotated by
    ``rope_by_positions`` before the attention, as LB/codec_native_attention.py:713-716 does.

    q [B,Q,H,D]; segments as produced by ``encode_rows``.  Read path
    MGM/nanokv_codec.py:393-455 (decode) + MGC/core.py:45-72 (attention).
    Returns (O [B,Q,H,D], lse [B,H,Q]).
    """
    batch, _, _, head_dim = q.shape
    keys = [decode_rows(s, decoder=k_decoder, mean=k_mean, dtype=dtype) for s in k_segments]
    values = [decode_rows(s, decoder=v_decoder, mean=v_mean, dtype=dtype) for s in v_segments]
    if keys:
        key = torch.cat(keys, 1).reshape(batch, -1, heads, head_dim)
        if rope is not None and rope.get("indices") is not None:
            key = rope_selected(key.permute(0, 2, 1, 3), rope["positions"], rope["freqs"],
                                frame_seqlen=rope["frame_seqlen"], width=rope["width"],
                                indices=rope["indices"]).permute(0, 2, 1, 3)
        elif rope is not None:
            key = rope_by_positions(key, rope["positions"], rope["freqs"],
                                    frame_seqlen=rope["frame_seqlen"], width=rope["width"])
        key = key.permute(0, 2, 1, 3)
        value = torch.cat(values, 1).reshape(batch, -1, heads, head_dim).permute(0, 2, 1, 3)
    else:
        key = q.new_zeros(batch, heads, 0, head_dim)
        value = q.new_zeros(batch, heads, 0, head_dim)
    out, lse = attention_lse(q.permute(0, 2, 1, 3).to(dtype), key, value, scale=scale)
    return out.permute(0, 2, 1, 3).contiguous(), lse


# --------------------------------------------------------------------------- #
# NanoKV-Fast: reader projections and the hybrid attention
# --------------------------------------------------------------------------- #


def reader_read(group: dict, latent, centers, ids, mean, *, target: str, dtype,
                native_dim: int):
    """Low-width K or V for one reader group: [B,h,n,d].

    out = latent @ read^T + (mean_h @ affine) inside the GEMM, then the
    projected centre table gathered by id is added.  MGC/core.py:168-200.
    """
    weight = group[target + "_read"].to(dtype)
    affine = group[target + "_affine"].to(dtype)
    heads = group["heads"].long()
    mean_heads = mean.reshape(-1, native_dim).index_select(0, heads).to(dtype)
    bias = torch.einsum("hd,hde->he", mean_heads, affine)
    output = F.linear(latent.to(dtype), weight.flatten(0, 1), bias.flatten())
    output = output.reshape(latent.shape[0], latent.shape[1], len(heads), weight.shape[1])
    output = output.permute(0, 2, 1, 3)
    if centers is None:
        return output
    table = centers.reshape(centers.shape[0], centers.shape[1], -1, native_dim)
    table = table.index_select(2, heads)
    projected = torch.einsum("bchd,hde->bhce", table.to(dtype), affine)
    assigned = projected.gather(
        2, ids[:, None, :, None].expand(-1, len(heads), -1, projected.shape[-1]))
    return output + assigned


def compressed_value_mean(low_segments, *, decoder: torch.Tensor, heads: int, native_dim: int):
    """Mean decoded V over the low history from latent sums and centre counts, fp32
    (LB/codec_native_attention.py:465-501): decoder (sum latent / n) + bf16(mean) + (counts^T
    centres) / n, as [B, heads, 1, native_dim]."""
    latent_sum = center_sum = None
    count = 0
    for item in low_segments:
        latent, centers, ids, mean = item["v"]
        counts = torch.zeros(centers.shape[:2], dtype=torch.float32)
        counts.scatter_add_(1, ids, torch.ones_like(ids, dtype=torch.float32))
        ls = latent.float().sum(1)
        cs = torch.einsum("bc,bcd->bd", counts, centers.float())
        latent_sum = ls if latent_sum is None else latent_sum + ls
        center_sum = cs if center_sum is None else center_sum + cs
        count += latent.shape[1]
    value = F.linear(latent_sum / count, decoder.float(), mean.to(torch.bfloat16).float()) + center_sum / count
    return value.reshape(latent_sum.shape[0], heads, 1, native_dim)


def hybrid_attention(q_pre, q_native, native_segments, low_segments, reader: dict, rope=None,
                     value_mean=None, camera=None):
    """Mixed-dimensional read; positional hooks are the identity unless ``rope`` is given.

    ``rope`` = dict(freqs, frame_seqlen, width, q_positions): the reduced query and every
    low-width key read are rotated with the native pairs the group retains (group["indices"]),
    by q_positions and segment["positions"] (LB/codec_native_attention.py:757, :779).
    ``value_mean`` [B,H,1,D] switches on the value-mean residual of groups narrower than the head:
    lifted + value_mean[heads] - lift(mean over tokens of the low-width V), in fp32 (:793-796); it
    applies to the single joined low partition, as the reference concatenates its segments.
    ``camera`` = dict(q=P^T, out=P) with segment["camera"] = P^-1 (each [1, frames, 4, 4, 4]) is
    Matrix-Game's PRoPE: query, low-width keys and values and the low-width output are transformed
    block-wise after the rotation (MGC/mg35.py:318-347).

    q_* [B,H,Q,D]; native_segments [(K,V) or (K,V,mask)] full-width [B,H,n,D]; low_segments
    [{"k": (latent, centers, ids, mean), "v": (...), optional "mask"}]; a mask is a boolean
    visibility [1,1,Q or 1,n] (MGC/core.py:55-65, :290-291, :303); reader {"native_dim",
    "groups": [...]}.  Per group the low-width partitions are merged into the
    native (protected) partition by LSE.  MGC/core.py:278-310.
    """
    native_dim = int(reader["native_dim"])
    scale = native_dim ** -0.5
    dtype = q_native.dtype
    native_out = torch.zeros_like(q_native)
    native_lse = torch.full(q_native.shape[:-1], -math.inf)
    for key, value, *visible in native_segments:
        out, lse = attention_lse(q_native, key, value, visible[0] if visible else None, scale=scale)
        native_out, native_lse = merge(native_out, native_lse, out, lse)
    result = torch.zeros_like(q_native)
    for group in reader["groups"]:
        head = group["heads"].long()
        query = torch.einsum("bhnd,hde->bhne", q_pre.index_select(1, head),
                             group["q_reduce"].to(dtype))
        if rope is not None:
            query = rope_selected(query, rope["q_positions"], rope["freqs"],
                                  frame_seqlen=rope["frame_seqlen"], width=rope["width"],
                                  indices=group["indices"])
        if camera is not None:
            query = camera_selected(query, camera["q"], group["indices"])
        out = native_out.index_select(1, head)
        lse = native_lse.index_select(1, head)
        if value_mean is not None:   # LingBot's form: one joined low partition per group
            kk = torch.cat([reader_read(group, *seg["k"], target="k", dtype=dtype, native_dim=native_dim)
                            for seg in low_segments], dim=2)
            vv = torch.cat([reader_read(group, *seg["v"], target="v", dtype=dtype, native_dim=native_dim)
                            for seg in low_segments], dim=2)
            if rope is not None:
                kk = rope_selected(kk, torch.cat([seg["positions"] for seg in low_segments]),
                                   rope["freqs"], frame_seqlen=rope["frame_seqlen"],
                                   width=rope["width"], indices=group["indices"])
            oo, ll = attention_lse(query, kk, vv, scale=scale)
            lifted = torch.einsum("bhne,hed->bhnd", oo, group["lift"].to(dtype))
            if group["lift"].shape[1] < native_dim:
                projected = torch.einsum("bhse,hed->bhsd", vv.float().mean(2, keepdim=True),
                                         group["lift"].to(dtype).float())
                lifted = lifted.float() + value_mean.index_select(1, head) - projected
            out, lse = merge(out, lse, lifted, ll)
            result.index_copy_(1, head, out.to(dtype))
            continue
        for segment in low_segments:
            kk = reader_read(group, *segment["k"], target="k", dtype=dtype, native_dim=native_dim)
            vv = reader_read(group, *segment["v"], target="v", dtype=dtype, native_dim=native_dim)
            if rope is not None:
                kk = rope_selected(kk, segment["positions"], rope["freqs"],
                                   frame_seqlen=rope["frame_seqlen"], width=rope["width"],
                                   indices=group["indices"])
            if camera is not None:
                kk = camera_selected(kk, segment["camera"], group["indices"])
                vv = camera_selected(vv, segment["camera"], group.get("v_indices", group["indices"]))
            oo, ll = attention_lse(query, kk, vv, segment.get("mask"), scale=scale)
            if camera is not None:
                oo = camera_selected(oo, camera["out"], group.get("v_indices", group["indices"]))
            lifted = torch.einsum("bhne,hed->bhnd", oo, group["lift"].to(dtype))
            out, lse = merge(out, lse, lifted, ll)
        result.index_copy_(1, head, out)
    return result


# ---------------------------------------------------------------- positional restore
def rope_table(max_len: int, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [max_len, head_dim/2] rotation table of the 3-D RoPE: the columns are the
    temporal, vertical and horizontal bands side by side
    (wan/modules/model.py:29-36 rope_params, :426-430 the three-band concatenation)."""
    def band(dim):
        angles = torch.outer(torch.arange(max_len),
                             1.0 / torch.pow(theta, torch.arange(0, dim, 2).to(torch.float64).div(dim)))
        return torch.polar(torch.ones_like(angles), angles)
    d = head_dim
    return torch.cat([band(d - 4 * (d // 6)), band(2 * (d // 6)), band(2 * (d // 6))], dim=1)


def rope_coordinates(positions: torch.Tensor, frame_seqlen: int, width: int):
    """absolute token position -> (frame, row, column)
    (wan/modules/lingbot_v2_cache_runtime.py:64-68)."""
    positions = positions.long()
    frame = torch.div(positions, frame_seqlen, rounding_mode="floor")
    spatial = positions.remainder(frame_seqlen)
    return frame, torch.div(spatial, width, rounding_mode="floor"), spatial.remainder(width)


def rope_by_positions(key: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, *,
                      frame_seqlen: int, width: int) -> torch.Tensor:
    """key [1,S,H,D] before RoPE -> after, each token rotated by its own absolute position:
    adjacent element pairs are complex numbers multiplied in float64 by the table row of the
    token's frame (temporal band), row (vertical band) and column (horizontal band), one
    rounding back to the key's dtype (wan/modules/lingbot_v2_cache_runtime.py:19-76)."""
    half = key.shape[-1] // 2
    split = [half - 2 * (half // 3), half // 3, half // 3]
    temporal, vertical, horizontal = freqs.split(split, dim=1)
    frame, row, column = rope_coordinates(positions, frame_seqlen, width)
    multiplier = torch.cat((temporal.index_select(0, frame), vertical.index_select(0, row),
                            horizontal.index_select(0, column)), dim=1)[:, None]
    pairs = torch.view_as_complex(key[0].to(torch.float64).reshape(key.shape[1], key.shape[2], -1, 2))
    return torch.view_as_real(pairs * multiplier).flatten(2)[None].to(key.dtype)


def rope_selected(value: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, *,
                  frame_seqlen: int, width: int, indices: torch.Tensor) -> torch.Tensor:
    """value [B,h,S,e] of a low-width reader -> rotated: pair p of head h is the native pair
    indices[h, 2p] // 2, and is multiplied by that column of the token's full multiplier row
    (wan/modules/codec_native_attention.py:416-438 _selected_multiplier / _rope_low)."""
    original_half = freqs.shape[1]
    split = [original_half - 2 * (original_half // 3), original_half // 3, original_half // 3]
    temporal, vertical, horizontal = freqs.split(split, dim=1)
    frame, row, column = rope_coordinates(positions, frame_seqlen, width)
    multiplier = torch.cat((temporal[frame], vertical[row], horizontal[column]), 1)   # [S, native half]
    pair = indices.long()[:, ::2] // 2                                                # [h, e/2]
    selected = multiplier[:, pair].permute(1, 0, 2)                                   # [h, S, e/2]
    pairs = torch.view_as_complex(value.double().reshape(*value.shape[:-1], -1, 2).contiguous())
    return torch.view_as_real(pairs * selected[None]).flatten(-2).to(value.dtype)


def rope_per_token(value: torch.Tensor, multiplier: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Matrix-Game's form: value [B,h,S,e], multiplier complex [S, native half] given per token,
    indices [h,e] the native dimensions each head retains (whole pairs); float64 complex product,
    one rounding (MGC/core.py:75-91 rope_selected)."""
    chosen = multiplier[:, indices.long()[:, ::2] // 2].permute(1, 0, 2)
    pairs = torch.view_as_complex(value.double().reshape(*value.shape[:-1], -1, 2).contiguous())
    return torch.view_as_real(pairs * chosen[None]).flatten(-2).to(value.dtype)


def camera_selected(x: torch.Tensor, matrix: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """PRoPE camera transform of rows x [B,h,S,e] that retain whole 8-wide native blocks:
    a block holds four (j) two-element (r) slots; slot j of the output block is sum_j' M[i, j'] of
    the input slots, with M = matrix[b, frame, camera] (4 x 4), camera = native block id % 4 and
    the S tokens split evenly over the matrix's frames; operands in x's dtype
    (MGC/core.py:110-137 camera_selected, full layout)."""
    blocks = indices.long().reshape(indices.shape[0], -1, 8)
    if not torch.equal(blocks, blocks[..., :1] + torch.arange(8)) or bool((blocks[..., 0] % 8).any()):
        raise ValueError("Invalid MG camera blocks")
    cams = (blocks[..., 0] // 8) % 4                                     # [h, G]
    frames = int(matrix.shape[1])
    if x.shape[-2] % frames:
        raise ValueError("PRoPE frame count must divide the token sequence")
    selected = matrix[:, :, cams].permute(0, 2, 1, 3, 4, 5)             # B, h, F, G, 4, 4
    values = x.reshape(x.shape[0], x.shape[1], frames, -1, blocks.shape[1], 4, 2)
    out = torch.einsum("bhfgij,bhftgjr->bhftgir", selected.to(x.dtype), values)
    return out.reshape(x.shape)


# ---------------------------------------------------------------- INT8 operator storage
def pack_int8_weight(weight: torch.Tensor, group_size: int = 0):
    """fp32 weight [rows, in] -> (int8 codes, bf16 scale [rows, in/group], group): symmetric
    per-(row, group) quantisation, scale = max(amax, 1e-12) / 127 (MGM/nanokv_codec.py:108-131)."""
    weight = weight.detach().float().cpu().contiguous()
    in_features = int(weight.shape[1])
    group = in_features if group_size <= 0 else int(group_size)
    if group > in_features or in_features % group:
        raise ValueError(f"INT8 group size {group} must divide {in_features}")
    grouped = weight.reshape(weight.shape[0], -1, group)
    scale = grouped.abs().amax(dim=2).clamp_min(1e-12) / 127.0
    codes = (grouped / scale[:, :, None]).round().clamp(-127, 127).to(torch.int8)
    return codes.reshape_as(weight), scale.to(torch.bfloat16), group


def unpack_int8_weight(qweight: torch.Tensor, scale: torch.Tensor, group_size: int) -> torch.Tensor:
    """bf16 weight the reference multiplies with: bf16(q) * scale, a bf16 product
    (MGM/nanokv_codec.py:147-152; LB/lingbot_v2_kv_codec.py:107 per row)."""
    rows = qweight.shape[0]
    return (qweight.reshape(rows, -1, group_size).to(torch.bfloat16)
            * scale.to(torch.bfloat16).reshape(rows, -1)[:, :, None]).reshape_as(qweight)
