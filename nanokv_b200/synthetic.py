"""Seeded synthetic stand-ins for rollout KV, operators and readers.

The reference measures on rollouts of trained video models; those weights and
inputs are not distributable, so every test and benchmark uses tensors of the
same shapes and value distributions drawn from a seeded CPU generator:
centres ~ N(0,1); history rows = centre[uniform id] + noise * N(0,1);
encoder ~ N(0, 1/J); decoder ~ N(0, 1/r); queries ~ N(0,1).
"""
from __future__ import annotations

import dataclasses
import math

import torch


@dataclasses.dataclass(frozen=True)
class Shape:
    """One workload of the compressed-KV path."""
    name: str
    heads: int
    head_dim: int
    rank: int
    centers: int
    history: int          # history tokens N (per layer)
    queries: int          # query tokens Q
    dtype: str            # "f32" | "bf16"
    chunk: int = 1560     # tokens per encoded segment
    layers: int = 1

    @property
    def joint(self) -> int:
        return self.heads * self.head_dim

    @property
    def torch_dtype(self) -> torch.dtype:
        return {"f32": torch.float32, "bf16": torch.bfloat16}[self.dtype]


# The five configurations the headline metric is defined on.
CONFIGS = {
    "c1_roundtrip_f32": Shape("c1_roundtrip_f32", 12, 128, 192, 16, 2048, 256, "f32", chunk=2048),
    "c2_hy_shaped": Shape("c2_hy_shaped", 24, 128, 384, 256, 24960, 4680, "bf16"),
    "c3_wan_shaped": Shape("c3_wan_shaped", 40, 128, 640, 512, 99840, 4680, "bf16", layers=40),
    "c4_fast_mixed": Shape("c4_fast_mixed", 24, 128, 384, 256, 49920, 4680, "bf16"),
    "c5_streaming": Shape("c5_streaming", 40, 128, 640, 512, 399360, 4680, "bf16"),
}


def generator(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def make_centers(shape: Shape, gen: torch.Generator) -> torch.Tensor:
    """[C, J] fp32 ~ N(0,1)."""
    return torch.randn(shape.centers, shape.joint, generator=gen)


def make_rows(count: int, centers: torch.Tensor, gen: torch.Generator, *, noise: float = 0.3,
              dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """[count, J]: a uniformly drawn centre plus noise, rounded to ``dtype``."""
    pick = torch.randint(centers.shape[0], (count,), generator=gen)
    rows = centers.index_select(0, pick) + noise * torch.randn(
        count, centers.shape[1], generator=gen)
    return rows.to(dtype)


def make_operator(shape: Shape, gen: torch.Generator, *, mean_std: float = 0.0,
                  dtype: torch.dtype | None = None) -> dict:
    """{"mean" f32 [J], "encoder" [r,J], "decoder" [J,r]} in the operator dtype."""
    dtype = shape.torch_dtype if dtype is None else dtype
    joint, rank = shape.joint, shape.rank
    encoder = torch.randn(rank, joint, generator=gen) / math.sqrt(joint)
    decoder = torch.randn(joint, rank, generator=gen) / math.sqrt(rank)
    mean = mean_std * torch.randn(joint, generator=gen)
    return {"mean": mean, "encoder": encoder.to(dtype).contiguous(),
            "decoder": decoder.to(dtype).contiguous()}


def make_queries(shape: Shape, gen: torch.Generator, count: int | None = None) -> torch.Tensor:
    """[Q, H, D] ~ N(0,1) in the workload dtype."""
    count = shape.queries if count is None else count
    return torch.randn(count, shape.heads, shape.head_dim, generator=gen).to(shape.torch_dtype)


def make_reader(shape: Shape, gen: torch.Generator, groups: list[tuple[list[int], int]],
                *, k_decoder: torch.Tensor | None = None,
                v_decoder: torch.Tensor | None = None) -> dict:
    """Reader payload in the reference's ReaderLayer layout.

    ``groups`` = [(head ids, width)].  Width == head_dim with decoders given
    yields the exact decoder-slice reader; otherwise read weights ~ N(0, 1/r)
    and q_reduce / affine / lift keep the first ``width`` native channels,
    scaled so logits keep their magnitude (sqrt(D/width)).
    """
    native, rank = shape.head_dim, shape.rank
    payload = {"heads": shape.heads, "native_dim": native, "rank": rank, "groups": []}
    for head_ids, width in groups:
        heads = torch.tensor(head_ids, dtype=torch.long)
        count = len(head_ids)
        indices = torch.arange(width).expand(count, width).contiguous()
        select = torch.zeros(count, native, width)
        select.scatter_(1, indices[:, None, :], 1.0)
        if width == native and k_decoder is not None:
            k_read = k_decoder.float().reshape(shape.heads, native, rank).index_select(0, heads)
            v_read = v_decoder.float().reshape(shape.heads, native, rank).index_select(0, heads)
            gain = 1.0
        else:
            k_read = torch.randn(count, width, rank, generator=gen) / math.sqrt(rank)
            v_read = torch.randn(count, width, rank, generator=gen) / math.sqrt(rank)
            gain = math.sqrt(native / width)
        payload["groups"].append({
            "heads": heads, "indices": indices,
            "q_reduce": (select * gain).contiguous(),
            "k_read": k_read.contiguous(), "v_read": v_read.contiguous(),
            "k_affine": select.clone(), "v_affine": select.clone(),
            "lift": select.transpose(1, 2).contiguous(),
        })
    return payload


def checksum(tensor: torch.Tensor) -> int:
    """Order-sensitive 64-bit digest of a tensor's bytes (for fixtures)."""
    import hashlib
    data = tensor.detach().contiguous().view(torch.uint8).numpy().tobytes()
    return int.from_bytes(hashlib.sha256(data).digest()[:8], "little")
