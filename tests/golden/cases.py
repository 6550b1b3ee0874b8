"""Seeded case definitions shared by the fixture generator and the tests."""
from __future__ import annotations

import dataclasses
import math

import torch

from nanokv_b200 import synthetic
from nanokv_b200.synthetic import Shape


@dataclasses.dataclass(frozen=True)
class CodecCase:
    name: str
    shape: Shape
    segments: tuple[int, ...]   # tokens per encoded segment
    layer: int = 0
    iters: int = 2
    seed: int = 0
    mean_std: float = 0.0
    attn_stride: int = 1        # query rows stored in the fixture


@dataclasses.dataclass(frozen=True)
class FastCase:
    name: str
    codec: CodecCase
    low_segments: int                       # leading segments read through readers
    groups: tuple[tuple[tuple[int, ...], int], ...]


C1 = CodecCase("c1_roundtrip_f32", synthetic.CONFIGS["c1_roundtrip_f32"], (2048,),
               attn_stride=4)
MINI_F32 = CodecCase(
    "mini_mg_f32", Shape("mini_f32", 2, 128, 64, 8, 512, 70, "f32"), (300, 212),
    layer=5, seed=11, mean_std=0.05)
MINI_BF16 = CodecCase(
    "mini_mg_bf16", Shape("mini_bf16", 2, 128, 64, 8, 512, 70, "bf16"), (300, 212),
    layer=3, seed=7, mean_std=0.05)
MINI_LB = CodecCase(
    "mini_lb_bf16", Shape("mini_lb", 2, 128, 64, 8, 300, 70, "bf16"), (300,),
    layer=1, seed=5, mean_std=0.05)

MG_CASES = (C1, MINI_F32, MINI_BF16)
LINGBOT_CASES = (MINI_LB,)

_FAST_SHAPE_F32 = Shape("fast_f32", 4, 128, 64, 8, 640, 70, "f32")
_FAST_SHAPE_BF16 = Shape("fast_bf16", 4, 128, 64, 8, 640, 70, "bf16")
FAST_CASES = (
    FastCase("fast_mini_f32",
             CodecCase("fast_mini_f32", _FAST_SHAPE_F32, (256, 256, 128), layer=2, seed=21,
                       mean_std=0.05),
             2, (((0, 2), 32), ((1, 3), 128))),
    FastCase("fast_mini_bf16",
             CodecCase("fast_mini_bf16", _FAST_SHAPE_BF16, (256, 256, 128), layer=2, seed=23,
                       mean_std=0.05),
             2, (((0, 2), 32), ((1, 3), 128))),
)


def build(case: CodecCase) -> dict:
    """All inputs of a codec case, deterministically from its seed."""
    shape = case.shape
    gen = synthetic.generator(case.seed)
    dtype = shape.torch_dtype
    out = {}
    for kind in ("k", "v"):
        centers = synthetic.make_centers(shape, gen)
        out[f"{kind}_true_centers"] = centers
        out[f"{kind}_chunks"] = [synthetic.make_rows(n, centers, gen, dtype=dtype)
                                 for n in case.segments]
        out[f"{kind}_op"] = synthetic.make_operator(shape, gen, mean_std=case.mean_std)
    out["q"] = synthetic.make_queries(shape, gen)
    return out


def build_reader(case: FastCase, data: dict) -> dict:
    gen = synthetic.generator(case.codec.seed + 1000)
    groups = [(list(heads), width) for heads, width in case.groups]
    return synthetic.make_reader(case.codec.shape, gen, groups,
                                 k_decoder=data["k_op"]["decoder"],
                                 v_decoder=data["v_op"]["decoder"])


def build_visibility(case: FastCase):
    """Matrix-Game style visibility: three query groups, each seeing its own subset of every
    segment (the first token of a segment is visible to all, so no partition is empty).
    Returns (query_groups i64 [Q], [bool [3, tokens of segment s]])."""
    gen = synthetic.generator(case.codec.seed + 2000)
    queries = case.codec.shape.queries
    groups = torch.arange(queries) * 3 // queries
    masks = [torch.rand(3, n, generator=gen) < 0.7 for n in case.codec.segments]
    for mask in masks:
        mask[:, 0] = True
    return groups, masks


def build_merge():
    """Two partitions with every -inf combination among the rows."""
    gen = synthetic.generator(99)
    out_a = torch.randn(1, 3, 16, 128, generator=gen).to(torch.bfloat16)
    out_b = torch.randn(1, 3, 16, 128, generator=gen).to(torch.bfloat16)
    lse_a = 3.0 * torch.randn(1, 3, 16, generator=gen)
    lse_b = 3.0 * torch.randn(1, 3, 16, generator=gen)
    lse_a[0, 0, :4] = -math.inf
    lse_b[0, 0, 2:6] = -math.inf
    lse_b[0, 1, 0] = lse_a[0, 1, 0]
    out_a[0, 0, :4] = 0
    out_b[0, 0, 2:6] = 0
    return out_a, lse_a, out_b, lse_b


@dataclasses.dataclass(frozen=True)
class RopeCase:
    name: str
    tokens: int
    heads: int
    head_dim: int
    height: int
    width: int
    dtype: torch.dtype


ROPE_CASES = (RopeCase("rope_d128_bf16", 112, 3, 128, 6, 8, torch.bfloat16),
              RopeCase("rope_d64_f32", 60, 2, 64, 5, 4, torch.float32))


def build_rope(case: RopeCase) -> dict:
    """Pre-RoPE keys and the absolute positions of a rolling cache: a sink run from position 0,
    then a recent run far from it (not one contiguous interval)."""
    gen = synthetic.generator(777 + case.head_dim)
    key = torch.randn(1, case.tokens, case.heads, case.head_dim, generator=gen).to(case.dtype)
    frame_seqlen = case.height * case.width
    sink = case.tokens // 3
    recent_start = 19 * frame_seqlen + 5
    positions = torch.cat([torch.arange(sink), torch.arange(recent_start, recent_start + case.tokens - sink)])
    return {"key": key, "positions": positions, "frame_seqlen": frame_seqlen,
            "grid_sizes": torch.tensor([[32, case.height, case.width]])}


def build_int8_weight() -> torch.Tensor:
    """An operator-shaped fp32 matrix with rows of very different magnitude (and one zero row)."""
    gen = synthetic.generator(4321)
    weight = torch.randn(96, 256, generator=gen) * torch.logspace(-3, 1, 96)[:, None]
    weight[17] = 0
    return weight


# Rolling window (LingBot lifecycle): four committed chunks, the window cuts the first and the third
ROLLING = CodecCase("rolling_lb_bf16", Shape("rolling_lb", 2, 128, 64, 8, 250, 70, "bf16"),
                    (70, 64, 64, 52), layer=2, seed=23, mean_std=0.05)
ROLLING_POLICY = dict(capacity=150, sink_tokens=40)
ROLLING_GRID = dict(height=4, width=5)      # frame_seqlen 20


def rolling_policy_cases():
    """(segment ranges, committed_end, capacity, sink_tokens) covering the policy's branches."""
    uniform = [(i * 30, (i + 1) * 30) for i in range(8)]
    ragged = [(0, 7), (7, 50), (50, 51), (51, 120), (120, 200)]
    return [
        (uniform, 240, 100, 30), (uniform, 240, 100, 0), (uniform, 240, 1000, 30),
        (uniform, 240, 30, 30), (uniform, 240, 20, 30), (uniform[:1], 30, 100, 50),
        (ragged, 200, 64, 10), (ragged, 200, 150, 49), (ragged, 200, 81, 7), ([], 0, 10, 2),
    ]


def select_indices(case: CodecCase) -> torch.Tensor:
    """Window compaction: drop the head of the first segment and two of its later tokens, keep the
    rest of the history (the second segment whole)."""
    first = case.segments[0]
    keep = [t for t in range(40, first) if t not in (100, 101)]
    return torch.tensor(keep + list(range(first, sum(case.segments))))


def build_rope_selected():
    """A low-width reader's rows [1, heads, tokens, 32] with the native pairs (of 64) each head keeps."""
    gen = synthetic.generator(901)
    heads, tokens, width, native = 3, 90, 32, 128
    value = torch.randn(1, heads, tokens, width, generator=gen).to(torch.bfloat16)
    pairs = torch.stack([torch.randperm(native // 2, generator=gen)[:width // 2].sort().values
                         for _ in range(heads)])
    indices = torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(heads, width)
    positions = torch.cat([torch.arange(25), torch.arange(700, 765)])
    return {"value": value, "indices": indices, "positions": positions, "frame_seqlen": 35,
            "grid_sizes": torch.tensor([[40, 5, 7]]), "native_dim": native}


def value_mean_interval(case: CodecCase, index: int) -> tuple[int, int]:
    """Local token interval of segment ``index`` that belongs to the low history."""
    count = case.segments[index]
    return (17, count) if index == 0 else (0, count)


def per_token_multiplier(data: dict) -> torch.Tensor:
    """complex128 [tokens, native half]: unit-modulus multipliers with seeded angles, one row per token."""
    gen = synthetic.generator(902)
    tokens = data["value"].shape[2]
    angles = (torch.rand(tokens, data["native_dim"] // 2, generator=gen, dtype=torch.float64) - 0.5) * 40.0
    return torch.polar(torch.ones_like(angles), angles)


def build_camera():
    """Low-width rows [1, heads, tokens, 32] that retain four of the sixteen native 8-wide blocks,
    and per-frame camera matrices [1, frames, 4 cameras, 4, 4]."""
    gen = synthetic.generator(903)
    heads, frames, per_frame, width = 3, 5, 18, 32
    value = torch.randn(1, heads, frames * per_frame, width, generator=gen).to(torch.bfloat16)
    blocks = torch.stack([torch.randperm(16, generator=gen)[:width // 8].sort().values for _ in range(heads)])
    indices = (blocks[:, :, None] * 8 + torch.arange(8)).reshape(heads, width)
    matrix = torch.randn(1, frames, 4, 4, 4, generator=gen)
    return {"value": value, "indices": indices, "matrix": matrix}


# Matrix-Game positional hooks around the mixed-width read (rotation by per-token multipliers, PRoPE
# camera blocks): FAST_CASES[1] with seeded multipliers and matrices
HOOK_FRAMES = dict(query=2, low=4)


def build_hooks(case: FastCase) -> dict:
    """q_multiplier complex128 [Q, D/2]; per low segment "freqs" complex128 [tokens, D/2] and "camera"
    (P^-1) [1, frames, 4, 4, 4]; "q_camera" (P^T) and "out_camera" (P) [1, frames, 4, 4, 4]."""
    gen = synthetic.generator(case.codec.seed + 3000)
    shape = case.codec.shape
    half = shape.head_dim // 2

    def multiplier(tokens):
        angles = (torch.rand(tokens, half, generator=gen, dtype=torch.float64) - 0.5) * 40.0
        return torch.polar(torch.ones_like(angles), angles)

    def matrix(frames):
        return torch.randn(1, frames, 4, 4, 4, generator=gen) * 0.5

    out = {"q_multiplier": multiplier(shape.queries), "q_camera": matrix(HOOK_FRAMES["query"]),
           "out_camera": matrix(HOOK_FRAMES["query"]), "segments": []}
    for tokens in case.codec.segments[:case.low_segments]:
        out["segments"].append({"freqs": multiplier(tokens), "camera": matrix(HOOK_FRAMES["low"])})
    return out


# LingBot streaming: the ROLLING chunks pushed through codec_cache_attention_inputs one by one, with
# an attention limit small enough that the overflow cut applies to the late chunks
STREAM_POLICY = dict(capacity=150, sink_tokens=40, max_attention_size=170)


def protected_token_cases():
    """(frame ids, recent, stride, sink): chronological frame runs with repeated ids, empty input."""
    runs = lambda ids, per: torch.tensor([i for i in ids for _ in range(per)])
    return [
        (runs(range(12), 3), 4, 3, 1), (runs(range(12), 3), 0, 2, 0), (runs(range(12), 3), 20, 5, 0),
        (runs([5, 5, 7, 5, 9, 9, 2], 2), 2, 2, 1), (runs(range(9), 1), 3, 0, 2),
        (torch.tensor([], dtype=torch.long), 2, 1, 1), (runs(range(30), 2), 5, 7, 3),
    ]


# LingBot NanoKV-Fast step (attend): three ROLLING chunks committed, the fourth attends; one frame of
# sink and one recent frame stay full width, the rest of the window is read through the readers
ATTEND_POLICY = {"recent_native_frames": 1, "sink_native_frames": 1}
ATTEND_GROUPS = (((0,), 64), ((1,), 128))


def build_attend_reader(case: CodecCase, data: dict) -> dict:
    gen = synthetic.generator(case.seed + 4000)
    return synthetic.make_reader(case.shape, gen, [(list(heads), width) for heads, width in ATTEND_GROUPS],
                                 k_decoder=data["k_op"]["decoder"], v_decoder=data["v_op"]["decoder"])


# HY-WorldPlay two-branch dictionary reader (Main-RoPE branch + PRoPE branch over all heads)
HY_SHAPE = dict(heads=4, head_dim=128, rank=64, centres=16, history=512, history_cameras=4, queries=96,
                query_cameras=2, text=24, main_width=64, prope_quartets=16)


def _se3(count: int, gen) -> torch.Tensor:
    """Random rigid transforms [1, count, 4, 4]."""
    rotation, _ = torch.linalg.qr(torch.randn(count, 3, 3, generator=gen))
    out = torch.zeros(1, count, 4, 4)
    out[0, :, :3, :3] = rotation
    out[0, :, :3, 3] = 0.3 * torch.randn(count, 3, generator=gen)
    out[0, :, 3, 3] = 1.0
    return out


def _rope_tables(tokens: int, dim: int, gen):
    """(cos, sin) [tokens, dim] with every pair of neighbouring channels sharing its angle."""
    angles = (torch.rand(tokens, dim // 2, generator=gen) - 0.5) * 30.0
    return angles.cos().repeat_interleave(2, dim=1), angles.sin().repeat_interleave(2, dim=1)


def build_hy() -> dict:
    """State, cache payloads and call inputs of one HY two-branch read, seeded."""
    cfg = HY_SHAPE
    gen = synthetic.generator(6001)
    H, D, r, C, N, S, E = (cfg[k] for k in ("heads", "head_dim", "rank", "centres", "history", "queries", "text"))
    dm, dp = cfg["main_width"], 4 * cfg["prope_quartets"]
    bf = torch.bfloat16
    pairs = torch.stack([torch.randperm(D // 2, generator=gen)[:dm // 2].sort().values for _ in range(H)])
    state = {
        "main_indices": torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(H, dm),
        "q_main_reduce": (torch.randn(H, dm, D, generator=gen) / math.sqrt(D) * 1.5).to(bf),
        "q_prope_mix": torch.randn(H, cfg["prope_quartets"], D // 4, generator=gen) / math.sqrt(D // 4) * 1.5,
        "k_main_read": (torch.randn(H, dm, r, generator=gen) / math.sqrt(r)).to(bf),
        "k_prope_read": (torch.randn(H, dp, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_main_read": (torch.randn(H, dm, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_prope_read": (torch.randn(H, dp, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_main_lift": (torch.randn(H, dm, D, generator=gen) / math.sqrt(dm)).to(bf),
        "v_prope_mix": torch.randn(H, cfg["prope_quartets"], D // 4, generator=gen) / math.sqrt(cfg["prope_quartets"]),
        "log_residual_scale_main": 0.2 * torch.randn(H, generator=gen),
        "log_residual_scale_prope": 0.2 * torch.randn(H, generator=gen),
    }

    def payload():
        codes = torch.randint(-7, 8, (1, N, r), generator=gen, dtype=torch.int8)
        return {"codes": codes,
                "latent_scale": (torch.rand(1, N, 1, generator=gen) * 0.3 + 0.05).to(bf),
                "latent_shape": (1, N, r), "latent_numel": N * r,
                "centre_main": (0.5 * torch.randn(1, H, C, dm, generator=gen)).to(bf),
                "centre_prope": (0.5 * torch.randn(1, H, C, dp, generator=gen)).to(bf),
                "semantic_ids": torch.randint(C, (1, N), generator=gen)}

    out = {"state": state, "k_vision": payload(), "v_vision": payload(),
           "vision_freqs": _rope_tables(N, D, gen), "current_freqs": _rope_tables(S, D, gen),
           "vision_viewmats": _se3(cfg["history_cameras"], gen), "current_viewmats": _se3(cfg["query_cameras"], gen),
           "q_pre": torch.randn(1, S, H, D, generator=gen).to(bf),
           "query": torch.randn(2, H, S, D, generator=gen).to(bf),
           "current_key": torch.randn(2, H, S, D, generator=gen).to(bf),
           "current_value": torch.randn(2, H, S, D, generator=gen).to(bf),
           "encoder_key": torch.randn(2, H, E, D, generator=gen).to(bf),
           "encoder_value": torch.randn(2, H, E, D, generator=gen).to(bf)}
    return out


# HY-WorldPlay's codec entry points: joint dimension 2048 (fixed in the reference), layout [B, H, S, D]
HY_CODEC = CodecCase("hy_codec_bf16", Shape("hy_codec", 16, 128, 128, 16, 200, 8, "bf16"), (200,),
                     layer=4, seed=31, mean_std=0.05)

HY_WRITE = dict(heads=16, head_dim=128, rank=64, centres=16, tokens=160, main_width=32, prope_quartets=8, layer=6)


def build_hy_write() -> dict:
    """Raw K / V history of one HY layer, its codec operators and the reader state the write side
    projects the centre tables with, seeded."""
    cfg = HY_WRITE
    gen = synthetic.generator(6101)
    H, D, r, C, S = (cfg[k] for k in ("heads", "head_dim", "rank", "centres", "tokens"))
    dm, quartets = cfg["main_width"], cfg["prope_quartets"]
    shape = Shape("hy_write", H, D, r, C, S, 8, "bf16")
    pairs = torch.stack([torch.randperm(D // 2, generator=gen)[:dm // 2].sort().values for _ in range(H)])
    out = {"operators": {}, "attention": {
        "main_indices": torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(H, dm),
        "k_main_anchor_reduce": torch.randn(H, dm, D, generator=gen) / math.sqrt(D),
        "q_prope_mix": torch.randn(H, quartets, D // 4, generator=gen) / math.sqrt(D // 4),
        "v_main_anchor_reduce": torch.randn(H, dm, D, generator=gen) / math.sqrt(D),
        "v_prope_anchor_mix": torch.randn(H, quartets, D // 4, generator=gen) / math.sqrt(D // 4),
    }}
    for name in ("k", "v"):
        centers = synthetic.make_centers(shape, gen)
        rows = synthetic.make_rows(S, centers, gen, dtype=torch.bfloat16)
        out[f"{name}_vision"] = rows.reshape(1, S, H, D).permute(0, 2, 1, 3).contiguous()
        op = synthetic.make_operator(shape, gen, mean_std=0.05)
        out["operators"][name] = {"mean": op["mean"], "encoder": op["encoder"]}
    return out


HY_CHAIN = dict(HY_WRITE, queries=64, text=16, history_cameras=4, query_cameras=2, layer=8)   # 32-wide branches


def build_hy_chain() -> dict:
    """One HY layer end to end: raw history -> compress_layer_cache -> two-branch read, seeded."""
    cfg = HY_CHAIN
    gen = synthetic.generator(6201)
    H, D, r, C, N, S, E = (cfg[k] for k in ("heads", "head_dim", "rank", "centres", "tokens", "queries", "text"))
    dm, quartets = cfg["main_width"], cfg["prope_quartets"]
    dp = 4 * quartets
    bf = torch.bfloat16
    shape = Shape("hy_chain", H, D, r, C, N, S, "bf16")
    pairs = torch.stack([torch.randperm(D // 2, generator=gen)[:dm // 2].sort().values for _ in range(H)])
    state = {
        "main_indices": torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(H, dm),
        "q_main_reduce": (torch.randn(H, dm, D, generator=gen) / math.sqrt(D) * 1.5).to(bf),
        "q_prope_mix": torch.randn(H, quartets, D // 4, generator=gen) / math.sqrt(D // 4) * 1.5,
        "k_main_read": (torch.randn(H, dm, r, generator=gen) / math.sqrt(r)).to(bf),
        "k_prope_read": (torch.randn(H, dp, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_main_read": (torch.randn(H, dm, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_prope_read": (torch.randn(H, dp, r, generator=gen) / math.sqrt(r)).to(bf),
        "v_main_lift": (torch.randn(H, dm, D, generator=gen) / math.sqrt(dm)).to(bf),
        "v_prope_mix": torch.randn(H, quartets, D // 4, generator=gen) / math.sqrt(quartets),
        "log_residual_scale_main": 0.2 * torch.randn(H, generator=gen),
        "log_residual_scale_prope": 0.2 * torch.randn(H, generator=gen),
        "k_main_anchor_reduce": torch.randn(H, dm, D, generator=gen) / math.sqrt(D),
        "v_main_anchor_reduce": torch.randn(H, dm, D, generator=gen) / math.sqrt(D),
        "v_prope_anchor_mix": torch.randn(H, quartets, D // 4, generator=gen) / math.sqrt(D // 4),
    }
    out = {"attention": state, "operators": {}}
    for name in ("k", "v"):
        centers = synthetic.make_centers(shape, gen)
        rows = synthetic.make_rows(N, centers, gen, dtype=bf)
        out[f"{name}_vision"] = rows.reshape(1, N, H, D).permute(0, 2, 1, 3).contiguous()
        op = synthetic.make_operator(shape, gen, mean_std=0.05)
        out["operators"][name] = {"mean": op["mean"], "encoder": op["encoder"]}
    out.update({
        "vision_freqs": _rope_tables(N, D, gen), "current_freqs": _rope_tables(S, D, gen),
        "vision_viewmats": _se3(cfg["history_cameras"], gen), "current_viewmats": _se3(cfg["query_cameras"], gen),
        "q_pre": torch.randn(1, S, H, D, generator=gen).to(bf),
        "query": torch.randn(2, H, S, D, generator=gen).to(bf),
        "current_key": torch.randn(2, H, S, D, generator=gen).to(bf),
        "current_value": torch.randn(2, H, S, D, generator=gen).to(bf),
        "encoder_key": torch.randn(2, H, E, D, generator=gen).to(bf),
        "encoder_value": torch.randn(2, H, E, D, generator=gen).to(bf)})
    return out


def hy_chain_runtime(data: dict) -> dict:
    cfg = HY_CHAIN
    return {"operators": data["operators"], "attention": data["attention"], "payload_mode": "dictionary_lowkv",
            "main_k_mode": "learned_rope", "recent_native_frames": 0,
            "shape": (cfg["heads"], cfg["head_dim"], cfg["heads"], cfg["head_dim"])}

