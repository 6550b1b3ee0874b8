"""GPU parity of the fused read at the head / rank / centre counts of the headline configurations.

The histories are encoded on the GPU (the encoder has its own bit-exact tests), copied to the
host and read there by the oracle; the fused kernel reads the device copy.  A strided subset of
the query rows is compared (every query row is independent of the others), which keeps the CPU
side to seconds at 40 heads.  Shapes: Matrix-Game / HY-like (24 heads, rank 384, 256 centres,
8-bit ids), Wan-like (40 heads, rank 640, 512 centres per segment, 16-bit ids, four history
splits, a query count that leaves the last query block with one tile) and the NanoKV-Fast
mixture (18 heads at width 32, 6 at full width, protected tokens left compressed).
"""
import pytest
import torch

from helpers import BF16_REL_TOL, oracle_segments_of, rel_err
from nanokv_b200 import attention, synthetic
from nanokv_b200.cache import CompressedHistory
from nanokv_b200.codec import Operator, QuantSpec, encode_append
from oracle import nkv_oracle as oracle

pytestmark = pytest.mark.gpu

FRAME = 1560


def encoded_history(shape, tokens, seed, *, segment=3120):
    """One (K or V) history of `tokens` rows = centre + 0.3 noise, own centre table per segment."""
    device = torch.device("cuda")
    gen = synthetic.generator(seed)
    operator = synthetic.make_operator(shape, gen, mean_std=0.05)
    op = Operator(operator["mean"], operator["encoder"], operator["decoder"], device=device)
    segments = -(-tokens // segment)
    hist = CompressedHistory(joint=shape.joint, rank=shape.rank, capacity=tokens, max_segments=segments,
                             centers_per_segment=shape.centers, device=device)
    dev_gen = torch.Generator(device=device).manual_seed(seed)
    for first in range(0, tokens, segment):
        count = min(segment, tokens - first)
        centers = torch.randn(shape.centers, shape.joint, generator=dev_gen, device=device)
        pick = torch.randint(shape.centers, (count,), generator=dev_gen, device=device)
        rows = centers.index_select(0, pick)
        rows.add_(torch.randn(count, shape.joint, generator=dev_gen, device=device), alpha=0.3)
        encode_append(hist, rows.to(torch.bfloat16), op, QuantSpec(), centers=centers)
    return hist, op, operator


@pytest.mark.parametrize("name,heads,rank,centers,tokens,queries,splits", [
    ("c2_hy_shaped", 24, 384, 256, 8 * FRAME, 700, None),
    ("c3_wan_shaped", 40, 640, 512, 8 * FRAME, 1100, 4),
    ("c3_wan_shaped_ragged", 40, 640, 512, 8 * FRAME + 77, 1030, 3),
], ids=lambda v: v if isinstance(v, str) else None)
def test_codec_attention_at_headline_shapes(name, heads, rank, centers, tokens, queries, splits):
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    shape = synthetic.Shape(name, heads, 128, rank, centers, tokens, queries, "bf16")
    hist_k, op_k, host_k = encoded_history(shape, tokens, 11)
    hist_v, op_v, host_v = encoded_history(shape, tokens, 12)
    assert hist_k.ids.element_size() == (2 if centers > 256 else 1)
    q = synthetic.make_queries(shape, synthetic.generator(13))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = attention.codec_attention(q.cuda(), hist_k, hist_v, op_k, op_v, status=status,
                                         splits=splits)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device-side wait gave up at site {int(status.item())}"
    rows = torch.arange(0, queries, 13)
    rows = torch.unique(torch.cat([rows, torch.tensor([255, 256, 511, 1023, 1024, queries - 1])
                                   .clamp_max(queries - 1)]))
    want, want_lse = oracle.codec_attention(
        q[rows][None], oracle_segments_of(hist_k, shape.joint), oracle_segments_of(hist_v, shape.joint),
        k_decoder=host_k["decoder"], k_mean=host_k["mean"], v_decoder=host_v["decoder"],
        v_mean=host_v["mean"], heads=heads, dtype=torch.bfloat16)
    got = out.cpu()[rows]
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert rel_err(got, want[0]) <= BF16_REL_TOL
    assert float((lse.cpu()[rows] - want_lse[0].t()).abs().max()) <= BF16_REL_TOL


def test_hybrid_attention_at_the_fast_mixture_shape():
    """18 heads read at width 32, 6 at full width, protected tokens rebuilt from their codes."""
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    heads, rank, centers = 24, 384, 256
    low_tokens, protected_tokens, queries = 6 * FRAME, 2 * FRAME, 600
    shape = synthetic.Shape("c4_fast_mixed", heads, 128, rank, centers, low_tokens, queries, "bf16")
    hist_k, op_k, host_k = encoded_history(shape, low_tokens, 21)
    hist_v, op_v, host_v = encoded_history(shape, low_tokens, 22)
    # protected tokens: encoded with the same operators (one codec per layer and tensor)
    prot = {}
    for kind, op, seed in (("k", op_k, 23), ("v", op_v, 24)):
        device = torch.device("cuda")
        dev_gen = torch.Generator(device=device).manual_seed(seed)
        hist = CompressedHistory(joint=shape.joint, rank=rank, capacity=protected_tokens, max_segments=1,
                                 centers_per_segment=centers, device=device)
        table = torch.randn(centers, shape.joint, generator=dev_gen, device=device)
        pick = torch.randint(centers, (protected_tokens,), generator=dev_gen, device=device)
        rows = table.index_select(0, pick)
        rows.add_(torch.randn(protected_tokens, shape.joint, generator=dev_gen, device=device), alpha=0.3)
        encode_append(hist, rows.to(torch.bfloat16), op, QuantSpec(), centers=table)
        prot[kind] = hist
    gen = synthetic.generator(25)
    payload = synthetic.make_reader(shape, gen, [(list(range(18)), 32), (list(range(18, 24)), 128)],
                                    k_decoder=host_k["decoder"], v_decoder=host_v["decoder"])
    reader = attention.Reader(payload, dtype=torch.bfloat16)
    q = synthetic.make_queries(shape, gen)
    got = attention.hybrid_attention(
        q.cuda(), q.cuda(), [{"k": prot["k"], "v": prot["v"], "op_k": op_k, "op_v": op_v}],
        [{"k": hist_k, "v": hist_v, "k_mean": op_k.mean, "v_mean": op_v.mean}], reader)
    torch.cuda.synchronize()
    # oracle on a strided subset of the queries
    rows = torch.arange(0, queries, 9)
    low = []
    for seg_k, seg_v in zip(oracle_segments_of(hist_k, shape.joint), oracle_segments_of(hist_v, shape.joint)):
        entry = {}
        for kind, seg, host in (("k", seg_k, host_k), ("v", seg_v, host_v)):
            latent = oracle.dequantize_rows(seg["codes"], seg["scale"])[None]
            entry[kind] = (latent, seg["centers"].float(), seg["ids"].long(), host["mean"])
        low.append(entry)
    native = []
    pair = []
    for kind, host in (("k", host_k), ("v", host_v)):
        seg = oracle_segments_of(prot[kind], shape.joint)[0]
        full = oracle.decode_rows(seg, decoder=host["decoder"], mean=host["mean"], dtype=torch.bfloat16)
        pair.append(full.reshape(1, -1, heads, 128).permute(0, 2, 1, 3))
    native.append(tuple(pair))
    qs = q[rows][None].permute(0, 2, 1, 3).contiguous()
    want = oracle.hybrid_attention(qs, qs, native, low, payload)[0]      # [H, rows, D]
    assert torch.isfinite(got.float()).all()
    assert rel_err(got.cpu()[rows].permute(1, 0, 2), want) <= BF16_REL_TOL
