"""GPU parity of the read path: decode, fused codec-attention, merge, hybrid attention."""
import math

import numpy as np
import pytest
import torch

import cases
from helpers import (BF16_REL_TOL, F32_REL_TOL, device_operator, history_from_segments, rel_err)
from nanokv_b200 import attention, codec, ops, synthetic
from oracle import nkv_oracle as oracle
from test_oracle_golden import encode_all, from_bits, load

pytestmark = pytest.mark.gpu


def oracle_segments(case):
    data = cases.build(case)
    return data, encode_all(case, data)


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.MINI_BF16], ids=lambda c: c.name)
def test_decode_rows_matches_oracle(case):
    data, segments = oracle_segments(case)
    dtype = case.shape.torch_dtype
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        hist = history_from_segments(segments[kind], joint=case.shape.joint, rank=case.shape.rank)
        want = torch.cat([oracle.decode_rows(s, decoder=op["decoder"], mean=op["mean"], dtype=dtype)
                          for s in segments[kind]], 1)[0]
        dev = device_operator(op)
        got = codec.decode(hist, dev, dtype=dtype).cpu()
        if dtype == torch.float32:
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
        else:
            assert rel_err(got, want) <= 2.0 ** -7
            assert float((got != want).float().mean()) < 0.02
        rows = torch.tensor([0, 299, 300, 511, 17, 17], dtype=torch.int32)
        picked = codec.decode(hist, dev, rows=rows.cuda(), dtype=dtype).cpu()
        assert torch.equal(picked, got[rows.long()])


def run_codec_attention(case, data, segments, *, group=None, scale_dtype=torch.bfloat16):
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank,
                                   group=group, scale_dtype=scale_dtype)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank,
                                   group=group, scale_dtype=scale_dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = attention.codec_attention(data["q"].cuda(), hist_k, hist_v, ops_k, ops_v,
                                         status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device-side wait gave up at site {int(status.item())}"
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.C1], ids=lambda c: c.name)
def test_codec_attention_f32_against_reference_fixture(case):
    gold = load(case.name)
    data, segments = oracle_segments(case)
    out, lse = run_codec_attention(case, data, segments)
    want_rows = torch.from_numpy(gold["attn_rows"])            # [H, Q/stride, D]
    got_rows = out.permute(1, 0, 2)[:, ::case.attn_stride]
    assert rel_err(got_rows, want_rows) <= F32_REL_TOL
    assert float((lse.t() - torch.from_numpy(gold["lse"])).abs().max()) <= F32_REL_TOL


def test_codec_attention_bf16_against_reference_fixture():
    case = cases.MINI_BF16
    gold = load(case.name)
    data, segments = oracle_segments(case)
    out, lse = run_codec_attention(case, data, segments)
    want_rows = from_bits(gold["attn_rows"], torch.bfloat16)
    assert rel_err(out.permute(1, 0, 2), want_rows) <= BF16_REL_TOL
    assert float((lse.t() - torch.from_numpy(gold["lse"])).abs().max()) <= BF16_REL_TOL


@pytest.mark.parametrize("heads,rank,history,queries,group,scale_dtype", [
    (2, 64, 128, 128, None, torch.bfloat16),      # exactly one tile each way
    (2, 64, 1, 1, None, torch.bfloat16),          # single token, single query
    (3, 128, 517, 300, None, torch.bfloat16),     # ragged everything, two query tiles
    (2, 192, 700, 257, 32, torch.float16),        # grouped scales in fp16
    (2, 640, 300, 130, None, torch.bfloat16),     # Wan-shaped rank
])
def test_codec_attention_bf16_shapes(heads, rank, history, queries, group, scale_dtype):
    shape = synthetic.Shape("t", heads, 128, rank, 8, history, queries, "bf16")
    segs = (history,) if history < 200 else (history - 130, 130)
    case = cases.CodecCase("t", shape, segs, seed=31, mean_std=0.05)
    data = cases.build(case)
    segments = {"k": [], "v": []}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        for chunk in data[f"{kind}_chunks"]:
            segments[kind].append(oracle.encode_rows(
                chunk[None], encoder=op["encoder"], mean=op["mean"],
                centers=data[f"{kind}_true_centers"][None].to(torch.bfloat16), group=group,
                scale_dtype=scale_dtype))
    out, lse = run_codec_attention(case, data, segments, group=group, scale_dtype=scale_dtype)
    k_op, v_op = data["k_op"], data["v_op"]
    want, want_lse = oracle.codec_attention(
        data["q"][None], segments["k"], segments["v"], k_decoder=k_op["decoder"],
        k_mean=k_op["mean"], v_decoder=v_op["decoder"], v_mean=v_op["mean"], heads=heads,
        dtype=torch.bfloat16)
    assert rel_err(out, want[0]) <= BF16_REL_TOL
    assert float((lse - want_lse[0].t()).abs().max()) <= BF16_REL_TOL


def test_codec_attention_bf16_tensor_core_vs_cuda_core_emulation():
    """Same inputs through the tcgen05 kernel and the fp32 CUDA-core kernel with bf16 rounding."""
    shape = synthetic.Shape("t", 4, 128, 256, 16, 1500, 520, "bf16")
    case = cases.CodecCase("t", shape, (700, 800), seed=41, mean_std=0.05)
    data, segments = oracle_segments(case)
    out_tc, lse_tc = run_codec_attention(case, data, segments)
    ops.force_simt(True)
    try:
        out_sm, lse_sm = run_codec_attention(case, data, segments)
    finally:
        ops.force_simt(False)
    assert rel_err(out_tc, out_sm) <= BF16_REL_TOL
    assert float((lse_tc - lse_sm).abs().max()) <= 5e-3


def test_codec_attention_history_splits_agree():
    """One launch with the history cut into runs merged by LSE equals the unsplit launch."""
    shape = synthetic.Shape("t", 2, 128, 128, 16, 1300, 300, "bf16")
    case = cases.CodecCase("t", shape, (600, 700), seed=43, mean_std=0.05)
    data, segments = oracle_segments(case)
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=shape.joint, rank=shape.rank)
    hist_v = history_from_segments(segments["v"], joint=shape.joint, rank=shape.rank)
    q = data["q"].cuda()
    whole, whole_lse = attention.codec_attention(q, hist_k, hist_v, ops_k, ops_v, splits=1)
    for splits in (2, 3, 16):
        out, lse = attention.codec_attention(q, hist_k, hist_v, ops_k, ops_v, splits=splits)
        assert rel_err(out.cpu(), whole.cpu()) <= 2.0 ** -6
        assert float((lse - whole_lse).abs().max()) <= 1e-3
    with pytest.raises(ValueError):
        attention.codec_attention(q, hist_k, hist_v, ops_k, ops_v, splits=17)


def test_codec_attention_empty_history():
    shape = synthetic.Shape("t", 2, 128, 64, 8, 0, 40, "bf16")
    gen = synthetic.generator(1)
    op = device_operator(synthetic.make_operator(shape, gen))
    hist = history_from_segments([], joint=256, rank=64)
    q = synthetic.make_queries(shape, gen).cuda()
    for query in (q, q.float()):
        opx = op if query.dtype == torch.bfloat16 else device_operator(
            synthetic.make_operator(shape, gen, dtype=torch.float32))
        out, lse = attention.codec_attention(query, hist, hist, opx, opx)
        assert float(out.abs().max()) == 0.0
        assert bool(torch.isinf(lse).all()) and bool((lse < 0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_attention_lse(dtype):
    gen = synthetic.generator(5)
    q = torch.randn(200, 3, 128, generator=gen).to(dtype)
    k = torch.randn(333, 3, 128, generator=gen).to(dtype)
    v = torch.randn(333, 3, 128, generator=gen).to(dtype)
    want, want_lse = oracle.attention_lse(q.permute(1, 0, 2)[None], k.permute(1, 0, 2)[None],
                                          v.permute(1, 0, 2)[None])
    out, lse = ops.attention_lse(q.cuda(), k.cuda(), v.cuda(), scale=128 ** -0.5)
    tol = F32_REL_TOL if dtype == torch.float32 else BF16_REL_TOL
    assert rel_err(out.cpu(), want[0].permute(1, 0, 2)) <= tol
    assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= tol


def test_merge_edge_cases_against_reference_fixture():
    gold = load("merge_edge")
    out_a, lse_a, out_b, lse_b = (t.cuda() for t in cases.build_merge())
    out, lse = attention.merge(out_a, lse_a, out_b, lse_b)
    want = from_bits(gold["out"], torch.bfloat16)
    want_lse = torch.from_numpy(gold["lse"])
    got_lse = lse.cpu()
    finite = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(got_lse), finite)
    assert torch.allclose(got_lse[finite], want_lse[finite], rtol=1e-6, atol=1e-6)
    assert rel_err(out.cpu(), want) <= 2.0 ** -7
    assert float(out.cpu()[0, 0, 2:4].abs().max()) == 0.0    # both partitions empty -> zeros


def test_merge_many_partitions_equals_unsplit_attention():
    gen = synthetic.generator(6)
    q = torch.randn(150, 2, 128, generator=gen).cuda()
    k = torch.randn(1000, 2, 128, generator=gen).cuda()
    v = torch.randn(1000, 2, 128, generator=gen).cuda()
    scale = 128 ** -0.5
    whole, whole_lse = ops.attention_lse(q, k, v, scale=scale)
    bounds = [0, 100, 100, 400, 777, 1000]        # includes an empty shard
    parts = [ops.attention_lse(q, k[a:b].contiguous(), v[a:b].contiguous(), scale=scale)
             for a, b in zip(bounds[:-1], bounds[1:])]
    out, lse = ops.lse_merge(parts)
    assert rel_err(out.cpu(), whole.cpu()) <= 1e-5
    assert float((lse - whole_lse).abs().max()) <= 1e-5


@pytest.mark.parametrize("case", cases.FAST_CASES, ids=lambda c: c.name)
def test_hybrid_attention_against_reference_fixture(case):
    gold = load(case.name)
    codec_case = case.codec
    shape = codec_case.shape
    dtype = shape.torch_dtype
    data, segments = oracle_segments(codec_case)
    low = case.low_segments
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    low_k = history_from_segments(segments["k"][:low], joint=shape.joint, rank=shape.rank)
    low_v = history_from_segments(segments["v"][:low], joint=shape.joint, rank=shape.rank)
    native = []
    for sk, sv in zip(segments["k"][low:], segments["v"][low:]):
        hk = history_from_segments([sk], joint=shape.joint, rank=shape.rank)
        hv = history_from_segments([sv], joint=shape.joint, rank=shape.rank)
        native.append((codec.decode(hk, ops_k, dtype=dtype).view(-1, shape.heads, shape.head_dim),
                       codec.decode(hv, ops_v, dtype=dtype).view(-1, shape.heads, shape.head_dim)))
    reader = attention.Reader(cases.build_reader(case, data), dtype=dtype)
    q = data["q"].cuda()
    got = attention.hybrid_attention(
        q, q, native, [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean}],
        reader)
    want = from_bits(gold["hybrid"], dtype)                  # [H, Q, D]
    tol = F32_REL_TOL if dtype == torch.float32 else BF16_REL_TOL
    assert rel_err(got.cpu().permute(1, 0, 2), want) <= tol
    # protected tokens left compressed and rebuilt inside the fused kernel: same result
    compressed = [{"k": history_from_segments([sk], joint=shape.joint, rank=shape.rank),
                   "v": history_from_segments([sv], joint=shape.joint, rank=shape.rank),
                   "op_k": ops_k, "op_v": ops_v}
                  for sk, sv in zip(segments["k"][low:], segments["v"][low:])]
    fused = attention.hybrid_attention(
        q, q, compressed, [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean}], reader)
    assert rel_err(fused.cpu().permute(1, 0, 2), want) <= tol


def test_hybrid_attention_with_visibility_masks_against_reference_fixture():
    """Boolean visibility per query group on every segment: the compressed segments are gathered
    (codes, scales, ids), not decoded, and read by the unmasked kernels; against the reference's
    masked hybrid_attention (MGC/core.py:278-310 with masks, :55-65)."""
    case = cases.FAST_CASES[1]
    gold = load("fast_masked_bf16")
    codec_case, shape = case.codec, case.codec.shape
    dtype = shape.torch_dtype
    data, segments = oracle_segments(codec_case)
    low = case.low_segments
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    low_k = history_from_segments(segments["k"][:low], joint=shape.joint, rank=shape.rank)
    low_v = history_from_segments(segments["v"][:low], joint=shape.joint, rank=shape.rank)
    groups, visible = cases.build_visibility(case)
    native = []
    for sk, sv, mask in zip(segments["k"][low:], segments["v"][low:], visible[low:]):
        hk = history_from_segments([sk], joint=shape.joint, rank=shape.rank)
        hv = history_from_segments([sv], joint=shape.joint, rank=shape.rank)
        native.append((codec.decode(hk, ops_k, dtype=dtype).view(-1, shape.heads, shape.head_dim),
                       codec.decode(hv, ops_v, dtype=dtype).view(-1, shape.heads, shape.head_dim),
                       mask.cuda()))
    reader = attention.Reader(cases.build_reader(case, data), dtype=dtype)
    q = data["q"].cuda()
    got = attention.hybrid_attention(
        q, q, native, [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean,
                        "mask": torch.cat(visible[:low], dim=1).cuda()}],
        reader, query_groups=groups.cuda())
    want = from_bits(gold["hybrid"], dtype)                  # [H, Q, D]
    assert rel_err(got.cpu().permute(1, 0, 2), want) <= BF16_REL_TOL
    # the masks matter: the unmasked read of the same inputs is far from the masked fixture
    plain = attention.hybrid_attention(
        q, q, [pair[:2] for pair in native],
        [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean}], reader)
    assert rel_err(plain.cpu().permute(1, 0, 2), want) > 4 * BF16_REL_TOL


def test_gather_view_keeps_the_segment_of_every_token():
    """Gathered tokens decode to the same rows as the same tokens of the whole history, across
    segment boundaries and with a segment that loses all its tokens."""
    case = cases.MINI_BF16
    shape = case.shape
    data, segments = oracle_segments(case)
    op = device_operator(data["k_op"])
    hist = history_from_segments(segments["k"] + segments["k"][:1], joint=shape.joint, rank=shape.rank)
    whole = codec.decode(hist, op, dtype=torch.bfloat16)
    first, second = case.segments
    index = torch.tensor([0, 5, first - 1, first + second, first + second + 7, hist.tokens - 1], device="cuda")
    view = ops.gather_view(hist.view(), index)                     # the middle segment is empty
    assert view.tokens == index.numel() and view.seg_start[:4].tolist() == [0, 3, 3, 6]
    rows = ops.decode_rows(view, op.decoder, op.mean, dtype=torch.bfloat16)
    assert torch.equal(rows, whole.index_select(0, index))


@pytest.mark.parametrize("heads,dim,tokens,queries", [(3, 128, 517, 300), (2, 64, 1, 1), (2, 128, 33000, 40)])
def test_plain_attention_bf16_runs_on_the_fused_kernel(heads, dim, tokens, queries):
    """bf16 plain attention (the Fast path's protected / current branch) enters the tcgen05 kernel
    with the rows as an exact centre table; it must agree with the oracle and with the fp32
    CUDA-core kernel, also past the 32,768-token segment boundary of the 16-bit ids."""
    gen = torch.Generator().manual_seed(tokens)
    q = torch.randn(queries, heads, dim, generator=gen).to(torch.bfloat16)
    k = torch.randn(tokens, heads, dim, generator=gen).to(torch.bfloat16)
    v = torch.randn(tokens, heads, dim, generator=gen).to(torch.bfloat16)
    scale = dim ** -0.5
    out, lse = ops.attention_lse(q.cuda(), k.cuda(), v.cuda(), scale=scale)
    ops.force_simt(True)
    try:
        ref_out, ref_lse = ops.attention_lse(q.cuda(), k.cuda(), v.cuda(), scale=scale)
    finally:
        ops.force_simt(False)
    torch.cuda.synchronize()
    assert rel_err(out.cpu(), ref_out.cpu()) <= BF16_REL_TOL
    assert float((lse - ref_lse).abs().max()) <= BF16_REL_TOL
    if tokens <= 1000:
        want, want_lse = oracle.attention_lse(q.permute(1, 0, 2)[None], k.permute(1, 0, 2)[None],
                                              v.permute(1, 0, 2)[None], scale=scale)
        assert rel_err(out.cpu(), want[0].permute(1, 0, 2)) <= BF16_REL_TOL
        assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= BF16_REL_TOL


def test_history_moments_match_the_oracle():
    case = cases.MINI_BF16
    data, segments = oracle_segments(case)
    hist = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    latent_sum, counts = ops.history_moments(hist.view())
    want_sum = sum(oracle.dequantize_rows(s["codes"], s["scale"]).float().sum(0) for s in segments["v"])
    assert torch.allclose(latent_sum.cpu(), want_sum.reshape(-1), rtol=1e-5, atol=1e-4)
    want_counts = torch.cat([torch.bincount(s["ids"].reshape(-1).long(), minlength=case.shape.centers)
                             for s in segments["v"]])
    assert torch.equal(counts.cpu()[:want_counts.numel()].long(), want_counts)
    again, _ = ops.history_moments(hist.view())
    assert torch.equal(again, latent_sum)                      # fixed summation order


@pytest.mark.parametrize("case", cases.FAST_CASES, ids=lambda c: c.name)
def test_hybrid_attention_value_mean_residual(case):
    """First-moment correction of the groups narrower than the head (LingBot's opt-in residual)."""
    codec_case = case.codec
    shape = codec_case.shape
    dtype = shape.torch_dtype
    data, segments = oracle_segments(codec_case)
    n_low = case.low_segments
    low, native = [], []
    for index in range(len(codec_case.segments)):
        seg_k, seg_v = segments["k"][index], segments["v"][index]
        if index < n_low:
            entry = {}
            for kind, seg in (("k", seg_k), ("v", seg_v)):
                latent = oracle.dequantize_rows(seg["codes"], seg["scale"])[None]
                entry[kind] = (latent, seg["centers"].float(), seg["ids"].long(), data[f"{kind}_op"]["mean"])
            low.append(entry)
        else:
            pair = []
            for kind, seg in (("k", seg_k), ("v", seg_v)):
                op = data[f"{kind}_op"]
                rows = oracle.decode_rows(seg, decoder=op["decoder"], mean=op["mean"], dtype=dtype)
                pair.append(rows.reshape(1, -1, shape.heads, shape.head_dim).permute(0, 2, 1, 3))
            native.append(tuple(pair))
    reader_payload = cases.build_reader(case, data)
    q = data["q"][None].permute(0, 2, 1, 3).contiguous()
    value_mean = oracle.compressed_value_mean(low, decoder=data["v_op"]["decoder"].to(dtype),
                                              heads=shape.heads, native_dim=shape.head_dim)
    want = oracle.hybrid_attention(q, q, native, low, reader_payload, value_mean=value_mean)[0]
    plain = oracle.hybrid_attention(q, q, native, low, reader_payload)[0]
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    low_k = history_from_segments(segments["k"][:n_low], joint=shape.joint, rank=shape.rank)
    low_v = history_from_segments(segments["v"][:n_low], joint=shape.joint, rank=shape.rank)
    native_dev = [(k[0].permute(1, 0, 2).contiguous().cuda(), v[0].permute(1, 0, 2).contiguous().cuda())
                  for k, v in native]
    reader = attention.Reader(reader_payload, dtype=dtype)
    got = attention.hybrid_attention(
        data["q"].cuda(), data["q"].cuda(), native_dev,
        [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean, "v_decoder": ops_v.decoder}],
        reader, value_mean_residual=True)
    tol = F32_REL_TOL if dtype == torch.float32 else BF16_REL_TOL
    assert rel_err(got.cpu().permute(1, 0, 2), want) <= tol
    assert rel_err(plain, want) > 2 * tol, "the correction must matter in this case"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("correct", [False, True])
def test_fast_finish_is_the_reference_blend_bit_for_bit(dtype, correct):
    """One launch = value-mean correction + LSE merge + head scatter, in the reference's fp32 order
    (finish, LingBot fast tree wan/modules/codec_native_finish_triton.py:21-35): compared bit for bit
    with the same expression evaluated by torch in fp32, infinite LSEs included."""
    gen = torch.Generator().manual_seed(11)
    Q, H, D = 37, 6, 64
    heads = torch.tensor([4, 0, 3], dtype=torch.int32)
    G = heads.numel()
    native = torch.randn(Q, H, D, generator=gen).to(dtype)
    lifted = torch.randn(Q, G, D, generator=gen).to(dtype)
    native_lse = torch.randn(Q, H, generator=gen) * 3
    low_lse = torch.randn(Q, G, generator=gen) * 3
    native_lse[0], low_lse[0] = -math.inf, -math.inf            # both partitions empty
    native_lse[1] = -math.inf                                    # only the low partition
    low_lse[2] = -math.inf                                       # only the native partition
    mean = torch.randn(H, D, generator=gen) if correct else None
    projected = torch.randn(G, D, generator=gen) if correct else None

    dev = torch.device("cuda", 0)
    pick = heads.long().to(dev)
    x, z = native_lse.to(dev)[:, pick], low_lse.to(dev)
    lse = torch.logaddexp(x, z)
    origin = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    low = lifted.to(dev).float()
    if correct:
        low = (low + mean.to(dev)[pick][None]) - projected.to(dev)[None]
    want = (native.to(dev)[:, pick].float() * (x - origin).exp()[..., None]
            + low * (z - origin).exp()[..., None]).to(dtype).cpu()
    lse = lse.cpu()

    out = torch.full((Q, H, D), 7.0, dtype=dtype, device=dev)
    out_lse = torch.full((Q, H), 7.0, device=dev)
    ops.fast_finish(native.to(dev), native_lse.to(dev), lifted.to(dev), low_lse.to(dev), heads.to(dev), out,
                    value_mean=None if mean is None else mean.to(dev),
                    projected_mean=None if projected is None else projected.to(dev), out_lse=out_lse)
    got = out.cpu()
    assert torch.equal(got[:, heads.long()].view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    untouched = [h for h in range(H) if h not in heads.tolist()]
    assert torch.all(got[:, untouched].float() == 7.0) and torch.all(out_lse.cpu()[:, untouched] == 7.0)
    got_lse = out_lse.cpu()[:, heads.long()]
    finite = torch.isfinite(lse)
    assert torch.equal(torch.isfinite(got_lse), finite)
    assert torch.allclose(got_lse[finite], lse[finite], rtol=0, atol=2e-6)

    # in place: the running output may be the full-width input itself
    running = native.to(dev).clone()
    ops.fast_finish(running, native_lse.to(dev), lifted.to(dev), low_lse.to(dev), heads.to(dev), running,
                    value_mean=None if mean is None else mean.to(dev),
                    projected_mean=None if projected is None else projected.to(dev))
    assert torch.equal(running.cpu()[:, heads.long()].float(), want.float())


def test_fast_finish_rejects_bad_arguments():
    dev = torch.device("cuda", 0)
    native = torch.zeros(4, 2, 16, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(4, 2, device=dev)
    heads = torch.tensor([1], dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        ops.fast_finish(native, lse, native[:, :1].contiguous().float(), lse[:, :1].contiguous(), heads, native)
    with pytest.raises(ValueError):
        ops.fast_finish(native, lse, native[:, :1].contiguous(), lse[:, :1].contiguous(), heads, native,
                        value_mean=torch.zeros(2, 16, device=dev))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("din,dout,pad", [(128, 32, 64), (32, 128, 128), (128, 128, 128), (24, 40, 48)])
def test_head_linear_is_the_per_head_matrix_product(dtype, din, dout, pad):
    """q_reduce / lift of a reader group on the library's own kernel against fp64 arithmetic."""
    gen = torch.Generator().manual_seed(din * 1000 + dout)
    x = torch.randn(77, 6, max(din, 64), generator=gen).to(dtype).cuda()
    w = (torch.randn(3, din, dout, generator=gen) / din ** 0.5).to(dtype).cuda()
    heads = torch.tensor([4, 0, 5])
    got = ops.head_linear(x, w, heads=heads.cuda(), din=din, pad_to=pad)
    want = torch.einsum("nhd,hde->nhe", x.cpu().double()[:, heads, :din], w.cpu().double())
    assert got.shape == (77, 3, pad) and got.dtype == dtype
    assert bool((got[..., dout:] == 0).all())
    tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
    assert float((got[..., :dout].cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
    # without a head list: head g of x goes with matrix g
    same = ops.head_linear(x[:, :3], w, din=din)
    plain = torch.einsum("nhd,hde->nhe", x.cpu().double()[:, :3, :din], w.cpu().double())
    assert float((same.cpu().double() - plain).abs().max()) <= tol * float(plain.abs().max())
