"""GPU parity of the positional restore inside the fused read: the kernel's rotation of the
rebuilt keys against the oracle's float64 complex restatement of the reference."""
import pytest
import torch

import cases
from helpers import BF16_REL_TOL, F32_REL_TOL, device_operator, history_from_segments, rel_err
from nanokv_b200 import attention, ops, synthetic
from oracle import nkv_oracle as oracle

pytestmark = pytest.mark.gpu


def build(heads, head_dim, rank, history, queries, dtype_name, height, width):
    shape = synthetic.Shape("rope", heads, head_dim, rank, 8, history, queries, dtype_name)
    segs = (history,) if history < 200 else (history - 130, 130)
    case = cases.CodecCase("rope", shape, segs, seed=47, mean_std=0.05)
    data = cases.build(case)
    segments = {"k": [], "v": []}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        for chunk in data[f"{kind}_chunks"]:
            segments[kind].append(oracle.encode_rows(
                chunk[None], encoder=op["encoder"], mean=op["mean"],
                centers=data[f"{kind}_true_centers"][None].to(torch.bfloat16)))
    frame_seqlen = height * width
    sink = history // 4                           # sink + recent: two separate position runs
    recent = 23 * frame_seqlen + 3
    positions = torch.cat([torch.arange(sink), torch.arange(recent, recent + history - sink)])
    # queries: random rows plus unit vectors, whose LSE is a log-sum-exp of single key columns
    q = data["q"].clone()
    for i in range(min(queries, head_dim)):
        q[i] = 0
        q[i, :, (7 * i) % head_dim] = 6.0
    return case, data, segments, positions, frame_seqlen, q


def run(case, data, segments, positions, frame_seqlen, width, q):
    dtype = case.shape.torch_dtype
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    freqs = oracle.rope_table(1024, case.shape.head_dim)
    table = attention.RopeTable(freqs, frame_seqlen=frame_seqlen, width=width)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = attention.codec_attention(q.cuda(), hist_k, hist_v, ops_k, ops_v, status=status,
                                         rope=table, positions=positions.cuda())
    plain, _ = attention.codec_attention(q.cuda(), hist_k, hist_v, ops_k, ops_v, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    k_op, v_op = data["k_op"], data["v_op"]
    want, want_lse = oracle.codec_attention(
        q[None], segments["k"], segments["v"], k_decoder=k_op["decoder"], k_mean=k_op["mean"],
        v_decoder=v_op["decoder"], v_mean=v_op["mean"], heads=case.shape.heads, dtype=dtype,
        rope=dict(positions=positions, freqs=freqs, frame_seqlen=frame_seqlen, width=width))
    return out.cpu(), lse.cpu(), want[0], want_lse[0].t(), plain.cpu()


@pytest.mark.parametrize("heads,head_dim,rank,history,queries,height,width", [
    (2, 128, 128, 517, 300, 6, 8),
    (3, 128, 640, 300, 130, 5, 4),
    (2, 64, 64, 260, 140, 3, 7),
])
@pytest.mark.parametrize("simt", [False, True], ids=["tcgen05", "cuda-core"])
def test_rope_read_bf16(heads, head_dim, rank, history, queries, height, width, simt):
    built = build(heads, head_dim, rank, history, queries, "bf16", height, width)
    case, data, segments, positions, frame_seqlen, q = built
    ops.force_simt(simt)
    try:
        out, lse, want, want_lse, plain = run(case, data, segments, positions, frame_seqlen, width, q)
    finally:
        ops.force_simt(False)
    assert rel_err(out, want) <= BF16_REL_TOL
    assert float((lse - want_lse).abs().max()) <= BF16_REL_TOL
    assert rel_err(plain, want) > 3 * BF16_REL_TOL, "the rotation must matter in this case"


def test_rope_read_f32():
    built = build(2, 64, 64, 260, 140, "f32", 3, 7)
    case, data, segments, positions, frame_seqlen, q = built
    out, lse, want, want_lse, _ = run(case, data, segments, positions, frame_seqlen, 7, q)
    assert rel_err(out, want) <= F32_REL_TOL
    assert float((lse - want_lse).abs().max()) <= F32_REL_TOL


def test_rope_argument_errors():
    freqs = oracle.rope_table(64, 128)
    with pytest.raises(ValueError):
        attention.RopeTable(freqs, frame_seqlen=48, width=7)          # width must divide the frame
    table = attention.RopeTable(freqs, frame_seqlen=48, width=8)
    built = build(2, 128, 128, 130, 4, "bf16", 6, 8)
    case, data, segments, positions, frame_seqlen, q = built
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    with pytest.raises(ValueError):                                    # position / K length mismatch
        attention.codec_attention(q.cuda(), hist_k, hist_v, ops_k, ops_v, rope=table,
                                  positions=positions[:-1].cuda())
    with pytest.raises(ValueError):
        attention.codec_attention(q.cuda(), hist_k, hist_v, ops_k, ops_v, rope=table)


def pair_index_of(indices: torch.Tensor) -> torch.Tensor:
    """reader indices [h, e] (retained native dimensions) -> native pair of every pair, i32 [h, e/2]."""
    return (indices[:, ::2] // 2).to(torch.int32)


def test_rope_rows_against_the_reference_fixtures():
    from test_oracle_golden import from_bits, load
    # full-width rows: rope_pre_key_by_positions
    case = cases.ROPE_CASES[0]
    gold, data = load(case.name), cases.build_rope(case)
    freqs = oracle.rope_table(1024, case.head_dim)
    table = attention.RopeTable(freqs, frame_seqlen=data["frame_seqlen"], width=case.width)
    got = table.rotate(data["key"][0].cuda(), data["positions"].cuda()).cpu()
    want = from_bits(gold["rotated"], torch.bfloat16)[0]
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    assert float((got != want).float().mean()) < 0.01          # fp32 instead of fp64: rare last-bit ties
    # a low-width reader's rows: _rope_low with selected native pairs
    gold, data = load("rope_selected_bf16"), cases.build_rope_selected()
    freqs = oracle.rope_table(1024, data["native_dim"])
    table = attention.RopeTable(freqs, frame_seqlen=data["frame_seqlen"], width=int(data["grid_sizes"][0, 2]))
    rows = data["value"][0].permute(1, 0, 2).contiguous()       # [S, h, e]
    got = table.rotate(rows.cuda(), data["positions"].cuda(), pair_index_of(data["indices"]).cuda()).cpu()
    want = from_bits(gold["rotated"], torch.bfloat16)[0].permute(1, 0, 2)
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    assert float((got != want).float().mean()) < 0.01
    # fp32 rows, strided input
    x = torch.randn(50, 4, 2 * 64, generator=torch.Generator().manual_seed(3))[:, :, :64]
    positions = torch.arange(100, 150)
    freqs = oracle.rope_table(1024, 64)
    table = attention.RopeTable(freqs, frame_seqlen=12, width=4)
    got = table.rotate(x.cuda(), positions.cuda()).cpu()
    want = oracle.rope_by_positions(x[None].contiguous(), positions, freqs, frame_seqlen=12, width=4)[0]
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("simt", [False, True], ids=["tcgen05", "cuda-core"])
def test_selected_pair_rope_inside_the_low_width_read(simt):
    """A 64-wide reader whose pairs are 32 selected native pairs of a 128-wide head."""
    heads, width, native = 3, 64, 128
    built = build(heads, width, 128, 400, 150, "bf16", 5, 6)
    case, data, segments, positions, frame_seqlen, q = built
    gen = torch.Generator().manual_seed(11)
    pairs = torch.stack([torch.randperm(native // 2, generator=gen)[:width // 2].sort().values
                         for _ in range(heads)])
    indices = torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(heads, width)
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    freqs = oracle.rope_table(1024, native)
    table = attention.RopeTable(freqs, frame_seqlen=frame_seqlen, width=6)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    view = table.view(positions.cuda(), pair_index_of(indices).cuda())
    ops.force_simt(simt)
    try:
        out, lse = ops.attn_codec(
            q.cuda(), hist_k.view(), hist_v.view(), ops_k.decoder.view(heads, width, -1),
            ops_k.bias.view(heads, width), ops_v.decoder.view(heads, width, -1),
            ops_v.bias.view(heads, width), scale=width ** -0.5, status=status, rope=view)
        torch.cuda.synchronize()
    finally:
        ops.force_simt(False)
    assert int(status.item()) == 0
    k_op, v_op = data["k_op"], data["v_op"]
    want, want_lse = oracle.codec_attention(
        q[None], segments["k"], segments["v"], k_decoder=k_op["decoder"], k_mean=k_op["mean"],
        v_decoder=v_op["decoder"], v_mean=v_op["mean"], heads=heads, dtype=torch.bfloat16,
        rope=dict(positions=positions, freqs=freqs, frame_seqlen=frame_seqlen, width=6, indices=indices))
    assert rel_err(out.cpu(), want[0]) <= BF16_REL_TOL
    assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= BF16_REL_TOL


@pytest.mark.parametrize("case", cases.FAST_CASES, ids=lambda c: c.name)
def test_hybrid_attention_with_selected_rope(case):
    """NanoKV-Fast with real positional hooks: the reduced query and the low-width keys are
    rotated with the native pairs each reader group keeps (LingBot's attend loop)."""
    from helpers import F32_REL_TOL
    from nanokv_b200 import codec
    from test_oracle_golden import encode_all
    data = cases.build(case.codec)
    shape = case.codec.shape
    dtype = shape.torch_dtype
    segments = encode_all(case.codec, data)
    frame_seqlen, width = 24, 6
    freqs = oracle.rope_table(1024, shape.head_dim)
    q_positions = torch.arange(5000, 5000 + shape.queries)
    starts = [0]
    for count in case.codec.segments:
        starts.append(starts[-1] + count)
    # oracle inputs (as in the fixture test) plus positions
    low, native = [], []
    for index in range(len(case.codec.segments)):
        seg_k, seg_v = segments["k"][index], segments["v"][index]
        if index < case.low_segments:
            entry = {"positions": torch.arange(starts[index], starts[index + 1]) + 300}
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
    want = oracle.hybrid_attention(q, q, native, low, reader_payload,
                                   rope=dict(freqs=freqs, frame_seqlen=frame_seqlen, width=width,
                                             q_positions=q_positions))[0]
    # product path
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    n_low = case.low_segments
    low_k = history_from_segments(segments["k"][:n_low], joint=shape.joint, rank=shape.rank)
    low_v = history_from_segments(segments["v"][:n_low], joint=shape.joint, rank=shape.rank)
    native_dev = [(k[0].permute(1, 0, 2).contiguous().cuda(), v[0].permute(1, 0, 2).contiguous().cuda())
                  for k, v in native]
    reader = attention.Reader(reader_payload, dtype=dtype)
    table = attention.RopeTable(freqs, frame_seqlen=frame_seqlen, width=width)
    low_positions = torch.cat([entry["positions"] for entry in low]).cuda()
    got = attention.hybrid_attention(
        data["q"].cuda(), data["q"].cuda(), native_dev,
        [{"k": low_k, "v": low_v, "k_mean": ops_k.mean, "v_mean": ops_v.mean, "positions": low_positions}],
        reader, rope=table, q_positions=q_positions.cuda())
    tol = F32_REL_TOL if dtype == torch.float32 else BF16_REL_TOL
    assert rel_err(got.cpu().permute(1, 0, 2), want) <= tol


def test_per_token_multipliers_matrix_game_form():
    """One table row per token (Matrix-Game hands its multipliers over that way): rows through
    nkv_rope_rows against the reference fixture, and the same table inside the fused read."""
    from test_oracle_golden import from_bits, load
    gold, data = load("rope_per_token_bf16"), cases.build_rope_selected()
    multiplier = cases.per_token_multiplier(data)
    table = attention.RopeTable.per_token(multiplier)
    rows = data["value"][0].permute(1, 0, 2).contiguous()
    tokens = rows.shape[0]
    got = table.rotate(rows.cuda(), torch.arange(tokens).cuda(), pair_index_of(data["indices"]).cuda()).cpu()
    want = from_bits(gold["rotated"], torch.bfloat16)[0].permute(1, 0, 2)
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    assert float((got != want).float().mean()) < 0.01
    # inside the read: a 64-wide reader over 128-wide heads, multipliers per history token
    heads, width, native = 2, 64, 128
    built = build(heads, width, 64, 300, 130, "bf16", 5, 6)
    case, bdata, segments, _, _, q = built
    gen = torch.Generator().manual_seed(13)
    angles = (torch.rand(300, native // 2, generator=gen, dtype=torch.float64) - 0.5) * 30.0
    mult = torch.polar(torch.ones_like(angles), angles)
    pairs = torch.stack([torch.randperm(native // 2, generator=gen)[:width // 2].sort().values
                         for _ in range(heads)])
    indices = torch.stack((2 * pairs, 2 * pairs + 1), dim=2).reshape(heads, width)
    ops_k, ops_v = device_operator(bdata["k_op"]), device_operator(bdata["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    view = attention.RopeTable.per_token(mult).view(torch.arange(300).cuda(), pair_index_of(indices).cuda())
    out, lse = ops.attn_codec(
        q.cuda(), hist_k.view(), hist_v.view(), ops_k.decoder.view(heads, width, -1),
        ops_k.bias.view(heads, width), ops_v.decoder.view(heads, width, -1),
        ops_v.bias.view(heads, width), scale=width ** -0.5, rope=view)
    k_op, v_op = bdata["k_op"], bdata["v_op"]
    keys = torch.cat([oracle.decode_rows(s, decoder=k_op["decoder"], mean=k_op["mean"], dtype=torch.bfloat16)
                      for s in segments["k"]], 1).reshape(1, -1, heads, width).permute(0, 2, 1, 3)
    values = torch.cat([oracle.decode_rows(s, decoder=v_op["decoder"], mean=v_op["mean"], dtype=torch.bfloat16)
                        for s in segments["v"]], 1).reshape(1, -1, heads, width).permute(0, 2, 1, 3)
    keys = oracle.rope_per_token(keys, mult, indices)
    want, want_lse = oracle.attention_lse(q.permute(1, 0, 2)[None], keys, values, scale=width ** -0.5)
    assert rel_err(out.cpu(), want[0].permute(1, 0, 2)) <= BF16_REL_TOL
    assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= BF16_REL_TOL
