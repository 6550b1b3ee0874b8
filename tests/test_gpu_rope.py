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
