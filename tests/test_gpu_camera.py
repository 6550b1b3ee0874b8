"""PRoPE camera transform on the GPU: explicit rows against the reference fixture, and inside the
fused read (keys and values) against the oracle."""
import pytest
import torch

import cases
from helpers import BF16_REL_TOL, F32_REL_TOL, device_operator, history_from_segments, rel_err
from nanokv_b200 import attention, ops
from oracle import nkv_oracle as oracle
from test_gpu_rope import build
from test_oracle_golden import from_bits, load

pytestmark = pytest.mark.gpu


def test_camera_rows_against_the_reference_fixture():
    gold, data = load("camera_bf16"), cases.build_camera()
    rows = data["value"][0].permute(1, 0, 2).contiguous()                  # [S, h, e]
    view = attention.camera_view(data["matrix"], data["indices"], rows.shape[0])
    got = ops.camera_rows(rows.cuda(), view).cpu()
    want = from_bits(gold["transformed"], torch.bfloat16)[0].permute(1, 0, 2)
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    assert float((got != want).float().mean()) < 0.01
    with pytest.raises(ValueError):
        attention.camera_view(data["matrix"], data["indices"], rows.shape[0] + 1)
    with pytest.raises(ValueError):
        attention.camera_index(data["indices"] + 1)


@pytest.mark.parametrize("heads,head_dim,rank,history,queries,frames,dtype_name", [
    (2, 128, 128, 520, 200, 4, "bf16"),
    (3, 64, 64, 300, 130, 5, "bf16"),
    (2, 64, 64, 260, 70, 2, "f32"),
])
@pytest.mark.parametrize("simt", [False, True], ids=["tcgen05", "cuda-core"])
def test_camera_inside_the_read(heads, head_dim, rank, history, queries, frames, dtype_name, simt):
    if dtype_name == "f32" and not simt:
        pytest.skip("fp32 always runs on the CUDA-core kernel")
    case, data, segments, positions, frame_seqlen, q = build(heads, head_dim, rank, history, queries,
                                                            dtype_name, 5, 4)
    dtype = case.shape.torch_dtype
    gen = torch.Generator().manual_seed(17)
    native = 128
    blocks = torch.stack([torch.randperm(native // 8, generator=gen)[:head_dim // 8].sort().values
                          for _ in range(heads)])
    indices = (blocks[:, :, None] * 8 + torch.arange(8)).reshape(heads, head_dim)
    m_k = torch.randn(1, frames, 4, 4, 4, generator=gen)
    m_v = torch.randn(1, frames, 4, 4, 4, generator=gen)
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    hist_k = history_from_segments(segments["k"], joint=case.shape.joint, rank=case.shape.rank)
    hist_v = history_from_segments(segments["v"], joint=case.shape.joint, rank=case.shape.rank)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.force_simt(simt)
    try:
        out, lse = ops.attn_codec(
            q.cuda(), hist_k.view(), hist_v.view(), ops_k.decoder.view(heads, head_dim, -1),
            ops_k.bias.view(heads, head_dim), ops_v.decoder.view(heads, head_dim, -1),
            ops_v.bias.view(heads, head_dim), scale=head_dim ** -0.5, status=status,
            camera_k=attention.camera_view(m_k, indices, history),
            camera_v=attention.camera_view(m_v, indices, history))
        torch.cuda.synchronize()
    finally:
        ops.force_simt(False)
    assert int(status.item()) == 0
    k_op, v_op = data["k_op"], data["v_op"]
    keys = torch.cat([oracle.decode_rows(s, decoder=k_op["decoder"], mean=k_op["mean"], dtype=dtype)
                      for s in segments["k"]], 1).reshape(1, -1, heads, head_dim).permute(0, 2, 1, 3)
    values = torch.cat([oracle.decode_rows(s, decoder=v_op["decoder"], mean=v_op["mean"], dtype=dtype)
                        for s in segments["v"]], 1).reshape(1, -1, heads, head_dim).permute(0, 2, 1, 3)
    keys = oracle.camera_selected(keys, m_k, indices)
    values = oracle.camera_selected(values, m_v, indices)
    want, want_lse = oracle.attention_lse(q.permute(1, 0, 2)[None].to(dtype), keys, values,
                                          scale=head_dim ** -0.5)
    tol = F32_REL_TOL if dtype == torch.float32 else BF16_REL_TOL
    assert rel_err(out.cpu(), want[0].permute(1, 0, 2)) <= tol
    assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= tol * max(1.0, float(want_lse.abs().max()))


def test_hybrid_attention_with_camera_hooks():
    """Matrix-Game's PRoPE around the low-width read: query (P^T), keys / values (P^-1, inside the
    kernel) and the low-width output (P)."""
    from test_oracle_golden import encode_all
    case = cases.FAST_CASES[1]                                   # bf16
    data = cases.build(case.codec)
    shape = case.codec.shape
    dtype = shape.torch_dtype
    segments = encode_all(case.codec, data)
    gen = torch.Generator().manual_seed(29)
    q_frames, low_frames = 2, 4
    cam = {"q": torch.randn(1, q_frames, 4, 4, 4, generator=gen) * 0.5,
           "out": torch.randn(1, q_frames, 4, 4, 4, generator=gen) * 0.5}
    low, native = [], []
    for index in range(len(case.codec.segments)):
        seg_k, seg_v = segments["k"][index], segments["v"][index]
        if index < case.low_segments:
            entry = {"camera": torch.randn(1, low_frames, 4, 4, 4, generator=gen) * 0.5}
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
    want = oracle.hybrid_attention(q, q, native, low, reader_payload, camera=cam)[0]
    plain = oracle.hybrid_attention(q, q, native, low, reader_payload)[0]
    ops_k, ops_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    native_dev = [(k[0].permute(1, 0, 2).contiguous().cuda(), v[0].permute(1, 0, 2).contiguous().cuda())
                  for k, v in native]
    reader = attention.Reader(reader_payload, dtype=dtype)
    low_dev = []
    for index, entry in enumerate(low):
        low_dev.append({"k": history_from_segments([segments["k"][index]], joint=shape.joint, rank=shape.rank),
                        "v": history_from_segments([segments["v"][index]], joint=shape.joint, rank=shape.rank),
                        "k_mean": ops_k.mean, "v_mean": ops_v.mean, "camera": entry["camera"]})
    got = attention.hybrid_attention(data["q"].cuda(), data["q"].cuda(), native_dev, low_dev, reader,
                                     camera=cam)
    assert rel_err(got.cpu().permute(1, 0, 2), want) <= BF16_REL_TOL
    assert rel_err(plain, want) > 2 * BF16_REL_TOL, "the transform must matter in this case"
