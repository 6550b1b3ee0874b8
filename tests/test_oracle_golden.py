"""The CPU oracle against outputs of the unmodified reference (tests/golden/*.npz)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from nanokv_b200.synthetic import checksum
from oracle import nkv_oracle as oracle

GOLDEN = Path(__file__).parent / "golden"


def load(name):
    return np.load(GOLDEN / f"{name}.npz")


def from_bits(array, dtype):
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    return tensor.view(dtype) if dtype in (torch.bfloat16, torch.float16) else tensor


def encode_all(case, data, *, lingbot=False):
    """Oracle encode of every segment with the reference flavour's parameters."""
    segments = {"k": [], "v": []}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        for chunk in data[f"{kind}_chunks"]:
            if lingbot:
                seed = 20260826 + case.layer * 17 + (kind == "v")
                flavour = dict(eps=1e-12, in_coeff_dtype=False)
            else:
                seed = 20260804 + case.layer
                flavour = dict(eps=oracle.F32_EPS, in_coeff_dtype=True)
            segments[kind].append(oracle.encode_rows(
                chunk[None], encoder=op["encoder"], mean=op["mean"],
                clusters=case.shape.centers, iters=case.iters, seed=seed, **flavour))
    return segments


def check_segments(gold, segments):
    for kind in ("k", "v"):
        for index, seg in enumerate(segments[kind]):
            assert np.array_equal(gold[f"{kind}{index}_ids"].reshape(-1),
                                  seg["ids"].reshape(-1).numpy()), "centre ids"
            assert np.array_equal(gold[f"{kind}{index}_packed"], seg["packed"].numpy()), "codes"
            assert np.array_equal(gold[f"{kind}{index}_scale"].reshape(-1),
                                  seg["scale"].view(torch.int16).reshape(-1).numpy()), "scales"
            assert np.array_equal(gold[f"{kind}{index}_centers"],
                                  seg["centers"].view(torch.int16).numpy()), "centres"


@pytest.mark.parametrize("case", cases.MG_CASES, ids=lambda c: c.name)
def test_mg_codec_and_attention(case):
    torch.set_num_threads(1)
    gold = load(case.name)
    data = cases.build(case)
    for kind in ("k", "v"):
        digests = [checksum(t) for t in data[f"{kind}_chunks"]]
        assert digests == list(gold[f"{kind}_input_digest"]), "seeded inputs drifted"
    segments = encode_all(case, data)
    check_segments(gold, segments)
    dtype = case.shape.torch_dtype
    heads = case.shape.heads
    k_op, v_op = data["k_op"], data["v_op"]
    for kind, op in (("k", k_op), ("v", v_op)):
        decoded = torch.cat([oracle.decode_rows(s, decoder=op["decoder"], mean=op["mean"],
                                                dtype=dtype) for s in segments[kind]], 1)
        assert checksum(decoded) == int(gold[f"{kind}_decoded_digest"][0]), "decoded rows"
    out, lse = oracle.codec_attention(
        data["q"][None], segments["k"], segments["v"], k_decoder=k_op["decoder"],
        k_mean=k_op["mean"], v_decoder=v_op["decoder"], v_mean=v_op["mean"], heads=heads,
        dtype=dtype)
    out_bhqd = out.permute(0, 2, 1, 3).contiguous()
    assert checksum(out_bhqd) == int(gold["attn_digest"][0]), "attention output"
    assert np.array_equal(gold["lse"], lse[0].numpy())


@pytest.mark.parametrize("case", cases.LINGBOT_CASES, ids=lambda c: c.name)
def test_lingbot_codec(case):
    torch.set_num_threads(1)
    gold = load(case.name)
    data = cases.build(case)
    segments = encode_all(case, data, lingbot=True)
    check_segments(gold, segments)
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        decoded = oracle.decode_rows(segments[kind][0], decoder=op["decoder"], mean=op["mean"],
                                     dtype=torch.bfloat16)
        assert np.array_equal(gold[f"{kind}_decoded"],
                              decoded.reshape(-1, case.shape.joint).view(torch.int16).numpy())


@pytest.mark.parametrize("case", cases.FAST_CASES, ids=lambda c: c.name)
def test_hybrid_attention(case, masked=False):
    torch.set_num_threads(1)
    gold = load("fast_masked_bf16" if masked else case.name)
    data = cases.build(case.codec)
    shape = case.codec.shape
    dtype = shape.torch_dtype
    segments = encode_all(case.codec, data)
    low, native = [], []
    for index in range(len(case.codec.segments)):
        seg_k, seg_v = segments["k"][index], segments["v"][index]
        if index < case.low_segments:
            entry = {}
            for kind, seg in (("k", seg_k), ("v", seg_v)):
                latent = oracle.dequantize_rows(seg["codes"], seg["scale"])[None]
                entry[kind] = (latent, seg["centers"].float(), seg["ids"].long(),
                               data[f"{kind}_op"]["mean"])
            low.append(entry)
        else:
            pair = []
            for kind, seg in (("k", seg_k), ("v", seg_v)):
                op = data[f"{kind}_op"]
                rows = oracle.decode_rows(seg, decoder=op["decoder"], mean=op["mean"], dtype=dtype)
                pair.append(rows.reshape(1, -1, shape.heads, shape.head_dim).permute(0, 2, 1, 3))
            native.append(tuple(pair))
    if masked:
        groups, visible = cases.build_visibility(case)
        full = [mask[groups][None, None] for mask in visible]
        for entry, mask in zip(low, full):
            entry["mask"] = mask
        native = [pair + (mask,) for pair, mask in zip(native, full[case.low_segments:])]
    reader = cases.build_reader(case, data)
    q = data["q"][None].permute(0, 2, 1, 3).contiguous()
    result = oracle.hybrid_attention(q, q, native, low, reader)
    want = from_bits(gold["hybrid"], dtype)
    assert torch.equal(result[0], want)


def test_hybrid_attention_with_visibility_masks():
    """Boolean visibility per query group on every segment, against the reference's masked read."""
    test_hybrid_attention(cases.FAST_CASES[1], masked=True)


def test_merge_edge_cases():
    gold = load("merge_edge")
    out, lse = oracle.merge(*cases.build_merge())
    assert np.array_equal(gold["out"], out.view(torch.int16).numpy())
    assert np.array_equal(gold["lse"], lse.numpy(), equal_nan=True)


def test_pack_roundtrip_and_nibble_order():
    codes = torch.tensor([[-7, 7, 0, 3], [1, -1, 6, -6]], dtype=torch.int8)
    packed, count = oracle.pack_int4(codes)
    assert packed.tolist() == [0 | (14 << 4), 7 | (10 << 4), 8 | (6 << 4), 13 | (1 << 4)]
    assert torch.equal(oracle.unpack_int4(packed, count, codes.shape), codes)


@pytest.mark.parametrize("case", cases.ROPE_CASES, ids=lambda c: c.name)
def test_rope_by_positions(case):
    gold = load(case.name)
    data = cases.build_rope(case)
    assert int(gold["key_digest"][0]) == checksum(data["key"]), "input generator drifted"
    freqs = oracle.rope_table(1024, case.head_dim)
    assert np.array_equal(gold["freqs_head"], torch.view_as_real(freqs[:64]).numpy()), "rotation table"
    assert int(gold["freqs_digest"][0]) == checksum(torch.view_as_real(freqs).contiguous())
    got = oracle.rope_by_positions(data["key"], data["positions"], freqs,
                                   frame_seqlen=data["frame_seqlen"], width=case.width)
    want = from_bits(gold["rotated"], case.dtype)
    assert torch.equal(got.view(torch.int16) if case.dtype == torch.bfloat16 else got, 
                       want.view(torch.int16) if case.dtype == torch.bfloat16 else want)


@pytest.mark.parametrize("name,group", [("per_row", 0), ("group64", 64)])
def test_int8_operator_storage(name, group):
    gold = load("int8_operator")
    weight = cases.build_int8_weight()
    assert int(gold["weight_digest"][0]) == checksum(weight), "input generator drifted"
    codes, scale, group_size = oracle.pack_int8_weight(weight, group)
    assert np.array_equal(gold[f"{name}_qweight"], codes.numpy())
    assert np.array_equal(gold[f"{name}_scale"], scale.view(torch.int16).numpy())
    dense = oracle.unpack_int8_weight(codes, scale, group_size)
    assert np.array_equal(gold[f"{name}_dense"], dense.view(torch.int16).numpy())


def test_rope_selected_pairs():
    gold = load("rope_selected_bf16")
    data = cases.build_rope_selected()
    assert int(gold["value_digest"][0]) == checksum(data["value"]), "input generator drifted"
    assert np.array_equal(gold["indices"], data["indices"].numpy())
    freqs = oracle.rope_table(1024, data["native_dim"])
    got = oracle.rope_selected(data["value"], data["positions"], freqs, frame_seqlen=data["frame_seqlen"],
                               width=int(data["grid_sizes"][0, 2]), indices=data["indices"])
    assert torch.equal(got.view(torch.int16), from_bits(gold["rotated"], torch.bfloat16).view(torch.int16))


def test_compressed_value_mean():
    gold = load("value_mean_lb_bf16")
    case = cases.ROLLING
    data = cases.build(case)
    assert int(gold["input_digest"][0]) == checksum(torch.cat(data["v_chunks"])), "input generator drifted"
    segments = encode_all(case, data, lingbot=True)["v"]
    low = []
    for index, seg in enumerate(segments):
        lo, hi = cases.value_mean_interval(case, index)
        latent = oracle.dequantize_rows(seg["codes"], seg["scale"])[None][:, lo:hi]
        low.append({"v": (latent, seg["centers"][None] if seg["centers"].dim() == 2 else seg["centers"],
                          seg["ids"].long().reshape(1, -1)[:, lo:hi], data["v_op"]["mean"])})
    got = oracle.compressed_value_mean(low, decoder=data["v_op"]["decoder"], heads=case.shape.heads,
                                       native_dim=case.shape.head_dim)
    assert np.array_equal(gold["value_mean"], got.numpy())


def test_rope_per_token_multipliers():
    gold = load("rope_per_token_bf16")
    data = cases.build_rope_selected()
    assert int(gold["value_digest"][0]) == checksum(data["value"]), "input generator drifted"
    got = oracle.rope_per_token(data["value"], cases.per_token_multiplier(data), data["indices"])
    assert torch.equal(got.view(torch.int16), from_bits(gold["rotated"], torch.bfloat16).view(torch.int16))


def test_camera_selected():
    gold = load("camera_bf16")
    data = cases.build_camera()
    assert int(gold["value_digest"][0]) == checksum(data["value"]), "input generator drifted"
    got = oracle.camera_selected(data["value"], data["matrix"], data["indices"])
    assert torch.equal(got.view(torch.int16), from_bits(gold["transformed"], torch.bfloat16).view(torch.int16))


@pytest.mark.parametrize("name,group", [("per_row", 0), ("group64", 64)])
def test_mg_operator_int8_packing_matches_the_reference(name, group, monkeypatch):
    """mg_codec._pack_int8 (what an operator read from the reference's artefact files is stored as in
    its default weight mode) against the bits the reference's own packer produced."""
    from nanokv_b200 import mg_codec
    gold = load("int8_operator")
    monkeypatch.setenv("MG35_KVCODEC_INT8_WEIGHT_GROUP_SIZE", str(group))
    packed = mg_codec._pack_int8(cases.build_int8_weight())
    assert np.array_equal(packed["qweight"].numpy(), gold[f"{name}_qweight"])
    assert np.array_equal(packed["scale"].view(torch.int16).numpy(), gold[f"{name}_scale"])


def test_hy_codec_entry_points():
    """The oracle's restatement of HY-WorldPlay's compress / decompress against the reference's own
    payload and decoded rows (bit-exact: same arithmetic, same CPU library)."""
    case = cases.HY_CODEC
    gold = load(case.name)
    data = cases.build(case)
    shape = case.shape
    for name in ("k", "v"):
        op = data[f"{name}_op"]
        rows = data[f"{name}_chunks"][0]
        x = rows.reshape(1, -1, shape.heads, shape.head_dim).permute(0, 2, 1, 3).contiguous()
        assert int(gold[f"{name}_digest"][0]) == checksum(x), "input generator drifted from the fixture"
        seg = oracle.hy_compress(x, encoder=op["encoder"], mean=op["mean"], clusters=shape.centers,
                                 iters=case.iters, layer=case.layer)
        assert np.array_equal(seg["ids"].numpy(), gold[f"{name}_ids"])
        assert torch.equal(seg["centers"], from_bits(gold[f"{name}_centers"], torch.bfloat16))
        assert np.array_equal(seg["packed"].numpy(), gold[f"{name}_packed"])
        assert torch.equal(seg["scale"].reshape(1, -1, 1), from_bits(gold[f"{name}_scale"], torch.bfloat16))
        out = oracle.hy_decompress(seg, decoder=op["decoder"], mean=op["mean"], heads=shape.heads,
                                   dtype=torch.bfloat16)
        assert torch.equal(out[:, :, :48], from_bits(gold[f"{name}_decoded_bf16"], torch.bfloat16))
        out32 = oracle.hy_decompress(seg, decoder=op["decoder"], mean=op["mean"], heads=shape.heads,
                                     dtype=torch.float32)
        assert torch.equal(out32[:, :, :16], torch.from_numpy(gold[f"{name}_decoded_f32"]))

