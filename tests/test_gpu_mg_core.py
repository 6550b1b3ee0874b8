"""The Matrix-Game codec-native attention interface (names, argument order and [1,H,tokens,D]
layout of the reference's codec_native/core.py) on the GPU, against fixtures the unmodified
reference produced."""
import os

import pytest
import torch

import cases
from helpers import BF16_REL_TOL, rel_err
from nanokv_b200 import mg_codec, mg_core
from oracle import nkv_oracle as oracle
from test_oracle_golden import from_bits, load

pytestmark = pytest.mark.gpu


def build_inputs(case, *, masked=False):
    """What the reference's fixture run builds, through this library's interface modules."""
    data = cases.build(case.codec)
    shape = case.codec.shape
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.codec.iters)
    dtype, heads, dim = shape.torch_dtype, shape.heads, shape.head_dim
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        mg_codec.register_operator(kind, case.codec.layer, mean=op["mean"], encoder=op["encoder"],
                                   decoder=op["decoder"])
    payloads = {kind: [mg_codec.encode_tensor(kind, case.codec.layer, chunk[None].cuda())
                       for chunk in data[f"{kind}_chunks"]] for kind in ("k", "v")}
    n_low = case.low_segments
    low = mg_codec.direct_latent_pair_segments(
        {"codec": mg_codec.SEGMENTS, "segments": payloads["k"][:n_low]},
        {"codec": mg_codec.SEGMENTS, "segments": payloads["v"][:n_low]}, device="cuda")
    native = []
    for pk, pv in zip(payloads["k"][n_low:], payloads["v"][n_low:]):
        key = mg_codec.decode_tensor(pk, dtype=dtype, device="cuda")
        value = mg_codec.decode_tensor(pv, dtype=dtype, device="cuda")
        native.append((key.reshape(1, -1, heads, dim).permute(0, 2, 1, 3),
                       value.reshape(1, -1, heads, dim).permute(0, 2, 1, 3), None))
    if masked:
        groups, visible = cases.build_visibility(case)
        full = [mask[groups][None, None].cuda() for mask in visible]           # [1, 1, Q, tokens]
        for segment, mask in zip(low, full[:n_low]):
            segment["mask"] = mask
        native = [(key, value, mask) for (key, value, _), mask in zip(native, full[n_low:])]
    reader = mg_core.ReaderLayer(cases.build_reader(case, data), dtype=dtype)
    q = data["q"][None].permute(0, 2, 1, 3).contiguous().cuda()
    return q, native, low, reader


@pytest.mark.parametrize("case", [cases.FAST_CASES[1]], ids=lambda c: c.name)
def test_hybrid_attention_identity_hooks(case):
    gold = load(case.name)
    q, native, low, reader = build_inputs(case)
    want = from_bits(gold["hybrid"], torch.bfloat16)
    # the reference's own call: identity lambdas are arbitrary callables here -> the unfused route
    loose = mg_core.hybrid_attention(
        q, q, native, low, reader, query_position=lambda value, group: value,
        kv_position=lambda kk, vv, segment, group: (kk, vv))
    assert loose.shape == q.shape
    assert rel_err(loose[0].cpu(), want) <= BF16_REL_TOL
    fused = mg_core.hybrid_attention(q, q, native, low, reader)
    assert rel_err(fused[0].cpu(), want) <= BF16_REL_TOL


def test_hybrid_attention_with_masks_in_the_reference_form():
    case = cases.FAST_CASES[1]
    gold = load("fast_masked_bf16")
    q, native, low, reader = build_inputs(case, masked=True)
    want = from_bits(gold["hybrid"], torch.bfloat16)
    fused = mg_core.hybrid_attention(q, q, native, low, reader)
    assert rel_err(fused[0].cpu(), want) <= BF16_REL_TOL
    loose = mg_core.hybrid_attention(
        q, q, native, low, reader, query_position=lambda value, group: value,
        kv_position=lambda kk, vv, segment, group: (kk, vv))
    assert rel_err(loose[0].cpu(), want) <= BF16_REL_TOL


def test_hybrid_attention_with_the_matrix_game_hooks_against_the_reference_fixture():
    """rope_selected on the reduced query and the low keys, camera_selected on query, keys, values
    and output: as data (fused, the kernel rotates and transforms its tiles) and as callables."""
    case = cases.FAST_CASES[1]
    gold = load("fast_hooks_bf16")
    q, native, low, reader = build_inputs(case)
    extra = cases.build_hooks(case)
    for segment, more in zip(low, extra["segments"]):
        segment.update({name: value.cuda() for name, value in more.items()})
    want = from_bits(gold["hybrid"], torch.bfloat16)
    hooks = mg_core.PositionHooks(q_multiplier=extra["q_multiplier"].cuda(), q_camera=extra["q_camera"].cuda(),
                                  out_camera=extra["out_camera"].cuda())
    fused = mg_core.hybrid_attention(q, q, native, low, reader, query_position=hooks.query_position,
                                     kv_position=hooks.kv_position, output_position=hooks.output_position)
    assert rel_err(fused[0].cpu(), want) <= BF16_REL_TOL

    # the call site's own closures (MGC/mg35.py:318-347 shape): arbitrary callables
    def query_position(value, group):
        value = mg_core.rope_selected(value, extra["q_multiplier"].cuda(), group.indices)
        return mg_core.camera_selected(value, extra["q_camera"].cuda(), group.indices)

    def kv_position(kk, vv, segment, group):
        kk = mg_core.rope_selected(kk, segment["freqs"], group.indices)
        return (mg_core.camera_selected(kk, segment["camera"], group.indices),
                mg_core.camera_selected(vv, segment["camera"], group.v_indices))

    def output_position(value, group):
        return mg_core.camera_selected(value, extra["out_camera"].cuda(), group.v_indices)

    loose = mg_core.hybrid_attention(q, q, native, low, reader, query_position=query_position,
                                     kv_position=kv_position, output_position=output_position)
    assert rel_err(loose[0].cpu(), want) <= BF16_REL_TOL
    # rotation alone
    rope_only = mg_core.PositionHooks(q_multiplier=extra["q_multiplier"].cuda())
    got = mg_core.hybrid_attention(q, q, native, low, reader, query_position=rope_only.query_position,
                                   kv_position=rope_only.kv_position)
    want_rope = from_bits(gold["rope_only"], torch.bfloat16)
    assert rel_err(got[0].cpu(), want_rope) <= BF16_REL_TOL
    assert rel_err(want_rope, want) > 2 * BF16_REL_TOL, "the camera transform must matter in this case"


def test_attention_lse_and_merge_in_the_reference_layout():
    gen = torch.Generator().manual_seed(77)
    q = torch.randn(1, 3, 90, 128, generator=gen).to(torch.bfloat16)
    k = torch.randn(1, 3, 400, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(1, 3, 400, 128, generator=gen).to(torch.bfloat16)
    want, want_lse = oracle.attention_lse(q, k, v)
    out, lse = mg_core.attention_lse(q.cuda(), k.cuda(), v.cuda())
    assert out.shape == want.shape and lse.shape == want_lse.shape
    assert rel_err(out.cpu(), want) <= BF16_REL_TOL and float((lse.cpu() - want_lse).abs().max()) <= 2e-2
    # row-constant mask, per-query mask, empty keys
    shared = torch.rand(1, 1, 1, 400, generator=gen) < 0.6
    want, want_lse = oracle.attention_lse(q, k, v, shared)
    out, lse = mg_core.attention_lse(q.cuda(), k.cuda(), v.cuda(), shared.cuda(), scale=128 ** -0.5)
    assert rel_err(out.cpu(), want) <= BF16_REL_TOL and float((lse.cpu() - want_lse).abs().max()) <= 2e-2
    groups = torch.arange(90) * 3 // 90
    rows = torch.rand(3, 400, generator=gen) < 0.5
    rows[:, 0] = True
    per_query = rows[groups][None, None]
    want, want_lse = oracle.attention_lse(q, k, v, per_query)
    out, lse = mg_core.attention_lse(q.cuda(), k.cuda(), v.cuda(), per_query.cuda())
    assert rel_err(out.cpu(), want) <= BF16_REL_TOL and float((lse.cpu() - want_lse).abs().max()) <= 2e-2
    out2, lse2 = mg_core.attention_grouped_mask(q.cuda(), k.cuda(), v.cuda(), per_query.cuda(), groups.cuda(),
                                                scale=128 ** -0.5)
    assert torch.equal(out2, out) and torch.equal(lse2, lse)
    empty, empty_lse = mg_core.attention_lse(q.cuda(), k[:, :, :0].cuda(), v[:, :, :0].cuda())
    assert float(empty.abs().max()) == 0 and bool(torch.isinf(empty_lse).all())
    with pytest.raises(ValueError):
        mg_core.attention_lse(q.cuda(), k.cuda(), v.cuda(), shared.float().cuda())
    gold = load("merge_edge")
    a, la, b, lb = (t.cuda() for t in cases.build_merge())
    merged, merged_lse = mg_core.merge(a, la, b, lb)
    assert rel_err(merged.cpu(), from_bits(gold["out"], torch.bfloat16)) <= 2.0 ** -7


def test_position_functions_against_the_reference_fixtures():
    data = cases.build_rope_selected()
    multiplier = cases.per_token_multiplier(data)
    got = mg_core.rope_selected(data["value"].cuda(), multiplier.cuda(), data["indices"].cuda()).cpu()
    want = from_bits(load("rope_per_token_bf16")["rotated"], torch.bfloat16)
    assert got.shape == want.shape
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    with pytest.raises(ValueError):
        mg_core.rope_selected(data["value"].cuda(), multiplier.cuda(), (data["indices"] + 1).cuda())
    cam = cases.build_camera()
    got = mg_core.camera_selected(cam["value"].cuda(), cam["matrix"].cuda(), cam["indices"].cuda()).cpu()
    want = from_bits(load("camera_bf16")["transformed"], torch.bfloat16)
    assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -6 * float(want.float().abs().max())
    with pytest.raises(ValueError):
        mg_core.camera_selected(cam["value"].cuda(), cam["matrix"].cuda(), cam["indices"].cuda(), layout="split")
