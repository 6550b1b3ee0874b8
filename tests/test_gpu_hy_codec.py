"""HY-WorldPlay's codec entry points (names, layouts and payload keys of the reference's
hyvideo/models/transformers/modules/kv_codecs.py) on the GPU, against a fixture the unmodified
reference produced."""
import os

import numpy as np
import pytest
import torch

import cases
from nanokv_b200 import hy_codec
from test_oracle_golden import from_bits, load

pytestmark = pytest.mark.gpu


def environment(case):
    for name in list(os.environ):
        if name.startswith("HY_KV_CODEC"):
            os.environ.pop(name)
    os.environ.update({
        "HY_KV_CODEC_ENABLE": "1", "HY_KV_CODEC_MODE": "global_pca", "HY_KV_CODEC_COEFF_QUANT": "int4",
        "HY_KV_CODEC_GLOBAL_PCA_RANK": str(case.shape.rank),
        "HY_KV_CODEC_SEMANTIC_SMOOTH_K": "1", "HY_KV_CODEC_SEMANTIC_SMOOTH_V": "1",
        "HY_KV_CODEC_SEMANTIC_CLUSTERS": str(case.shape.centers), "HY_KV_CODEC_SEMANTIC_ITERS": str(case.iters),
    })


def inputs(case, name, data):
    shape = case.shape
    op = data[f"{name}_op"]
    hy_codec.register_operator(name, case.layer, mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
    rows = data[f"{name}_chunks"][0]
    return rows.reshape(1, -1, shape.heads, shape.head_dim).permute(0, 2, 1, 3).contiguous().cuda()


def test_compress_matches_the_reference_payload():
    case = cases.HY_CODEC
    gold = load(case.name)
    environment(case)
    data = cases.build(case)
    flips = 0
    for name in ("k", "v"):
        x = inputs(case, name, data)
        payload, stats = hy_codec.compress_kv_tensor(x, case.layer, name)
        assert payload["codec"] == "global_pca" and payload["coeff_quant"] == "int4" and payload["kv_codec"]
        assert payload["shape"] == tuple(x.shape) and payload["semantic_smooth"]
        assert payload["latent_shape"] == (1, x.shape[2], case.shape.rank)
        assert tuple(payload["latent_scale"].shape) == (1, x.shape[2], 1)
        assert tuple(payload["semantic_centers"].shape) == (1, case.shape.centers, 2048)
        assert np.array_equal(payload["semantic_ids"].cpu().numpy(), gold[f"{name}_ids"])
        assert torch.equal(payload["semantic_centers"].cpu(), from_bits(gold[f"{name}_centers"], torch.bfloat16))
        assert torch.equal(payload["latent_scale"].cpu(), from_bits(gold[f"{name}_scale"], torch.bfloat16))
        got = hy_codec.unpack_quantized_codes(payload["latent_int8"].cpu(), 4, payload["latent_numel"])
        want = hy_codec.unpack_quantized_codes(torch.from_numpy(gold[f"{name}_packed"]), 4, payload["latent_numel"])
        delta = (got.int() - want.int()).abs()
        assert int(delta.max()) <= 1, "a code may move by one step at an exact rounding tie only"
        flips += int(delta.sum())
        assert int(stats["actual_bytes"]) == int(gold[f"{name}_bytes"][0])
    print(f"code flips against the reference: {flips}")
    assert flips <= 4


def test_decompress_of_the_reference_payload():
    case = cases.HY_CODEC
    gold = load(case.name)
    environment(case)
    data = cases.build(case)
    shape = case.shape
    for name in ("k", "v"):
        x = inputs(case, name, data)
        sequence = x.shape[2]
        payload = {
            "kv_codec": True, "codec": "global_pca", "coeff_quant": "int4", "rank": shape.rank,
            "shape": tuple(x.shape), "layer_idx": case.layer, "tensor_name": name, "semantic_smooth": True,
            "semantic_centers": from_bits(gold[f"{name}_centers"], torch.bfloat16),
            "semantic_ids": torch.from_numpy(gold[f"{name}_ids"]),
            "latent_int8": torch.from_numpy(gold[f"{name}_packed"]),
            "latent_scale": from_bits(gold[f"{name}_scale"], torch.bfloat16),
            "latent_shape": (1, sequence, shape.rank), "latent_numel": sequence * shape.rank,
        }
        out = hy_codec.decompress_kv_tensor(payload, torch.bfloat16, "cuda")
        want = from_bits(gold[f"{name}_decoded_bf16"], torch.bfloat16)
        assert out.shape == x.shape and out.dtype == torch.bfloat16     # the fixture keeps the first 48 tokens
        # the decoder GEMM accumulates in another order than the CPU BLAS of the fixture run: bf16 results
        # may differ by one rounding step of the larger operand
        err = (out[:, :, :48].cpu().float() - want.float()).abs().max() / want.float().abs().max()
        assert float(err) <= 2.0 ** -7
        out32 = hy_codec.decompress_kv_tensor(payload, torch.float32, "cuda")
        want32 = torch.from_numpy(gold[f"{name}_decoded_f32"])
        err32 = (out32[:, :, :16].cpu() - want32).abs().max() / want32.abs().max()
        assert out32.dtype == torch.float32 and float(err32) <= 2.0 ** -7
        # fp32 rows carry the centre in full precision: they are not the bf16 rows widened
        assert not torch.equal(out32, out.float())
        assert float((out32 - out.float()).abs().max() / out.float().abs().max()) <= 2.0 ** -8
        # this module's own payload of the same input decodes to the same rows (up to the few codes that
        # may differ by one step at an exact rounding tie)
        back = hy_codec.decompress_kv_tensor(hy_codec.compress_kv_tensor(x, case.layer, name)[0], x.dtype, "cuda")
        assert float((back.float() - out.float()).abs().mean() / out.float().abs().mean()) < 1e-3


def test_layer_cache_entry_point_and_errors():
    case = cases.HY_CODEC
    environment(case)
    data = cases.build(case)
    cache = {"k_vision": inputs(case, "k", data), "v_vision": inputs(case, "v", data), "other": 3}
    shapes = {key: tuple(cache[key].shape) for key in ("k_vision", "v_vision")}
    hy_codec.apply_codec_to_layer_cache(cache, case.layer)
    for key in ("k_vision", "v_vision"):
        assert isinstance(cache[key], dict) and cache[key]["shape"] == shapes[key]
    assert cache["other"] == 3
    again = hy_codec.apply_codec_to_layer_cache(cache, case.layer)   # payloads are left alone
    assert again is cache and isinstance(cache["k_vision"], dict)
    plain = torch.zeros(1, 16, 8, 128, device="cuda")
    assert hy_codec.decompress_kv_tensor(plain) is plain
    with pytest.raises(ValueError):
        hy_codec.compress_kv_tensor(torch.zeros(1, 8, 64, 128, device="cuda"), case.layer, "k")   # H*D != 2048
    with pytest.raises(ValueError):
        hy_codec.compress_kv_tensor(torch.zeros(16, 64, 128, device="cuda"), case.layer, "k")
    with pytest.raises(KeyError):
        hy_codec.compress_kv_tensor(cache_input := torch.zeros(1, 16, 64, 128, device="cuda"), 99, "k")
    os.environ["HY_KV_CODEC_MODE"] = "bogus"
    with pytest.raises(ValueError):
        hy_codec.mode()
    os.environ["HY_KV_CODEC_MODE"] = "int8"
    with pytest.raises(NotImplementedError):
        hy_codec.compress_kv_tensor(cache_input, case.layer, "k")
    os.environ["HY_KV_CODEC_ENABLE"] = "0"
    untouched = {"k_vision": plain}
    assert hy_codec.apply_codec_to_layer_cache(untouched, 0)["k_vision"] is plain


def test_quantiser_entry_points():
    gen = torch.Generator().manual_seed(5)
    coeff = torch.randn(1, 40, 128, generator=gen).to(torch.bfloat16)
    codes, scale = hy_codec.quantize_kv_tensor(coeff.cuda(), 4, "per_token")
    work = coeff.float()
    want_scale = work.abs().amax(dim=-1, keepdim=True).clamp_min(torch.finfo(torch.float32).eps) / 7
    want = (work / want_scale).round().clamp(-7, 7).to(torch.int8)
    assert torch.equal(scale.cpu(), want_scale)
    assert int((codes.cpu().int() - want.int()).abs().max()) <= 1
    packed = hy_codec.pack_quantized_codes(want, 4)
    assert packed.dtype == torch.uint8 and packed.numel() == want.numel() // 2
    assert torch.equal(hy_codec.unpack_quantized_codes(packed, 4, want.numel(), tuple(want.shape)), want)
    with pytest.raises(ValueError):
        hy_codec.quantize_kv_tensor(coeff.cuda(), 5, "per_token")
    with pytest.raises(ValueError):
        hy_codec.pack_quantized_codes(torch.full((4,), 9, dtype=torch.int8), 4)
