"""Host-side logic of the HY-WorldPlay codec interface that needs no GPU: environment parsing, the nibble
packer against the oracle's and against the reference's packed bytes, payload accounting, argument errors."""
import numpy as np
import pytest
import torch

import cases
from nanokv_b200 import hy_codec
from oracle import nkv_oracle as oracle
from test_oracle_golden import load


def test_mode_and_flags(monkeypatch):
    for name in ("HY_KV_CODEC_ENABLE", "HY_KV_CODEC_MODE", "HY_KV_CODEC_TARGET", "HY_KV_CODEC_SCALE_DTYPE"):
        monkeypatch.delenv(name, raising=False)
    assert hy_codec.mode() == "none" and not hy_codec.enabled()
    monkeypatch.setenv("HY_KV_CODEC_MODE", "Global_PCA ")
    assert hy_codec.mode() == "global_pca" and not hy_codec.enabled()
    monkeypatch.setenv("HY_KV_CODEC_ENABLE", "yes")
    assert hy_codec.enabled()
    monkeypatch.setenv("HY_KV_CODEC_MODE", "zip")
    with pytest.raises(ValueError):
        hy_codec.mode()
    monkeypatch.setenv("HY_KV_CODEC_TARGET", "k")
    assert hy_codec._target_enabled("k") and not hy_codec._target_enabled("v")
    monkeypatch.setenv("HY_KV_CODEC_TARGET", "q")
    with pytest.raises(ValueError):
        hy_codec._target_enabled("k")
    assert hy_codec._scale_storage_dtype() == torch.bfloat16
    monkeypatch.setenv("HY_KV_CODEC_SCALE_DTYPE", "fp16")
    assert hy_codec._scale_storage_dtype() == torch.float16
    monkeypatch.setenv("HY_KV_CODEC_SCALE_DTYPE", "fp8")
    with pytest.raises(ValueError):
        hy_codec._scale_storage_dtype()
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_SMOOTH_K", "1")
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_SMOOTH_LAYERS", "3, 5")
    assert hy_codec._semantic_smooth_enabled(5, "k") and not hy_codec._semantic_smooth_enabled(4, "k")
    assert not hy_codec._semantic_smooth_enabled(5, "v")


def test_packer_matches_the_oracle_and_the_reference_bytes():
    gen = torch.Generator().manual_seed(9)
    codes = torch.randint(-7, 8, (37, 6), generator=gen, dtype=torch.int8)
    packed = hy_codec.pack_quantized_codes(codes, 4)
    want, count = oracle.pack_int4(codes)
    assert count == codes.numel() and torch.equal(packed, want)
    assert torch.equal(hy_codec.unpack_quantized_codes(packed, 4, codes.numel(), tuple(codes.shape)), codes)
    odd = torch.randint(-7, 8, (5,), generator=gen, dtype=torch.int8)           # odd count: padded nibble
    assert hy_codec.pack_quantized_codes(odd, 4).numel() == 3
    assert torch.equal(hy_codec.unpack_quantized_codes(hy_codec.pack_quantized_codes(odd, 4), 4, 5), odd)
    # the reference's own packed bytes unpack and repack to themselves
    gold = load(cases.HY_CODEC.name)
    stored = torch.from_numpy(gold["k_packed"])
    count = cases.HY_CODEC.segments[0] * cases.HY_CODEC.shape.rank
    assert torch.equal(hy_codec.pack_quantized_codes(hy_codec.unpack_quantized_codes(stored, 4, count), 4), stored)
    with pytest.raises(NotImplementedError):
        hy_codec.pack_quantized_codes(codes, 8)
    with pytest.raises(ValueError):
        hy_codec.pack_quantized_codes(torch.tensor([9], dtype=torch.int8), 4)


def test_payload_accounting_and_passthrough():
    payload = {"a": torch.zeros(3, 4, dtype=torch.bfloat16), "b": [torch.zeros(5, dtype=torch.uint8), 7],
               "c": {"d": torch.zeros(2, dtype=torch.float32)}, "e": "text"}
    assert hy_codec._payload_tensor_bytes(payload) == 24 + 5 + 8
    plain = torch.zeros(2, 2)
    assert hy_codec.decompress_kv_tensor(plain) is plain
    assert hy_codec.decompress_kv_tensor({"kv_codec": False, "x": 1})["x"] == 1
    with pytest.raises(ValueError):
        hy_codec.decompress_kv_tensor({"kv_codec": True, "codec": "uniform_packed"})
    with pytest.raises(ValueError):
        hy_codec.register_operator("q", 0, mean=torch.zeros(2048), encoder=torch.zeros(8, 2048),
                                   decoder=torch.zeros(2048, 8), device="cpu")
