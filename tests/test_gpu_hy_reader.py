"""HY-WorldPlay's two-branch dictionary reader (the reference function's argument list) on the GPU,
against a fixture the reference function produced (its CUDA-only attention call replaced by exact
fp32 softmax attention for the CPU run; everything else unmodified)."""
import numpy as np
import pytest
import torch

import cases
from helpers import BF16_REL_TOL, rel_err
from nanokv_b200 import hy_reader, ops
from oracle import nkv_oracle as oracle
from test_oracle_golden import from_bits, load

pytestmark = pytest.mark.gpu


def build_call(data):
    cfg = cases.HY_SHAPE
    cache = {"vision_freqs_cis": data["vision_freqs"], "vision_viewmats": data["vision_viewmats"],
             "vision_Ks": None}
    for name in ("k_vision", "v_vision"):
        part = dict(data[name])
        codes = part.pop("codes")
        packed, _ = oracle.pack_int4(codes.reshape(-1, cfg["rank"]))
        part["latent_int4"] = packed
        cache[name] = part
    runtime = {"recent_native_frames": 0, "attention": data["state"], "main_k_mode": "learned_rope",
               "shape": (cfg["heads"], cfg["head_dim"], cfg["heads"], cfg["head_dim"])}
    return cache, runtime


def test_two_branch_reader_against_the_reference_fixture():
    gold, data = load("hy_two_branch_bf16"), cases.build_hy()
    cache, runtime = build_call(data)
    # the packed bytes the reference's own packer made are the bytes this library reads
    assert np.array_equal(gold["packed_k"], cache["k_vision"]["latent_int4"].numpy())
    cuda = lambda name: data[name].cuda()
    main, prope = hy_reader.attend_dictionary_lowkv(
        0, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"), cuda("encoder_key"),
        cuda("encoder_value"), cache, data["current_freqs"], data["current_viewmats"], None, runtime)
    ops.check_status()
    cfg = cases.HY_SHAPE
    assert main.shape == prope.shape == (1, cfg["queries"], cfg["heads"] * cfg["head_dim"])
    want_main = from_bits(gold["main"], torch.bfloat16)
    want_prope = from_bits(gold["prope"], torch.bfloat16)
    assert rel_err(main.cpu(), want_main) <= BF16_REL_TOL
    assert rel_err(prope.cpu(), want_prope) <= BF16_REL_TOL
    # the two branches are different reads: neither output equals the other
    assert rel_err(main.cpu(), want_prope) > 4 * BF16_REL_TOL
    # second call on the same state reuses the prepared operands and the cached views
    again, _ = hy_reader.attend_dictionary_lowkv(
        0, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"), cuda("encoder_key"),
        cuda("encoder_value"), cache, data["current_freqs"], data["current_viewmats"], None, runtime)
    assert torch.equal(again, main)
    # the public entry point: the runtime registered per layer, the reference's two checks
    hy_reader.register_runtime(11, dict(runtime, payload_mode="dictionary_lowkv"))
    with pytest.raises(RuntimeError):
        hy_reader.attend(11, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"),
                         cuda("encoder_key"), cuda("encoder_value"), cache, data["current_freqs"],
                         data["current_viewmats"], None)          # the cache is not marked as compressed
    marked = dict(cache, direct_codec_latent=True)
    public, _ = hy_reader.attend(11, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"),
                                 cuda("encoder_key"), cuda("encoder_value"), marked, data["current_freqs"],
                                 data["current_viewmats"], None)
    assert torch.equal(public, main)
    with pytest.raises(RuntimeError):
        hy_reader.attend(11, cuda("q_pre"), cuda("query")[:1], cuda("current_key"), cuda("current_value"),
                         cuda("encoder_key"), cuda("encoder_value"), marked, data["current_freqs"],
                         data["current_viewmats"], None)
    with pytest.raises(KeyError):
        hy_reader.attend(12, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"),
                         cuda("encoder_key"), cuda("encoder_value"), marked, data["current_freqs"],
                         data["current_viewmats"], None)
    with pytest.raises(NotImplementedError):
        hy_reader.attend_dictionary_lowkv(
            0, cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"), cuda("encoder_key"),
            cuda("encoder_value"), cache, data["current_freqs"], data["current_viewmats"], None,
            dict(runtime, recent_native_frames=2))


def test_projection_matrices_match_the_closed_forms():
    gen = torch.Generator().manual_seed(4)
    view = cases._se3(3, gen)
    P, P_T, P_inv = hy_reader.projection_matrices(view, None)
    assert torch.allclose(P @ P_inv, torch.eye(4).expand(1, 3, 4, 4), atol=1e-5)
    assert torch.equal(P_T, P.transpose(-1, -2))
    Ks = torch.zeros(1, 3, 3, 3)
    Ks[..., 0, 0], Ks[..., 1, 1], Ks[..., 2, 2] = 1.3, 0.8, 1.0
    Ks[..., 0, 2], Ks[..., 1, 2] = 0.4, 0.6          # the principal point is dropped by the reference
    P, _, P_inv = hy_reader.projection_matrices(view, Ks)
    assert torch.allclose(P @ P_inv, torch.eye(4).expand(1, 3, 4, 4), atol=1e-5)
    assert torch.allclose(P[..., 0, :], 1.3 * view[..., 0, :], atol=1e-6)


def write_runtime(data):
    cfg = cases.HY_WRITE
    return {"operators": data["operators"], "attention": data["attention"], "payload_mode": "dictionary_lowkv",
            "main_k_mode": "learned_rope", "recent_native_frames": 0,
            "shape": (cfg["heads"], cfg["head_dim"], cfg["heads"], cfg["head_dim"])}


def test_compress_layer_cache_against_the_reference_fixture(monkeypatch):
    """The write side (`compress_layer_cache` / `_compress_one` of the reference module): packed codes,
    fp32 scales and ids as the reference made them, the branches' centre tables within a bf16 step."""
    cfg = cases.HY_WRITE
    gold, data = load("hy_write_bf16"), cases.build_hy_write()
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_CLUSTERS", str(cfg["centres"]))
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_ITERS", "2")
    hy_reader.register_runtime(cfg["layer"], write_runtime(data))
    cache = {"k_vision": data["k_vision"].cuda(), "v_vision": data["v_vision"].cuda(), "vision_thw": (1, 1, 1),
             "_direct_codec_positioned_history": object()}
    out = hy_reader.compress_layer_cache(cache, cfg["layer"])
    assert out is cache and cache["direct_codec_latent"] and "_direct_codec_positioned_history" not in cache
    flips = 0
    for name in ("k", "v"):
        payload = cache[f"{name}_vision"]
        S, r = cfg["tokens"], cfg["rank"]
        assert payload["shape"] == (1, 16, S, 128) and payload["latent_shape"] == (1, S, r)
        assert payload["payload_mode"] == "dictionary_lowkv" and payload["tensor_name"] == name
        assert np.array_equal(payload["semantic_ids"].cpu().numpy(), gold[f"{name}_ids"])
        assert payload["latent_scale"].dtype == torch.float32
        assert np.array_equal(payload["latent_scale"].cpu().numpy(), gold[f"{name}_scale"])
        got, _ = None, None
        got = torch.from_numpy(gold[f"{name}_packed"])
        mine = payload["latent_int4"].cpu()
        assert mine.shape == got.shape
        lo = (mine & 15).int() - (got & 15).int()
        hi = (mine >> 4).int() - (got >> 4).int()
        assert int(lo.abs().max()) <= 1 and int(hi.abs().max()) <= 1
        flips += int(lo.abs().sum() + hi.abs().sum())
        for table in ("centre_main", "centre_prope"):
            want = from_bits(gold[f"{name}_{table}"], torch.bfloat16)
            assert payload[table].shape == want.shape and payload[table].dtype == torch.bfloat16
            assert rel_err(payload[table].cpu(), want) <= 2.0 ** -7
    print(f"code flips against the reference: {flips}")
    assert flips <= 4
    again = hy_reader.compress_layer_cache(dict(k_vision=data["k_vision"].cuda(), v_vision=data["v_vision"].cuda()), 99)
    assert isinstance(again["k_vision"], torch.Tensor)            # no runtime for that layer: left alone
    with pytest.raises(RuntimeError):
        hy_reader.compress_layer_cache(cache, cfg["layer"])       # already compressed
    with pytest.raises(NotImplementedError):
        hy_reader.register_runtime(3, dict(write_runtime(data), grouped_attention=[{}]))


def test_write_then_read_of_one_layer_against_the_reference_chain(monkeypatch):
    """compress_layer_cache followed by attend on the payloads it made, against the reference's
    _compress_one + _attend_dictionary_lowkv on the same raw history and queries."""
    cfg = cases.HY_CHAIN
    gold, data = load("hy_chain_bf16"), cases.build_hy_chain()
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_CLUSTERS", str(cfg["centres"]))
    monkeypatch.setenv("HY_KV_CODEC_SEMANTIC_ITERS", "2")
    hy_reader.register_runtime(cfg["layer"], cases.hy_chain_runtime(data))
    cache = {"k_vision": data["k_vision"].cuda(), "v_vision": data["v_vision"].cuda(),
             "vision_freqs_cis": data["vision_freqs"], "vision_viewmats": data["vision_viewmats"], "vision_Ks": None}
    hy_reader.compress_layer_cache(cache, cfg["layer"])
    assert np.array_equal(cache["k_vision"]["semantic_ids"].cpu().numpy(), gold["k_ids"])
    cuda = lambda name: data[name].cuda()
    main, prope = hy_reader.attend(
        cfg["layer"], cuda("q_pre"), cuda("query"), cuda("current_key"), cuda("current_value"), cuda("encoder_key"),
        cuda("encoder_value"), cache, data["current_freqs"], data["current_viewmats"], None)
    ops.check_status()
    assert main.shape == prope.shape == (1, cfg["queries"], cfg["heads"] * cfg["head_dim"])
    assert rel_err(main[:, ::4].cpu(), from_bits(gold["main"], torch.bfloat16)) <= BF16_REL_TOL
    assert rel_err(prope[:, ::4].cpu(), from_bits(gold["prope"], torch.bfloat16)) <= BF16_REL_TOL
