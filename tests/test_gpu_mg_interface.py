"""The Matrix-Game codec interface (same names and payloads as the reference module) on the GPU."""
import os

import numpy as np
import pytest
import torch

import cases
from helpers import code_flip_report
from nanokv_b200 import mg_codec
from oracle import nkv_oracle as oracle
from test_oracle_golden import encode_all, load

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.MINI_BF16], ids=lambda c: c.name)
def test_encode_decode_through_the_reference_interface(case):
    gold = load(case.name)
    data = cases.build(case)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.iters)
    dtype = case.shape.torch_dtype
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        mg_codec.register_operator(kind, case.layer, mean=op["mean"], encoder=op["encoder"],
                                   decoder=op["decoder"])
        container = None
        for index, chunk in enumerate(data[f"{kind}_chunks"]):
            payload = mg_codec.encode_tensor(kind, case.layer, chunk[None].cuda())
            assert payload["codec"] == "worldplay_c64_pca_int4_v1"
            assert payload["ids"].dtype == torch.uint8 and payload["scale"].dtype == torch.bfloat16
            assert np.array_equal(gold[f"{kind}{index}_ids"], payload["ids"].cpu().numpy())
            n, r = payload["latent_shape"]
            want = oracle.unpack_int4(torch.from_numpy(gold[f"{kind}{index}_packed"]), n * r, (n, r))
            got = oracle.unpack_int4(payload["packed_codes"].cpu(), n * r, (n, r))
            report = code_flip_report(got, want)
            assert report["max_step"] <= 1 and report["flips"] <= 2e-3 * report["total"], report
            container = mg_codec.concat_values(container, payload)
        total = sum(case.segments)
        assert mg_codec.value_shape(container) == (1, total, case.shape.joint)
        assert mg_codec.payload_bytes(container) > 0
        decoded = mg_codec.decode_value(container, dtype=dtype, device="cuda")
        segments = encode_all(case, data)[kind]
        want_rows = torch.cat([oracle.decode_rows(s, decoder=op["decoder"], mean=op["mean"],
                                                  dtype=dtype) for s in segments], 1)
        err = float((decoded.cpu().float() - want_rows.float()).abs().max())
        assert err <= 2.0 ** -6 * float(want_rows.float().abs().max())


def test_interface_errors_match_the_reference():
    with pytest.raises(ValueError):
        mg_codec.encode_tensor("q", 0, torch.zeros(1, 8, 256, device="cuda"))
    with pytest.raises(KeyError):
        mg_codec.encode_tensor("k", 91, torch.zeros(1, 300, 256, device="cuda"))
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = "64"
    mg_codec.register_operator("k", 92, mean=torch.zeros(256), encoder=torch.zeros(64, 256),
                               decoder=torch.zeros(256, 64))
    with pytest.raises(ValueError):      # more clusters than tokens
        mg_codec.encode_tensor("k", 92, torch.zeros(1, 8, 256, device="cuda"))
    with pytest.raises(RuntimeError):
        mg_codec.concat_values({"codec": "worldplay_raw_v1", "tensor": torch.zeros(1)}, torch.zeros(1))
    with pytest.raises(RuntimeError):
        mg_codec.decode_tensor({"codec": "something_else"}, dtype=torch.float32, device="cuda")


def test_select_value_cuts_and_reuses_segments_like_the_reference():
    """A window compaction that cuts the first segment and keeps the second whole: the kept
    segment is reused, the cut one is decoded, gathered and encoded again; the result is compared
    with what the reference's select_value produced from the same inputs."""
    from test_oracle_golden import from_bits
    case = cases.MINI_BF16
    gold = load("select_mg_bf16")
    data = cases.build(case)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.iters)
    op = data["k_op"]
    mg_codec.register_operator("k", case.layer, mean=op["mean"], encoder=op["encoder"],
                               decoder=op["decoder"])
    value = None
    for chunk in data["k_chunks"]:
        value = mg_codec.concat_values(value, mg_codec.encode_tensor("k", case.layer, chunk[None].cuda()))
    token_idx = cases.select_indices(case)
    picked = mg_codec.select_value(value, token_idx.cuda(), kind="k", layer=case.layer,
                                   dtype=torch.bfloat16, device="cuda")
    parts = picked["segments"]
    assert len(parts) == 2 and parts[1] is value["segments"][1]          # whole segment reused
    cut = parts[0]
    assert tuple(cut["shape"]) == tuple(int(v) for v in gold["cut_shape"])
    same_ids = float((cut["ids"].cpu().numpy() == gold["cut_ids"]).mean())
    assert same_ids >= 0.98, same_ids
    decoded = mg_codec.decode_value(picked, dtype=torch.bfloat16, device="cuda")[0].cpu().float()
    want = from_bits(gold["decoded"], torch.bfloat16).float()
    assert decoded.shape == want.shape
    assert float((decoded - want).norm() / want.norm()) <= 2e-2
    # selections that need no work, or nothing
    whole = mg_codec.select_value(value, torch.arange(sum(case.segments)), kind="k", layer=case.layer,
                                  dtype=torch.bfloat16, device="cuda")
    assert whole["segments"][0] is value["segments"][0] and whole["segments"][1] is value["segments"][1]
    second = mg_codec.select_value(value, torch.arange(case.segments[0], sum(case.segments)), kind="k",
                                   layer=case.layer, dtype=torch.bfloat16, device="cuda")
    assert second is value["segments"][1]
    assert mg_codec.select_value(value, torch.empty(0, dtype=torch.long), kind="k", layer=case.layer,
                                 dtype=torch.bfloat16, device="cuda") is None
    with pytest.raises(RuntimeError):
        mg_codec.select_value(value, torch.tensor([5, 3]), kind="k", layer=case.layer,
                              dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        mg_codec.select_value(value, torch.tensor([5, 9999]), kind="k", layer=case.layer,
                              dtype=torch.bfloat16, device="cuda")


def test_selected_decode_and_direct_rows_follow_the_token_mask():
    """decode_pair_selected and direct_latent_pair_segments(token_keep=) on a two-segment history:
    the selected rows equal the same rows of the whole decode; a segment the mask empties is left out."""
    case = cases.MINI_BF16
    data = cases.build(case)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.iters)
    containers = {}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        mg_codec.register_operator(kind, case.layer, mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
        container = None
        for chunk in data[f"{kind}_chunks"]:
            container = mg_codec.concat_values(container, mg_codec.encode_tensor(kind, case.layer, chunk[None].cuda()))
        containers[kind] = container
    total = sum(case.segments)
    gen = torch.Generator().manual_seed(3)
    keep = torch.rand(total, generator=gen) < 0.3
    key_rows, value_rows = mg_codec.decode_pair_selected(containers["k"], containers["v"], keep,
                                                         dtype=torch.bfloat16, device="cuda")
    whole_k, whole_v = mg_codec.decode_pair_values(containers["k"], containers["v"], dtype=torch.bfloat16,
                                                   device="cuda")
    assert torch.equal(key_rows, whole_k[:, keep.cuda()]) and torch.equal(value_rows, whole_v[:, keep.cuda()])
    none_k, none_v = mg_codec.decode_pair_selected(containers["k"], containers["v"], torch.zeros(total, dtype=torch.bool),
                                                   dtype=torch.bfloat16, device="cuda")
    assert none_k.shape == (1, 0, case.shape.joint) and none_v.shape == none_k.shape
    with pytest.raises(ValueError):
        mg_codec.decode_pair_selected(containers["k"], containers["v"], keep[:-1], dtype=torch.bfloat16, device="cuda")
    only_second = torch.zeros(total, dtype=torch.bool)
    only_second[case.segments[0] + 3:case.segments[0] + 40] = True
    low = mg_codec.direct_latent_pair_segments(containers["k"], containers["v"], device="cuda", token_keep=only_second)
    assert len(low) == 1 and low[0]["length"] == 37 and low[0]["k"].tokens == 37
    assert low[0]["logical_indices"].tolist() == list(range(case.segments[0] + 3, case.segments[0] + 40))
    everything = mg_codec.direct_latent_pair_segments(containers["k"], containers["v"], device="cuda")
    assert [item["length"] for item in everything] == list(case.segments)
    with pytest.raises(ValueError):
        mg_codec.direct_latent_pair_segments(containers["k"], containers["v"], device="cuda", token_keep=keep[:-1])


@pytest.mark.parametrize("mode", ["bf16", "int8", "fp32"])
def test_operators_load_from_the_reference_artefact_layout(tmp_path, monkeypatch, mode):
    """With nothing registered for a layer the module reads the reference's artefact files (K basis
    directory, V-QAT checkpoint directory, weight mode variable), as the backbone's environment names
    them; the result equals registering the same weights by hand."""
    case = cases.MINI_BF16
    data = cases.build(case)
    layer = 31                                   # a layer nothing else registers
    k_op, v_op = data["k_op"], data["v_op"]
    basis = tmp_path / "basis" / "k_c64"
    basis.mkdir(parents=True)
    torch.save({"mean": k_op["mean"].float(), "components": k_op["encoder"].float()}, basis / f"layer_{layer:02d}.pt")
    vdir = tmp_path / "vqat"
    vdir.mkdir()
    torch.save({"format": "mg35_worldplay_v_c64_int4_qat_v1", "mean": v_op["mean"].float(),
                "encoder": v_op["encoder"].float(), "decoder": v_op["decoder"].float()}, vdir / f"layer_{layer:02d}.pt")
    monkeypatch.setenv("MG35_KVCODEC_BASIS_DIR", str(tmp_path / "basis"))
    monkeypatch.setenv("MG35_KVCODEC_DECODER_DIR_V", str(vdir))
    monkeypatch.delenv("MG35_KVCODEC_DECODER_DIR_K", raising=False)
    monkeypatch.delenv("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", raising=False)
    monkeypatch.setenv("MG35_KVCODEC_OPERATOR_WEIGHT_MODE", mode)
    monkeypatch.setenv("MG35_KVCODEC_C64_CLUSTERS", str(case.shape.centers))
    monkeypatch.setenv("MG35_KVCODEC_C64_ITERS", str(case.iters))
    for key in [k for k in mg_codec._OPERATORS if k[1] in (layer, layer + 1)]:
        del mg_codec._OPERATORS[key]
    rows = data["k_chunks"][0][None].cuda()
    rows = rows.float() if mode == "fp32" else rows
    loaded = {kind: mg_codec.encode_tensor(kind, layer, rows) for kind in ("k", "v")}
    # the same weights handed over explicitly (K decoder = encoder transposed, as the basis file implies)
    cast = (lambda w: w.float()) if mode == "fp32" else (lambda w: w.float().to(torch.bfloat16))
    if mode == "int8":
        from nanokv_b200.codec import Operator
        for kind, op, decoder in (("k", k_op, k_op["encoder"].float().t().contiguous()), ("v", v_op, v_op["decoder"].float())):
            mg_codec._OPERATORS[(kind, layer + 1, "cuda")] = Operator.from_int8(
                op["mean"].float(), mg_codec._pack_int8(op["encoder"].float()), mg_codec._pack_int8(decoder))
    else:
        mg_codec.register_operator("k", layer + 1, mean=k_op["mean"], encoder=cast(k_op["encoder"]),
                                   decoder=cast(k_op["encoder"].float().t().contiguous()))
        mg_codec.register_operator("v", layer + 1, mean=v_op["mean"], encoder=cast(v_op["encoder"]),
                                   decoder=cast(v_op["decoder"]))
    for kind in ("k", "v"):
        by_hand = mg_codec.encode_tensor(kind, layer + 1, rows)
        # the seed of the online C-means depends on the layer: compare through a decode of the same payload
        dtype = torch.float32 if mode == "fp32" else torch.bfloat16
        a = mg_codec.decode_tensor(loaded[kind], dtype=dtype, device="cuda")
        redo = dict(loaded[kind], layer=layer + 1)
        b = mg_codec.decode_tensor(redo, dtype=dtype, device="cuda")
        assert torch.equal(a, b)
        assert by_hand["packed_codes"].shape == loaded[kind]["packed_codes"].shape
    monkeypatch.delenv("MG35_KVCODEC_BASIS_DIR")
    with pytest.raises(KeyError):
        mg_codec.encode_tensor("k", 77, rows)


def test_preload_operator_weights_reads_the_prepacked_file(tmp_path, monkeypatch):
    """preload_operator_weights (MGM/nanokv_codec.py:258-279): every entry of the prepacked INT8 file
    becomes resident; encoding then needs no other artefact and gives the bytes of the same operator
    registered by hand."""
    case = cases.MINI_BF16
    data = cases.build(case)
    layers = (41, 42)
    for key in [k for k in mg_codec._OPERATORS if k[1] in layers or k[1] == 43]:
        del mg_codec._OPERATORS[key]
    entries = {}
    for layer in layers:
        for kind in ("k", "v"):
            op = data[f"{kind}_op"]
            entries[f"{kind}:{layer:02d}"] = {"mean": op["mean"].float(),
                                              "encoder": mg_codec._pack_int8(op["encoder"].float()),
                                              "decoder": mg_codec._pack_int8(op["decoder"].float())}
    path = tmp_path / "operators.pt"
    torch.save({"format": "mg35_worldplay_operator_int8_v1", "entries": entries}, path)
    monkeypatch.delenv("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", raising=False)
    with pytest.raises(RuntimeError):
        mg_codec.preload_operator_weights(torch.device("cuda"))
    monkeypatch.setenv("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", str(path))
    mg_codec.preload_operator_weights(torch.device("cuda"))
    assert all((kind, layer, "cuda") in mg_codec._OPERATORS for kind in ("k", "v") for layer in layers)
    monkeypatch.delenv("MG35_KVCODEC_PREPACKED_OPERATOR_PATH")      # resident: the file is not needed again
    monkeypatch.setenv("MG35_KVCODEC_C64_CLUSTERS", str(case.shape.centers))
    monkeypatch.setenv("MG35_KVCODEC_C64_ITERS", str(case.iters))
    rows = data["k_chunks"][0][None].cuda()
    from nanokv_b200.codec import Operator
    op = data["k_op"]
    mg_codec._OPERATORS[("k", 43, "cuda")] = Operator.from_int8(
        op["mean"].float(), mg_codec._pack_int8(op["encoder"].float()), mg_codec._pack_int8(op["decoder"].float()))
    loaded = mg_codec.encode_tensor("k", 41, rows)
    by_hand = dict(mg_codec.encode_tensor("k", 43, rows))
    a = mg_codec.decode_tensor(loaded, dtype=torch.bfloat16, device="cuda")
    b = mg_codec.decode_tensor(dict(loaded, layer=43), dtype=torch.bfloat16, device="cuda")
    assert torch.equal(a, b) and by_hand["packed_codes"].shape == loaded["packed_codes"].shape
    bad = tmp_path / "bad.pt"
    torch.save({"format": "something else", "entries": {}}, bad)
    monkeypatch.setenv("MG35_KVCODEC_PREPACKED_OPERATOR_PATH", str(bad))
    with pytest.raises(RuntimeError):
        mg_codec.preload_operator_weights(torch.device("cuda"))
