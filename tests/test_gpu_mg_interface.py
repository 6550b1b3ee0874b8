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
