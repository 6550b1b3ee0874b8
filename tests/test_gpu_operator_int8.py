"""INT8 operator storage on the GPU: the unpack kernel against the reference fixture, and an
operator built from INT8 storage against the same operator given as dense bf16."""
import numpy as np
import pytest
import torch

import cases
from nanokv_b200 import codec, ops
from oracle import nkv_oracle as oracle
from test_oracle_golden import load

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,group", [("per_row", 0), ("group64", 64)])
def test_unpack_matches_reference_fixture(name, group):
    gold = load("int8_operator")
    q = torch.from_numpy(gold[f"{name}_qweight"]).cuda()
    scale = torch.from_numpy(gold[f"{name}_scale"]).view(torch.bfloat16).cuda()
    dense = ops.unpack_int8_weight(q, scale, group)
    assert np.array_equal(dense.cpu().view(torch.int16).numpy(), gold[f"{name}_dense"])


def test_unpack_argument_errors():
    q = torch.zeros(4, 48, dtype=torch.int8, device="cuda")
    scale = torch.ones(4, 1, dtype=torch.bfloat16, device="cuda")
    ops.unpack_int8_weight(q, scale)                                   # per row, 48 = 3 x 16 columns
    with pytest.raises(ValueError):
        ops.unpack_int8_weight(q, scale, 36)                           # group must divide the columns
    with pytest.raises(ValueError):
        ops.unpack_int8_weight(q[:, :40].contiguous(), scale)          # columns not a multiple of 16
    with pytest.raises(ValueError):
        ops.unpack_int8_weight(q.float(), scale)


def test_operator_from_int8_equals_dense_operator():
    gen = torch.Generator().manual_seed(5)
    rank, joint = 64, 256
    encoder = torch.randn(rank, joint, generator=gen) / joint ** 0.5
    decoder = torch.randn(joint, rank, generator=gen) / rank ** 0.5
    mean = torch.randn(joint, generator=gen) * 0.05
    packed = {}
    dense = {}
    for name, weight, group in (("encoder", encoder, 0), ("decoder", decoder, 32)):
        codes, scale, group_size = oracle.pack_int8_weight(weight, group)
        packed[name] = {"qweight": codes, "scale": scale, "group_size": group_size}
        dense[name] = oracle.unpack_int8_weight(codes, scale, group_size)
    op = codec.Operator.from_int8(mean, packed["encoder"], packed["decoder"])
    assert torch.equal(op.encoder.cpu(), dense["encoder"]) and torch.equal(op.decoder.cpu(), dense["decoder"])
    assert op.dtype == torch.bfloat16 and op.rank == rank and op.joint == joint
