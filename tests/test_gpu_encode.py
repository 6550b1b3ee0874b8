"""GPU parity of the encoder (assign / C-means / project / quantise+pack / append)."""
import math

import numpy as np
import pytest
import torch

import cases
from helpers import code_flip_report, device_operator, unpack_device_codes
from nanokv_b200 import codec, ops, synthetic
from nanokv_b200.cache import CompressedHistory
from oracle import nkv_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("group", [None, 32])
@pytest.mark.parametrize("in_coeff_dtype", [False, True])
@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float16])
def test_quant_pack_is_bit_exact(dtype, group, in_coeff_dtype, scale_dtype):
    if in_coeff_dtype and dtype != torch.bfloat16:
        pytest.skip("coefficient-dtype arithmetic only differs for bf16 coefficients")
    gen = synthetic.generator(3)
    coeff = torch.randn(777, 192, generator=gen).to(dtype)
    coeff[5] = 0            # all-zero row: the eps clamp decides the scale
    coeff[6, 10] = 1e-9     # tiny row
    coeff[7] *= 1e4
    # exact .5 quotients exercise round-half-even: row amax 7 -> scale 1
    coeff[8] = torch.tensor([7.0, 0.5, 1.5, 2.5, -0.5, -1.5, 3.5, -2.5] * 24).to(dtype)
    eps = oracle.F32_EPS
    want_codes, want_scale = oracle.quantize_rows(coeff, group=group, eps=eps,
                                                  in_coeff_dtype=in_coeff_dtype,
                                                  scale_dtype=scale_dtype)
    want_packed, _ = oracle.pack_int4(want_codes)
    got_packed, got_scale = ops.quant_pack(coeff.cuda(), group=group, eps=eps,
                                           in_coeff_dtype=in_coeff_dtype, scale_dtype=scale_dtype)
    assert torch.equal(got_packed.cpu().reshape(-1), want_packed)
    assert torch.equal(got_scale.cpu().view(torch.int16), want_scale.view(torch.int16))


@pytest.mark.parametrize("rank", [64, 320, 384, 640, 1024])
@pytest.mark.parametrize("group", [None, 32])
@pytest.mark.parametrize("in_coeff_dtype", [False, True])
def test_quant_pack_row_widths_are_bit_exact(rank, group, in_coeff_dtype):
    """Every lanes-per-token layout of the vectorised kernel (8, 16, 32 lanes), a token count that
    leaves the last warp partly empty, ties at exact halves."""
    gen = synthetic.generator(rank)
    coeff = (torch.randn(1001, rank, generator=gen) * torch.logspace(-2, 2, 1001)[:, None]).to(torch.bfloat16)
    coeff[3] = 0
    coeff[4, ::2] = 3.5
    coeff[4, 1] = 7.0
    want_codes, want_scale = oracle.quantize_rows(coeff, group=group, eps=oracle.F32_EPS,
                                                  in_coeff_dtype=in_coeff_dtype)
    want_packed, _ = oracle.pack_int4(want_codes)
    got_packed, got_scale = ops.quant_pack(coeff.cuda(), group=group, eps=oracle.F32_EPS,
                                           in_coeff_dtype=in_coeff_dtype)
    assert torch.equal(got_packed.cpu().reshape(-1), want_packed)
    assert torch.equal(got_scale.cpu().view(torch.int16), want_scale.view(torch.int16))


@pytest.mark.parametrize("rank,group", [(640, None), (384, None), (1024, None), (64, None), (640, 32)])
@pytest.mark.parametrize("in_coeff_dtype", [False, True])
def test_quant_pack_streaming_form_is_bit_exact(rank, group, in_coeff_dtype):
    """Inputs of 8,192 tokens and more stream through a shared-memory ring; a token count that ends
    in a partial tile, rows of very different magnitude, against the oracle."""
    gen = synthetic.generator(rank + 9)
    tokens = 20011
    coeff = (torch.randn(tokens, rank, generator=gen) * torch.logspace(-3, 3, tokens)[:, None]).to(torch.bfloat16)
    coeff[11] = 0
    coeff[tokens - 1, ::2] = 2.5
    coeff[tokens - 1, 1] = 7.0
    want_codes, want_scale = oracle.quantize_rows(coeff, group=group, eps=oracle.F32_EPS,
                                                  in_coeff_dtype=in_coeff_dtype)
    want_packed, _ = oracle.pack_int4(want_codes)
    got_packed, got_scale = ops.quant_pack(coeff.cuda(), group=group, eps=oracle.F32_EPS,
                                           in_coeff_dtype=in_coeff_dtype)
    assert torch.equal(got_packed.cpu().reshape(-1), want_packed)
    assert torch.equal(got_scale.cpu().view(torch.int16), want_scale.view(torch.int16))


@pytest.mark.parametrize("S,J,rank,clusters", [(1000, 512, 640, 64), (12480, 1024, 640, 64), (300, 256, 384, 16),
                                               (129, 256, 64, 8), (2000, 512, 320, 32), (700, 256, 1024, 8)])
@pytest.mark.parametrize("in_coeff_dtype", [False, True])
@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float16])
def test_project_quant_equals_project_then_quant_pack(S, J, rank, clusters, in_coeff_dtype, scale_dtype):
    """The single-kernel projection + quantiser + packing (coefficients kept on chip, per-token
    maximum swapped between the two column-half thread blocks) writes the same bytes as the
    projection kernel followed by the quantiser kernel; shapes outside it take the two kernels."""
    gen = synthetic.generator(S + rank)
    centers = torch.randn(clusters, J, generator=gen).to(torch.bfloat16).cuda()
    ids = torch.randint(clusters, (S,), generator=gen).to(torch.uint8).cuda()
    rows = (centers[ids.long()].float().cpu() + 0.4 * torch.randn(S, J, generator=gen)).to(torch.bfloat16).cuda()
    mean = (0.05 * torch.randn(J, generator=gen)).cuda()
    encoder = (torch.randn(rank, J, generator=gen) / math.sqrt(J)).to(torch.bfloat16).cuda()
    coeff = ops.project(rows, centers, ids, mean, encoder)
    want_codes, want_scales = ops.quant_pack(coeff, eps=oracle.F32_EPS, in_coeff_dtype=in_coeff_dtype,
                                             scale_dtype=scale_dtype)
    got_codes, got_scales = ops.project_quant(rows, centers, ids, mean, encoder, eps=oracle.F32_EPS,
                                              in_coeff_dtype=in_coeff_dtype, scale_dtype=scale_dtype)
    assert torch.equal(got_codes, want_codes)
    assert torch.equal(got_scales.view(torch.int16), want_scales.view(torch.int16))
    # 32-wide groups are outside the single-kernel form: same entry point, two kernels
    grouped = ops.project_quant(rows, centers, ids, mean, encoder, group=32, eps=oracle.F32_EPS,
                                in_coeff_dtype=in_coeff_dtype, scale_dtype=scale_dtype)
    want_grouped = ops.quant_pack(coeff, group=32, eps=oracle.F32_EPS, in_coeff_dtype=in_coeff_dtype,
                                  scale_dtype=scale_dtype)
    assert torch.equal(grouped[0], want_grouped[0])
    assert torch.equal(grouped[1].view(torch.int16), want_grouped[1].view(torch.int16))


def test_quant_pack_empty_input():
    packed, scale = ops.quant_pack(torch.zeros(0, 64, device="cuda"))
    assert packed.shape == (0, 32) and scale.shape == (0, 1)


@pytest.mark.parametrize("dtype,S,J,C", [
    (torch.float32, 300, 256, 8), (torch.float32, 2048, 1536, 16),
    (torch.bfloat16, 300, 256, 16), (torch.bfloat16, 1000, 1024, 256),
    (torch.bfloat16, 333, 512, 512), (torch.bfloat16, 129, 256, 80),
])
def test_assign_matches_oracle(dtype, S, J, C):
    gen = synthetic.generator(17)
    centers = torch.randn(C, J, generator=gen)
    rows = synthetic.make_rows(S, centers, gen, dtype=dtype)
    stored = centers.to(torch.bfloat16)
    table = stored if dtype == torch.bfloat16 else stored.float()
    want = oracle.assign_labels(rows[None].float(), stored[None].float())[0]
    got = ops.assign(rows.cuda(), table.cuda())
    got = got.cpu().to(torch.int64) & 0xFFFF
    assert torch.equal(got, want)


def test_assign_ties_take_the_lowest_index():
    centers = torch.zeros(32, 256)
    centers[3] = 1.0
    centers[9] = 1.0          # duplicate of centre 3
    rows = torch.ones(70, 256)
    got = ops.assign(rows.to(torch.bfloat16).cuda(), centers.to(torch.bfloat16).cuda())
    assert got.cpu().tolist() == [3] * 70
    got = ops.assign(rows.cuda(), centers.cuda())
    assert got.cpu().tolist() == [3] * 70


@pytest.mark.parametrize("S,J,C,spread", [(3000, 1024, 64, 0.3), (4100, 512, 256, 0.3), (1560, 1024, 256, 1.0),
                                          (2500, 768, 512, 0.5)])
def test_kmeans_tensor_core_assignment_matches_oracle(S, J, C, spread):
    """bf16 rows with 16 | C: the assignment inside the online C-means runs on the tensor cores
    against the fp32 centres split into three bf16 planes.  Ids must equal the fp32 CPU oracle's
    (sequential-order means included), also when clusters overlap (spread 1.0) and for C > 256."""
    gen = synthetic.generator(S + C)
    true_centers = torch.randn(C, J, generator=gen)
    pick = torch.randint(C, (S,), generator=gen)
    rows = (true_centers[pick] + spread * torch.randn(S, J, generator=gen)).to(torch.bfloat16)
    seed = 424242 + C
    want_centers, want_labels = oracle.kmeans(rows[None].float(), C, 2, seed)
    init = codec.kmeans_init_rows(S, C, seed)
    got_centers, got_ids = ops.kmeans(rows.cuda(), C, 2, init.cuda())
    assert torch.equal(got_ids.cpu().long(), want_labels[0])
    got = got_centers.cpu().float()
    want = want_centers[0].to(torch.bfloat16).float()
    assert (got - want).abs().max() <= 2.0 ** -7 * want.abs().max()
    assert (got != want).float().mean() < 0.02
    # and the CUDA-core path (forced) gives the same ids: the two assignments agree
    ops.force_simt(True)
    try:
        _, simt_ids = ops.kmeans(rows.cuda(), C, 2, init.cuda())
    finally:
        ops.force_simt(False)
    assert torch.equal(simt_ids, got_ids)


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.MINI_BF16, cases.C1], ids=lambda c: c.name)
def test_kmeans_matches_oracle(case):
    data = cases.build(case)
    rows = data["k_chunks"][0]
    S = rows.shape[0]
    seed = 20260804 + case.layer
    C = case.shape.centers
    want_centers, want_labels = oracle.kmeans(rows[None].float(), C, case.iters, seed)
    init = codec.kmeans_init_rows(S, C, seed)
    got_centers, got_ids = ops.kmeans(rows.cuda(), C, case.iters, init.cuda())
    assert torch.equal(got_ids.cpu().long(), want_labels[0])
    # centre means are fp32 sums in a different order: bf16 storage may differ in the last bit
    got = got_centers.cpu().float()
    want = want_centers[0].to(torch.bfloat16).float()
    assert (got - want).abs().max() <= 2.0 ** -7 * want.abs().max()
    assert (got != want).float().mean() < 0.02


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.MINI_BF16], ids=lambda c: c.name)
def test_project_matches_oracle(case):
    data = cases.build(case)
    rows, op = data["k_chunks"][0], data["k_op"]
    _, stored, ids = oracle.semantic_residual(rows[None], case.shape.centers, case.iters, 1)
    residual = rows[None].float() - torch.gather(
        stored.float(), 1, ids.long()[..., None].expand(-1, -1, rows.shape[-1]))
    want = oracle.operator_linear(residual[0] - op["mean"], op["encoder"])
    got = ops.project(rows.cuda(), stored[0].cuda(), ids[0].cuda(), op["mean"].cuda(),
                      op["encoder"].cuda()).cpu()
    if case.shape.dtype == "f32":
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    else:
        # bf16 outputs of fp32 accumulations in another order: equal except at rounding boundaries
        ulp = (got.float() - want.float()).abs() / want.float().abs().clamp_min(1e-3)
        assert float(ulp.max()) <= 2.0 ** -7
        assert float((got != want).float().mean()) < 0.02


def _encode_on_device(case, data, kind, quant, *, fixed_centers):
    op = device_operator(data[f"{kind}_op"])
    chunks = data[f"{kind}_chunks"]
    total = sum(c.shape[0] for c in chunks)
    hist = CompressedHistory(joint=case.shape.joint, rank=case.shape.rank, capacity=total,
                             max_segments=len(chunks), centers_per_segment=case.shape.centers,
                             group=quant.group, scale_dtype=quant.scale_dtype)
    for index, chunk in enumerate(chunks):
        centers = None
        if fixed_centers:
            centers = data[f"{kind}_true_centers"].to(torch.bfloat16).cuda()
        codec.encode_append(hist, chunk.cuda(), op, quant, centers=centers,
                            clusters=case.shape.centers, iters=case.iters,
                            seed=20260804 + case.layer)
    return hist


@pytest.mark.parametrize("case", [cases.C1, cases.MINI_F32, cases.MINI_BF16], ids=lambda c: c.name)
def test_online_encode_against_reference_fixture(case):
    """encode (C-means + project + quantise + pack + append) vs the reference's stored outputs."""
    gold = np.load(cases_dir() / f"{case.name}.npz")
    data = cases.build(case)
    for kind in ("k", "v"):
        hist = _encode_on_device(case, data, kind, codec.MG_QUANT, fixed_centers=False)
        offset = 0
        for index, n in enumerate(case.segments):
            want_ids = torch.from_numpy(gold[f"{kind}{index}_ids"]).reshape(-1).long()
            got_ids = hist.ids[offset:offset + n].cpu().long()
            assert torch.equal(got_ids, want_ids), "centre ids must be bit-exact"
            want_codes = oracle.unpack_int4(torch.from_numpy(gold[f"{kind}{index}_packed"]),
                                            n * case.shape.rank, (n, case.shape.rank))
            got_codes = unpack_device_codes(hist.codes[offset:offset + n], case.shape.rank)
            report = code_flip_report(got_codes, want_codes)
            print(f"{case.name}/{kind}{index}: {report}")
            assert report["max_step"] <= 1, "a code may only flip by one step"
            assert report["flips"] <= 2e-3 * report["total"], report
            offset += n


@pytest.mark.parametrize("case", [cases.MINI_F32, cases.MINI_BF16], ids=lambda c: c.name)
@pytest.mark.parametrize("quant", [codec.MG_QUANT, codec.LINGBOT_QUANT, codec.GROUP32_FP16],
                         ids=["mg", "lingbot", "group32_fp16"])
def test_fixed_centre_encode_matches_oracle(case, quant):
    data = cases.build(case)
    hist = _encode_on_device(case, data, "k", quant, fixed_centers=True)
    op = data["k_op"]
    offset = 0
    for chunk in data["k_chunks"]:
        n = chunk.shape[0]
        want = oracle.encode_rows(
            chunk[None], encoder=op["encoder"], mean=op["mean"],
            centers=data["k_true_centers"][None].to(torch.bfloat16), group=quant.group,
            eps=quant.eps, in_coeff_dtype=quant.in_coeff_dtype, scale_dtype=quant.scale_dtype)
        assert torch.equal(hist.ids[offset:offset + n].cpu().long(), want["ids"][0].long())
        got_codes = unpack_device_codes(hist.codes[offset:offset + n], case.shape.rank)
        report = code_flip_report(got_codes, want["codes"])
        print(f"{case.name}/{quant}: {report}")
        assert report["max_step"] <= 1
        assert report["flips"] <= 2e-3 * report["total"], report
        offset += n


def test_encode_rejects_bad_arguments():
    hist = CompressedHistory(joint=256, rank=64, capacity=100, max_segments=1,
                             centers_per_segment=8)
    gen = synthetic.generator(0)
    shape = synthetic.Shape("x", 2, 128, 64, 8, 100, 8, "bf16")
    op = device_operator(synthetic.make_operator(shape, gen))
    with pytest.raises(ValueError):
        codec.encode_append(hist, torch.zeros(10, 128, device="cuda", dtype=torch.bfloat16), op)
    with pytest.raises(ValueError):   # more clusters than tokens, as the reference raises
        codec.encode_append(hist, torch.zeros(4, 256, device="cuda", dtype=torch.bfloat16), op,
                            clusters=8)
    with pytest.raises(ValueError):   # capacity
        codec.encode_append(hist, torch.zeros(200, 256, device="cuda", dtype=torch.bfloat16), op,
                            clusters=8)


def cases_dir():
    from pathlib import Path
    return Path(__file__).parent / "golden"
