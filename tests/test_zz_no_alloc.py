"""nkv_encode_append_static: the encoder for callers that cannot allocate device memory.

Such callers (a server whose own pool owns the whole GPU, a plugin that must
not trigger a cudaMalloc mid-rollout) pass inputs and outputs only; the
coefficient scratch is a fixed array inside the library.  The entry point has
to give exactly what nkv_encode_append gives with caller scratch, also on a
second call that finds the first call's leftovers in the array.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import pytest
import torch

from nanokv_b200 import _lib, ops, synthetic

pytestmark = pytest.mark.gpu


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def _encode(entry, rows, centers, mean, encoder, group, *, workspace):
    """Call one of the two entry points through the C ABI into fresh output buffers."""
    lib = _lib.library()
    S, J = rows.shape
    r, C = encoder.shape[0], centers.shape[0]
    codes = torch.zeros(S + 3, r // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(S + 3, r // group, dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros(S + 3, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = (_ptr(rows), ops.dtype_code(rows.dtype), _ptr(centers), C, _ptr(mean), _ptr(encoder),
            ops.dtype_code(encoder.dtype), S, J, r, group, 1e-12, _lib.NKV_QUANT_F32,
            _lib.NKV_BF16, 1, 3, _ptr(codes), _ptr(scales), _ptr(ids))
    if workspace:
        scratch = torch.empty(S * r, dtype=encoder.dtype, device="cuda")
        status = lib.nkv_encode_append(*head, _ptr(scratch), scratch.numel() * scratch.element_size(),
                                       stream)
    else:
        status = getattr(lib, entry)(*head, stream)
    _lib.check(status)
    torch.cuda.synchronize()
    return codes.cpu(), scales.cpu().view(torch.int16), ids.cpu()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_encoder_equals_the_allocating_one_twice_in_a_row(dtype):
    shape = synthetic.Shape("s", 2, 128, 64, 16, 0, 0, "bf16" if dtype == torch.bfloat16 else "f32")
    gen = synthetic.generator(123)
    op = synthetic.make_operator(shape, gen, mean_std=0.05)
    centers = synthetic.make_centers(shape, gen)
    mean, encoder = op["mean"].cuda(), op["encoder"].cuda()
    stored = centers.to(torch.bfloat16).cuda()
    # two calls with different inputs and sizes: the second one starts from a dirty array
    for count in (700, 333):
        rows = synthetic.make_rows(count, centers, gen, dtype=dtype).cuda()
        want = _encode(None, rows, stored, mean, encoder, 64, workspace=True)
        got = _encode("nkv_encode_append_static", rows, stored, mean, encoder, 64, workspace=False)
        for name, a, b in zip(("codes", "scales", "ids"), got, want):
            assert torch.equal(a, b), f"{name} differ on the {count}-token call"
        assert int(got[0][:3].sum()) == 0, "rows before the append offset must stay untouched"


def test_static_scratch_encoder_rejects_oversized_chunks():
    lib = _lib.library()
    limit = 4 * 1024 * 1024
    S, r = limit // (1024 * 4) + 1, 1024      # one row too many for fp32 coefficients
    status = lib.nkv_encode_append_static(None, _lib.NKV_F32, None, 16, None, None, _lib.NKV_F32, S,
                                          2048, r, r, 1e-12, 0, _lib.NKV_BF16, 1, 0, None, None,
                                          None, None)
    assert status == _lib.NKV_ERR_TOO_LARGE
    assert b"coefficient scratch" in lib.nkv_last_error()
    with pytest.raises(ValueError):
        _lib.check(status)


def test_static_scratch_encoder_takes_no_device_memory():
    """With every buffer allocated beforehand and one warmed call behind it, a call of the static
    entry point leaves the device's free memory exactly where it was: nothing inside allocates."""
    lib = _lib.library()
    shape = synthetic.Shape("s", 2, 128, 64, 16, 0, 0, "bf16")
    gen = synthetic.generator(7)
    op = synthetic.make_operator(shape, gen, mean_std=0.05)
    centers = synthetic.make_centers(shape, gen)
    mean, encoder = op["mean"].cuda(), op["encoder"].cuda()
    stored = centers.to(torch.bfloat16).cuda()
    rows = synthetic.make_rows(512, centers, gen, dtype=torch.bfloat16).cuda()
    S, J = rows.shape
    r, C = encoder.shape[0], stored.shape[0]
    codes = torch.zeros(S, r // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(S, 1, dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros(S, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (_ptr(rows), ops.dtype_code(rows.dtype), _ptr(stored), C, _ptr(mean), _ptr(encoder),
            ops.dtype_code(encoder.dtype), S, J, r, r, 1e-12, _lib.NKV_QUANT_F32, _lib.NKV_BF16, 1, 0,
            _ptr(codes), _ptr(scales), _ptr(ids), stream)
    _lib.check(lib.nkv_encode_append_static(*args))    # first call: symbol look-up, module load
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    _lib.check(lib.nkv_encode_append_static(*args))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
