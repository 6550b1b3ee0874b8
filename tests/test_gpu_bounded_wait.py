"""The bounded device-side waits are seen to give up.

Every wait inside the fused read (on a shared-memory barrier, on a counter another CTA advances)
carries a cycle budget; when it runs out the kernel records the wait site, drains and returns.
Here the two kinds of wait run on their own with a short budget and nobody to satisfy them: the
kernel must come back, report the site, and leave the context usable.  Nothing faults or hangs.
"""
import ctypes

import pytest
import torch

from nanokv_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,site", [(0, 990), (1, 991)], ids=["barrier", "global-counter"])
def test_a_wait_nobody_satisfies_gives_up_and_reports_its_site(kind, site):
    lib = _lib.library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.nkv_selftest_bounded_wait(kind, 1 << 17, ctypes.c_void_p(status.data_ptr()), stream))
    torch.cuda.synchronize()                       # returns: the kernel did not hang
    assert int(status.item()) == site
    # the context is still usable, and the status maps to the ABI's error class
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    with pytest.raises(RuntimeError, match="device-side wait"):
        _lib.check_device_status(int(status.item()))


def test_the_wait_self_test_rejects_bad_arguments():
    lib = _lib.library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for kind, budget in ((2, 1000), (0, 0), (1, 1 << 40)):
        assert lib.nkv_selftest_bounded_wait(kind, budget, ctypes.c_void_p(status.data_ptr()), None) \
            == _lib.NKV_ERR_INVALID
