"""Context-parallel exchange on the GPU: the peer-memory merge kernel against the plain merge
kernel (one GPU, ranks emulated by local buffers) and, where the box has two GPUs, two real
ranks mapping each other's buffers."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_peer_merge_matches_lse_merge_bitwise(world, dtype):
    from nanokv_b200 import context_parallel, ops
    device = torch.device("cuda", 0)
    queries, heads, width = 77, 3, 64
    rows = queries * heads
    gen = torch.Generator().manual_seed(7 + world)
    parts = []
    for p in range(world):
        out = torch.randn(queries, heads, width, generator=gen).to(dtype).to(device)
        lse = (torch.randn(queries, heads, generator=gen) * 4.0).to(device)
        if p == world - 1 and world > 1:
            lse[5:9] = float("-inf")
            out[5:9] = 0
        parts.append((out, lse))
    for out, lse in parts:                          # rows empty in every partition
        lse[0] = float("-inf")
        out[0] = 0
    want_out, want_lse = ops.lse_merge(parts)
    # every emulated rank merges its slice into every rank's result buffer
    results = [(torch.full_like(parts[0][0], float("nan")), torch.full_like(parts[0][1], float("nan")))
               for _ in range(world)]
    for r, (begin, end) in enumerate(context_parallel.shard_bounds(rows, world)):
        ops.cp_merge_peer([o.data_ptr() for o, _ in parts], [l.data_ptr() for _, l in parts],
                          [o.data_ptr() for o, _ in results], [l.data_ptr() for _, l in results],
                          rows=rows, width=width, row_begin=begin, row_end=end, dtype=dtype,
                          device=device)
    torch.cuda.synchronize()
    for got_out, got_lse in results:
        assert torch.equal(got_out.view(torch.uint8), want_out.view(torch.uint8))
        assert torch.equal(got_lse.view(torch.int32), want_lse.view(torch.int32))
    assert torch.isinf(want_lse[0]).all() and (want_out[0] == 0).all()


def test_peer_merge_rejects_bad_arguments():
    from nanokv_b200 import ops
    device = torch.device("cuda", 0)
    out = torch.zeros(4, 1, 8, dtype=torch.bfloat16, device=device)
    lse = torch.zeros(4, 1, device=device)
    ptrs = ([out.data_ptr()], [lse.data_ptr()], [out.data_ptr()], [lse.data_ptr()])
    with pytest.raises(ValueError):
        ops.cp_merge_peer(*ptrs, rows=4, width=8, row_begin=3, row_end=9, dtype=torch.bfloat16,
                          device=device)
    with pytest.raises(ValueError):
        ops.cp_merge_peer(*ptrs, rows=4, width=12, row_begin=0, row_end=4, dtype=torch.bfloat16,
                          device=device)
    with pytest.raises(ValueError, match="not 16-byte aligned"):   # partial / result pointers off by 2 bytes
        ops.cp_merge_peer(*[[v + 2 for v in p] for p in ptrs], rows=4, width=8, row_begin=0, row_end=4,
                          dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError):                                  # more ranks than the kernel folds
        ops.cp_merge_peer(*[p * 17 for p in ptrs], rows=4, width=8, row_begin=0, row_end=4,
                          dtype=torch.bfloat16, device=device)


def test_peer_buffer_tensor_window():
    from nanokv_b200 import ops
    device = torch.device("cuda", 0)
    block = ops.PeerBuffer.allocate(4096, device)
    assert len(block.handle) == 64
    a = block.tensor(0, (8, 16), torch.float32)
    b = block.tensor(512, (8, 16), torch.float32)
    a.fill_(3.0)
    b.copy_(a * 2)
    torch.cuda.synchronize()
    assert float(block.tensor(512, (128,), torch.float32).sum()) == 768.0
    with pytest.raises(ValueError):
        block.tensor(4000, (64,), torch.float32)
    del a, b
    block.release()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_exchange_over_peer_memory():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    port = 29600 + os.getpid() % 1000
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(port),
         str(ROOT / "tests" / "cp_peer_worker.py")],
        env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]


def test_flag_ordered_exchange_of_one_rank_matches_the_merge():
    """world = 1: the flag protocol is satisfied by the rank itself; the result is the plain merge's."""
    from nanokv_b200 import ops
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    out = torch.randn(50, 2, 64, generator=gen).to(torch.bfloat16).to(device)
    lse = torch.randn(50, 2, generator=gen).to(device)
    got_out, got_lse = torch.full_like(out, float("nan")), torch.full_like(lse, float("nan"))
    flags = torch.zeros(ops.PEER_FLAG_WORDS, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for epoch in (1, 2, 3):                                   # the same buffers, call after call
        ops.cp_exchange_peer([out.data_ptr()], [lse.data_ptr()], [got_out.data_ptr()], [got_lse.data_ptr()],
                             [flags.data_ptr()], rank=0, rows=100, width=64, row_begin=0, row_end=100,
                             dtype=torch.bfloat16, epoch=epoch, device=device, status=status)
    torch.cuda.synchronize()
    want_out, want_lse = ops.lse_merge([(out, lse)])
    assert int(status.item()) == 0
    assert torch.equal(got_out.view(torch.int16), want_out.view(torch.int16))
    assert torch.equal(got_lse, want_lse)
    assert flags[:1].tolist() == [3] and flags[16:17].tolist() == [3] and int(flags[32]) == 0


def test_exchange_gives_up_when_a_peer_never_arrives():
    """Two ranks' buffers on one GPU, only rank 0's kernel runs: rank 1 never reports its partial, so
    rank 0's wait runs out of its (short) budget, the kernel returns without merging and the status
    word names the wait site.  Nothing hangs or faults; the context stays usable."""
    from nanokv_b200 import _lib, ops
    device = torch.device("cuda", 0)
    parts = [(torch.ones(8, 1, 8, dtype=torch.bfloat16, device=device), torch.zeros(8, 1, device=device))
             for _ in range(2)]
    results = [(torch.full((8, 1, 8), 5.0, dtype=torch.bfloat16, device=device),
                torch.full((8, 1), 5.0, device=device)) for _ in range(2)]
    flags = [torch.zeros(ops.PEER_FLAG_WORDS, dtype=torch.int32, device=device) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ops.cp_exchange_peer([o.data_ptr() for o, _ in parts], [l.data_ptr() for _, l in parts],
                         [o.data_ptr() for o, _ in results], [l.data_ptr() for _, l in results],
                         [f.data_ptr() for f in flags], rank=0, rows=8, width=8, row_begin=0, row_end=4,
                         dtype=torch.bfloat16, epoch=1, device=device, status=status, budget_cycles=1 << 17)
    torch.cuda.synchronize()
    assert int(status.item()) == 980
    assert all(bool((o == 5.0).all()) and bool((l == 5.0).all()) for o, l in results)   # nothing merged
    assert flags[1][0].item() == 1                      # rank 0 did announce its partial to rank 1
    with pytest.raises(RuntimeError, match="device-side wait"):
        _lib.check_device_status(int(status.item()))
    assert float(torch.ones(3, device=device).sum()) == 3.0
