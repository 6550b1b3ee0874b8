"""Context-parallel host logic on CPU: world_size-2 gloo ranks shard the history by frames,
gather (O, lse) partials and merge them; the result must equal the unsplit attention.

The device merge kernel is exercised by the GPU tests; here the gathered partials are merged by
the oracle's fold of the reference's two-way merge, which is the arithmetic statement of the
exchange step.
"""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank: int, world: int, port: int, frames: int, results):
    sys.path.insert(0, str(ROOT))
    from nanokv_b200 import context_parallel
    from oracle import nkv_oracle as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                      # identical tensors on every rank
        frame, heads, dim, queries = 37, 2, 32, 50
        q = torch.randn(1, heads, queries, dim)
        k = torch.randn(1, heads, frames * frame, dim)
        v = torch.randn(1, heads, frames * frame, dim)
        start, stop = context_parallel.shard_bounds(frames, world)[rank]
        out, lse = oracle.attention_lse(q, k[:, :, start * frame:stop * frame],
                                        v[:, :, start * frame:stop * frame])
        partials = context_parallel.gather_partials(out, lse)
        assert len(partials) == world
        merged, merged_lse = oracle.merge_many(partials)
        whole, whole_lse = oracle.attention_lse(q, k, v)
        results[rank] = (float((merged - whole).abs().max()),
                         float((merged_lse - whole_lse).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("frames", [5, 1])       # 1 frame over 2 ranks: one shard is empty
def test_two_rank_gather_and_merge(frames):
    manager = mp.Manager()
    results = manager.dict()
    port = 29500 + (os.getpid() % 2000) + frames
    mp.spawn(_worker, args=(2, port, frames, results), nprocs=2, join=True)
    assert sorted(results.keys()) == [0, 1]
    for err, lse_err in results.values():
        assert err < 1e-5 and lse_err < 1e-5


def test_shard_bounds_are_contiguous_and_balanced():
    from nanokv_b200.context_parallel import shard_bounds
    for units in (0, 1, 7, 64):
        for world in (1, 2, 3, 8):
            bounds = shard_bounds(units, world)
            assert bounds[0][0] == 0 and bounds[-1][1] == units
            assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
            sizes = [b - a for a, b in bounds]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 0)
