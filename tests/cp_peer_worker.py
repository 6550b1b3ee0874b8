"""One rank of the peer-memory context-parallel exchange check (launched by
test_gpu_context_parallel.py through torch.distributed.run, one process per GPU).

Every rank fills its peer-visible partial buffers with seeded (O, lse), runs the fused
merge + all-gather kernel over peer memory and compares the result bit for bit with the plain
exchange (NCCL all-gather of whole partials, then the P-way merge kernel).  Several rounds reuse
the same buffers; one round has an empty shard (lse = -inf, O = 0) and rows empty on every rank.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    from nanokv_b200 import context_parallel
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    failures = []
    for dtype, (queries, heads, width) in ((torch.bfloat16, (301, 5, 128)),
                                           (torch.float32, (64, 3, 64)),
                                           (torch.bfloat16, (1, 1, 8))):
        exchange = context_parallel.PeerExchange(queries, heads, width, dtype, device)
        for round_index in range(3):
            gen = torch.Generator().manual_seed(1000 * round_index + rank)
            out = torch.randn(queries, heads, width, generator=gen).to(dtype)
            lse = torch.randn(queries, heads, generator=gen) * 3.0
            if round_index == 1:
                if rank == world - 1:                    # an empty shard
                    out.zero_()
                    lse.fill_(float("-inf"))
                lse[0].fill_(float("-inf"))              # a row empty on every rank
                out[0].zero_()
            exchange.partial_out.copy_(out.to(device))
            exchange.partial_lse.copy_(lse.to(device))
            got_out, got_lse = exchange.merge()
            want_out, want_lse = context_parallel.gather_and_merge(
                exchange.partial_out.clone(), exchange.partial_lse.clone())
            torch.cuda.synchronize()
            if not (torch.equal(got_out.view(torch.uint8), want_out.view(torch.uint8))
                    and torch.equal(got_lse.view(torch.int32), want_lse.view(torch.int32))):
                failures.append((str(dtype), round_index))
        exchange.close()
    flag = torch.tensor([len(failures)], device=device)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    if failures:
        print(f"rank {rank}: peer merge differs from all-gather + merge in {failures}", file=sys.stderr)
    return 1 if int(flag.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
