"""Headline benchmark: fused INT4 codec-attention (and encode) on the Wan-shaped history.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of codec-attention over every layer's compressed history
(99,840 tokens per layer, 4,680 queries, 40 layers, H 40 x D 128, rank 640,
512 centres) on synthetic, seeded inputs.  With N > 1 (torchrun) the history
is sharded by token range over the ranks; each rank attends its shard, the
(O, lse) partials are all-gathered over NCCL and merged by log-sum-exp.
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from nanokv_b200 import synthetic  # noqa: E402

SHAPE = synthetic.CONFIGS["c3_wan_shaped"]
FRAME = 1560
METRIC = "codec_attention_history_tokens_per_s"
UNIT = "history-tokens/s"


def measured_traffic(kernel: str, workload: str):
    """DRAM bytes per launch of `kernel` on `workload`, from the figures file written next to the ncu
    summary of that kernel (dram__bytes_read.sum + dram__bytes_write.sum of one launch); None when
    no capture of the kernel as built is on record."""
    path = ROOT / "profiles" / "ncu_figures.json"
    if not path.exists():
        return None
    try:
        entry = json.loads(path.read_text()).get(f"{kernel}:{workload}")
    except (ValueError, AttributeError):
        return None
    return None if entry is None else entry.get("dram_bytes_per_launch")


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def attention_flops(tokens: int, queries: int, joint: int, rank: int) -> float:
    """Algorithmic flops of one layer: QK^T + PV (4*Q*J) plus one decode of K and V (4*r*J)."""
    return float(tokens) * (4.0 * queries * joint + 4.0 * rank * joint)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, peak, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 9:
                continue
            try:
                clocks.append(float(row[1]))
                peak = float(row[2])
            except ValueError:
                continue
            for name, flag in zip(names, row[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "samples": len(clocks), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------- workload
def rope_freqs(rows: int, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [rows, head_dim/2]: temporal, vertical and horizontal bands side by side."""
    def band(dim):
        angles = torch.outer(torch.arange(rows),
                             1.0 / torch.pow(theta, torch.arange(0, dim, 2).to(torch.float64).div(dim)))
        return torch.polar(torch.ones_like(angles), angles)
    d = head_dim
    return torch.cat([band(d - 4 * (d // 6)), band(2 * (d // 6)), band(2 * (d // 6))], dim=1)


def build_layers(shape, frames: range, layers: int, device, encode_frames: int = 8):
    """Encode this rank's frames of every layer into compressed histories (fixed centres).

    Returns (layer list, seconds spent in encode kernels, tokens encoded).  Rows are
    drawn on the device from a seeded generator: centre[uniform id] + 0.3 * N(0,1).
    """
    from nanokv_b200.cache import CompressedHistory
    from nanokv_b200.codec import Operator, QuantSpec, encode_append
    gen = torch.Generator(device=device).manual_seed(1234)
    tokens = len(frames) * FRAME
    segments = (len(frames) + encode_frames - 1) // encode_frames
    result = []
    quant = QuantSpec()
    for layer in range(layers):
        entry = {}
        for kind in ("k", "v"):
            cpu_gen = synthetic.generator(1000 * layer + (kind == "v"))
            operator = synthetic.make_operator(shape, cpu_gen)
            op = Operator(operator["mean"], operator["encoder"], operator["decoder"], device=device)
            centers = torch.randn(shape.centers, shape.joint, generator=gen, device=device)
            hist = CompressedHistory(joint=shape.joint, rank=shape.rank, capacity=max(tokens, 1),
                                     max_segments=max(segments, 1),
                                     centers_per_segment=shape.centers, device=device,
                                     shared_centers=True)
            hist.centers.copy_(centers.to(torch.bfloat16))
            for first in range(0, len(frames), encode_frames):
                count = min(encode_frames, len(frames) - first) * FRAME
                pick = torch.randint(shape.centers, (count,), generator=gen, device=device)
                rows = centers.index_select(0, pick)
                rows.add_(torch.randn(count, shape.joint, generator=gen, device=device), alpha=0.3)
                encode_append(hist, rows.to(torch.bfloat16), op, quant, centers="resident")
            entry[kind] = (hist, op)
        result.append(entry)
    return result


def time_encode(shape, device, steps: int, warmup: int, frames: int = 8):
    """Encode tokens/s: K and V rows of `frames` frames (fixed centres), device resident."""
    from nanokv_b200.cache import CompressedHistory
    from nanokv_b200.codec import Operator, QuantSpec, encode_append
    gen = torch.Generator(device=device).manual_seed(77)
    cpu_gen = synthetic.generator(5)
    operator = synthetic.make_operator(shape, cpu_gen)
    op = Operator(operator["mean"], operator["encoder"], operator["decoder"], device=device)
    centers = torch.randn(shape.centers, shape.joint, generator=gen, device=device)
    count = frames * FRAME
    pick = torch.randint(shape.centers, (count,), generator=gen, device=device)
    rows = (centers.index_select(0, pick) +
            0.3 * torch.randn(count, shape.joint, generator=gen, device=device)).to(torch.bfloat16)
    total = steps + warmup
    hist = CompressedHistory(joint=shape.joint, rank=shape.rank, capacity=count * total * 2,
                             max_segments=2 * total, centers_per_segment=shape.centers,
                             device=device, shared_centers=True)
    hist.centers.copy_(centers.to(torch.bfloat16))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for index in range(total):
        if index == warmup:
            torch.cuda.synchronize()
            start.record()
        encode_append(hist, rows, op, QuantSpec(), centers="resident")   # "K"
        encode_append(hist, rows, op, QuantSpec(), centers="resident")   # "V"
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / steps
    # the HBM-bound stage alone: quantise + pack of 399,360 tokens' coefficients (inputs > L2)
    from nanokv_b200 import ops
    coeff = torch.randn(399360, shape.rank, generator=gen, device=device).to(torch.bfloat16)
    codes = torch.empty(coeff.shape[0], shape.rank // 2, dtype=torch.uint8, device=device)
    scales = torch.empty(coeff.shape[0], 1, dtype=torch.bfloat16, device=device)
    q_start, q_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for index in range(3 + 5):
        if index == 3:
            q_start.record()
        ops.quant_pack(coeff, codes=codes, scales=scales)
    q_stop.record()
    torch.cuda.synchronize()
    quant_seconds = q_start.elapsed_time(q_stop) / 1e3 / 5
    quant_bytes = coeff.shape[0] * (shape.rank * 2 + shape.rank // 2 + 2)
    # the same with Matrix-Game's rule (quotient rounded to bf16 before rint)
    for index in range(3 + 5):
        if index == 3:
            q_start.record()
        ops.quant_pack(coeff, codes=codes, scales=scales, in_coeff_dtype=True)
    q_stop.record()
    torch.cuda.synchronize()
    quant_bf16_seconds = q_start.elapsed_time(q_stop) / 1e3 / 5
    del coeff, codes, scales
    # online C-means form (the reference's encode_tensor: 2 iterations from a seeded permutation,
    # then projection + quantiser): one chunk (1 frame) and one encode call (`frames` frames)
    from nanokv_b200.codec import kmeans_init_rows
    online = {}
    for label, tokens in (("chunk", FRAME), ("call", count)):
        piece = rows[:tokens].contiguous()
        clusters = min(shape.centers, 256)
        target = CompressedHistory(joint=shape.joint, rank=shape.rank, capacity=tokens * 8, max_segments=8,
                                   centers_per_segment=clusters, device=device)
        k_start, k_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for index in range(3 + 5):
            if index == 3:
                k_start.record()
            encode_append(target, piece, op, QuantSpec(), clusters=clusters, iters=2, seed=20260804)
        k_stop.record()
        torch.cuda.synchronize()
        online[label] = tokens / (k_start.elapsed_time(k_stop) / 1e3 / 5)
    flops = count * 2 * 2.0 * shape.joint * (shape.centers + shape.rank)
    bytes_ = count * 2 * (shape.joint * 2 + shape.rank // 2 + 2 + 2)
    return {"tokens_per_s": count / seconds, "ms": seconds * 1e3, "tokens_per_call": count,
            "tflops": flops / seconds / 1e12, "gbs": bytes_ / seconds / 1e9,
            "fused": True,
            "form": "given centres: assign kernel, then projection + quantise + pack in one kernel",
            "quant_pack_gbs": quant_bytes / quant_seconds / 1e9,
            "quant_pack_bf16_rule_gbs": quant_bytes / quant_bf16_seconds / 1e9,
            "quant_pack_tokens": 399360,
            "kmeans_tokens_per_s": online["call"], "kmeans_tokens_per_s_one_frame": online["chunk"],
            "kmeans_form": "online C-means (256 centres, 2 iterations, host-seeded start rows) + projection "
                           "+ quantise + pack, per encode call of %d tokens / of one frame" % count}


def run_ours(args) -> dict:
    import torch.distributed as dist
    from nanokv_b200 import attention, context_parallel
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        # keep stdout to the one JSON line (NCCL prints its version banner there at VERSION level)
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)
    shape, layers = SHAPE, args.layers
    total_frames = args.history_frames or shape.history // FRAME
    history_tokens = total_frames * FRAME
    bounds = context_parallel.shard_bounds(total_frames, world)
    frames = range(*bounds[rank])
    built = build_layers(shape, frames, layers, device)
    local_tokens = len(frames) * FRAME
    gen = synthetic.generator(4242)
    q_host = synthetic.make_queries(shape, gen).pin_memory()          # same queries on every rank
    q_dev = q_host.to(device, non_blocking=True)
    out_host = torch.empty(shape.queries, shape.heads, shape.head_dim, dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty(shape.queries, shape.heads, dtype=torch.float32).pin_memory()
    status = torch.zeros(1, dtype=torch.int32, device=device)
    rope_args = {}
    if args.rope:   # positional restore inside the read: 30 x 52 token frames, this rank's positions
        table = attention.RopeTable(rope_freqs(1024, shape.head_dim), frame_seqlen=FRAME, width=52,
                                    device=device)
        start = frames.start * FRAME
        rope_args = dict(rope=table, positions=torch.arange(start, start + local_tokens,
                                                            dtype=torch.int32, device=device))
    exchange = None
    if world > 1 and args.exchange != "nccl":
        exchange = context_parallel.PeerExchange(shape.queries, shape.heads, shape.head_dim,
                                                 torch.bfloat16, device,
                                                 ordering="flags" if args.exchange == "peer" else "nccl")
        # the fused exchange must reproduce all-gather + merge bit for bit on this workload
        (hk, ok), (hv, ov) = built[0]["k"], built[0]["v"]
        attention.codec_attention(q_dev, hk, hv, ok, ov, status=status, out=exchange.partial_out,
                                  lse=exchange.partial_lse, **rope_args)
        fused_out, fused_lse = exchange.merge()
        plain_out, plain_lse = context_parallel.gather_and_merge(exchange.partial_out.clone(),
                                                                 exchange.partial_lse.clone())
        if not (torch.equal(fused_out.view(torch.int16), plain_out.view(torch.int16))
                and torch.equal(fused_lse.view(torch.int32), plain_lse.view(torch.int32))):
            raise RuntimeError("peer-memory exchange differs from all-gather + merge")

    # end-to-end I/O of a sharded job: every rank copies in its 1/P slice of the queries (then an
    # NVLink all-gather makes them whole on every rank) and copies out its 1/P slice of the merged
    # rows, so the job moves each input and result byte across PCIe once
    rows = shape.queries * shape.heads
    per_rank_q = -(-shape.queries // world)
    q_lo, q_hi = min(shape.queries, rank * per_rank_q), min(shape.queries, (rank + 1) * per_rank_q)
    row_lo, row_hi = context_parallel.shard_bounds(rows, world)[rank]
    # The copies run on their own streams: layer l+1's queries are uploaded (two buffers) and layer
    # l-1's rows downloaded while layer l attends, every copy still inside the timed region.
    upload_stream, download_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)
    if world > 1:
        q_stage = [torch.zeros(per_rank_q, shape.heads, shape.head_dim, dtype=torch.bfloat16, device=device)
                   for _ in range(2)]
        q_whole = [torch.empty(world * per_rank_q, shape.heads, shape.head_dim, dtype=torch.bfloat16,
                               device=device) for _ in range(2)]
    else:
        q_slots = [torch.empty_like(q_dev) for _ in range(2)]

    def queries_from_host(slot: int):
        """Enqueued on the upload stream; returns the device queries and the event that says they are there."""
        with torch.cuda.stream(upload_stream):
            if world == 1:
                q_slots[slot].copy_(q_host, non_blocking=True)
                q = q_slots[slot]
            else:
                q_stage[slot][:q_hi - q_lo].copy_(q_host[q_lo:q_hi], non_blocking=True)
                dist.all_gather_into_tensor(q_whole[slot], q_stage[slot])
                q = q_whole[slot][:shape.queries]
            landed = torch.cuda.Event()
            landed.record(upload_stream)
        return q, landed

    def attend_layer(entry, q):
        (hk, ok), (hv, ov) = entry["k"], entry["v"]
        if exchange is not None:
            attention.codec_attention(q, hk, hv, ok, ov, status=status, **rope_args,
                                      out=exchange.partial_out, lse=exchange.partial_lse)
            return None
        return attention.codec_attention(q, hk, hv, ok, ov, status=status, **rope_args)

    def merge_layer(partial):
        if exchange is not None:
            return exchange.merge()
        return context_parallel.gather_and_merge(*partial)

    def step(host_io: bool):
        merged = None
        if not host_io:
            for entry in built:
                merged = merge_layer(attend_layer(entry, q_dev))
            return merged
        main = torch.cuda.current_stream(device)
        upload_stream.wait_stream(main)
        download_stream.wait_stream(main)
        slot_free = [None, None]          # the attention that read this query buffer has run
        drained = None                    # the previous layer's rows have left the merged buffers
        q_next, landed = queries_from_host(0)
        for index, entry in enumerate(built):
            slot = index & 1
            q = q_next
            main.wait_event(landed)
            if index + 1 < len(built):
                if slot_free[slot ^ 1] is not None:
                    upload_stream.wait_event(slot_free[slot ^ 1])
                q_next, landed = queries_from_host(slot ^ 1)
            partial = attend_layer(entry, q)
            slot_free[slot] = torch.cuda.Event()
            slot_free[slot].record(main)
            if drained is not None:
                main.wait_event(drained)
            merged = merge_layer(partial)
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(download_stream):
                download_stream.wait_event(ready)
                out_host.view(rows, -1)[row_lo:row_hi].copy_(
                    merged[0].view(rows, -1)[row_lo:row_hi], non_blocking=True)
                lse_host.view(rows)[row_lo:row_hi].copy_(merged[1].view(rows)[row_lo:row_hi],
                                                         non_blocking=True)
                drained = torch.cuda.Event()
                drained.record(download_stream)
            merged[0].record_stream(download_stream)
            merged[1].record_stream(download_stream)
        main.wait_event(drained)
        return merged

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(host_io: bool, steps: int, warmup: int) -> float:
        for _ in range(warmup):
            step(host_io)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step(host_io)
        stop.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / 1e3

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    seconds = timed(False, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    e2e_seconds = timed(True, max(1, args.steps // 2), 1)
    e2e_steps = max(1, args.steps // 2)
    # the overlapped copies must have delivered the last layer's rows
    merged = step(True)
    barrier()
    if not (torch.equal(out_host.view(rows, -1)[row_lo:row_hi], merged[0].view(rows, -1)[row_lo:row_hi].cpu())
            and torch.equal(lse_host.view(rows)[row_lo:row_hi], merged[1].view(rows)[row_lo:row_hi].cpu())):
        raise RuntimeError("end-to-end path: the rows on the host differ from the rows on the device")
    if int(status.item()) != 0:
        raise RuntimeError(f"device-side wait gave up at site {int(status.item())}")

    # the dominant kernel alone, on this rank's shard: per-launch duration for the roofline
    kernel_ms = []
    entry = built[0]
    (hk, ok), (hv, ov) = entry["k"], entry["v"]
    for index in range(3 + 5):
        other = built[index % len(built)]
        (hk, ok), (hv, ov) = other["k"], other["v"]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        attention.codec_attention(q_dev, hk, hv, ok, ov, status=status, **rope_args)
        stop.record()
        torch.cuda.synchronize()
        if index >= 3:
            kernel_ms.append(start.elapsed_time(stop))
    kernel_s = statistics.mean(kernel_ms) / 1e3

    # the exchange step alone (collective: every rank runs it), max over ranks
    exchange_ms = None
    if world > 1:
        part_out, part_lse = attention.codec_attention(q_dev, hk, hv, ok, ov, status=status)
        if exchange is not None:
            exchange.partial_out.copy_(part_out)
            exchange.partial_lse.copy_(part_lse)
        rounds = 10
        for index in range(2 + rounds):
            if index == 2:
                barrier()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            if exchange is not None:
                exchange.merge()
            else:
                context_parallel.gather_and_merge(part_out, part_lse)
        stop.record()
        barrier()
        took = torch.tensor([start.elapsed_time(stop) / rounds], device=device)
        dist.all_reduce(took, op=dist.ReduceOp.MAX)
        exchange_ms = float(took.item())
    # every rank encodes the chunks it owns (ownership is by chunk, no data-path exchange), so the
    # job's encode rate is the sum over ranks; measured on all ranks at once
    if world > 1:
        dist.barrier()
    encode = time_encode(shape, device, steps=5, warmup=3)
    if world > 1:
        rates = torch.tensor([encode["tokens_per_s"], encode["kmeans_tokens_per_s"]], device=device)
        slowest = rates.clone()
        dist.all_reduce(rates, op=dist.ReduceOp.SUM)
        dist.all_reduce(slowest, op=dist.ReduceOp.MIN)
        encode["all_ranks_tokens_per_s"] = float(rates[0].item())
        encode["all_ranks_kmeans_tokens_per_s"] = float(rates[1].item())
        encode["slowest_rank_tokens_per_s"] = float(slowest[0].item())
    else:
        encode["all_ranks_tokens_per_s"] = encode["tokens_per_s"]
        encode["all_ranks_kmeans_tokens_per_s"] = encode["kmeans_tokens_per_s"]
    encode["ranks"] = world

    # the same end-to-end step with the copies IN LINE on the compute stream: queries in, attention,
    # rows out, layer after layer -- what a layer stack whose next queries depend on this layer's
    # output pays (the overlapped form above is the upper bound a pipelined caller can reach)
    def step_inline():
        merged = None
        for entry in built:
            if world > 1:
                q_stage[0][:q_hi - q_lo].copy_(q_host[q_lo:q_hi], non_blocking=True)
                dist.all_gather_into_tensor(q_whole[0], q_stage[0])
                q = q_whole[0][:shape.queries]
            else:
                q_slots[0].copy_(q_host, non_blocking=True)
                q = q_slots[0]
            merged = merge_layer(attend_layer(entry, q))
            out_host.view(rows, -1)[row_lo:row_hi].copy_(merged[0].view(rows, -1)[row_lo:row_hi],
                                                         non_blocking=True)
            lse_host.view(rows)[row_lo:row_hi].copy_(merged[1].view(rows)[row_lo:row_hi], non_blocking=True)
        return merged

    step_inline()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(e2e_steps):
        step_inline()
    stop.record()
    barrier()
    inline_ms = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(inline_ms, op=dist.ReduceOp.MAX)
    inline_seconds = float(inline_ms.item()) / 1e3

    # parity of what was timed, on rank 0: the first frames of layer 0's history through the fused
    # read against the CPU oracle on a strided subset of the query rows, and (one GPU) the stock
    # torch GPU path on the whole layer as the comparison arm
    parity, gpu_ref = None, None
    if rank == 0 and not args.no_cpu:
        parity = parity_sample(shape, built[0], q_dev, q_host)
    if rank == 0 and world == 1 and not args.no_gpu_reference:
        gpu_ref = gpu_reference(shape, built[0], q_dev)
        ours = attention.codec_attention(q_dev, built[0]["k"][0], built[0]["v"][0], built[0]["k"][1],
                                         built[0]["v"][1])[0]
        theirs = gpu_ref.pop("out", None)
        if theirs is not None:
            gpu_ref["rel_diff_vs_fused"] = float((ours.float() - theirs.float()).abs().max() /
                                                 theirs.float().abs().max())
        del ours, theirs
        torch.cuda.empty_cache()

    if exchange is not None:
        exchange.close()
    del built
    torch.cuda.empty_cache()
    if rank != 0:
        return {}
    peaks, peak_kind = measured_peaks()
    step_ms = seconds / args.steps * 1e3
    tokens_per_step = history_tokens * layers
    flops_launch = attention_flops(local_tokens, shape.queries, shape.joint, shape.rank)
    achieved = flops_launch / kernel_s / 1e12
    peak = float(peaks["bf16_tflops_sustained"])
    q_bytes = q_host.numel() * 2
    o_bytes = out_host.numel() * 2 + lse_host.numel() * 4
    cpu = cpu_baseline(shape) if world == 1 and not args.no_cpu else None
    line = {
        "metric": METRIC, "value": tokens_per_step / (seconds / args.steps), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": shape.name, "heads": shape.heads, "head_dim": shape.head_dim,
                   "rank": shape.rank, "centers": shape.centers, "history_tokens": history_tokens,
                   "queries": shape.queries, "layers": layers, "quant_group": shape.rank,
                   "scale_dtype": "bf16", "parallelism": f"cp{world}",
                   "positional_restore": "3-D RoPE of the rebuilt keys inside the read" if args.rope else "none",
                   "exchange": ("none" if world == 1 else
                                "peer-memory merge + all-gather kernel, ranks ordered by flag words in peer memory"
                                if exchange is not None and args.exchange == "peer" else
                                "peer-memory merge + all-gather kernel between two NCCL all-reduces"
                                if exchange is not None else "nccl all-gather + merge kernel"),
                   "e2e_io": (("whole queries in, whole (O, lse) out" if world == 1 else
                               "each rank copies its 1/P slice of the queries in (NVLink all-gather "
                               "makes them whole) and its 1/P slice of the merged rows out; bytes are "
                               "job totals") + "; every layer's copies are inside the timed region, on "
                              "their own streams, overlapping the neighbouring layers' attention"),
                   "l2_policy": "inputs larger than L2 (distinct compressed history per layer)"},
        "e2e": {"value": tokens_per_step / (e2e_seconds / e2e_steps), "unit": UNIT,
                "h2d_bytes_per_step": q_bytes * layers, "d2h_bytes_per_step": o_bytes * layers},
        "e2e_inline": {"value": tokens_per_step / (inline_seconds / e2e_steps), "unit": UNIT,
                       "note": "copies in line on the compute stream, no overlap with other layers"},
        # per layer: fused attention + LSE merge of its history splits (+ the CP merge when sharded)
        "gpu_launches": args.steps * layers * (2 + (1 if world > 1 else 0)),
        "exchange_ms_per_layer": exchange_ms,
        "roofline": {"bound": "tensor", "kernel": "attn_codec_kernel<128>", "achieved": achieved,
                     "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_source": f"bf16_tflops_sustained of {peak_kind}",
                     "launch_ms": kernel_s * 1e3, "flops_per_launch": flops_launch,
                     # DRAM bytes of one launch over the full layer from an ncu capture of this
                     # kernel, when one is on record (per-rank shards are not captured separately)
                     "traffic": (measured_traffic("attn_codec_kernel", shape.name)
                                 if world == 1 and not args.history_frames else None)},
        "encode": encode,
        "clocks": clocks,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    if parity:
        line["parity"] = parity
    if gpu_ref:
        line["gpu_reference"] = gpu_ref
    return line


# ------------------------------------------------------------------ CPU baseline / reference arm
def cpu_sample(shape, sample_tokens: int):
    """The oracle port (CPU restatement of the reference) on a history subsample, all host threads."""
    from oracle import nkv_oracle as oracle
    torch.set_num_threads(os.cpu_count() or 1)
    gen = synthetic.generator(9)
    segments, ops_ = {"k": [], "v": []}, {}
    for kind in ("k", "v"):
        centers = synthetic.make_centers(shape, gen)
        rows = synthetic.make_rows(sample_tokens, centers, gen, dtype=torch.bfloat16)
        ops_[kind] = synthetic.make_operator(shape, gen)
        segments[kind].append(oracle.encode_rows(
            rows[None], encoder=ops_[kind]["encoder"], mean=ops_[kind]["mean"],
            centers=centers[None].to(torch.bfloat16), eps=oracle.F32_EPS))
    q = synthetic.make_queries(shape, gen)

    def run():
        return oracle.codec_attention(
            q[None], segments["k"], segments["v"], k_decoder=ops_["k"]["decoder"],
            k_mean=ops_["k"]["mean"], v_decoder=ops_["v"]["decoder"], v_mean=ops_["v"]["mean"],
            heads=shape.heads, dtype=torch.bfloat16)
    return run


def cpu_baseline(shape, sample_tokens: int = 2048, runs: int = 2) -> dict:
    run = cpu_sample(shape, sample_tokens)
    run()
    times = []
    for _ in range(runs):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    seconds = statistics.median(times)
    return {"value": sample_tokens / seconds, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"one layer, {sample_tokens}-token history subsample x {shape.queries} queries, "
                      f"decode K+V + tiled attention; linear in history length"}


def run_reference(args) -> dict:
    """Reference arm: the reference's CPU arithmetic (oracle port; the reference itself is a
    Python tree that is not present on the benchmark host) on a bounded sample per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    shape = SHAPE
    sample = 1024
    run = cpu_sample(shape, sample)
    for _ in range(min(args.warmup, 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    seconds = (time.perf_counter() - t0) / args.steps
    value = sample / seconds
    desc = (f"one layer, {sample}-token history subsample x {shape.queries} queries per step, "
            f"decode K+V + tiled attention; linear in history length")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": shape.name, "heads": shape.heads, "head_dim": shape.head_dim,
                   "rank": shape.rank, "centers": shape.centers, "history_tokens": shape.history,
                   "queries": shape.queries, "layers": args.layers, "sample_tokens": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }



# ------------------------------------------------------------------ parity of the timed path
def parity_sample(shape, entry, q_dev, q_host, frames: int = 4, stride: int = 73) -> dict:
    """The fused read over the first `frames` frames of a layer's history (a view of the cache the
    bench times) against the CPU oracle reading the same codes, on every `stride`-th query row."""
    from nanokv_b200 import attention
    from oracle import nkv_oracle as oracle
    (hk, ok), (hv, ov) = entry["k"], entry["v"]
    tokens = min(frames * FRAME, hk.tokens)
    out, lse = attention.codec_attention(q_dev, hk.view_tokens(0, tokens), hv.view_tokens(0, tokens), ok, ov)
    torch.cuda.synchronize()
    rows = torch.arange(0, shape.queries, stride)

    def segment(hist):
        codes = hist.codes[:tokens].cpu()
        return {"shape": (1, tokens, shape.joint), "rank": hist.rank, "packed": codes.reshape(-1),
                "count": tokens * hist.rank, "scale": hist.scales[:tokens].cpu(),
                "centers": hist.centers[:hist.centers_per_segment].cpu()[None],
                "ids": hist.ids[:tokens].cpu().to(torch.int64).bitwise_and(0xFFFF)[None]}

    torch.set_num_threads(os.cpu_count() or 1)
    want, want_lse = oracle.codec_attention(
        q_host[rows][None], [segment(hk)], [segment(hv)], k_decoder=ok.decoder.cpu(), k_mean=ok.mean.cpu(),
        v_decoder=ov.decoder.cpu(), v_mean=ov.mean.cpu(), heads=shape.heads, dtype=torch.bfloat16)
    got = out.cpu()[rows].float()
    rel = float((got - want[0].float()).abs().max() / want[0].float().abs().max())
    lse_err = float((lse.cpu()[rows] - want_lse[0].t()).abs().max())
    if not (rel <= 2e-2 and lse_err <= 2e-2):
        raise RuntimeError(f"fused read differs from the oracle: rel {rel:.3e}, lse {lse_err:.3e}")
    return {"parity_rel_err": rel, "lse_abs_err": lse_err, "tolerance": 2e-2,
            "sample": f"layer 0, first {tokens} history tokens, {rows.numel()} of {shape.queries} query "
                      f"rows x {shape.heads} heads, against the CPU oracle"}


# ------------------------------------------------------------------ GPU comparison arm
def gpu_reference(shape, entry, q, steps: int = 3, warmup: int = 2) -> dict:
    """The reference's own GPU arithmetic for one layer with stock torch operators, per stage:
    nibble unpack x bf16 scale, F.linear with the decoder and the bf16 mean, centre add (K and V
    rows of history size written to HBM), then scaled-dot-product attention by the library kernel
    torch picks (MGM/nanokv_codec.py:393-455, MGC/core.py:50-53).  A comparison arm: it calls
    library kernels and is never part of the product path."""
    import torch.nn.functional as F
    (hk, ok), (hv, ov) = entry["k"], entry["v"]
    H, D = shape.heads, shape.head_dim

    def rebuild(hist, op):
        n = hist.tokens
        codes = hist.codes[:n]
        nibbles = torch.stack((codes & 0x0F, codes >> 4), dim=-1).reshape(n, hist.rank)
        latent = (nibbles.to(torch.bfloat16) - 7) * hist.scales[:n]
        rows = F.linear(latent, op.decoder, op.mean.to(torch.bfloat16))
        ids = hist.ids[:n].long() & 0xFFFF
        rows += hist.centers.index_select(0, ids)
        return rows.view(n, H, D)

    def attend(k, v, backend):
        qq, kk, vv = (t.permute(1, 0, 2)[None] for t in (q, k, v))
        if backend == "aten_flash":
            res = torch.ops.aten._scaled_dot_product_flash_attention(qq, kk, vv, 0.0, False, False,
                                                                     scale=D ** -0.5)
            return res[0], res[1]
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            return F.scaled_dot_product_attention(qq, kk, vv, scale=D ** -0.5), None

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        # every iteration on its own: the arm allocates gigabytes of temporaries, and an iteration in
        # which the caching allocator goes back to the driver is not the library's time -- the arm
        # is credited with its best iteration
        times = []
        for _ in range(steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return min(times), out

    result = {"layer_tokens": hk.tokens}
    decode_ms, kv = timed(lambda: (rebuild(hk, ok), rebuild(hv, ov)))
    result["decode_ms"] = decode_ms
    best = None
    for backend in ("aten_flash", "cudnn"):
        try:
            ms, (out, _) = timed(lambda: attend(kv[0], kv[1], backend))
        except Exception as exc:   # the backend is not built for this GPU / shape
            result[backend + "_error"] = str(exc).splitlines()[0][:120]
            continue
        result[backend + "_attention_ms"] = ms
        if best is None or ms < best[0]:
            best = (ms, backend, out)
    if best is not None:
        result.update(attention_ms=best[0], backend=best[1], total_ms=decode_ms + best[0])
        result["out"] = best[2][0].permute(1, 0, 2)      # [Q, H, D], dropped before printing
    result["kv_hbm_bytes"] = 2 * hk.tokens * shape.joint * 2
    return result


def run_torch_gpu(args) -> dict:
    """bench.py --impl torch_gpu: one c3 layer through stock torch operators on one GPU."""
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    shape = SHAPE
    built = build_layers(shape, range(shape.history // FRAME), 1, device)
    q = synthetic.make_queries(shape, synthetic.generator(4242)).to(device)
    ref = gpu_reference(shape, built[0], q, steps=args.steps, warmup=max(args.warmup, 1))
    ref.pop("out", None)
    total = ref.get("total_ms")
    return {"impl": "torch_gpu", "metric": METRIC, "unit": UNIT,
            "value": (shape.history / (total / 1e3)) if total else None, "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": shape.name, "layers": 1},
            "gpu_reference": ref}

# ------------------------------------------------------------------ secondary workloads
def run_fast(args) -> dict:
    """c4: NanoKV-Fast mixed-dimensional read, one layer, one GPU.  History 32 frames; the last 2
    are protected (rebuilt at full width inside the fused kernel); the older 30 are read through reader
    projections: 18 heads at width 32, 6 heads at full width; partitions merged by LSE."""
    from nanokv_b200 import attention, codec
    shape = synthetic.CONFIGS["c4_fast_mixed"]
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    frames, protected = shape.history // FRAME, 2
    old = build_layers(shape, range(frames - protected), 1, device)[0]
    recent = build_layers(shape, range(protected), 1, device)[0]
    (hk, ok), (hv, ov) = old["k"], old["v"]
    (pk, _), (pv, _) = recent["k"], recent["v"]
    gen = synthetic.generator(77)
    reader = attention.Reader(
        synthetic.make_reader(shape, gen, [(list(range(18)), 32), (list(range(18, 24)), 128)],
                              k_decoder=ok.decoder.cpu(), v_decoder=ov.decoder.cpu()),
        dtype=torch.bfloat16, device=device)
    q = synthetic.make_queries(shape, gen).to(device)

    def step():
        native = [{"k": pk, "v": pv, "op_k": ok, "op_v": ov}]    # protected rows rebuilt inside the kernel
        low = [{"k": hk, "v": hv, "k_mean": ok.mean, "v_mean": ov.mean}]
        return attention.hybrid_attention(q, q, native, low, reader)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / args.steps
    peaks, peak_kind = measured_peaks()
    Q, r, D = shape.queries, shape.rank, shape.head_dim
    low_tokens, prot_tokens = (frames - protected) * FRAME, protected * FRAME
    # algorithmic flops: per low-width token and head group 4 Q d + 4 r d, per protected token the full read
    flops = (low_tokens * (18 * (4.0 * Q * 32 + 4.0 * r * 32) + 6 * (4.0 * Q * D + 4.0 * r * D)) +
             prot_tokens * (4.0 * Q * shape.joint + 4.0 * r * shape.joint))
    roofline = {"bound": "tensor", "kernel": "attn_codec_kernel<64> + attn_codec_kernel<128>",
                "achieved": flops / seconds / 1e12, "peak": float(peaks["bf16_tflops_sustained"]),
                "unit": "TFLOP/s", "frac": flops / seconds / 1e12 / float(peaks["bf16_tflops_sustained"]),
                "peak_source": f"bf16_tflops_sustained of {peak_kind}", "flops_per_layer": flops,
                "traffic": None}
    return {"roofline": roofline,
            "metric": "fast_attention_history_tokens_per_s", "value": shape.history / seconds,
            "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": shape.name, "heads": shape.heads, "rank": shape.rank,
                       "history_tokens": shape.history, "protected_tokens": protected * FRAME,
                       "queries": shape.queries, "low_heads": 18, "low_width": 32, "layers": 1}}


def run_streaming(args, standalone: bool = True) -> dict:
    """c5: streaming rollout, one layer.  Per chunk: encode + append 1,560 new K and V tokens
    (chunk c belongs to rank c % world, which encodes it into its own shard: ownership is
    round-robin by chunk, so shards stay balanced as the history grows), then 4,680-query
    codec-attention against the grown history (each rank its shard; the partials are merged by the
    peer-memory exchange, or by NCCL all-gather + merge with --exchange nccl)."""
    import torch.distributed as dist
    from nanokv_b200 import attention, context_parallel
    from nanokv_b200.cache import CompressedHistory
    from nanokv_b200.codec import Operator, QuantSpec, encode_append
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1 and standalone:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)
    shape, chunks = synthetic.CONFIGS["c5_streaming"], args.chunks
    exchange = None
    if world > 1 and args.exchange != "nccl":
        exchange = context_parallel.PeerExchange(shape.queries, shape.heads, shape.head_dim,
                                                 torch.bfloat16, device,
                                                 ordering="flags" if args.exchange == "peer" else "nccl")
    mine = (chunks + world - 1 - rank) // world
    gen = torch.Generator(device=device).manual_seed(99 + rank)
    hists, ops_ = {}, {}
    for kind in ("k", "v"):
        operator = synthetic.make_operator(shape, synthetic.generator(kind == "v"))
        ops_[kind] = Operator(operator["mean"], operator["encoder"], operator["decoder"], device=device)
        hist = CompressedHistory(joint=shape.joint, rank=shape.rank, capacity=max(mine, 1) * FRAME,
                                 max_segments=max(mine, 1), centers_per_segment=shape.centers,
                                 device=device, shared_centers=True)
        centers = torch.randn(shape.centers, shape.joint, generator=gen, device=device)
        hist.centers.copy_(centers.to(torch.bfloat16))
        hists[kind] = (hist, centers)
    q = synthetic.make_queries(shape, synthetic.generator(4242)).to(device)
    rows = {}
    for kind in ("k", "v"):
        centers = hists[kind][1]
        pick = torch.randint(shape.centers, (FRAME,), generator=gen, device=device)
        rows[kind] = (centers.index_select(0, pick) + 0.3 * torch.randn(
            FRAME, shape.joint, generator=gen, device=device)).to(torch.bfloat16)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    attended = 0
    for chunk in range(chunks):
        if chunk % world == rank:
            for kind in ("k", "v"):
                encode_append(hists[kind][0], rows[kind], ops_[kind], QuantSpec(), centers="resident")
        if exchange is not None:
            attention.codec_attention(q, hists["k"][0], hists["v"][0], ops_["k"], ops_["v"],
                                      out=exchange.partial_out, lse=exchange.partial_lse)
            exchange.merge()
        else:
            out, lse = attention.codec_attention(q, hists["k"][0], hists["v"][0], ops_["k"], ops_["v"])
            context_parallel.gather_and_merge(out, lse)
        attended += (chunk + 1) * FRAME
    stop.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if exchange is not None:
        exchange.close()
    if world > 1 and standalone:
        dist.destroy_process_group()
    if rank != 0:
        return {}
    seconds = float(ms.item()) / 1e3
    return {"metric": "streaming_history_tokens_per_s", "value": attended / seconds, "unit": UNIT,
            "n_gpus": world, "steps": chunks, "warmup": 0, "ms_per_step": seconds * 1e3 / chunks,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": shape.name, "heads": shape.heads, "rank": shape.rank,
                       "chunks": chunks, "tokens_per_chunk": FRAME, "queries": shape.queries,
                       "final_history_tokens": chunks * FRAME, "layers": 1,
                       "sharding": "chunk c is encoded into and owned by rank c % world (round-robin)",
                       "exchange": ("none" if world == 1 else
                                    "peer-memory merge + all-gather kernel" if args.exchange != "nccl" else
                                    "nccl all-gather + merge kernel")},
            "encode_tokens_per_s_incl_attention": chunks * FRAME / seconds}


def run_aux(args) -> dict:
    """The HBM-bound helpers around the read, one GPU, c3 shapes: INT8 operator expansion, first
    moments of a 99,840-token history, rotation of the 4,680 query rows, the P-way merge, the finish of the
    mixed-dimensional read, and the rolling-window prune.  Each is timed alone with CUDA events (inputs larger than L2 or an L2
    flush between iterations) and reported in GB/s of its algorithmic bytes against the measured
    copy bandwidth."""
    from nanokv_b200 import attention, ops
    shape = SHAPE
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device)
    gen = torch.Generator(device=device).manual_seed(5)

    def timed(fn, steps=args.steps, warmup=max(args.warmup, 3)):
        times = []
        for index in range(warmup + steps):
            flush.fill_(index & 255)                      # evict L2 between iterations
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            if index >= warmup:
                times.append(start.elapsed_time(stop))
        return statistics.mean(times) / 1e3

    results = {}

    def report(name, seconds, nbytes):
        results[name] = {"ms": seconds * 1e3, "gbs": nbytes / seconds / 1e9,
                         "frac_of_hbm": nbytes / seconds / 1e9 / hbm, "bytes": nbytes}

    # INT8 operator -> bf16: one decoder [J, r]
    q8 = torch.randint(-127, 128, (shape.joint, shape.rank), generator=gen, device=device, dtype=torch.int8)
    scale = torch.rand(shape.joint, 1, generator=gen, device=device).to(torch.bfloat16)
    report("operator_unpack_int8", timed(lambda: ops.unpack_int8_weight(q8, scale)),
           q8.numel() * 3 + scale.numel() * 2)
    # first moments of one layer's V history
    layer = build_layers(shape, range(shape.history // FRAME), 1, device)[0]
    (hk, ok), (hv, ov) = layer["k"], layer["v"]
    view = hv.view()
    per_token = shape.rank // 2 + 2 + hv.ids.element_size()
    report("history_moments", timed(lambda: ops.history_moments(view)), view.tokens * per_token)
    # rotation of the query rows
    table = attention.RopeTable(rope_freqs(1024, shape.head_dim), frame_seqlen=FRAME, width=52, device=device)
    q = synthetic.make_queries(shape, synthetic.generator(1)).to(device)
    positions = torch.arange(90000, 90000 + shape.queries, dtype=torch.int32, device=device)
    report("rope_rows", timed(lambda: table.rotate(q, positions)), q.numel() * 2 * 2)
    # four-way merge of (O, lse) partials
    parts = [(torch.randn(shape.queries, shape.heads, shape.head_dim, generator=gen, device=device)
              .to(torch.bfloat16), torch.randn(shape.queries, shape.heads, generator=gen, device=device))
             for _ in range(4)]
    report("lse_merge_4way", timed(lambda: ops.lse_merge(parts)),
           5 * parts[0][0].numel() * 2 + 5 * parts[0][1].numel() * 4)
    # finish of the mixed-dimensional read: 18 of 24 heads corrected, merged and scattered in one launch
    fin_heads = torch.arange(18, dtype=torch.int32, device=device)
    native = torch.randn(shape.queries, 24, shape.head_dim, generator=gen, device=device).to(torch.bfloat16)
    native_lse = torch.randn(shape.queries, 24, generator=gen, device=device)
    lifted = native[:, :18].contiguous()
    low_lse = native_lse[:, :18].contiguous()
    mean = torch.randn(24, shape.head_dim, generator=gen, device=device)
    finished = torch.empty_like(native)
    report("fast_finish", timed(lambda: ops.fast_finish(native, native_lse, lifted, low_lse, fin_heads, finished,
                                                        value_mean=mean, projected_mean=mean[:18].contiguous())),
           3 * lifted.numel() * 2 + 2 * low_lse.numel() * 4)
    # rolling-window prune: drop the oldest non-sink segments of the history (device copies only)
    keep = [0] + list(range(3, hk.segments))
    moved = (hk.tokens - hk._starts[3]) * per_token
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    hk.retain(keep)
    stop.record()
    torch.cuda.synchronize()
    report("prune_retain", start.elapsed_time(stop) / 1e3, 2 * moved)
    return {"metric": "aux_kernels", "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "dtype": "u8/bf16", "data": "synthetic",
            "config": {"workload": "aux", "shape": shape.name, "l2_policy": "192 MiB flush between iterations"},
            "peak": hbm, "peak_source": f"hbm_gbs of {peak_kind}", "kernels": results}


def time_rope(shape, device, layers: int = 2, launches: int = 4) -> dict:
    """Positional restore inside the read: ms per layer launch with the rebuilt keys rotated (3-D RoPE
    by absolute position), one GPU, whole c3 history."""
    from nanokv_b200 import attention
    built = build_layers(shape, range(shape.history // FRAME), layers, device)
    q = synthetic.make_queries(shape, synthetic.generator(4242)).to(device)
    table = attention.RopeTable(rope_freqs(1024, shape.head_dim), frame_seqlen=FRAME, width=52, device=device)
    positions = torch.arange(shape.history, dtype=torch.int32, device=device)
    times = []
    for index in range(2 + launches):
        (hk, ok), (hv, ov) = built[index % layers]["k"], built[index % layers]["v"]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        attention.codec_attention(q, hk, hv, ok, ov, rope=table, positions=positions)
        stop.record()
        torch.cuda.synchronize()
        if index >= 2:
            times.append(start.elapsed_time(stop))
    ms = statistics.mean(times)
    peaks, peak_kind = measured_peaks()
    flops = attention_flops(shape.history, shape.queries, shape.joint, shape.rank)
    return {"ms_per_layer": ms, "history_tokens_per_s": shape.history / (ms / 1e3),
            "roofline": {"bound": "tensor", "kernel": "attn_codec_kernel<128, rope>",
                         "achieved": flops / (ms / 1e3) / 1e12, "peak": float(peaks["bf16_tflops_sustained"]),
                         "unit": "TFLOP/s",
                         "frac": flops / (ms / 1e3) / 1e12 / float(peaks["bf16_tflops_sustained"]),
                         "peak_source": f"bf16_tflops_sustained of {peak_kind}", "traffic": None}}


def run_secondary(args) -> dict:
    """Short versions of the secondary workloads, after the headline: c5 on every rank; c4 and the
    positional restore on one GPU only.  A failure is reported in place and does not void the headline."""
    import copy
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    result = {}

    def attempt(name, fn):
        try:
            value = fn()
            if rank == 0:
                result[name] = value
        except Exception as exc:   # keep the headline line
            if rank == 0:
                result[name] = {"error": f"{type(exc).__name__}: {str(exc).splitlines()[0][:160]}"}

    stream_args = copy.copy(args)
    stream_args.chunks = args.secondary_chunks
    attempt("c5_streaming", lambda: {k: v for k, v in run_streaming(stream_args, standalone=False).items()
                                     if k in ("metric", "value", "unit", "ms_per_step", "config",
                                              "encode_tokens_per_s_incl_attention")})
    if world == 1:
        fast_args = copy.copy(args)
        fast_args.steps, fast_args.warmup = 3, 2
        attempt("c4_fast_mixed", lambda: {k: v for k, v in run_fast(fast_args).items()
                                          if k in ("metric", "value", "unit", "ms_per_step", "config", "roofline")})
        attempt("c3_positional_restore", lambda: time_rope(SHAPE, torch.device("cuda", 0)))
    return result


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=3)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_gpu"])
    parser.add_argument("--layers", type=int, default=SHAPE.layers)
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg and the oracle parity sample")
    parser.add_argument("--no-gpu-reference", action="store_true",
                        help="skip the stock-torch GPU comparison arm (one GPU only)")
    parser.add_argument("--no-secondary", action="store_true",
                        help="skip the short secondary workloads (c4, c5, positional restore)")
    parser.add_argument("--history-frames", type=int, default=0,
                        help="history frames per layer (default: the workload's 64); smaller values are "
                             "for profiler captures")
    parser.add_argument("--rope", action="store_true",
                        help="rotate the rebuilt keys by absolute position inside the read (3-D RoPE)")
    parser.add_argument("--exchange", default="peer", choices=["peer", "peer_nccl_fences", "nccl"],
                        help="context-parallel exchange: fused peer-memory kernel ordered by flag words in peer "
                             "memory, the same kernel between two 4-byte NCCL all-reduces, or NCCL all-gather + merge")
    parser.add_argument("--workload", default="c3_wan_shaped",
                        choices=["c3_wan_shaped", "c4_fast_mixed", "c5_streaming", "aux", "encode"],
                        help="c3 is the headline; c4 / c5 / aux / encode are secondary measurements")
    parser.add_argument("--chunks", type=int, default=256, help="c5: chunks streamed")
    parser.add_argument("--secondary-chunks", type=int, default=256,
                        help="c5 chunks of the short secondary run behind the headline")
    args = parser.parse_args()
    # stdout carries the one JSON line and nothing else: whatever a library prints there while
    # the workloads run (the NCCL version banner, for one) goes to stderr instead
    sys.stdout.flush()
    json_out = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        line = run_reference(args)
    elif args.impl == "torch_gpu":
        line = run_torch_gpu(args)
    elif args.workload == "c4_fast_mixed":
        line = run_fast(args)
    elif args.workload == "c5_streaming":
        line = run_streaming(args)
    elif args.workload == "aux":
        line = run_aux(args)
    elif args.workload == "encode":
        torch.cuda.set_device(0)
        line = {"workload": "encode (c3 shapes, one GPU)", "n_gpus": 1,
                "encode": time_encode(SHAPE, torch.device("cuda", 0), steps=args.steps, warmup=max(args.warmup, 3))}
    else:
        line = run_ours(args)
        if not args.no_secondary and not args.history_frames:
            secondary = run_secondary(args)
            if line:
                line["secondary"] = secondary
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(json_out, 1)
    os.close(json_out)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
