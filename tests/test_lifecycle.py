"""Segment lifecycle: the window policy against the reference's fixture (CPU), and on the GPU the
rolling history (commit, prune, windowed read with positional restore) against the windowed
K / V / positions the reference decodes."""
import numpy as np
import pytest
import torch

import cases
from nanokv_b200 import lifecycle
from test_oracle_golden import from_bits, load


def test_window_policy_matches_reference_prune():
    gold = load(cases.ROLLING.name)
    for index, (ranges, end, capacity, sink) in enumerate(cases.rolling_policy_cases()):
        kept = lifecycle.kept_segments(ranges, committed_end=end, capacity=capacity, sink_tokens=sink)
        assert kept == gold[f"policy{index}_kept"].tolist(), (ranges, end, capacity, sink)
        # every piece lies inside a kept segment and inside the window, pieces cover the window's
        # intersection with the committed segments exactly once
        pieces = lifecycle.active_pieces(ranges, committed_end=end, capacity=capacity, sink_tokens=sink)
        covered = sorted(p for _, a, b in pieces for p in range(a, b))
        window = {p for a, b in lifecycle.active_intervals(end, capacity, sink) for p in range(a, b)}
        committed = {p for a, b in ranges for p in range(a, b)}
        assert covered == sorted(window & committed)
        assert {i for i, _, _ in pieces} <= set(kept)


def test_window_positions_match_reference_decode():
    gold = load(cases.ROLLING.name)
    case = cases.ROLLING
    ranges, start = [], 0
    for count in case.segments:
        ranges.append((start, start + count))
        start += count
    policy = dict(committed_end=start, **cases.ROLLING_POLICY)
    assert lifecycle.kept_segments(ranges, **policy) == gold["kept"].tolist()
    positions = [p for _, a, b in lifecycle.active_pieces(ranges, **policy) for p in range(a, b)]
    assert positions == gold["positions"].tolist()


def test_stream_window_and_overflow_cut_match_the_reference_entry_point():
    """The window + max_attention_size cut behind codec_cache_attention_inputs, on segment tables
    alone: positions and surviving segments of every step of the reference's streamed run."""
    from nanokv_b200 import lingbot_attention
    gold = load("stream_lb_bf16")
    policy = {k: v for k, v in cases.STREAM_POLICY.items() if k != "max_attention_size"}
    limit = cases.STREAM_POLICY["max_attention_size"]
    segments, start = [], 0
    for step, count in enumerate(cases.ROLLING.segments):
        _, runs = lingbot_attention._window(segments, committed_end=start, **policy)
        kept, lead = lingbot_attention._cut(runs, count, protected=min(policy["sink_tokens"], start, limit),
                                            limit=limit)
        positions = [p + i for a, b, p in kept for i in range(b - a)] + list(range(start + lead, start + count))
        assert positions == gold[f"step{step}_positions"].tolist()
        segments.append({"global_start": start, "global_end": start + count})
        start += count
        segments = lingbot_attention._prune_segments(segments, committed_end=start, **policy)
        assert [[s["global_start"], s["global_end"]] for s in segments] == gold[f"step{step}_segments"].tolist()
    # nothing to cut, everything cut, a cut inside the current chunk
    assert lingbot_attention._cut([(0, 10, 0)], 5, protected=4, limit=15) == ([(0, 10, 0)], 0)
    assert lingbot_attention._cut([(0, 10, 0)], 5, protected=4, limit=4) == ([(0, 4, 0)], 5)
    assert lingbot_attention._cut([(0, 10, 0)], 5, protected=4, limit=7) == ([(0, 4, 0)], 2)
    assert lingbot_attention._cut([(0, 10, 0), (10, 30, 50)], 5, protected=4, limit=12) == \
        ([(0, 4, 0), (27, 30, 67)], 0)


def test_protected_tokens_match_the_reference():
    from nanokv_b200 import mg_core
    gold = load("protected_tokens")
    for index, (ids, recent, stride, sink) in enumerate(cases.protected_token_cases()):
        got = mg_core.protected_tokens(ids, recent, stride, sink)
        assert got.dtype == torch.bool and got.tolist() == gold[f"keep{index}"].tolist(), index
    with pytest.raises(ValueError):
        mg_core.protected_tokens(torch.arange(4), -1, 1)


def test_active_intervals_edges():
    assert lifecycle.active_intervals(0, 10, 2) == []
    assert lifecycle.active_intervals(5, 10, 2) == [(0, 2), (2, 5)]
    assert lifecycle.active_intervals(50, 10, 2) == [(0, 2), (42, 50)]
    assert lifecycle.active_intervals(50, 10, 0) == [(40, 50)]
    assert lifecycle.active_intervals(50, 2, 5) == [(0, 5)]          # the sink alone fills the window


@pytest.mark.gpu
def test_rolling_history_read_matches_reference_window():
    from helpers import BF16_REL_TOL, device_operator, rel_err
    from nanokv_b200 import attention, codec
    from oracle import nkv_oracle as oracle
    gold = load(cases.ROLLING.name)
    case = cases.ROLLING
    data = cases.build(case)
    shape = case.shape
    op_k, op_v = device_operator(data["k_op"]), device_operator(data["v_op"])
    rolling = lifecycle.RollingHistory(joint=shape.joint, rank=shape.rank, capacity_tokens=shape.history,
                                       max_segments=len(case.segments), clusters=shape.centers,
                                       quant=codec.LINGBOT_QUANT)
    for key, value in zip(data["k_chunks"], data["v_chunks"]):
        rolling.commit(key.cuda(), value.cuda(), op_k, op_v, iters=case.iters,
                       seed_k=20260826 + case.layer * 17, seed_v=20260826 + case.layer * 17 + 1)
    policy = cases.ROLLING_POLICY
    dropped = rolling.prune(**policy)
    assert dropped == len(case.segments) - len(gold["kept"])
    assert rolling.k.segments == len(gold["kept"]) and rolling.k.tokens == rolling.v.tokens
    grid = cases.ROLLING_GRID
    freqs = oracle.rope_table(1024, shape.head_dim)
    table = attention.RopeTable(freqs, frame_seqlen=grid["height"] * grid["width"], width=grid["width"])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = data["q"]
    out, lse, positions = rolling.read(q.cuda(), op_k, op_v, rope=table, status=status, **policy)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert positions.cpu().tolist() == gold["positions"].tolist()
    # the reference's windowed, rotated keys and values -> attention by the oracle
    heads, dim = shape.heads, shape.head_dim
    key = from_bits(gold["key_rotated"], torch.bfloat16).reshape(-1, heads, dim)
    value = from_bits(gold["value"], torch.bfloat16).reshape(-1, heads, dim)
    want, want_lse = oracle.attention_lse(q.permute(1, 0, 2)[None], key.permute(1, 0, 2)[None],
                                          value.permute(1, 0, 2)[None])
    assert rel_err(out.cpu(), want[0].permute(1, 0, 2)) <= BF16_REL_TOL
    assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= BF16_REL_TOL
    # without pruning first, the same window is read from the uncompacted history
    again = lifecycle.RollingHistory(joint=shape.joint, rank=shape.rank, capacity_tokens=shape.history,
                                     max_segments=len(case.segments), clusters=shape.centers,
                                     quant=codec.LINGBOT_QUANT)
    for key_rows, value_rows in zip(data["k_chunks"], data["v_chunks"]):
        again.commit(key_rows.cuda(), value_rows.cuda(), op_k, op_v, iters=case.iters,
                     seed_k=20260826 + case.layer * 17, seed_v=20260826 + case.layer * 17 + 1)
    out2, lse2, positions2 = again.read(q.cuda(), op_k, op_v, rope=table, status=status, **policy)
    assert torch.equal(positions2, positions)
    assert rel_err(out2.cpu(), out.cpu()) <= 2.0 ** -7 and float((lse2 - lse).abs().max()) <= 1e-2


@pytest.mark.gpu
def test_retain_and_token_views():
    from helpers import device_operator
    from nanokv_b200 import codec
    case = cases.ROLLING
    data = cases.build(case)
    op = device_operator(data["k_op"])
    from nanokv_b200.cache import CompressedHistory
    hist = CompressedHistory(joint=case.shape.joint, rank=case.shape.rank, capacity=case.shape.history,
                             max_segments=4, centers_per_segment=case.shape.centers)
    for chunk in data["k_chunks"]:
        codec.encode_append(hist, chunk.cuda(), op, clusters=case.shape.centers, seed=3)
    whole = codec.decode(hist, op, dtype=torch.bfloat16)
    from nanokv_b200 import ops
    for a, b in ((0, 250), (5, 70), (60, 140), (134, 135), (199, 250)):
        part = ops.decode_rows(hist.view_tokens(a, b), op.decoder, op.mean, dtype=torch.bfloat16)
        assert torch.equal(part, whole[a:b]), (a, b)
    hist.retain([0, 2, 3])
    assert hist.tokens == 70 + 64 + 52 and hist.segments == 3
    kept = codec.decode(hist, op, dtype=torch.bfloat16)
    assert torch.equal(kept, torch.cat([whole[:70], whole[134:]]))
    hist.retain([0, 2])                                        # two single-segment runs
    assert hist.tokens == 70 + 52 and hist.segments == 2
    assert torch.equal(codec.decode(hist, op, dtype=torch.bfloat16), torch.cat([whole[:70], whole[198:]]))
    with pytest.raises(ValueError):
        hist.retain([1, 0])
    with pytest.raises(ValueError):
        hist.view_tokens(10, 500)


def test_retain_bookkeeping_on_random_histories():
    """Host logic of the in-place prune (tensors on the CPU, arrays filled directly): for random
    segment sizes and random kept subsets the moved codes, scales, ids, centre rows and both segment
    tables equal the concatenation of the kept segments."""
    import random
    from nanokv_b200.cache import CompressedHistory
    rng = random.Random(1)
    for _ in range(60):
        segments = rng.randint(1, 7)
        counts = [rng.randint(1, 40) for _ in range(segments)]
        clusters = [rng.randint(1, 5) for _ in range(segments)]
        hist = CompressedHistory(joint=8, rank=8, capacity=sum(counts) + 5, max_segments=8,
                                 centers_per_segment=5, device="cpu")
        tokens = rows = 0
        hist._starts, hist._center_rows = [0], []
        for count, k in zip(counts, clusters):
            hist.codes[tokens:tokens + count] = torch.randint(0, 255, (count, hist.codes.shape[1])).to(hist.codes.dtype)
            hist.scales[tokens:tokens + count] = torch.randn(count, hist.scales.shape[1]).to(hist.scales.dtype)
            hist.ids[tokens:tokens + count] = torch.randint(0, k, (count,)).to(hist.ids.dtype)
            hist.centers[rows:rows + k] = torch.randn(k, hist.centers.shape[1]).to(hist.centers.dtype)
            hist._center_rows.append(rows)
            tokens, rows = tokens + count, rows + k
            hist._starts.append(tokens)
        hist._center_used = rows
        keep = sorted(rng.sample(range(segments), rng.randint(0, segments)))

        def kept(array, bounds):
            parts = [array[bounds[i]:bounds[i + 1]].clone() for i in keep]
            return torch.cat(parts) if parts else array[:0].clone()
        row_bounds = hist._center_rows + [rows]
        want = {name: kept(getattr(hist, name), hist._starts) for name in ("codes", "scales", "ids")}
        want_centers = kept(hist.centers, row_bounds)
        starts, first_rows = [0], [0]
        for i in keep:
            starts.append(starts[-1] + counts[i])
            first_rows.append(first_rows[-1] + clusters[i])
        hist.retain(keep)
        assert hist._starts == starts and hist._center_rows == first_rows[:-1]
        assert hist.tokens == starts[-1] and hist.segments == len(keep)
        for name, expected in want.items():
            assert torch.equal(getattr(hist, name)[:starts[-1]], expected), name
        assert torch.equal(hist.centers[:first_rows[-1]], want_centers)
        assert hist.seg_start[:len(starts)].tolist() == starts
        assert hist.seg_center_row[:len(keep)].tolist() == first_rows[:-1]
