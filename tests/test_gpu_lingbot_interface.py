"""The LingBot codec and rolling-cache interfaces (the reference modules' names, argument lists and
payload dictionaries) on the GPU, against fixtures the unmodified reference produced."""
import numpy as np
import pytest
import torch

import cases
from helpers import BF16_REL_TOL, code_flip_report, rel_err
from nanokv_b200 import attention, lingbot_attention, lingbot_codec
from oracle import nkv_oracle as oracle
from test_oracle_golden import from_bits, load

pytestmark = pytest.mark.gpu


def register(case, data):
    for target in ("k", "v"):
        op = data[f"{target}_op"]
        lingbot_codec.register_operator(target, case.layer, mean=op["mean"], encoder=op["encoder"],
                                        decoder=op["decoder"])


def close_rows(got: torch.Tensor, want: torch.Tensor) -> None:
    """Decoded rows of an encode that may differ from the reference's by single code steps."""
    scale = float(want.float().abs().max())
    diff = (got.float() - want.float()).abs()
    assert float(diff.max()) <= 0.25 * scale
    assert float((diff > 2.0 ** -6 * scale).float().mean()) < 0.01


def test_encode_tensor_and_decode_tensor_with_the_reference_argument_list():
    case = cases.MINI_LB
    gold, data = load(case.name), cases.build(case)
    register(case, data)
    heads, dim, rank = case.shape.heads, case.shape.head_dim, case.shape.rank
    for target in ("k", "v"):
        chunk = data[f"{target}_chunks"][0]
        payload = lingbot_codec.encode_tensor(
            chunk.reshape(1, -1, heads, dim).cuda(), target=target, layer=case.layer, sp_rank=0,
            basis_root="synthetic", rank=rank, clusters=case.shape.centers, iters=case.iters)
        count = chunk.shape[0]
        assert payload["format"] == lingbot_codec.FORMAT and payload["shape"] == (1, count, heads, dim)
        assert payload["latent_shape"] == (1, count, rank) and payload["latent_count"] == count * rank
        assert np.array_equal(gold[f"{target}0_ids"], payload["ids"].cpu().numpy())
        assert np.array_equal(gold[f"{target}0_centers"],
                              payload["centers"].cpu().view(torch.int16).numpy())
        want = oracle.unpack_int4(torch.from_numpy(gold[f"{target}0_packed"]), count * rank, (count, rank))
        got = oracle.unpack_int4(payload["latent_packed"].cpu(), count * rank, (count, rank))
        report = code_flip_report(got, want)
        assert report["max_step"] <= 1 and report["flips"] <= 2e-3 * report["total"], report
        same = (got == want).all(dim=1)
        want_scale = from_bits(gold[f"{target}0_scale"], torch.bfloat16).reshape(-1)
        assert float((payload["latent_scale"].cpu().reshape(-1) != want_scale).float().mean()) < 0.01
        decoded = lingbot_codec.decode_tensor(payload, dtype=torch.bfloat16, device="cuda")
        assert decoded.shape == (1, count, heads, dim)
        want_rows = from_bits(gold[f"{target}_decoded"], torch.bfloat16)
        got_rows = decoded.cpu().reshape(count, -1)
        # rows whose codes equal the reference's decode to the reference's rows up to rounding
        err = (got_rows[same].float() - want_rows[same].float()).abs().max()
        assert float(err) <= 2.0 ** -6 * float(want_rows.float().abs().max())
        close_rows(got_rows, want_rows)
        # row and interval accessors agree with the whole decode
        index = torch.tensor([0, 5, count - 1, 17])
        picked = lingbot_codec.decode_tensor_rows(payload, index, dtype=torch.bfloat16, device="cuda")
        assert torch.equal(picked[0].cpu(), decoded[0].cpu()[index])
        part = lingbot_codec.decode_tensor_slice(payload, 30, 95, dtype=torch.bfloat16, device="cuda")
        assert torch.equal(part.cpu(), decoded.cpu()[:, 30:95])
        latent, (centers, ids), mean = lingbot_codec.direct_latent_slice(payload, 30, 95, device="cuda")
        assert latent.shape == (1, 65, rank) and ids.shape == (1, 65) and centers.shape[1] == case.shape.centers
        want_latent = oracle.dequantize_rows(got[30:95], payload["latent_scale"].cpu().reshape(-1, 1)[30:95])
        assert torch.equal(latent[0].cpu(), want_latent)
        rows_latent, _, _ = lingbot_codec.direct_latent_rows(payload, index, device="cuda")
        assert torch.equal(rows_latent[0].cpu(), oracle.dequantize_rows(
            got[index], payload["latent_scale"].cpu().reshape(-1, 1)[index]))
        with pytest.raises(ValueError):
            lingbot_codec.decode_tensor_slice(payload, 10, count + 1, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        lingbot_codec.encode_tensor(torch.zeros(2, 8, heads, dim, device="cuda"), target="k", layer=case.layer,
                                    sp_rank=0, basis_root="synthetic", rank=rank)
    with pytest.raises(RuntimeError):
        lingbot_codec.decode_tensor({"format": "other"}, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(KeyError):
        lingbot_codec.encode_tensor(torch.zeros(1, 80, heads, dim, device="cuda"), target="k", layer=77,
                                    sp_rank=0, basis_root="nowhere", rank=rank)


def stream_cache(case):
    cache = {"global_end_index": torch.zeros(1, dtype=torch.long),
             "local_end_index": torch.zeros(1, dtype=torch.long)}
    lingbot_attention.configure_cache(cache, layer=case.layer, sp_rank=0, options={
        "codec_rank": case.shape.rank, "codec_clusters": case.shape.centers, "codec_iters": case.iters,
        "codec_basis_root_k": "synthetic", "codec_basis_root_v": "synthetic"})
    cache["codec_commit"] = True
    return cache


def test_encode_pair_then_the_windowed_decode_against_the_reference_fixture():
    """encode_pair per chunk, _prune_segments, _decode_active_history (decode_segments underneath)."""
    case = cases.ROLLING
    gold, data = load(case.name), cases.build(case)
    register(case, data)
    heads, dim = case.shape.heads, case.shape.head_dim
    segments, start = [], 0
    for key, value in zip(data["k_chunks"], data["v_chunks"]):
        cache = {"codec_layer": case.layer, "codec_rank": case.shape.rank,
                 "codec_clusters": case.shape.centers, "codec_iters": case.iters,
                 "codec_commit_start": start, "codec_basis_root_k": "synthetic",
                 "codec_basis_root_v": "synthetic"}
        segments.append(lingbot_codec.encode_pair(key.reshape(1, -1, heads, dim).cuda(),
                                                  value.reshape(1, -1, heads, dim).cuda(), cache=cache))
        assert segments[-1]["global_start"] == start and segments[-1]["resident_bytes"] > 0
        start += key.shape[0]
    policy = dict(committed_end=start, **cases.ROLLING_POLICY)
    kept = lingbot_attention._prune_segments(segments, **policy)
    assert [segments.index(s) for s in kept] == gold["kept"].tolist()
    key, value, positions = lingbot_attention._decode_active_history(
        kept, dtype=torch.bfloat16, device=torch.device("cuda"), **policy)
    assert positions.cpu().tolist() == gold["positions"].tolist()
    close_rows(key[0].cpu(), from_bits(gold["key"], torch.bfloat16))
    close_rows(value[0].cpu(), from_bits(gold["value"], torch.bfloat16))
    whole = lingbot_codec.decode_segments(kept, dtype=torch.bfloat16, device="cuda")
    assert whole[0].shape[1] == sum(s["global_end"] - s["global_start"] for s in kept)
    assert lingbot_codec.decode_segments([], dtype=torch.bfloat16, device="cuda") is None


def test_codec_cache_attention_inputs_stream_against_the_reference_fixture():
    """Chunk by chunk through the reference-named entry point: positions, segment table and cache
    counters exactly; K / V rows as the reference's; then the fused step on the same cache state
    against attention over the reference's rows."""
    case = cases.ROLLING
    gold, data = load("stream_lb_bf16"), cases.build(case)
    register(case, data)
    heads, dim = case.shape.heads, case.shape.head_dim
    cache, fused_cache = stream_cache(case), stream_cache(case)
    grid = cases.ROLLING_GRID
    freqs = oracle.rope_table(1024, dim)
    frame_seqlen = grid["height"] * grid["width"]
    table = attention.RopeTable(freqs, frame_seqlen=frame_seqlen, width=grid["width"])
    start = 0
    for step, (key, value) in enumerate(zip(data["k_chunks"], data["v_chunks"])):
        key4 = key.reshape(1, -1, heads, dim).cuda()
        value4 = value.reshape(1, -1, heads, dim).cuda()
        key_cache, value_cache, positions = lingbot_attention.codec_cache_attention_inputs(
            cache, key4, value4, current_start=start, **cases.STREAM_POLICY)
        assert positions.cpu().tolist() == gold[f"step{step}_positions"].tolist()
        assert [[s["global_start"], s["global_end"]] for s in cache["codec_segments"]] == \
            gold[f"step{step}_segments"].tolist()
        want_key = from_bits(gold[f"step{step}_key"], torch.bfloat16)
        want_value = from_bits(gold[f"step{step}_value"], torch.bfloat16)
        close_rows(key_cache[0].cpu(), want_key)
        close_rows(value_cache[0].cpu(), want_value)
        # the fused step: queries of this chunk (rotated) over window + current, keys rotated inside
        count = key.shape[0]
        q_positions = torch.arange(start, start + count)
        q = data["q"][:min(count, data["q"].shape[0])]
        q_rot = oracle.rope_by_positions(q[None], q_positions[:q.shape[0]], freqs, frame_seqlen=frame_seqlen,
                                         width=grid["width"])[0]
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out, lse = lingbot_attention.codec_cache_attention(
            fused_cache, q_rot[None].cuda(), key4, value4, current_start=start, rope=table, status=status,
            **cases.STREAM_POLICY)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        rotated = oracle.rope_by_positions(want_key[None], torch.from_numpy(gold[f"step{step}_positions"]),
                                           freqs, frame_seqlen=frame_seqlen, width=grid["width"])[0]
        want, want_lse = oracle.attention_lse(q_rot.permute(1, 0, 2)[None], rotated.permute(1, 0, 2)[None],
                                              want_value.permute(1, 0, 2)[None])
        assert rel_err(out[0].cpu(), want[0].permute(1, 0, 2)) <= BF16_REL_TOL
        assert float((lse.cpu() - want_lse[0].t()).abs().max()) <= BF16_REL_TOL
        start += count
    assert cache["global_end_index"].tolist() == gold["global_end"].tolist()
    assert cache["local_end_index"].tolist() == gold["local_end"].tolist()
    assert fused_cache["codec_committed_end"] == cache["codec_committed_end"] == start
    # a commit that does not continue the cache is refused like the reference refuses it
    with pytest.raises(RuntimeError):
        lingbot_attention.codec_cache_attention_inputs(
            cache, key4, value4, current_start=start + 5, **cases.STREAM_POLICY)


def test_attend_against_the_reference_fixture(monkeypatch):
    """NanoKV-Fast step with the reference's argument list: committed chunks, then a chunk that
    attends (sink and recent frame at full width, the rest through a 64-wide and a 128-wide reader
    group), without and with the value-mean residual; and the calls that fall back (None)."""
    case = cases.ROLLING
    gold, data = load("attend_lb_bf16"), cases.build(case)
    register(case, data)
    heads, dim = case.shape.heads, case.shape.head_dim
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy=cases.ATTEND_POLICY)
    cache = stream_cache(case)
    chunks = list(zip(data["k_chunks"], data["v_chunks"]))
    start = 0
    for key, value in chunks[:-1]:
        lingbot_attention.codec_cache_attention_inputs(
            cache, key.reshape(1, -1, heads, dim).cuda(), value.reshape(1, -1, heads, dim).cuda(),
            current_start=start, **cases.STREAM_POLICY)
        start += key.shape[0]
    assert start == int(gold["start"][0])
    cache["codec_commit"] = False
    key, value = (t.reshape(1, -1, heads, dim).cuda() for t in chunks[-1])
    grid = cases.ROLLING_GRID
    frame_seqlen = grid["height"] * grid["width"]
    freqs = oracle.rope_table(1024, dim)
    count = key.shape[1]
    q_pre = data["q"][:count][None].cuda()
    q_native = from_bits(gold["q_native"], torch.bfloat16)[None].cuda()
    common = dict(current_start=start, grid_sizes=torch.tensor([[64, grid["height"], grid["width"]]]),
                  freqs=freqs, frame_seqlen=frame_seqlen, **cases.STREAM_POLICY)
    monkeypatch.setenv("LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL", "0")
    plain = lingbot_attention.attend(q_pre, q_native, key, value, cache, **common)
    assert plain.shape == q_pre.shape
    want = from_bits(gold["plain"], torch.bfloat16)
    assert rel_err(plain[0].cpu(), want) <= BF16_REL_TOL
    monkeypatch.setenv("LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL", "1")
    corrected = lingbot_attention.attend(q_pre, q_native, key, value, cache, **common)
    want_corrected = from_bits(gold["corrected"], torch.bfloat16)
    assert rel_err(corrected[0].cpu(), want_corrected) <= BF16_REL_TOL
    assert rel_err(want, want_corrected) > 1e-3, "the residual must matter in this case"
    monkeypatch.setenv("LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL", "0")
    assert cache["codec_committed_end"] == start and len(cache["codec_segments"]) == 3   # nothing committed
    # fallbacks: no reader for the layer; everything protected; policy says native
    other = dict(cache, codec_layer=case.layer + 40)
    assert lingbot_attention.attend(q_pre, q_native, key, value, other, **common) is None
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy={"recent_native_frames": 1000})
    assert lingbot_attention.attend(q_pre, q_native, key, value, cache, **common) is None
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy=dict(cases.ATTEND_POLICY, native_prefix_chunks=3))
    assert lingbot_attention.attend(q_pre, q_native, key, value, dict(cache, codec_chunk_id=2), **common) is None
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy=dict(cases.ATTEND_POLICY, native_denoise_calls=[0, 2]))
    seen = [lingbot_attention.attend(q_pre, q_native, key, value, cache, **common) is None for _ in range(4)]
    assert seen == [True, False, True, False]
    # anchors: every second frame stays full width; same softmax over the same tokens, so the
    # result stays close to the unanchored one while taking the non-contiguous path
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy=dict(cases.ATTEND_POLICY, anchor_stride=2))
    anchored = lingbot_attention.attend(q_pre, q_native, key, value, cache, **common)
    assert anchored.shape == q_pre.shape and bool(torch.isfinite(anchored.float()).all())
    # a committing call appends and prunes like the reference
    lingbot_attention.register_reader(case.layer, cases.build_attend_reader(case, data),
                                      policy=cases.ATTEND_POLICY)
    cache["codec_commit"] = True
    lingbot_attention.attend(q_pre, q_native, key, value, cache, **common)
    assert cache["codec_committed_end"] == start + count
    assert [[s["global_start"], s["global_end"]] for s in cache["codec_segments"]] == \
        load("stream_lb_bf16")["step3_segments"].tolist()
    with pytest.raises(ValueError):
        lingbot_attention.attend(q_pre[:, :, :1], q_native[:, :, :1], key, value, cache, **common)
