"""Generate the golden fixtures by running the UNMODIFIED reference on CPU.

    python tests/golden/make_golden.py --reference /path/to/NanoKV   (or NANOKV_REFERENCE_ROOT)

Needs a checkout of the reference project (it is imported, never copied).
Inputs are regenerated from seeds by ``tests/golden/cases.py``; only the
reference's outputs (and a digest of each input, to detect generator drift)
are stored, as compressed ``.npz`` files next to this script.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE))

import cases  # noqa: E402
from nanokv_b200.synthetic import checksum  # noqa: E402
from oracle import ref_import  # noqa: E402


def bits(tensor: torch.Tensor) -> np.ndarray:
    """Store 16-bit floats as their bit patterns (numpy has no bf16)."""
    tensor = tensor.detach().contiguous()
    if tensor.dtype in (torch.bfloat16, torch.float16):
        return tensor.view(torch.int16).numpy()
    return tensor.numpy()


def save(name: str, arrays: dict) -> None:
    arrays["torch_version"] = np.frombuffer(torch.__version__.encode(), dtype=np.uint8)
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    size = (HERE / f"{name}.npz").stat().st_size
    print(f"wrote {name}.npz ({size / 1024:.0f} KiB)")


def mg_segment_arrays(prefix: str, payload: dict, out: dict) -> None:
    out[f"{prefix}_ids"] = payload["ids"].numpy()
    out[f"{prefix}_packed"] = payload["packed_codes"].numpy()
    out[f"{prefix}_scale"] = bits(payload["scale"])
    out[f"{prefix}_centers"] = bits(payload["centers"])


def run_mg_case(case: cases.CodecCase, root) -> dict:
    """encode_tensor / decode_value / attention_lse of the Matrix-Game modules."""
    codec = ref_import.load_mg_codec(root)
    core = ref_import.load_mg_core(root)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.iters)
    data = cases.build(case)
    out = {}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_mg_operator(codec, kind, case.layer, mean=op["mean"],
                                      encoder=op["encoder"], decoder=op["decoder"])
        out[f"{kind}_input_digest"] = np.array([checksum(t) for t in data[f"{kind}_chunks"]],
                                               dtype=np.uint64)
    containers = {}
    for kind in ("k", "v"):
        container = None
        for index, chunk in enumerate(data[f"{kind}_chunks"]):
            payload = codec.encode_tensor(kind, case.layer, chunk[None])
            mg_segment_arrays(f"{kind}{index}", payload, out)
            container = codec.concat_values(container, payload)
        containers[kind] = container
    dtype = case.shape.torch_dtype
    key, value = codec.decode_pair_values(containers["k"], containers["v"], dtype=dtype,
                                          device=torch.device("cpu"))
    out["k_decoded_head"] = bits(key[0, :64])
    out["v_decoded_head"] = bits(value[0, :64])
    out["k_decoded_digest"] = np.array([checksum(key)], dtype=np.uint64)
    out["v_decoded_digest"] = np.array([checksum(value)], dtype=np.uint64)
    heads, dim = case.shape.heads, case.shape.head_dim
    q = data["q"][None].permute(0, 2, 1, 3).contiguous()
    kk = key.reshape(1, -1, heads, dim).permute(0, 2, 1, 3)
    vv = value.reshape(1, -1, heads, dim).permute(0, 2, 1, 3)
    attn, lse = core.attention_lse(q, kk, vv)
    out["q_digest"] = np.array([checksum(data["q"])], dtype=np.uint64)
    out["attn_rows"] = bits(attn[0, :, ::case.attn_stride])
    out["attn_digest"] = np.array([checksum(attn)], dtype=np.uint64)
    out["lse"] = lse[0].numpy()
    return out


def run_lingbot_case(case: cases.CodecCase, root) -> dict:
    """encode_tensor / decode_tensor of the LingBot module (always bf16 operators)."""
    codec = ref_import.load_lingbot_codec(root)
    data = cases.build(case)
    heads, dim = case.shape.heads, case.shape.head_dim
    out = {}
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_lingbot_operator(
            codec, "synthetic", kind, case.layer, joint_dim=case.shape.joint,
            rank=case.shape.rank, mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
        chunk = data[f"{kind}_chunks"][0]
        payload = codec.encode_tensor(
            chunk.reshape(1, -1, heads, dim), target=kind, layer=case.layer, sp_rank=0,
            basis_root="synthetic", rank=case.shape.rank, clusters=case.shape.centers,
            iters=case.iters)
        out[f"{kind}_input_digest"] = np.array([checksum(chunk)], dtype=np.uint64)
        out[f"{kind}0_ids"] = payload["ids"].numpy()
        out[f"{kind}0_packed"] = payload["latent_packed"].numpy()
        out[f"{kind}0_scale"] = bits(payload["latent_scale"])
        out[f"{kind}0_centers"] = bits(payload["centers"])
        decoded = codec.decode_tensor(payload, dtype=torch.bfloat16, device=torch.device("cpu"))
        out[f"{kind}_decoded"] = bits(decoded.reshape(-1, case.shape.joint))
    return out


def run_fast_case(case: cases.FastCase, root, masked: bool = False) -> dict:
    """hybrid_attention of codec_native/core.py over MG payloads; ``masked`` hands every segment
    a boolean visibility mask [1, 1, Q, tokens] that is constant within a query group."""
    codec = ref_import.load_mg_codec(root)
    core = ref_import.load_mg_core(root)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.codec.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.codec.iters)
    data = cases.build(case.codec)
    shape = case.codec.shape
    heads, dim, dtype = shape.heads, shape.head_dim, shape.torch_dtype
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_mg_operator(codec, kind, case.codec.layer, mean=op["mean"],
                                      encoder=op["encoder"], decoder=op["decoder"])
    payloads = {kind: [codec.encode_tensor(kind, case.codec.layer, chunk[None])
                       for chunk in data[f"{kind}_chunks"]] for kind in ("k", "v")}
    device = torch.device("cpu")
    low_k = {"codec": "worldplay_segments_v1", "segments": payloads["k"][:case.low_segments]}
    low_v = {"codec": "worldplay_segments_v1", "segments": payloads["v"][:case.low_segments]}
    low = codec.direct_latent_pair_segments(low_k, low_v, device=device)
    native = []
    for pk, pv in zip(payloads["k"][case.low_segments:], payloads["v"][case.low_segments:]):
        key = codec.decode_tensor(pk, dtype=dtype, device=device)
        value = codec.decode_tensor(pv, dtype=dtype, device=device)
        native.append((key.reshape(1, -1, heads, dim).permute(0, 2, 1, 3),
                       value.reshape(1, -1, heads, dim).permute(0, 2, 1, 3), None))
    if masked:
        groups, visible = cases.build_visibility(case)
        full = [mask[groups][None, None] for mask in visible]           # [1, 1, Q, tokens]
        for segment, mask in zip(low, full[:case.low_segments]):
            segment["mask"] = mask
        native = [(key, value, mask) for (key, value, _), mask in zip(native, full[case.low_segments:])]
    reader_payload = cases.build_reader(case, data)
    reader = core.ReaderLayer(reader_payload)
    q = data["q"][None].permute(0, 2, 1, 3).contiguous()
    result = core.hybrid_attention(
        q, q, native, low, reader,
        query_position=lambda value, group: value,
        kv_position=lambda kk, vv, segment, group: (kk, vv))
    return {"hybrid": bits(result[0]), "q_digest": np.array([checksum(data["q"])], dtype=np.uint64)}


def run_merge_case(root) -> dict:
    core = ref_import.load_mg_core(root)
    out_a, lse_a, out_b, lse_b = cases.build_merge()
    out, lse = core.merge(out_a, lse_a, out_b, lse_b)
    return {"out": bits(out), "lse": lse.numpy()}


def reference_rope_params(root):
    """The reference's ``rope_params`` (wan/modules/model.py), taken out of its module by name and
    executed as is: the module itself imports packages that are not installed here."""
    import ast
    path = root / ref_import.LB / "wan/modules/model.py"
    tree = ast.parse(path.read_text())
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "rope_params")
    scope = {"torch": torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec"), scope)
    return scope["rope_params"]


def run_select_case(case: cases.CodecCase, root) -> dict:
    """select_value of the MG module over two payload segments: the selection cuts the first
    segment (decode, gather, re-encode) and takes the second whole (reused)."""
    codec = ref_import.load_mg_codec(root)
    data = cases.build(case)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.iters)
    op = data["k_op"]
    ref_import.inject_mg_operator(codec, "k", case.layer, mean=op["mean"], encoder=op["encoder"],
                                  decoder=op["decoder"])
    value = None
    for chunk in data["k_chunks"]:
        value = codec.concat_values(value, codec.encode_tensor("k", case.layer, chunk[None]))
    token_idx = cases.select_indices(case)
    picked = codec.select_value(value, token_idx, kind="k", layer=case.layer, dtype=torch.bfloat16,
                                device=torch.device("cpu"))
    parts = picked["segments"]
    assert len(parts) == 2 and parts[1] is value["segments"][1]
    cut = parts[0]
    decoded = codec.decode_value(picked, dtype=torch.bfloat16, device=torch.device("cpu"))
    return {"cut_ids": cut["ids"].numpy(), "cut_packed": cut["packed_codes"].numpy(),
            "cut_scale": bits(cut["scale"]), "cut_centers": bits(cut["centers"]),
            "cut_shape": np.array(cut["shape"], dtype=np.int64), "decoded": bits(decoded[0]),
            "input_digest": np.array([checksum(torch.cat(data["k_chunks"]))], dtype=np.uint64)}


def load_lingbot_runtime(root):
    ref_import.load_lingbot_codec(root)
    return ref_import._load("wan.modules.lingbot_v2_cache_runtime",
                            root / ref_import.LB / "wan/modules/lingbot_v2_cache_runtime.py")


def run_rolling_case(case: cases.CodecCase, root) -> dict:
    """LingBot lifecycle on real payloads: encode_pair per chunk, _prune_segments,
    _decode_active_history (windowed K / V / positions), rope_pre_key_by_positions."""
    codec = ref_import.load_lingbot_codec(root)
    runtime = load_lingbot_runtime(root)
    data = cases.build(case)
    heads, dim = case.shape.heads, case.shape.head_dim
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_lingbot_operator(
            codec, "synthetic", kind, case.layer, joint_dim=case.shape.joint,
            rank=case.shape.rank, mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
    segments, start = [], 0
    for key, value in zip(data["k_chunks"], data["v_chunks"]):
        cache = {"codec_layer": case.layer, "codec_rank": case.shape.rank,
                 "codec_clusters": case.shape.centers, "codec_iters": case.iters,
                 "codec_commit_start": start, "codec_basis_root_k": "synthetic",
                 "codec_basis_root_v": "synthetic"}
        segments.append(codec.encode_pair(key.reshape(1, -1, heads, dim),
                                          value.reshape(1, -1, heads, dim), cache=cache))
        start += key.shape[0]
    policy = dict(committed_end=start, **cases.ROLLING_POLICY)
    kept = runtime._prune_segments(segments, **policy)
    kept_index = [next(i for i, s in enumerate(segments) if s is k) for k in kept]
    key, value, positions = runtime._decode_active_history(
        kept, dtype=torch.bfloat16, device=torch.device("cpu"), **policy)
    grid = cases.ROLLING_GRID
    rope_params = reference_rope_params(root)
    freqs = torch.cat([rope_params(1024, dim - 4 * (dim // 6)), rope_params(1024, 2 * (dim // 6)),
                       rope_params(1024, 2 * (dim // 6))], dim=1)
    os.environ["LINGBOT_PRE_ROPE_TRITON"] = "0"
    rotated = runtime.rope_pre_key_by_positions(
        key, positions, grid_sizes=torch.tensor([[64, grid["height"], grid["width"]]]), freqs=freqs,
        frame_seqlen=grid["height"] * grid["width"])
    out = {"kept": np.array(kept_index, dtype=np.int64), "positions": positions.numpy(),
           "key": bits(key[0]), "value": bits(value[0]), "key_rotated": bits(rotated[0]),
           "q_digest": np.array([checksum(data["q"])], dtype=np.uint64)}
    # the policy alone, on synthetic segment tables
    for index, (ranges, end, capacity, sink) in enumerate(cases.rolling_policy_cases()):
        table = [{"global_start": a, "global_end": b} for a, b in ranges]
        survivors = runtime._prune_segments(table, committed_end=end, capacity=capacity, sink_tokens=sink)
        out[f"policy{index}_kept"] = np.array([table.index(s) for s in survivors], dtype=np.int64)
    return out


def run_rope_selected_case(root) -> dict:
    """_rope_low of the LingBot Fast attention module (selected native pairs per head)."""
    import types
    ref_import.load_lingbot_codec(root)
    load_lingbot_runtime(root)
    fast = ref_import._load("wan.modules.codec_native_attention",
                            root / ref_import.LB / "wan/modules/codec_native_attention.py")
    data = cases.build_rope_selected()
    rope_params = reference_rope_params(root)
    d = data["native_dim"]
    freqs = torch.cat([rope_params(1024, d - 4 * (d // 6)), rope_params(1024, 2 * (d // 6)),
                       rope_params(1024, 2 * (d // 6))], dim=1)
    os.environ["LINGBOT_CODEC_NATIVE_TRITON_ROPE"] = "0"
    out = fast._rope_low(data["value"], data["positions"], data["grid_sizes"], freqs,
                         data["frame_seqlen"], types.SimpleNamespace(indices=data["indices"]))
    return {"rotated": bits(out), "value_digest": np.array([checksum(data["value"])], dtype=np.uint64),
            "indices": data["indices"].numpy()}


def run_value_mean_case(case: cases.CodecCase, root) -> dict:
    """_compressed_value_mean of the LingBot Fast module over the V payloads of a rolling case:
    the first segment cut to an interval, the others whole."""
    codec = ref_import.load_lingbot_codec(root)
    load_lingbot_runtime(root)
    fast = ref_import._load("wan.modules.codec_native_attention",
                            root / ref_import.LB / "wan/modules/codec_native_attention.py")
    data = cases.build(case)
    heads, dim = case.shape.heads, case.shape.head_dim
    op = data["v_op"]
    ref_import.inject_lingbot_operator(
        codec, "synthetic", "v", case.layer, joint_dim=case.shape.joint, rank=case.shape.rank,
        mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
    low = []
    for index, chunk in enumerate(data["v_chunks"]):
        payload = codec.encode_tensor(
            chunk.reshape(1, -1, heads, dim), target="v", layer=case.layer, sp_rank=0,
            basis_root="synthetic", rank=case.shape.rank, clusters=case.shape.centers, iters=case.iters)
        lo, hi = cases.value_mean_interval(case, index)
        low.append({"v": codec.direct_latent_slice(payload, lo, hi, device=torch.device("cpu")),
                    "v_payload": payload, "bounds": (lo, hi)})
    value = fast._compressed_value_mean(low, torch.device("cpu"), None)
    return {"value_mean": value.numpy(),
            "input_digest": np.array([checksum(torch.cat(data["v_chunks"]))], dtype=np.uint64)}


def run_fast_hooks_case(case: cases.FastCase, root) -> dict:
    """hybrid_attention of codec_native/core.py with the Matrix-Game hooks: rope_selected on the
    reduced query and the low-width keys, camera_selected on query, keys, values and output."""
    codec = ref_import.load_mg_codec(root)
    core = ref_import.load_mg_core(root)
    os.environ["MG35_KVCODEC_C64_CLUSTERS"] = str(case.codec.shape.centers)
    os.environ["MG35_KVCODEC_C64_ITERS"] = str(case.codec.iters)
    for name in ("MG35_CODEC_NATIVE_FUSED_CAMERA", "MG35_CODEC_NATIVE_RUNTIME_OPT"):
        os.environ.pop(name, None)
    data = cases.build(case.codec)
    shape = case.codec.shape
    heads, dim, dtype = shape.heads, shape.head_dim, shape.torch_dtype
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_mg_operator(codec, kind, case.codec.layer, mean=op["mean"],
                                      encoder=op["encoder"], decoder=op["decoder"])
    payloads = {kind: [codec.encode_tensor(kind, case.codec.layer, chunk[None])
                       for chunk in data[f"{kind}_chunks"]] for kind in ("k", "v")}
    device = torch.device("cpu")
    low = codec.direct_latent_pair_segments(
        {"codec": "worldplay_segments_v1", "segments": payloads["k"][:case.low_segments]},
        {"codec": "worldplay_segments_v1", "segments": payloads["v"][:case.low_segments]}, device=device)
    hooks = cases.build_hooks(case)
    for segment, extra in zip(low, hooks["segments"]):
        segment.update(extra)
    native = []
    for pk, pv in zip(payloads["k"][case.low_segments:], payloads["v"][case.low_segments:]):
        key = codec.decode_tensor(pk, dtype=dtype, device=device)
        value = codec.decode_tensor(pv, dtype=dtype, device=device)
        native.append((key.reshape(1, -1, heads, dim).permute(0, 2, 1, 3),
                       value.reshape(1, -1, heads, dim).permute(0, 2, 1, 3), None))
    reader = core.ReaderLayer(cases.build_reader(case, data))

    def query_position(value, group):
        value = core.rope_selected(value, hooks["q_multiplier"], group.indices)
        return core.camera_selected(value, hooks["q_camera"], group.indices)

    def kv_position(kk, vv, segment, group):
        kk = core.rope_selected(kk, segment["freqs"], group.indices)
        return (core.camera_selected(kk, segment["camera"], group.indices),
                core.camera_selected(vv, segment["camera"], group.v_indices))

    def output_position(value, group):
        return core.camera_selected(value, hooks["out_camera"], group.v_indices)

    q = data["q"][None].permute(0, 2, 1, 3).contiguous()
    result = core.hybrid_attention(q, q, native, low, reader, query_position=query_position,
                                   kv_position=kv_position, output_position=output_position)
    rope_only = core.hybrid_attention(
        q, q, native, low, reader,
        query_position=lambda value, group: core.rope_selected(value, hooks["q_multiplier"], group.indices),
        kv_position=lambda kk, vv, segment, group: (core.rope_selected(kk, segment["freqs"], group.indices), vv))
    return {"hybrid": bits(result[0]), "rope_only": bits(rope_only[0]),
            "q_digest": np.array([checksum(data["q"])], dtype=np.uint64)}


def run_stream_case(case: cases.CodecCase, root) -> dict:
    """LingBot's codec_cache_attention_inputs chunk by chunk with codec_commit set: the returned
    K / V / positions of every step (history window + current chunk, cut to max_attention_size)."""
    codec = ref_import.load_lingbot_codec(root)
    runtime = load_lingbot_runtime(root)
    data = cases.build(case)
    heads, dim = case.shape.heads, case.shape.head_dim
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_lingbot_operator(
            codec, "synthetic", kind, case.layer, joint_dim=case.shape.joint,
            rank=case.shape.rank, mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"])
    cache = {"global_end_index": torch.zeros(1, dtype=torch.long),
             "local_end_index": torch.zeros(1, dtype=torch.long)}
    runtime.configure_cache(cache, layer=case.layer, sp_rank=0, options={
        "codec_rank": case.shape.rank, "codec_clusters": case.shape.centers, "codec_iters": case.iters,
        "codec_basis_root_k": "synthetic", "codec_basis_root_v": "synthetic"})
    cache["codec_commit"] = True
    out, start = {}, 0
    for step, (key, value) in enumerate(zip(data["k_chunks"], data["v_chunks"])):
        key_cache, value_cache, positions = runtime.codec_cache_attention_inputs(
            cache, key.reshape(1, -1, heads, dim), value.reshape(1, -1, heads, dim),
            current_start=start, **cases.STREAM_POLICY)
        out[f"step{step}_positions"] = positions.numpy()
        out[f"step{step}_key"] = bits(key_cache[0])
        out[f"step{step}_value"] = bits(value_cache[0])
        out[f"step{step}_segments"] = np.array(
            [[s["global_start"], s["global_end"]] for s in cache["codec_segments"]], dtype=np.int64)
        start += key.shape[0]
    out["global_end"] = cache["global_end_index"].numpy()
    out["local_end"] = cache["local_end_index"].numpy()
    return out


def run_attend_case(case: cases.CodecCase, root) -> dict:
    """attend of the LingBot Fast module: the first chunks are committed through
    codec_cache_attention_inputs, the last one attends (sink + recent frames at full width, the rest
    of the window through a two-group reader), without and with the value-mean residual."""
    codec = ref_import.load_lingbot_codec(root)
    runtime = load_lingbot_runtime(root)
    fast = ref_import._load("wan.modules.codec_native_attention",
                            root / ref_import.LB / "wan/modules/codec_native_attention.py")
    data = cases.build(case)
    heads, dim = case.shape.heads, case.shape.head_dim
    os.environ["LINGBOT_CODEC_NATIVE_ENABLE"] = "1"
    os.environ["LINGBOT_CODEC_NATIVE_MANIFEST"] = "synthetic_manifest.json"
    os.environ["LINGBOT_V2_KV_CODEC_PREPACKED_OPERATOR_PATH"] = "synthetic_operator.pt"
    for name in ("LINGBOT_CODEC_NATIVE_HOST_POLICY", "LINGBOT_CODEC_NATIVE_TRITON_ROPE",
                 "LINGBOT_CODEC_NATIVE_TRITON_NATIVE_ROPE", "LINGBOT_CODEC_NATIVE_FUSED_FINISH",
                 "LINGBOT_CODEC_NATIVE_BATCH_READ", "LINGBOT_CODEC_NATIVE_DUMP_ROOT",
                 "LINGBOT_CODEC_NATIVE_D128_JOINT"):
        os.environ.pop(name, None)
    os.environ["LINGBOT_PRE_ROPE_TRITON"] = "0"
    for kind in ("k", "v"):
        op = data[f"{kind}_op"]
        ref_import.inject_lingbot_operator(
            codec, "synthetic", kind, case.layer, joint_dim=case.shape.joint, rank=case.shape.rank,
            mean=op["mean"], encoder=op["encoder"], decoder=op["decoder"], prepacked="synthetic_operator.pt")
    manifest = {"format": "codec_native_manifest_v1", "model": "lingbot-world-v2",
                "policy": dict(cases.ATTEND_POLICY), "layers": {f"0:{case.layer}": {"calibrated": True}}}
    reader = fast._Layer(cases.build_attend_reader(case, data))
    fast._BANK[(str(Path("synthetic_manifest.json").resolve()), "cpu")] = (manifest, {(0, case.layer): reader})
    cache = {"global_end_index": torch.zeros(1, dtype=torch.long),
             "local_end_index": torch.zeros(1, dtype=torch.long)}
    runtime.configure_cache(cache, layer=case.layer, sp_rank=0, options={
        "codec_rank": case.shape.rank, "codec_clusters": case.shape.centers, "codec_iters": case.iters,
        "codec_basis_root_k": "synthetic", "codec_basis_root_v": "synthetic"})
    cache["codec_commit"] = True
    start = 0
    chunks = list(zip(data["k_chunks"], data["v_chunks"]))
    for key, value in chunks[:-1]:
        runtime.codec_cache_attention_inputs(
            cache, key.reshape(1, -1, heads, dim), value.reshape(1, -1, heads, dim),
            current_start=start, **cases.STREAM_POLICY)
        start += key.shape[0]
    cache["codec_commit"] = False
    key, value = (t.reshape(1, -1, heads, dim) for t in chunks[-1])
    grid = cases.ROLLING_GRID
    frame_seqlen = grid["height"] * grid["width"]
    rope_params = reference_rope_params(root)
    freqs = torch.cat([rope_params(1024, dim - 4 * (dim // 6)), rope_params(1024, 2 * (dim // 6)),
                       rope_params(1024, 2 * (dim // 6))], dim=1)
    grid_sizes = torch.tensor([[64, grid["height"], grid["width"]]])
    count = key.shape[1]
    q_pre = data["q"][:count][None]
    positions = torch.arange(start, start + count)
    q_native = runtime.rope_pre_key_by_positions(q_pre, positions, grid_sizes=grid_sizes, freqs=freqs,
                                                 frame_seqlen=frame_seqlen)
    common = dict(current_start=start, grid_sizes=grid_sizes, freqs=freqs, frame_seqlen=frame_seqlen,
                  **cases.STREAM_POLICY)
    os.environ["LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL"] = "0"
    plain = fast.attend(q_pre, q_native, key, value, cache, **common)
    os.environ["LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL"] = "1"
    corrected = fast.attend(q_pre, q_native, key, value, cache, **common)
    os.environ["LINGBOT_CODEC_NATIVE_VALUE_MEAN_RESIDUAL"] = "0"
    return {"plain": bits(plain[0]), "corrected": bits(corrected[0]), "q_native": bits(q_native[0]),
            "start": np.array([start], dtype=np.int64)}


def run_hy_case(root) -> dict:
    """_attend_dictionary_lowkv of HY-WorldPlay's direct latent attention module: Main-RoPE and PRoPE
    branches over a packed INT4 history with per-branch centre tables, native attention over the
    text and current tokens, lift and log-sum-exp combine.  The module's _flash_lse calls a
    CUDA-only ATen kernel; for this CPU run it is replaced by the exact fp32 softmax attention of
    the Matrix-Game core module (attention_lse), which is the only substituted piece."""
    hy = ref_import.load_hy_reader(root)
    core = ref_import.load_mg_core(root)
    from hyvideo.models.transformers.modules.kv_codecs import pack_quantized_codes
    data = cases.build_hy()
    for name in list(os.environ):
        if name.startswith("HY_DIRECT_CODEC"):
            os.environ.pop(name)
    os.environ["HY_DIRECT_CODEC_LATENT_READ_CACHE"] = "0"
    hy._flash_lse = lambda q, k, v, scale=None: core.attention_lse(q, k, v, scale=scale)
    cache = {"vision_freqs_cis": data["vision_freqs"], "vision_viewmats": data["vision_viewmats"],
             "vision_Ks": None}
    for name in ("k_vision", "v_vision"):
        part = dict(data[name])
        part["latent_int4"] = pack_quantized_codes(part.pop("codes"), 4)
        cache[name] = part
    cfg = cases.HY_SHAPE
    runtime = {"recent_native_frames": 0, "attention": data["state"], "main_k_mode": "learned_rope",
               "shape": (cfg["heads"], cfg["head_dim"], cfg["heads"], cfg["head_dim"])}
    main, prope = hy._attend_dictionary_lowkv(
        0, data["q_pre"], data["query"], data["current_key"], data["current_value"], data["encoder_key"],
        data["encoder_value"], cache, data["current_freqs"], data["current_viewmats"], None, runtime)
    return {"main": bits(main), "prope": bits(prope), "packed_k": cache["k_vision"]["latent_int4"].numpy(),
            "q_digest": np.array([checksum(data["q_pre"])], dtype=np.uint64)}


def hy_codec_environment(case: cases.CodecCase) -> None:
    """The environment the reference's HY codec reads for the global-PCA INT4 form with online
    joint-head C-means (kv_codecs.py:70-113,1009-1075)."""
    for name in list(os.environ):
        if name.startswith("HY_KV_CODEC"):
            os.environ.pop(name)
    os.environ.update({
        "HY_KV_CODEC_ENABLE": "1", "HY_KV_CODEC_MODE": "global_pca", "HY_KV_CODEC_COEFF_QUANT": "int4",
        "HY_KV_CODEC_GLOBAL_PCA_RANK": str(case.shape.rank), "HY_KV_CODEC_OPERATOR_WEIGHT_MODE": "bf16",
        "HY_KV_CODEC_SEMANTIC_SMOOTH_K": "1", "HY_KV_CODEC_SEMANTIC_SMOOTH_V": "1",
        "HY_KV_CODEC_SEMANTIC_CLUSTERS": str(case.shape.centers), "HY_KV_CODEC_SEMANTIC_ITERS": str(case.iters),
        "HY_KV_CODEC_DETERMINISTIC_CENTERS": "1", "HY_KV_CODEC_PROFILE": "0",
        "HY_KV_CODEC_SEMANTIC_BASIS_DIR_K": "synthetic_k", "HY_KV_CODEC_SEMANTIC_BASIS_DIR_V": "synthetic_v",
        "HY_KV_CODEC_SEMANTIC_LINEAR_DIR_K": "synthetic_k", "HY_KV_CODEC_SEMANTIC_LINEAR_DIR_V": "synthetic_v",
    })


def run_hy_codec_case(case: cases.CodecCase, root) -> dict:
    """compress_kv_tensor / decompress_kv_tensor of HY-WorldPlay's codec module on [1, H, S, D] tensors
    (global PCA, INT4 coefficients, online joint-head C-means, bf16 operators)."""
    codec = ref_import.load_hy_codec(root)
    hy_codec_environment(case)
    data = cases.build(case)
    shape = case.shape
    out = {}
    for name in ("k", "v"):
        op = data[f"{name}_op"]
        ref_import.inject_hy_operator(codec, name, case.layer, mean=op["mean"], encoder=op["encoder"],
                                      decoder=op["decoder"], storage="bf16")
        rows = data[f"{name}_chunks"][0]
        x = rows.reshape(1, -1, shape.heads, shape.head_dim).permute(0, 2, 1, 3).contiguous()
        payload, stats = codec.compress_kv_tensor(x, case.layer, name)
        out[f"{name}_ids"] = payload["semantic_ids"].numpy()
        out[f"{name}_centers"] = bits(payload["semantic_centers"])
        out[f"{name}_packed"] = payload["latent_int8"].numpy()
        out[f"{name}_scale"] = bits(payload["latent_scale"])
        out[f"{name}_bytes"] = np.array([int(stats["actual_bytes"])], dtype=np.int64)
        out[f"{name}_decoded_bf16"] = bits(codec.decompress_kv_tensor(payload, torch.bfloat16, "cpu")[:, :, :48])
        out[f"{name}_decoded_f32"] = codec.decompress_kv_tensor(payload, torch.float32, "cpu")[:, :, :16].numpy()
        out[f"{name}_digest"] = np.array([checksum(x)], dtype=np.uint64)
    return out


def hy_write_runtime(data: dict) -> dict:
    cfg = cases.HY_WRITE
    return {"operators": data["operators"], "attention": data["attention"], "payload_mode": "dictionary_lowkv",
            "main_k_mode": "learned_rope", "recent_native_frames": 0,
            "shape": (cfg["heads"], cfg["head_dim"], cfg["heads"], cfg["head_dim"])}


def run_hy_write_case(root) -> dict:
    """_compress_one of HY-WorldPlay's direct latent attention module (the body of compress_layer_cache)
    on raw [1, 16, S, 128] history: packed codes, fp32 scales, ids and the two branches' centre tables."""
    hy = ref_import.load_hy_reader(root)
    cfg = cases.HY_WRITE
    for name in list(os.environ):
        if name.startswith("HY_KV_CODEC") or name.startswith("HY_DIRECT_CODEC"):
            os.environ.pop(name)
    os.environ.update({"HY_KV_CODEC_SEMANTIC_CLUSTERS": str(cfg["centres"]), "HY_KV_CODEC_SEMANTIC_ITERS": "2",
                       "HY_KV_CODEC_DETERMINISTIC_CENTERS": "1", "HY_KV_CODEC_PROFILE": "0"})
    data = cases.build_hy_write()
    runtime = hy_write_runtime(data)
    out = {}
    for name in ("k", "v"):
        payload = hy._compress_one(data[f"{name}_vision"], cfg["layer"], name, runtime)
        out[f"{name}_packed"] = payload["latent_int4"].numpy()
        out[f"{name}_scale"] = payload["latent_scale"].numpy()
        out[f"{name}_ids"] = payload["semantic_ids"].numpy()
        out[f"{name}_centre_main"] = bits(payload["centre_main"])
        out[f"{name}_centre_prope"] = bits(payload["centre_prope"])
        out[f"{name}_digest"] = np.array([checksum(data[f"{name}_vision"])], dtype=np.uint64)
    return out


def run_hy_chain_case(root) -> dict:
    """HY-WorldPlay Fast end to end on one layer: the module's _compress_one on the raw K / V history,
    then its _attend_dictionary_lowkv over the payloads it made (the CUDA-only _flash_lse replaced by the
    exact fp32 attention of the Matrix-Game core module, as in the two-branch fixture)."""
    hy = ref_import.load_hy_reader(root)
    core = ref_import.load_mg_core(root)
    cfg = cases.HY_CHAIN
    for name in list(os.environ):
        if name.startswith("HY_KV_CODEC") or name.startswith("HY_DIRECT_CODEC"):
            os.environ.pop(name)
    os.environ.update({"HY_KV_CODEC_SEMANTIC_CLUSTERS": str(cfg["centres"]), "HY_KV_CODEC_SEMANTIC_ITERS": "2",
                       "HY_KV_CODEC_DETERMINISTIC_CENTERS": "1", "HY_KV_CODEC_PROFILE": "0",
                       "HY_DIRECT_CODEC_LATENT_READ_CACHE": "0"})
    hy._flash_lse = lambda q, k, v, scale=None: core.attention_lse(q, k, v, scale=scale)
    data = cases.build_hy_chain()
    runtime = cases.hy_chain_runtime(data)
    cache = {"vision_freqs_cis": data["vision_freqs"], "vision_viewmats": data["vision_viewmats"], "vision_Ks": None}
    for name in ("k", "v"):
        cache[f"{name}_vision"] = hy._compress_one(data[f"{name}_vision"], cfg["layer"], name, runtime)
    main, prope = hy._attend_dictionary_lowkv(
        cfg["layer"], data["q_pre"], data["query"], data["current_key"], data["current_value"], data["encoder_key"],
        data["encoder_value"], cache, data["current_freqs"], data["current_viewmats"], None, runtime)
    return {"main": bits(main[:, ::4]), "prope": bits(prope[:, ::4]),
            "k_ids": cache["k_vision"]["semantic_ids"].numpy(),
            "q_digest": np.array([checksum(data["q_pre"])], dtype=np.uint64)}


def run_protected_tokens_case(root) -> dict:
    """protected_tokens of the MG core module on seeded frame-id sequences."""
    core = ref_import.load_mg_core(root)
    return {f"keep{index}": core.protected_tokens(ids, recent, stride, sink).numpy()
            for index, (ids, recent, stride, sink) in enumerate(cases.protected_token_cases())}


def run_rope_per_token_case(root) -> dict:
    """rope_selected of the MG core module: multipliers handed over per token."""
    core = ref_import.load_mg_core(root)
    data = cases.build_rope_selected()
    out = core.rope_selected(data["value"], cases.per_token_multiplier(data), data["indices"])
    return {"rotated": bits(out), "value_digest": np.array([checksum(data["value"])], dtype=np.uint64)}


def run_camera_case(root) -> dict:
    """camera_selected of the MG core module (torch path)."""
    core = ref_import.load_mg_core(root)
    data = cases.build_camera()
    os.environ.pop("MG35_CODEC_NATIVE_FUSED_CAMERA", None)
    os.environ.pop("MG35_CODEC_NATIVE_RUNTIME_OPT", None)
    out = core.camera_selected(data["value"], data["matrix"], data["indices"])
    return {"transformed": bits(out), "value_digest": np.array([checksum(data["value"])], dtype=np.uint64)}


def run_int8_operator_case(root) -> dict:
    """The reference's INT8 operator packing and the bf16 weight it multiplies with."""
    codec = ref_import.load_mg_codec(root)
    out = {}
    for name, group in (("per_row", 0), ("group64", 64)):
        weight = cases.build_int8_weight()
        os.environ["MG35_KVCODEC_OPERATOR_WEIGHT_MODE"] = "int8"
        os.environ["MG35_KVCODEC_INT8_WEIGHT_GROUP_SIZE"] = str(group)
        packed = codec._pack_operator(weight, torch.device("cpu"))
        os.environ.pop("MG35_CODEC_NATIVE_WEIGHT_DEQUANT_OPT", None)
        # _operator_linear with an identity input returns the dequantised weight's transpose rows:
        eye = torch.eye(weight.shape[1], dtype=torch.bfloat16)
        dense = codec._operator_linear(eye, packed).t().contiguous()       # [rows, in] bf16
        out[f"{name}_qweight"] = packed["qweight"].numpy()
        out[f"{name}_scale"] = bits(packed["scale"])
        out[f"{name}_dense"] = bits(dense)
    os.environ["MG35_KVCODEC_OPERATOR_WEIGHT_MODE"] = "int8"
    os.environ.pop("MG35_KVCODEC_INT8_WEIGHT_GROUP_SIZE", None)
    out["weight_digest"] = np.array([checksum(cases.build_int8_weight())], dtype=np.uint64)
    return out


def run_rope_case(case: cases.RopeCase, root) -> dict:
    ref_import.load_lingbot_codec(root)
    runtime = ref_import._load("wan.modules.lingbot_v2_cache_runtime",
                               root / ref_import.LB / "wan/modules/lingbot_v2_cache_runtime.py")
    rope_params = reference_rope_params(root)
    d = case.head_dim
    freqs = torch.cat([rope_params(1024, d - 4 * (d // 6)), rope_params(1024, 2 * (d // 6)),
                       rope_params(1024, 2 * (d // 6))], dim=1)   # model.py:426-430
    data = cases.build_rope(case)
    os.environ["LINGBOT_PRE_ROPE_TRITON"] = "0"
    out = runtime.rope_pre_key_by_positions(data["key"], data["positions"],
                                            grid_sizes=data["grid_sizes"], freqs=freqs,
                                            frame_seqlen=data["frame_seqlen"])
    return {"rotated": bits(out), "freqs_head": torch.view_as_real(freqs[:64]).numpy(),   # rows in use
            "freqs_digest": np.array([checksum(torch.view_as_real(freqs).contiguous())], dtype=np.uint64),
            "key_digest": np.array([checksum(data["key"])], dtype=np.uint64)}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=None)
    parser.add_argument("--only", default="", help="regenerate only fixtures whose name starts with this")
    args = parser.parse_args()
    global save
    write = save
    save = lambda name, arrays: write(name, arrays()) if name.startswith(args.only) else None
    root = ref_import.reference_root(args.reference)
    torch.set_num_threads(1)  # one thread: bit-stable reductions in the stored outputs
    for case in cases.MG_CASES:
        save(case.name, lambda: run_mg_case(case, root))
    for case in cases.LINGBOT_CASES:
        save(case.name, lambda: run_lingbot_case(case, root))
    for case in cases.FAST_CASES:
        save(case.name, lambda: run_fast_case(case, root))
    save("fast_masked_bf16", lambda: run_fast_case(cases.FAST_CASES[1], root, masked=True))
    save("fast_hooks_bf16", lambda: run_fast_hooks_case(cases.FAST_CASES[1], root))
    save("stream_lb_bf16", lambda: run_stream_case(cases.ROLLING, root))
    save("attend_lb_bf16", lambda: run_attend_case(cases.ROLLING, root))
    save("hy_two_branch_bf16", lambda: run_hy_case(root))
    save(cases.HY_CODEC.name, lambda: run_hy_codec_case(cases.HY_CODEC, root))
    save("hy_write_bf16", lambda: run_hy_write_case(root))
    save("hy_chain_bf16", lambda: run_hy_chain_case(root))
    save("protected_tokens", lambda: run_protected_tokens_case(root))
    save("merge_edge", lambda: run_merge_case(root))
    save("select_mg_bf16", lambda: run_select_case(cases.MINI_BF16, root))
    save("rope_selected_bf16", lambda: run_rope_selected_case(root))
    save("rope_per_token_bf16", lambda: run_rope_per_token_case(root))
    save("camera_bf16", lambda: run_camera_case(root))
    save("value_mean_lb_bf16", lambda: run_value_mean_case(cases.ROLLING, root))
    save("int8_operator", lambda: run_int8_operator_case(root))
    save(cases.ROLLING.name, lambda: run_rolling_case(cases.ROLLING, root))
    for case in cases.ROPE_CASES:
        save(case.name, lambda: run_rope_case(case, root))


if __name__ == "__main__":
    main()
