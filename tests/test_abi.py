"""The C ABI: the library builds, loads, and exports every symbol the header declares."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "nanokv_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nkv_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("nkv_assign", "nkv_kmeans", "nkv_project", "nkv_quant_pack",
                     "nkv_encode_append", "nkv_decode_rows", "nkv_attn_codec",
                     "nkv_attention_lse", "nkv_lse_merge", "nkv_status_string", "nkv_version"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from nanokv_b200 import _lib
    lib = _lib.library()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.nkv_version() == 1
    assert lib.nkv_status_string(0) == b"ok"
    assert lib.nkv_status_string(-4) == b"device-side wait gave up"


def test_argument_errors_need_no_gpu():
    """Validation happens before any CUDA call, so bad arguments are reported on any host."""
    from nanokv_b200 import _lib
    lib = _lib.library()
    status = lib.nkv_quant_pack(None, _lib.NKV_BF16, 4, 64, 48, 1e-7, 0, _lib.NKV_BF16, None,
                                None, None)
    assert status == _lib.NKV_ERR_INVALID
    assert b"group" in lib.nkv_last_error()
    with pytest.raises(ValueError):
        _lib.check(status)
    status = lib.nkv_assign(None, _lib.NKV_BF16, None, _lib.NKV_BF16, 8, 64, 300, None, 1, None)
    assert status == _lib.NKV_ERR_INVALID


def test_product_path_has_no_cpu_fallback():
    import torch
    from nanokv_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.quant_pack(torch.zeros(4, 64))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.assign(torch.zeros(4, 64), torch.zeros(2, 64))


def test_product_never_imports_the_oracle():
    for path in (ROOT / "nanokv_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text.replace("no CPU", ""), f"{path} mentions the oracle"


def test_host_layer_exposes_a_wrapper_for_every_entry_point():
    """Each C entry point has its host-side caller (an edit that drops one must fail here, on CPU)."""
    from nanokv_b200 import attention, codec, context_parallel, lifecycle, mg_codec, ops
    expected = {
        ops: ["assign", "kmeans", "project", "quant_pack", "decode_rows", "attn_codec", "attention_lse",
              "lse_merge", "rope_rows", "RopeView", "HistoryView", "unpack_int8_weight", "PeerBuffer",
              "cp_merge_peer", "force_simt", "default_splits", "fast_finish", "history_moments",
              "camera_rows", "prepare_decoder"],
        attention: ["codec_attention", "merge", "RopeTable", "ReaderGroup", "Reader", "hybrid_attention"],
        codec: ["Operator", "QuantSpec", "encode_append", "decode", "kmeans_init_rows"],
        context_parallel: ["shard_bounds", "gather_partials", "merge_partials", "gather_and_merge",
                           "PeerExchange"],
        lifecycle: ["active_intervals", "kept_segments", "active_pieces", "RollingHistory"],
        mg_codec: ["register_operator", "encode_tensor", "decode_tensor", "decode_value", "concat_values",
                   "select_value", "value_shape", "payload_bytes", "history_from_payloads"],
    }
    for module, names in expected.items():
        missing = [name for name in names if not hasattr(module, name)]
        assert not missing, f"{module.__name__} lost {missing}"
