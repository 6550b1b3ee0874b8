"""ctypes binding of libnanokv_b200.so (the C ABI in include/nanokv_b200.h).

There is no fallback: if the shared library is missing and cannot be built,
importing the product path raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

from . import build as _build


class Rope(ctypes.Structure):
    """struct nkv_rope"""
    _fields_ = [("positions", c_void_p), ("cos_sin", c_void_p), ("table_rows", c_int32),
                ("frame_seqlen", c_int32), ("width", c_int32), ("table_half", c_int32),
                ("pair_index", c_void_p)]


class Camera(ctypes.Structure):
    """struct nkv_camera"""
    _fields_ = [("matrices", c_void_p), ("cam_index", c_void_p), ("frames", c_int32),
                ("tokens_per_frame", c_int32)]


NKV_OK = 0
NKV_ERR_INVALID, NKV_ERR_CUDA, NKV_ERR_UNSUPPORTED, NKV_ERR_DEVICE_WAIT, NKV_ERR_TOO_LARGE = (
    -1, -2, -3, -4, -5)
NKV_F32, NKV_BF16, NKV_F16 = 0, 1, 2
NKV_QUANT_F32, NKV_QUANT_IN_BF16 = 0, 1


class History(ctypes.Structure):
    """struct nkv_history"""
    _fields_ = [
        ("codes", c_void_p), ("scales", c_void_p), ("ids", c_void_p), ("centers", c_void_p),
        ("seg_start", c_void_p), ("seg_center_row", c_void_p),
        ("tokens", c_int32), ("segments", c_int32), ("rank", c_int32), ("group", c_int32),
        ("scale_dtype", c_int32), ("id_bytes", c_int32), ("center_rows", c_int32),
        ("center_width", c_int32),
    ]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "nkv_status_string": (c_char_p, [c_int]),
    "nkv_last_error": (c_char_p, []),
    "nkv_version": (c_int, []),
    "nkv_assign": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                           c_void_p]),
    "nkv_kmeans_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "nkv_kmeans": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "nkv_project": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_int, c_void_p, c_void_p]),
    "nkv_quant_pack": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                               c_void_p, c_void_p, c_void_p]),
    "nkv_project_quant": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p, c_size_t, c_void_p]),
    "nkv_encode_append": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "nkv_encode_append_static": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                         c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nkv_decode_rows": (c_int, [POINTER(History), c_void_p, c_int, c_void_p, c_int, c_void_p,
                                c_int, c_void_p, c_int, c_void_p]),
    "nkv_attn_codec": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int,
                               POINTER(History), POINTER(History), c_void_p, c_void_p, c_void_p,
                               c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nkv_attn_codec_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nkv_attn_codec_split": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                     POINTER(History), POINTER(History), c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_size_t, c_void_p]),
    "nkv_attn_codec_rope": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                    POINTER(History), POINTER(History), c_void_p, c_void_p,
                                    c_void_p, c_void_p, POINTER(Rope), c_float, c_void_p, c_void_p,
                                    c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "nkv_attn_codec_pos": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                   POINTER(History), POINTER(History), c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, POINTER(Rope), POINTER(Camera), POINTER(Camera),
                                   c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t,
                                   c_void_p]),
    "nkv_decoder_prepare": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "nkv_camera_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, POINTER(Camera),
                                c_void_p, c_void_p]),
    "nkv_rope_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, POINTER(Rope),
                              c_void_p, c_void_p]),
    "nkv_attention_lse": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                  c_int64, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                  c_void_p, c_void_p]),
    "nkv_lse_merge": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int64, c_int, c_int,
                              c_void_p, c_void_p, c_void_p]),
    "nkv_history_moments_workspace_bytes": (c_size_t, [c_int, c_int]),
    "nkv_history_moments": (c_int, [POINTER(History), c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "nkv_fast_finish": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "nkv_operator_unpack_int8": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nkv_peer_alloc": (c_int, [c_int64, POINTER(c_void_p), c_char_p]),
    "nkv_cp_exchange_peer": (c_int, [POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
                                     POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_int64, c_int,
                                     c_int64, c_int64, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p]),
    "nkv_head_linear": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                c_int, c_int, c_void_p, c_void_p]),
    "nkv_set_bf16_path": (c_int, [c_int]),
    "nkv_selftest_bounded_wait": (c_int, [c_int, ctypes.c_longlong, c_void_p, c_void_p]),
    "nkv_peer_open": (c_int, [c_char_p, POINTER(c_void_p)]),
    "nkv_peer_close": (c_int, [c_void_p]),
    "nkv_peer_free": (c_int, [c_void_p]),
    "nkv_cp_merge_peer": (c_int, [POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
                                  POINTER(c_void_p), c_int, c_int64, c_int, c_int64, c_int64, c_int,
                                  c_void_p]),
}

_EXCEPTIONS = {NKV_ERR_INVALID: ValueError, NKV_ERR_TOO_LARGE: ValueError}

_lib = None


def library() -> ctypes.CDLL:
    """Load (building first if the tree has no up-to-date .so) and bind."""
    global _lib
    if _lib is None:
        path = _build.build()
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int) -> None:
    """Map a status code to the exception class the reference API raises."""
    if status == NKV_OK:
        return
    lib = library()
    detail = lib.nkv_last_error().decode()
    kind = lib.nkv_status_string(status).decode()
    raise _EXCEPTIONS.get(status, RuntimeError)(f"nanokv_b200: {kind}: {detail}")


STATUS_SCORE_RANGE = 950


def check_device_status(word: int) -> None:
    """Raise for a non-zero status word that a kernel left behind.

    The fused read writes the site code of a bounded wait that gave up (its rows are then not
    results: their LSE is NaN), or STATUS_SCORE_RANGE when a row's scores left the window of the
    online softmax (that row's LSE is NaN).  NKV_OK from the launching call only says that the
    launch was accepted; the word is valid once the stream has been synchronised."""
    if word == 0:
        return
    if word == STATUS_SCORE_RANGE:
        raise RuntimeError("nanokv_b200: attention scores of a row rose more than 2^96 above the "
                           "maximum of the tiles before them; that row's LSE is NaN")
    kind = library().nkv_status_string(NKV_ERR_DEVICE_WAIT).decode()
    raise RuntimeError(f"nanokv_b200: {kind}: wait site {word}")
