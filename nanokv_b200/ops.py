"""Tensor-level wrappers over the C ABI.

Each function takes CUDA tensors, enqueues on torch's current stream and
returns without synchronising.  PyTorch is used for device memory and streams
only; all arithmetic happens in libnanokv_b200.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import NKV_BF16, NKV_F16, NKV_F32, NKV_QUANT_F32, NKV_QUANT_IN_BF16, History

_DTYPE = {torch.float32: NKV_F32, torch.bfloat16: NKV_BF16, torch.float16: NKV_F16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}") from None


def _ptr(tensor: torch.Tensor | None):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise RuntimeError("nanokv_b200 runs on CUDA tensors only (there is no CPU path)")
        if not tensor.is_contiguous():
            raise ValueError("nanokv_b200 expects contiguous tensors")
        device = device or tensor.device
    return device


def id_dtype(clusters: int) -> torch.dtype:
    """uint8 ids up to 256 centres (the reference's storage), int16 bit patterns beyond."""
    return torch.uint8 if clusters <= 256 else torch.int16


# --------------------------------------------------------------------------- encode
def assign(x: torch.Tensor, centers: torch.Tensor, ids: torch.Tensor | None = None) -> torch.Tensor:
    """Nearest-centre ids of rows x [S,J] against centers [C,J]."""
    device = _require_cuda(x, centers, ids)
    S, J = x.shape
    C = centers.shape[0]
    if ids is None:
        ids = torch.empty(S, dtype=id_dtype(C), device=device)
    _lib.check(_lib.library().nkv_assign(
        _ptr(x), dtype_code(x.dtype), _ptr(centers), dtype_code(centers.dtype), S, J, C,
        _ptr(ids), ids.element_size(), _stream(device)))
    return ids


def kmeans(x: torch.Tensor, clusters: int, iters: int, init_rows: torch.Tensor, *,
           centers: torch.Tensor | None = None, ids: torch.Tensor | None = None):
    """Online C-means of one chunk -> (stored centres bf16 [C,J], ids [S])."""
    device = _require_cuda(x, centers, ids)
    S, J = x.shape
    lib = _lib.library()
    if not 0 < clusters <= S:
        raise ValueError(f"clusters must be in [1, S]; got {clusters} for S={S}")
    if centers is None:
        centers = torch.empty(clusters, J, dtype=torch.bfloat16, device=device)
    if ids is None:
        ids = torch.empty(S, dtype=id_dtype(clusters), device=device)
    nbytes = lib.nkv_kmeans_workspace_bytes(S, J, clusters)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
    init_rows = init_rows.to(device=device, dtype=torch.int32).contiguous()
    _lib.check(lib.nkv_kmeans(
        _ptr(x), dtype_code(x.dtype), S, J, clusters, iters, _ptr(init_rows), _ptr(centers),
        _ptr(ids), ids.element_size(), _ptr(workspace), nbytes, _stream(device)))
    return centers, ids


def project(x, centers_bf16, ids, mean, encoder) -> torch.Tensor:
    """coeff [S,r] = ((x - centre[id]) - mean) @ encoder^T in the encoder dtype."""
    device = _require_cuda(x, centers_bf16, ids, mean, encoder)
    S, J = x.shape
    r = encoder.shape[0]
    coeff = torch.empty(S, r, dtype=encoder.dtype, device=device)
    _lib.check(_lib.library().nkv_project(
        _ptr(x), dtype_code(x.dtype), _ptr(centers_bf16), _ptr(ids), ids.element_size(),
        _ptr(mean), _ptr(encoder), dtype_code(encoder.dtype), S, J, r, _ptr(coeff),
        _stream(device)))
    return coeff


def quant_pack(coeff, *, group=None, eps=1.1920928955078125e-07, in_coeff_dtype=False,
               scale_dtype=torch.bfloat16, codes=None, scales=None):
    """INT4 quantise + pack -> (codes u8 [S,r/2], scales [S,r/group])."""
    device = _require_cuda(coeff, codes, scales)
    S, r = coeff.shape
    group = r if group is None else int(group)
    if codes is None:
        codes = torch.empty(S, r // 2, dtype=torch.uint8, device=device)
    if scales is None:
        scales = torch.empty(S, r // group, dtype=scale_dtype, device=device)
    _lib.check(_lib.library().nkv_quant_pack(
        _ptr(coeff), dtype_code(coeff.dtype), S, r, group, float(eps),
        NKV_QUANT_IN_BF16 if in_coeff_dtype else NKV_QUANT_F32, dtype_code(scales.dtype),
        _ptr(codes), _ptr(scales), _stream(device)))
    return codes, scales


def project_quant(x, centers_bf16, ids, mean, encoder, *, group=None, eps=1.1920928955078125e-07,
                  in_coeff_dtype=False, scale_dtype=torch.bfloat16, codes=None, scales=None):
    """project + quant_pack of rows whose centre ids are known -> (codes u8 [S,r/2], scales
    [S,r/group]); one kernel (coefficients never leave the chip) for bf16 operands with one scale per
    token, the two kernels through a scratch tensor otherwise.  Same bytes either way."""
    device = _require_cuda(x, centers_bf16, ids, mean, encoder, codes, scales)
    S, J = x.shape
    r = encoder.shape[0]
    group = r if group is None else int(group)
    if codes is None:
        codes = torch.empty(S, r // 2, dtype=torch.uint8, device=device)
    if scales is None:
        scales = torch.empty(S, r // group, dtype=scale_dtype, device=device)
    fused = (x.dtype == encoder.dtype == torch.bfloat16 and group == r and r % 64 == 0
             and not _SIMT_FORCED[0] and codes.data_ptr() % 16 == 0)
    workspace = None if fused else torch.empty(S, r, dtype=encoder.dtype, device=device)
    status = _lib.library().nkv_project_quant(
        _ptr(x), dtype_code(x.dtype), _ptr(centers_bf16), _ptr(ids), ids.element_size(), _ptr(mean),
        _ptr(encoder), dtype_code(encoder.dtype), S, J, r, group, float(eps),
        NKV_QUANT_IN_BF16 if in_coeff_dtype else NKV_QUANT_F32, dtype_code(scales.dtype), _ptr(codes),
        _ptr(scales), _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
        _stream(device))
    if status == _lib.NKV_ERR_INVALID and workspace is None:
        # the single-kernel form did not apply to this shape after all: once more with scratch
        workspace = torch.empty(S, r, dtype=encoder.dtype, device=device)
        status = _lib.library().nkv_project_quant(
            _ptr(x), dtype_code(x.dtype), _ptr(centers_bf16), _ptr(ids), ids.element_size(), _ptr(mean),
            _ptr(encoder), dtype_code(encoder.dtype), S, J, r, group, float(eps),
            NKV_QUANT_IN_BF16 if in_coeff_dtype else NKV_QUANT_F32, dtype_code(scales.dtype), _ptr(codes),
            _ptr(scales), _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(device))
    _lib.check(status)
    return codes, scales


# ---------------------------------------------------------------------- history view
@dataclass
class HistoryView:
    """Device arrays of one compressed tensor plus the struct the ABI takes."""
    codes: torch.Tensor
    scales: torch.Tensor
    ids: torch.Tensor
    centers: torch.Tensor
    seg_start: torch.Tensor
    seg_center_row: torch.Tensor
    tokens: int
    segments: int
    rank: int
    group: int

    def struct(self) -> History:
        return History(
            self.codes.data_ptr(), self.scales.data_ptr(), self.ids.data_ptr(),
            self.centers.data_ptr(), self.seg_start.data_ptr(), self.seg_center_row.data_ptr(),
            self.tokens, self.segments, self.rank, self.group, dtype_code(self.scales.dtype),
            self.ids.element_size(), self.centers.shape[0], self.centers.shape[1])


def gather_view(view: HistoryView, index: torch.Tensor) -> HistoryView:
    """The history restricted to the tokens listed in ``index`` (increasing, device i64): codes,
    scales and ids are gathered, every segment keeps its centre rows and shrinks to its listed
    tokens (a segment none of whose tokens is listed becomes empty).  This is how a boolean
    visibility mask over the keys is applied to a compressed history: nothing is decoded."""
    _require_cuda(view.codes, index)
    index = index.to(torch.int64)
    starts = view.seg_start[:view.segments + 1].to(torch.int64)
    seg_start = torch.searchsorted(index, starts).to(torch.int32)
    return HistoryView(
        codes=view.codes.index_select(0, index), scales=view.scales.index_select(0, index),
        ids=view.ids.index_select(0, index), centers=view.centers, seg_start=seg_start,
        seg_center_row=view.seg_center_row, tokens=int(index.numel()), segments=view.segments,
        rank=view.rank, group=view.group)


def decode_rows(view: HistoryView, decoder, mean, *, rows=None, dtype=None) -> torch.Tensor:
    """Reconstruct rows (all, or those listed in ``rows``) -> [n, J]."""
    device = _require_cuda(decoder, mean, rows)
    J = decoder.shape[0]
    n = view.tokens if rows is None else rows.numel()
    dtype = decoder.dtype if dtype is None else dtype
    out = torch.empty(n, J, dtype=dtype, device=device)
    if rows is not None:
        rows = rows.to(dtype=torch.int32).contiguous()
    struct = view.struct()
    _lib.check(_lib.library().nkv_decode_rows(
        ctypes.byref(struct), _ptr(rows), n, _ptr(decoder), dtype_code(decoder.dtype), _ptr(mean),
        J, _ptr(out), dtype_code(dtype), _stream(device)))
    return out


# ------------------------------------------------------------------------ attention
def default_splits(tokens: int) -> int:
    """Upper bound on the history splits of one fused launch; the library picks the count below it
    that fills its groups of thread blocks most evenly (runs of at least 24 tiles)."""
    return max(1, min(8, tokens // (24 * 128)))


_STATUS_WORDS: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The per-device int32 word the fused read reports into when the caller passes none."""
    key = torch.device(device)
    if key not in _STATUS_WORDS:
        _STATUS_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _STATUS_WORDS[key]


def check_status(device=None) -> None:
    """Synchronise and raise if a fused read on ``device`` (default: every device used so far) left a
    status behind: a bounded device-side wait that gave up, or a row whose scores left the softmax
    window.  The word is cleared.  Results of launches since the last check are only to be trusted
    after this returns."""
    words = [status_word(device)] if device is not None else list(_STATUS_WORDS.values())
    for word in words:
        value = int(word.item())      # synchronises the device
        if value:
            word.zero_()
            _lib.check_device_status(value)


def attn_codec(q, view_k: HistoryView, view_v: HistoryView, wk, bias_k, wv, bias_v, *,
               scale: float, status: torch.Tensor | None = None, splits: int | None = None,
               out: torch.Tensor | None = None, lse: torch.Tensor | None = None,
               rope: "RopeView | None" = None, camera_k: "CameraView | None" = None,
               camera_v: "CameraView | None" = None, prepared: bool = False):
    """Fused read: q [Q,H,dk] -> (O [Q,H,dv], lse f32 [Q,H]).

    wk [H,dk,r], wv [H,dv,r] in q's dtype; bias f32 [H,dk] / [H,dv].  ``splits`` cuts the
    history into that many runs attended in one launch and merged by LSE (None: automatic).
    ``out`` / ``lse`` name contiguous result buffers to fill (e.g. peer-visible ones).
    ``rope`` rotates the rebuilt keys by the absolute position of every history token;
    ``camera_k`` / ``camera_v`` apply the PRoPE camera transform to the rebuilt keys / values.
    ``prepared``: wk / wv came from :func:`prepare_decoder` (kernel order; bf16 tensor-core path only).
    """
    device = _require_cuda(wk, bias_k, wv, bias_v, status)
    if not q.is_cuda:
        raise RuntimeError("nanokv_b200 runs on CUDA tensors only (there is no CPU path)")
    Q, H, dk = q.shape
    dv = wv.shape[1]
    if q.stride(2) != 1:
        raise ValueError("queries must be contiguous along the head dimension")
    if out is None:
        out = torch.empty(Q, H, dv, dtype=q.dtype, device=device)
    if lse is None:
        lse = torch.empty(Q, H, dtype=torch.float32, device=device)
    if (tuple(out.shape) != (Q, H, dv) or out.dtype != q.dtype or not out.is_contiguous()
            or tuple(lse.shape) != (Q, H) or lse.dtype != torch.float32 or not lse.is_contiguous()):
        raise ValueError("result buffers must be contiguous [Q,H,dv] in q's dtype and f32 [Q,H]")
    _require_cuda(out, lse)
    if status is None:   # a launch always has somewhere to report a wait that gave up: check_status()
        status = status_word(device)
    sk, sv = view_k.struct(), view_v.struct()
    lib = _lib.library()
    if splits is None:
        splits = default_splits(view_k.tokens) if q.dtype == torch.bfloat16 else 1
    nbytes = lib.nkv_attn_codec_workspace_bytes(Q, H, dv, splits)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None
    rope_struct = None
    if rope is not None:
        if rope.positions.numel() < view_k.tokens:
            raise ValueError("RoPE position/K length mismatch")
        if rope.pair_index is None and rope.cos_sin.shape[1] != dk // 2:
            raise ValueError("rotation table width does not match the head width")
        if rope.pair_index is not None and tuple(rope.pair_index.shape) != (H, dk // 2):
            raise ValueError("pair index must be [heads, head_dim/2]")
        rope_struct = ctypes.byref(rope.struct())
    cameras = []
    for camera, width in ((camera_k, dk), (camera_v, dv)):
        if camera is not None and tuple(camera.cam_index.shape) != (H, width // 8):
            raise ValueError("camera index must be [heads, head_dim/8]")
        cameras.append(None if camera is None else ctypes.byref(camera.struct()))
    _lib.check(lib.nkv_attn_codec_pos(
        _ptr(q), dtype_code(q.dtype), q.stride(0), q.stride(1), Q, H, dk, dv, ctypes.byref(sk),
        ctypes.byref(sv), _ptr(wk), _ptr(bias_k), _ptr(wv), _ptr(bias_v), 1 if prepared else 0,
        rope_struct, cameras[0],
        cameras[1], float(scale), _ptr(out), _ptr(lse), _ptr(status), splits, _ptr(workspace), nbytes,
        _stream(device)))
    return out, lse


def prepare_decoder(weight: torch.Tensor) -> torch.Tensor:
    """bf16 decoder / reader rows [..., rank] in the order the tensor-core kernel expands code words
    (nkv_decoder_prepare): a one-time copy per operator; pass it with ``prepared=True``."""
    device = _require_cuda(weight)
    if weight.dtype != torch.bfloat16 or weight.shape[-1] % 8:
        raise ValueError("prepare_decoder takes bf16 rows whose length is a multiple of 8")
    out = torch.empty_like(weight)
    rank = weight.shape[-1]
    _lib.check(_lib.library().nkv_decoder_prepare(_ptr(weight), weight.numel() // rank, rank, _ptr(out),
                                                  _stream(device)))
    return out


def tensor_core_read(dtype: torch.dtype, dk: int, dv: int, rank: int) -> bool:
    """Whether nkv_attn_codec runs this shape on the tcgen05 kernel (and may take prepared weights)."""
    return (dtype == torch.bfloat16 and dk == dv and dk in (64, 128) and rank % 64 == 0
            and not _SIMT_FORCED[0])


_SIMT_FORCED = [False]


class CameraView:
    """struct nkv_camera over device tensors: matrices f32 [frames, 4, 4, 4], cam_index i32
    [heads, head_dim/8]; tokens are split evenly over the frames."""

    def __init__(self, matrices: torch.Tensor, cam_index: torch.Tensor, tokens_per_frame: int):
        _require_cuda(matrices, cam_index)
        if matrices.dtype != torch.float32 or matrices.dim() != 4 or tuple(matrices.shape[1:]) != (4, 4, 4):
            raise ValueError("camera matrices must be float32 [frames, 4, 4, 4]")
        if cam_index.dtype != torch.int32 or cam_index.dim() != 2:
            raise ValueError("camera index must be int32 [heads, head_dim/8]")
        if tokens_per_frame <= 0:
            raise ValueError("tokens_per_frame must be positive")
        self.matrices, self.cam_index, self.tokens_per_frame = matrices, cam_index, int(tokens_per_frame)

    def struct(self) -> "_lib.Camera":
        return _lib.Camera(self.matrices.data_ptr(), self.cam_index.data_ptr(),
                           int(self.matrices.shape[0]), self.tokens_per_frame)


def camera_rows(x: torch.Tensor, camera: CameraView) -> torch.Tensor:
    """PRoPE camera transform of explicit rows x [S,H,d] (nkv_camera_rows) -> contiguous [S,H,d]."""
    device = _require_cuda(camera.matrices)
    if not x.is_cuda or x.dim() != 3 or x.stride(2) != 1:
        raise ValueError("rows must be a CUDA [S,H,d] tensor, contiguous along d")
    S, H, d = x.shape
    if d % 8 or tuple(camera.cam_index.shape) != (H, d // 8):
        raise ValueError("camera index must be [heads, head_dim/8]")
    out = torch.empty(S, H, d, dtype=x.dtype, device=device)
    struct = camera.struct()
    _lib.check(_lib.library().nkv_camera_rows(_ptr(x), dtype_code(x.dtype), x.stride(0), x.stride(1), S,
                                              H, d, ctypes.byref(struct), _ptr(out), _stream(device)))
    return out


class RopeView:
    """struct nkv_rope over device tensors: positions i32 [tokens], cos_sin f32 [rows, D/2, 2]."""

    def __init__(self, positions: torch.Tensor, cos_sin: torch.Tensor, frame_seqlen: int, width: int,
                 pair_index: torch.Tensor | None = None):
        _require_cuda(positions, cos_sin, pair_index)
        if pair_index is not None and pair_index.dtype != torch.int32:
            raise ValueError("pair index must be int32")
        self.pair_index = pair_index
        if positions.dtype != torch.int32 or cos_sin.dtype != torch.float32:
            raise ValueError("positions must be int32 and the rotation table float32")
        if cos_sin.dim() != 3 or cos_sin.shape[2] != 2:
            raise ValueError("rotation table must be [rows, head_dim/2, 2]")
        if frame_seqlen != 0 and (frame_seqlen < 0 or width <= 0 or frame_seqlen % width):
            raise ValueError(f"frame_seqlen mismatch: width {width} does not divide {frame_seqlen}")
        self.positions, self.cos_sin = positions, cos_sin
        self.frame_seqlen, self.width = int(frame_seqlen), int(width)

    def struct(self) -> "_lib.Rope":
        return _lib.Rope(self.positions.data_ptr(), self.cos_sin.data_ptr(), int(self.cos_sin.shape[0]),
                         self.frame_seqlen, self.width, int(self.cos_sin.shape[1]),
                         None if self.pair_index is None else self.pair_index.data_ptr())


def rope_rows(x: torch.Tensor, rope: RopeView) -> torch.Tensor:
    """Rotate explicit rows x [S,H,d] by rope.positions (nkv_rope_rows) -> contiguous [S,H,d]."""
    device = _require_cuda(rope.positions)
    if not x.is_cuda or x.dim() != 3 or x.stride(2) != 1:
        raise ValueError("rows must be a CUDA [S,H,d] tensor, contiguous along d")
    S, H, d = x.shape
    if rope.positions.numel() != S:
        raise ValueError("RoPE position/row length mismatch")
    if rope.pair_index is None and rope.cos_sin.shape[1] != d // 2:
        raise ValueError("rotation table width does not match the head width")
    if rope.pair_index is not None and tuple(rope.pair_index.shape) != (H, d // 2):
        raise ValueError("pair index must be [heads, head_dim/2]")
    out = torch.empty(S, H, d, dtype=x.dtype, device=device)
    struct = rope.struct()
    _lib.check(_lib.library().nkv_rope_rows(_ptr(x), dtype_code(x.dtype), x.stride(0), x.stride(1), S, H,
                                            d, ctypes.byref(struct), _ptr(out), _stream(device)))
    return out


_PLAIN_CACHE: dict = {}


def _plain_history(k: torch.Tensor) -> HistoryView:
    """Full-width rows [N,H,D] dressed as a compressed history the fused kernel rebuilds exactly:
    rank-64 codes that all mean zero with zero scales (latent = 0), and the rows themselves as the
    centre table with ids 0, 1, 2 ... (segments of 32,768 tokens keep the ids in 16 bits), so that
    bf16(bf16(0 + 0) + centre) is the row."""
    N, H, D = k.shape
    key = (k.device, N)
    if key not in _PLAIN_CACHE:
        span = 32768
        segments = max(1, -(-N // span))
        index = torch.arange(N, device=k.device)
        for stale in [name for name in _PLAIN_CACHE if isinstance(name[0], torch.device)][:-7]:
            del _PLAIN_CACHE[stale]   # keep a handful of history lengths
        _PLAIN_CACHE[key] = dict(
            codes=torch.full((max(N, 1), 32), 0x77, dtype=torch.uint8, device=k.device),
            scales=torch.zeros(max(N, 1), 1, dtype=torch.bfloat16, device=k.device),
            ids=(index % span).to(torch.int16),
            seg_start=torch.tensor([min(s * span, N) for s in range(segments + 1)], dtype=torch.int32,
                                   device=k.device),
            seg_center_row=torch.arange(segments, dtype=torch.int32, device=k.device) * span,
            segments=segments)
    c = _PLAIN_CACHE[key]
    return HistoryView(codes=c["codes"], scales=c["scales"], ids=c["ids"], centers=k.view(N, H * D),
                       seg_start=c["seg_start"], seg_center_row=c["seg_center_row"], tokens=N,
                       segments=c["segments"], rank=64, group=64)


def attention_lse(q, k, v, *, scale: float):
    """Plain attention: q [Q,H,d], k [N,H,d], v [N,H,dv] -> (O [Q,H,dv], lse [Q,H]).

    bf16 rows of width 64 or 128 run on the tcgen05 kernel of the fused read (the rows enter as
    its centre table, see ``_plain_history``); everything else on the fp32 CUDA-core kernel."""
    device = _require_cuda(q, k, v)
    Q, H, d = q.shape
    N, dv = k.shape[0], v.shape[2]
    if (q.dtype == torch.bfloat16 and k.dtype == v.dtype == torch.bfloat16 and d == dv
            and d in (64, 128) and N > 0 and k.is_contiguous() and v.is_contiguous()
            and q.stride(2) == 1 and q.stride(0) % 8 == 0 and q.stride(1) % 8 == 0):
        zero_w = _PLAIN_CACHE.setdefault(("w", device, H, d),
                                         torch.zeros(H, d, 64, dtype=torch.bfloat16, device=device))
        zero_b = _PLAIN_CACHE.setdefault(("b", device, H, d),
                                         torch.zeros(H, d, dtype=torch.float32, device=device))
        view_k = _plain_history(k)
        view_v = _plain_history(v)
        # all-zero weights are their own kernel-order copy
        return attn_codec(q, view_k, view_v, zero_w, zero_b, zero_w, zero_b, scale=scale,
                          prepared=tensor_core_read(q.dtype, d, dv, 64))
    out = torch.empty(Q, H, dv, dtype=q.dtype, device=device)
    lse = torch.empty(Q, H, dtype=torch.float32, device=device)
    if k.stride() != v.stride() and d == dv:
        raise ValueError("k and v must share a layout")
    _lib.check(_lib.library().nkv_attention_lse(
        _ptr(q), _ptr(k), _ptr(v), dtype_code(q.dtype), q.stride(0), q.stride(1), k.stride(0),
        k.stride(1), Q, N, H, d, dv, float(scale), _ptr(out), _ptr(lse), _stream(device)))
    return out, lse


def history_moments(view: HistoryView):
    """(latent_sum f32 [rank], center_counts i32 [centre rows]) of a history (nkv_history_moments)."""
    device = _require_cuda(view.codes)
    lib = _lib.library()
    latent_sum = torch.empty(view.rank, dtype=torch.float32, device=device)
    counts = torch.empty(view.centers.shape[0], dtype=torch.int32, device=device)
    nbytes = lib.nkv_history_moments_workspace_bytes(view.tokens, view.rank)
    workspace = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
    struct = view.struct()
    _lib.check(lib.nkv_history_moments(ctypes.byref(struct), _ptr(latent_sum), _ptr(counts),
                                       _ptr(workspace), nbytes, _stream(device)))
    return latent_sum, counts


def unpack_int8_weight(qweight: torch.Tensor, scale: torch.Tensor, group_size: int | None = None):
    """INT8 operator storage -> bf16 weight: bf16(q) * scale per (row, group), one bf16 product.
    qweight i8 [rows, cols]; scale bf16 [rows, cols / group] (or [rows, 1] / [rows] per row)."""
    device = _require_cuda(qweight, scale)
    if qweight.dtype != torch.int8 or qweight.dim() != 2:
        raise ValueError("qweight must be an int8 matrix")
    rows, cols = qweight.shape
    group = cols if group_size in (None, 0) else int(group_size)
    if group <= 0 or cols % group:
        raise ValueError(f"INT8 group size {group} must divide {cols}")
    scale = scale.to(torch.bfloat16).reshape(rows, -1).contiguous()
    if scale.shape[1] != cols // group:
        raise ValueError("scale shape does not match the group size")
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
    _lib.check(_lib.library().nkv_operator_unpack_int8(
        _ptr(qweight), _ptr(scale), rows, cols, group, _ptr(out), _stream(device)))
    return out


def fast_finish(native: torch.Tensor, native_lse: torch.Tensor, lifted: torch.Tensor,
                low_lse: torch.Tensor, heads: torch.Tensor, out: torch.Tensor, *,
                value_mean: torch.Tensor | None = None, projected_mean: torch.Tensor | None = None,
                out_lse: torch.Tensor | None = None) -> torch.Tensor:
    """Finish of the mixed-dimensional read for one head group in one launch: value-mean
    correction, log-sum-exp merge of the full-width with the lifted low-width partial, scatter to
    the group's heads (finish, LingBot fast tree wan/modules/codec_native_finish_triton.py:37-46).

    native, out [Q, H, D]; lifted [Q, Hg, D]; native_lse [Q, H]; low_lse [Q, Hg] f32; heads i32 [Hg];
    value_mean f32 [H, D] with projected_mean f32 [Hg, D], or neither."""
    device = _require_cuda(native, native_lse, lifted, low_lse, heads, out)
    Q, H, D = native.shape
    G = heads.numel()
    if lifted.shape != (Q, G, D) or out.shape != native.shape or lifted.dtype != native.dtype \
            or out.dtype != native.dtype:
        raise ValueError("fast_finish: native/out [Q,H,D] and lifted [Q,Hg,D] of one dtype")
    if native_lse.shape != (Q, H) or low_lse.shape != (Q, G):
        raise ValueError("fast_finish: lse shapes do not match")
    if (value_mean is None) != (projected_mean is None):
        raise ValueError("fast_finish: the value mean and its projected part come together")
    for t in (native, lifted, out, native_lse, low_lse):
        if not t.is_contiguous():
            raise ValueError("fast_finish: contiguous tensors are required")
    if native_lse.dtype != torch.float32 or low_lse.dtype != torch.float32:
        raise ValueError("fast_finish: lse tensors are float32")
    heads = heads.to(torch.int32).contiguous()
    if value_mean is not None:
        if value_mean.shape != (H, D) or projected_mean.shape != (G, D):
            raise ValueError("fast_finish: value_mean [H,D], projected_mean [Hg,D]")
        value_mean = value_mean.float().contiguous()
        projected_mean = projected_mean.float().contiguous()
    if out_lse is not None and (out_lse.shape != (Q, H) or out_lse.dtype != torch.float32
                                or not out_lse.is_contiguous()):
        raise ValueError("fast_finish: out_lse is a contiguous float32 [Q,H]")
    _lib.check(_lib.library().nkv_fast_finish(
        _ptr(native), _ptr(native_lse), _ptr(lifted), _ptr(low_lse), _ptr(heads), _ptr(value_mean),
        _ptr(projected_mean), Q, H, G, D, dtype_code(native.dtype), _ptr(out), _ptr(out_lse),
        _stream(device)))
    return out


class PeerBuffer:
    """A device buffer other processes of the box can map (nkv_peer_alloc / nkv_peer_open).

    ``handle`` (64 bytes) is what a peer passes to :meth:`open`; tensors over the memory come from
    :meth:`tensor`.  The owner frees on :meth:`release`, a peer unmaps."""

    def __init__(self, pointer: int, nbytes: int, device: torch.device, handle: bytes | None):
        self.pointer, self.nbytes, self.device, self.handle = pointer, nbytes, device, handle

    @classmethod
    def allocate(cls, nbytes: int, device) -> "PeerBuffer":
        device = torch.device(device)
        handle = ctypes.create_string_buffer(64)
        pointer = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(_lib.library().nkv_peer_alloc(int(nbytes), ctypes.byref(pointer), handle))
        return cls(int(pointer.value), int(nbytes), device, handle.raw)

    @classmethod
    def open(cls, handle: bytes, nbytes: int, device) -> "PeerBuffer":
        device = torch.device(device)
        if len(handle) != 64:
            raise ValueError("a peer handle is 64 bytes")
        pointer = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(_lib.library().nkv_peer_open(handle, ctypes.byref(pointer)))
        return cls(int(pointer.value), int(nbytes), device, None)

    def tensor(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """Zero-copy tensor over [offset, offset + numel * itemsize) of the buffer."""
        count = 1
        for extent in shape:
            count *= int(extent)
        itemsize = torch.empty((), dtype=dtype).element_size()
        if offset < 0 or offset + count * itemsize > self.nbytes:
            raise ValueError("tensor window outside the peer buffer")
        window = _CudaWindow(self.pointer + offset, count * itemsize, self)
        flat = torch.as_tensor(window, device=self.device)
        return flat.view(dtype).view(*shape)

    def release(self) -> None:
        if self.pointer:
            lib = _lib.library()
            with torch.cuda.device(self.device):
                _lib.check(lib.nkv_peer_free(self.pointer) if self.handle is not None
                           else lib.nkv_peer_close(self.pointer))
            self.pointer = 0


class _CudaWindow:
    """__cuda_array_interface__ view (uint8) of a raw device range; keeps its owner alive."""

    def __init__(self, pointer: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (pointer, False), "version": 3, "strides": None}


def cp_merge_peer(part_out_ptrs, part_lse_ptrs, dst_out_ptrs, dst_lse_ptrs, *, rows: int, width: int,
                  row_begin: int, row_end: int, dtype: torch.dtype, device) -> None:
    """Merge rows [row_begin, row_end) of every rank's partial and store them into every rank's
    result buffer (nkv_cp_merge_peer).  The pointer lists are per rank, peers' as mapped here."""
    world = len(part_out_ptrs)
    arrays = [(ctypes.c_void_p * world)(*[int(v) for v in values])
              for values in (part_out_ptrs, part_lse_ptrs, dst_out_ptrs, dst_lse_ptrs)]
    device = torch.device(device)
    _lib.check(_lib.library().nkv_cp_merge_peer(
        arrays[0], arrays[1], arrays[2], arrays[3], world, int(rows), int(width), int(row_begin),
        int(row_end), dtype_code(dtype), _stream(device)))


def head_linear(x: torch.Tensor, w: torch.Tensor, *, heads: torch.Tensor | None = None,
                din: int | None = None, pad_to: int | None = None) -> torch.Tensor:
    """out[n, g, :] = x[n, head(g), :din] @ w[g]  (nkv_head_linear): the query reduction and the value
    lift of a reader group.  x [S, H, >= din] (last dimension contiguous), w [h, din, dout] in x's dtype,
    ``heads`` i32 [h] picks the heads of x (default: head g), ``pad_to`` zero-pads the output columns."""
    device = _require_cuda(w)
    if not x.is_cuda or x.device != device:
        raise RuntimeError("nanokv_b200 runs on CUDA tensors only (there is no CPU path)")
    if x.stride(2) != 1 or x.dtype != w.dtype:
        raise ValueError("head_linear takes rows contiguous along the last dimension, in the weights' dtype")
    h, w_in, dout = w.shape
    din = w_in if din is None else int(din)
    if din != w_in or x.shape[2] < din:
        raise ValueError("head_linear: input width does not match the weights")
    pad = dout if pad_to is None else int(pad_to)
    out = torch.empty(x.shape[0], h, pad, dtype=x.dtype, device=device)
    index = None if heads is None else heads.to(device=device, dtype=torch.int32).contiguous()
    _lib.check(_lib.library().nkv_head_linear(
        _ptr(x), dtype_code(x.dtype), x.stride(0), x.stride(1), _ptr(index), _ptr(w.contiguous()),
        x.shape[0], h, din, dout, pad, _ptr(out), _stream(device)))
    return out


PEER_FLAG_WORDS = 64


def cp_exchange_peer(part_out_ptrs, part_lse_ptrs, dst_out_ptrs, dst_lse_ptrs, flag_ptrs, *, rank: int,
                     rows: int, width: int, row_begin: int, row_end: int, dtype: torch.dtype, epoch: int,
                     device, status: torch.Tensor | None = None, budget_cycles: int = 0) -> None:
    """cp_merge_peer with the ranks ordered by flag words in peer memory instead of collectives
    (nkv_cp_exchange_peer): one launch per rank and layer."""
    world = len(part_out_ptrs)
    arrays = [(ctypes.c_void_p * world)(*[int(v) for v in values])
              for values in (part_out_ptrs, part_lse_ptrs, dst_out_ptrs, dst_lse_ptrs, flag_ptrs)]
    device = torch.device(device)
    if status is None:
        status = status_word(device)
    _lib.check(_lib.library().nkv_cp_exchange_peer(
        arrays[0], arrays[1], arrays[2], arrays[3], arrays[4], world, int(rank), int(rows), int(width),
        int(row_begin), int(row_end), dtype_code(dtype), int(epoch), int(budget_cycles), _ptr(status),
        _stream(device)))


def lse_merge(partials):
    """[(O [rows..., d], lse [rows...])] -> merged (O, lse); an empty partition is (0, -inf)."""
    outs = [o for o, _ in partials]
    lses = [l for _, l in partials]
    device = _require_cuda(*outs, *lses)
    first = outs[0]
    d = first.shape[-1]
    rows = first.numel() // d
    out = torch.empty_like(first)
    lse = torch.empty_like(lses[0])
    n = len(partials)
    out_ptrs = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
    lse_ptrs = (ctypes.c_void_p * n)(*[l.data_ptr() for l in lses])
    _lib.check(_lib.library().nkv_lse_merge(
        out_ptrs, lse_ptrs, n, rows, d, dtype_code(first.dtype), _ptr(out), _ptr(lse),
        _stream(device)))
    return out, lse


def force_simt(on: bool) -> None:
    """Triage hook: run bf16 work on the fp32 CUDA-core kernels (same rounding points)."""
    _SIMT_FORCED[0] = bool(on)
    _lib.check(_lib.library().nkv_set_bf16_path(1 if on else 0))
