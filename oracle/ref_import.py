"""Load the unmodified reference modules for golden-vector generation.

TEST INFRASTRUCTURE ONLY, and usable only where a checkout of the reference
project is present (pass its root, or set NANOKV_REFERENCE_ROOT).  The GPU
tests, the smoke entry and the benchmark never import this file: they use the
fixtures under ``tests/golden/`` that ``tests/golden/make_golden.py`` produced
with it.

The reference's package ``__init__`` files import whole model zoos, so the few
module files on the codec path are loaded by file path under empty stand-in
parent packages.  Nothing in the reference tree is modified or copied.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import torch

MG = "models/Matrix-Game-3.5/fast"
LB = "models/LingBot-World-2.0/fast"
HY = "models/HY-WorldPlay/fast"


def reference_root(root: str | os.PathLike | None = None) -> Path:
    root = root or os.environ.get("NANOKV_REFERENCE_ROOT")
    if not root:
        raise FileNotFoundError("pass the reference checkout's root or set NANOKV_REFERENCE_ROOT")
    root = Path(root)
    if not (root / MG / "diffsynth/models/nanokv_codec.py").exists():
        raise FileNotFoundError(f"no reference checkout at {root}")
    return root


def _stub_package(name: str, path: Path) -> None:
    if name not in sys.modules:
        module = types.ModuleType(name)
        module.__path__ = [str(path)]
        sys.modules[name] = module


def _load(name: str, path: Path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def load_mg_codec(root=None):
    """Matrix-Game codec module (diffsynth/models/nanokv_codec.py)."""
    root = reference_root(root)
    base = root / MG / "diffsynth"
    _stub_package("diffsynth", base)
    _stub_package("diffsynth.models", base / "models")
    os.environ["MG35_KVCODEC_MODE"] = "worldplay_method"
    return _load("diffsynth.models.nanokv_codec", base / "models/nanokv_codec.py")


def load_mg_core(root=None):
    """Model-independent attention_lse / merge / hybrid_attention (codec_native/core.py)."""
    root = reference_root(root)
    base = root / MG / "codec_native"
    _stub_package("codec_native", base)
    return _load("codec_native.core", base / "core.py")


def load_lingbot_codec(root=None):
    """LingBot codec module (wan/modules/lingbot_v2_kv_codec.py)."""
    root = reference_root(root)
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))  # for nanokv.artifacts
    base = root / LB / "wan"
    _stub_package("wan", base)
    _stub_package("wan.modules", base / "modules")
    return _load("wan.modules.lingbot_v2_kv_codec", base / "modules/lingbot_v2_kv_codec.py")


def inject_mg_operator(codec, kind: str, layer: int, *, mean, encoder, decoder) -> None:
    """Put synthetic operator weights where ``_operator`` looks them up
    (diffsynth/models/nanokv_codec.py:156-160).  dtype selects the storage."""
    def pack(weight):
        storage = {"torch.float32": "fp32", "torch.bfloat16": "bf16"}[str(weight.dtype)]
        return {"storage": storage, "weight": weight}
    codec._OPERATORS[(codec._rung(), kind, int(layer), "cpu")] = {
        "mean": mean.float(), "encoder": pack(encoder), "decoder": pack(decoder)}


def inject_lingbot_operator(codec, root_tag: str, target: str, layer: int, *, joint_dim: int,
                            rank: int, mean, encoder, decoder, prepacked: str = "") -> None:
    """Same for LingBot's ``_load_operator`` cache key
    (wan/modules/lingbot_v2_kv_codec.py:120-127)."""
    key = (codec._resolved_path(root_tag), "", codec._resolved_path(prepacked) if prepacked else "",
           target, 0, int(layer), int(joint_dim), int(rank), "cpu")
    codec._OPERATORS[key] = {"mean": mean.float(), "encoder": encoder, "decoder": decoder}


def load_hy_reader(root=None):
    """HY-WorldPlay's direct latent attention module (two-branch dictionary reader) and its codec
    helpers, under empty stand-in parent packages (hyvideo/.../direct_codec_latent_attention.py)."""
    root = reference_root(root)
    base = root / HY / "hyvideo"
    for name, path in (("hyvideo", base), ("hyvideo.models", base / "models"),
                       ("hyvideo.models.transformers", base / "models/transformers"),
                       ("hyvideo.models.transformers.modules", base / "models/transformers/modules"),
                       ("hyvideo.prope", base / "prope")):
        _stub_package(name, path)
    import importlib
    return importlib.import_module("hyvideo.models.transformers.modules.direct_codec_latent_attention")


def load_hy_codec(root=None):
    """HY-WorldPlay's codec module (hyvideo/models/transformers/modules/kv_codecs.py), imported under
    the same stand-in parent packages as the reader."""
    load_hy_reader(root)
    import importlib
    return importlib.import_module("hyvideo.models.transformers.modules.kv_codecs")


def inject_hy_operator(codec, tensor_name: str, layer: int, *, mean, encoder, decoder, storage: str) -> None:
    """Stand in for the artefact files of one (tensor, layer): global_pca_compress_v and
    decompress_kv_tensor obtain their operator from _global_device_operator_weights
    (kv_codecs.py:834-912), the available rank from _load_global_basis (:428-458) and the encoder-delta
    flag from _load_global_linear_delta (:542-582); the three are replaced by functions that return the
    given matrices, packed by the module's own _pack_operator_weight (:647-679)."""
    table = codec.__dict__.setdefault("_INJECTED_OPERATORS", {})
    table[(tensor_name, int(layer))] = {
        "mean": mean.float(),
        "encoder": codec._pack_operator_weight(encoder, storage, "cpu"),
        "decoder": codec._pack_operator_weight(decoder, storage, "cpu"),
        "mode": storage,
        "rank": int(encoder.shape[0]),
    }
    codec._global_device_operator_weights = (
        lambda root_, linear_root, layer_idx, name, rank, device: table[(name, int(layer_idx))])
    codec._load_global_basis = (
        lambda root_, layer_idx, name="v": {"components": torch.zeros(table[(name, int(layer_idx))]["rank"], 1),
                                              "mean": table[(name, int(layer_idx))]["mean"]})
    codec._load_global_linear_delta = lambda *args, **kwargs: {"model": {}}

