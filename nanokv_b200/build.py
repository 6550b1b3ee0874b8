"""Build libnanokv_b200.so in-tree with nvcc for sm_100a.

    python -m nanokv_b200.build [--force]

The shared library sits next to the sources (``nanokv_b200/_build/``) so that
it travels with a snapshot of the tree; it is never installed elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
BUILD = PACKAGE / "_build"
LIBRARY = BUILD / "libnanokv_b200.so"
SOURCES = ("nkv_api.cu", "nkv_simt.cu", "nkv_elementwise.cu", "nkv_tc_attn.cu", "nkv_tc_encode.cu",
           "nkv_static_scratch.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def flags() -> list[str]:
    """NKV_DEV=1 in the environment adds -DNKV_DEV: tuning knobs read from the environment by the
    fused read's planner (development builds only; the default build has none)."""
    extra = ["-DNKV_DEV"] if os.environ.get("NKV_DEV", "0") not in ("", "0") else []
    return NVCC_FLAGS + extra


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; it is required to build libnanokv_b200")
    return found


def sources() -> list[Path]:
    return [CSRC / name for name in SOURCES if (CSRC / name).exists()]


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    stamp = BUILD / "flags.txt"
    if not stamp.exists() or stamp.read_text() != " ".join(flags()):
        return True
    built = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(PACKAGE.parent / "include" / "nanokv_b200.h")
    return any(dep.stat().st_mtime > built for dep in deps)


def compile_one(source: Path) -> Path:
    obj = BUILD / (source.stem + ".o")
    cmd = [nvcc(), *flags(), "-c", str(source), "-o", str(obj)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    (BUILD / (source.stem + ".ptxas.log")).write_text(result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stderr[-4000:]}")
    return obj


def build(force: bool = False) -> Path:
    if not force and not stale():
        return LIBRARY
    BUILD.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources()))
    cmd = [nvcc(), "-shared", "-o", str(LIBRARY), *map(str, objects), "-lcudart"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode:
        raise RuntimeError(f"link failed:\n{result.stderr[-4000:]}")
    (BUILD / "flags.txt").write_text(" ".join(flags()))
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
