"""Builds libb200moe.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Run as ``python -m fused_moe_b200.build``; the repository's build hook calls :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libb200moe.so"
SOURCES = ["api.cu", "routing.cu", "sort.cu", "gemm.cu", "gemm_skinny.cu", "quant.cu", "sort_static.cu", "ep.cu", "decode.cu"]
HEADERS = [CSRC / "common.cuh", CSRC / "gemm_common.cuh", CSRC / "half_rows.cuh", PKG_DIR.parent / "include" / "b200moe.h"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + HEADERS
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xptxas", "-v" if verbose else "-warn-spills",
        "-o", str(LIB_PATH),
    ] + [str(CSRC / s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libb200moe.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
