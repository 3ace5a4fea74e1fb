"""Builds ``libwalk_b200.so`` (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m mlx_cluster_b200.build``. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libwalk_b200.so"
SOURCES = [CSRC / "walk_b200.cu", CSRC / "csr_build.cu", CSRC / "host_widen.cpp"]
HEADERS = [CSRC / "walk_kernels.cuh", CSRC / "philox.cuh", CSRC / "host_widen.h", CSRC / "n2v_pool.cuh", CSRC / "n2v_pool_tri.cuh", CSRC / "host_common.h", PKG.parent / "include" / "walk_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-pthread", "-shared",
    "--fmad=false",  # the uniform walk's float32 product must not be contracted
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set $NVCC")
    return cand


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [*SOURCES, *HEADERS])


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
           "-o", str(LIB), *map(str, SOURCES)]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
