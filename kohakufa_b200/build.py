"""Builds ``libkfa.so`` (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m kohakufa_b200.build            # rebuild if a source is newer than the library
    python -m kohakufa_b200.build --force

No GPU is needed to build (nvcc cross-compiles). The library is never built implicitly at
import time on a machine without nvcc: ``kohakufa_b200._lib`` raises instead.
"""

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libkfa.so"
SOURCES = [CSRC / "kfa_api.cu"]
HEADERS = [
    CSRC / "kfa_ptx.cuh",
    CSRC / "kfa_fwd.cuh",
    CSRC / "kfa_bwd.cuh",
    CSRC / "kfa_bwd_fused.cuh",
    CSRC / "kfa_selftest.cuh",
    CSRC / "kfa_cp.cuh",
    CSRC / "kfa_mask.cuh",
    CSRC / "kfa_scores.cuh",
    PKG.parent / "include" / "kfa.h",
]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: cannot build libkfa.so")
    return found


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, "-o", str(LIB), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (PKG / "build.log").write_text(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
