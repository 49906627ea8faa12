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
# The same library with every pipeline wait limited to a few hundred cycles, so that the first wait for
# a copy from global memory runs out by itself: what tests/test_abort.py loads to see the kernels'
# give-up path (status word, NaN outputs, clean teardown) run on a device without hanging anything.
LIB_SHORT_WAIT = PKG / "libkfa_shortwait.so"
SHORT_WAIT_FLAGS = ["-DKFA_WAIT_CYCLES=300ll"]
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


def stale(lib: Path = LIB) -> bool:
    if not lib.exists():
        return True
    built = lib.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def _compile(lib: Path, extra, log: str, verbose: bool) -> None:
    cmd = [nvcc_path(), *NVCC_FLAGS, *extra, "-o", str(lib), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (PKG / log).write_text(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)


def build(force: bool = False, verbose: bool = False, short_wait: bool = True) -> Path:
    """Compile the library (and, with ``short_wait``, its short-wait test twin) if missing or older than
    the sources; returns the library's path."""
    jobs = [(LIB, [], "build.log")] + ([(LIB_SHORT_WAIT, SHORT_WAIT_FLAGS, "build_shortwait.log")] if short_wait else [])
    for lib, extra, log in jobs:
        if force or stale(lib):
            _compile(lib, extra, log, verbose and lib is LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
