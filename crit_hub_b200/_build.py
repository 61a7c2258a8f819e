"""In-tree build of libqgemv.so (sm_100a only) with nvcc.

    python -m crit_hub_b200._build [--force] [--verbose]

The shared object is written next to this file so that it travels with the source tree;
nothing is installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libqgemv.so")

SOURCES = ["api.cu", "pack.cpp"]
HEADERS = ["ptx.cuh", "gemv_kernel.cuh", "gemv_stream.cuh", "moe_stream.cuh", "gemm_skinny.cuh", "gemv_tc.cuh", "gemv_seq.cuh", "gemm_tc_a4.cuh", "tp_allreduce.cuh", "aux_kernels.cuh", "qgemv_layout.h"]


def _newest_source_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    paths.append(os.path.join(INCLUDE, "qgemv.h"))
    return max(os.path.getmtime(p) for p in paths if os.path.exists(p))


def nvcc_path() -> str:
    cand = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile libqgemv.so if it is missing or older than its sources; return its path."""
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime():
        return LIB_PATH
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC,-fopenmp", "-diag-suppress", "177",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-o", LIB_PATH, "-lgomp"]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
