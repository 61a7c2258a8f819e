"""Build the CPU oracle shared library (test infrastructure, never shipped).

    python oracle/build.py        ->  oracle/_build/libqgemv_oracle.so

The reference project holds no implementation of the quantized GEMV path (its
engines' kernels live in a separate, un-vendored repository), so there is no
`oracle/_ref` to compile: the oracle is a restatement of the public formats.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "qgemv_oracle.cpp")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libqgemv_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = [
        "g++", "-std=c++17", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
        "-march=x86-64-v2", "-shared", "-fPIC", SRC, "-o", OUT,
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
