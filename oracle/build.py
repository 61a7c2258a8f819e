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


OUT_NATIVE = os.path.join(OUT_DIR, "libqgemv_oracle_native.so")


def build_native(force: bool = False) -> str | None:
    """The same source for the machine it is compiled on (-O3 -march=native): used only for the TIMED
    fp32 CPU baseline, and only on the machine that built it (the instruction set does not travel).
    A marker file records the CPU it was built for.  Returns None when the compile fails."""
    os.makedirs(OUT_DIR, exist_ok=True)
    marker = OUT_NATIVE + ".cpu"
    cpu = ""
    try:
        with open("/proc/cpuinfo") as f:
            cpu = next((ln.split(":", 1)[1].strip() for ln in f if ln.startswith("model name")), "")
    except OSError:
        pass
    fresh = (os.path.exists(OUT_NATIVE) and os.path.exists(marker)
             and os.path.getmtime(OUT_NATIVE) >= os.path.getmtime(SRC) and open(marker).read() == cpu)
    if fresh and not force:
        return OUT_NATIVE
    cmd = ["g++", "-std=c++17", "-O3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-march=native",
           "-shared", "-fPIC", SRC, "-o", OUT_NATIVE]
    try:
        subprocess.run(cmd, check=True, capture_output=True)
    except (subprocess.CalledProcessError, OSError):
        return None
    with open(marker, "w") as f:
        f.write(cpu)
    return OUT_NATIVE


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
