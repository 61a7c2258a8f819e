"""The C-ABI library: loads, exports every declared symbol, and refuses to compute without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(qgemv_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(qg):
    lib = ctypes.CDLL(qg.lib_path())
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"


def test_status_strings(qg):
    assert qg.status_string(0) == "ok"
    for code in range(-8, 0):
        assert qg.status_string(code) != "unknown status"
    assert qg.status_string(-99) == "unknown status"


def test_no_cpu_fallback(qg):
    """Without a CUDA device the library reports it; it never computes on the host."""
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(qg.QgemvError) as e:
        qg.QGemv(device=0)
    assert e.value.status == qg.ERR_NO_DEVICE


def test_package_does_not_import_oracle():
    """The shipped package must not reach into the oracle."""
    pkg = os.path.join(ROOT, "crit_hub_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "oracle" not in text.lower(), f"{fn} mentions the oracle"


def test_header_is_plain_c_and_links(qg, tmp_path):
    """include/qgemv.h compiles as C99 (no C++ or torch types at the boundary) and a C program that
    references the declared entry points links against the library and runs its host-only calls."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi.c"
    src.write_text(
        '#include <stdio.h>\n#include "qgemv.h"\n'
        "int main(void) {\n"
        "  qgemv_skinny_plan p;\n"
        "  qgemv_shard s = {0, 128, 0, 256};\n"
        "  if (qgemv_gemm_skinny_plan(QGEMV_FMT_NVFP4, 8192, 8192, 256, 148, &p) != QGEMV_OK) return 2;\n"
        "  if (p.ctas != 128 || p.tmem_columns != 512) return 3;\n"
        "  if (qgemv_packed_size(QGEMV_FMT_NVFP4, 256, 256, &s) == 0) return 4;\n"
        '  printf("%s\\n", qgemv_status_string(QGEMV_ERR_TIMEOUT));\n'
        "  /* the device entry points only need to link */\n"
        "  void* f[] = {(void*)qgemv_init, (void*)qgemv_load, (void*)qgemv_gemv, (void*)qgemv_gemm_skinny,\n"
        "               (void*)qgemv_moe_gemv, (void*)qgemv_tp_allreduce, (void*)qgemv_gemv_noalloc};\n"
        "  return f[0] == 0;\n}\n")
    exe = tmp_path / "abi"
    lib = qg.lib_path()
    cmd = [gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-Wno-pedantic", "-I", os.path.join(ROOT, "include"), str(src),
           "-o", str(exe), lib, "-Wl,-rpath," + os.path.dirname(lib)]
    out = subprocess.run(cmd, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stderr)
    assert run.stdout.strip()
