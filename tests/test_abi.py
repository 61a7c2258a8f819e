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
