"""The C-ABI shared library loads on a machine without a GPU and exports every
symbol that include/cortex_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

from cortex_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "cortex_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = _declared()
    assert len(names) >= 40
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_the_header():
    assert set(_declared()) == set(_lib.SIGNATURES)


def test_error_reporting_without_a_device():
    lib = _lib.load()
    rc = lib.cb200_unsupported(b"gemv!")
    assert rc == 2 and "gemv!" in _lib.last_error()
    # argument validation happens before any CUDA call
    rc = lib.cb200_gemm(None, 4, None, 0, 0, 0, 1.0, None, 0, 0, 0, None, 0, 0, 0.0)
    assert rc == 1 and "null" in _lib.last_error()
