"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/*.h declares (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header, macro):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(macro + r"\s+[\w\s\*]+?\b(\w+)\s*\(", text)))


def test_ops_library_exports_header_symbols():
    from megcc_b200 import _lib
    names = declared("megcc_b200.h", "MB200_API")
    assert len(names) >= 14
    L = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/megcc_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "python signatures out of sync with the header"
    assert b"sm_100a" in _lib.lib().mb200_version()


def test_lite_and_compiler_libraries_export_header_symbols():
    from megcc_b200 import _lib, compiler, lite
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = declared("megcc_b200_lite.h", "LITE_API")
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/megcc_b200_lite.h but not exported"
    assert sorted(lite.SIGNATURES) == names
    Lc = ctypes.CDLL(compiler.LIB_PATH)
    cnames = declared("megcc_b200_compiler.h", "MB200C_API")
    for n in cnames:
        assert hasattr(Lc, n), f"{n} declared in include/megcc_b200_compiler.h but not exported"
    assert sorted(compiler.SIGNATURES) == cnames


def test_missing_library_fails_loudly(monkeypatch):
    from megcc_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libmegcc_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
