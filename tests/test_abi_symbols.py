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


def test_verified_requant_constants_agree_with_the_reference_chain():
    """mb200_requant_fast_constants (host only): the one-FMA requantisation it licenses must
    give the reference's int8 on every accumulator; checked here independently, with exact
    rational arithmetic for the fused multiply-add, on all near-tie accumulators (those whose
    scaled value lies within 1e-4 of a half-integer), a dense band around zero, and the
    saturation edges."""
    import ctypes
    from fractions import Fraction
    import numpy as np
    from megcc_b200._lib import lib
    f32 = np.float32

    def constants(s_src, s_flt, s_dst, act):
        m, d = ctypes.c_float(), ctypes.c_float()
        ok = lib().mb200_requant_fast_constants(s_src, s_flt, s_dst, act, ctypes.byref(m),
                                                ctypes.byref(d))
        return ok, m.value, d.value

    found = 0
    rng = np.random.default_rng(7)
    triples = [(0.05, 0.01, 2.0, 1), (0.05, 0.01, 5.0, 1), (0.0473, 0.00731, 0.1931, 1),
               (0.02, 0.01, 0.5, 0), (0.05, 0.01, 0.77, 0), (0.3, 0.2, 0.01, 1)]
    triples += [(float(rng.uniform(0.01, 0.1)), float(rng.uniform(0.002, 0.02)),
                 float(rng.uniform(0.05, 3.0)), int(rng.integers(0, 2))) for _ in range(12)]
    for s_src, s_flt, s_dst, act in triples:
        ops, c, d = constants(s_src, s_flt, s_dst, act)
        if not ops:
            assert c == 0.0 and d == 0.0
            continue
        assert ops in (1, 2, 3)
        found += 1
        assert 0.0 < d < 1.0
        ratio = float(f32(s_src)) * float(f32(s_flt)) / float(f32(s_dst))
        r = int(130 / ratio) + 4
        acc = np.arange(-r, r + 1, dtype=np.int64)
        frac = np.abs((acc * ratio) % 1.0 - 0.5)
        pick = np.unique(np.concatenate([acc[frac < 1e-4], np.arange(-3000, 3001),
                                         acc[:50], acc[-50:], np.array([-2**31, 2**31 - 1])]))
        a = pick.astype(np.float32)
        t = (a * f32(s_src)).astype(np.float32) * f32(s_flt)
        x = (t.astype(np.float32) / f32(s_dst)).astype(np.float32)
        if act == 1:
            x = np.maximum(x, f32(0))
        want = np.clip(np.sign(x) * np.floor(np.abs(x.astype(np.float64)) + 0.5), -128, 127)
        off = Fraction(float(f32(d)))
        got = []
        lead = a
        if ops >= 2:
            lead = (lead * f32(s_src)).astype(np.float32)
        if ops >= 3:
            lead = (lead * f32(s_flt)).astype(np.float32)
        for v in lead:
            h = off if (act == 1 or not np.signbit(v)) else -off
            # exact sum, then one rounding to float32 (float64 in between is harmless: the
            # exact value has at most 48 + 24 significant bits and is nowhere near a float64 tie
            # that is also a float32 tie)
            y = f32(float(Fraction(float(v)) * Fraction(float(f32(c))) + h))
            q = int(np.clip(np.trunc(y), -128, 127))
            got.append(max(q, 0) if act == 1 else q)
        assert (np.array(got) == want).all(), (s_src, s_flt, s_dst, act)
    assert found >= 6
    # no licence without positive scales, nor for H_SWISH
    assert constants(0.05, -0.01, 2.0, 1)[0] == 0
    assert constants(0.05, 0.01, 2.0, 2)[0] == 0
