"""The CPU restatement against the reference's own kernels (oracle/_ref) run live, on
random shapes beyond the golden set, plus properties of the arithmetic that hold at any
size."""
import numpy as np
import pytest

import cases


def test_random_convs_match_reference(reference):
    O = reference
    r = cases.rng_for("random_convs")
    for i in range(40):
        k = int(r.choice([1, 2, 3, 5, 7]))
        stride = int(r.choice([1, 2, 3]))
        pad = int(r.choice([0, k // 2]))
        act = str(r.choice(["IDENTITY", "RELU", "H_SWISH"]))
        dw = bool(r.integers(0, 2))
        ic = int(r.integers(1, 24))
        oc = ic if dw else int(r.integers(1, 24))
        h, w = int(r.integers(k, 30)), int(r.integers(k, 30))
        n = int(r.integers(1, 4))
        src = r.integers(-128, 128, (n, ic, h, w), dtype=np.int8)
        flt = (r.integers(-127, 128, (ic, 1, 1, k, k), dtype=np.int8) if dw
               else r.integers(-127, 128, (oc, ic, k, k), dtype=np.int8))
        bias = r.integers(-2000, 2001, (oc,), dtype=np.int32)
        s = (float(r.uniform(0.01, 0.1)), float(r.uniform(0.005, 0.02)), float(r.uniform(0.05, 3)))
        g = ic if dw else 1
        a = O.conv_bias_qs8(src, flt, bias, stride, pad, *s, act, g)
        b = O.ref_conv_bias_qs8(src, flt, bias, stride, pad, *s, act, g)
        assert (a == b).all(), (i, k, stride, pad, act, dw)


def test_conv_without_bias_matches_reference(reference):
    O = reference
    r = cases.rng_for("nobias")
    src = r.integers(-128, 128, (2, 8, 9, 11), dtype=np.int8)
    flt = r.integers(-127, 128, (5, 8, 3, 3), dtype=np.int8)
    a = O.conv_bias_qs8(src, flt, None, 1, 1, 0.1, 0.1, 2.0, "RELU")
    b = O.ref_conv_bias_qs8(src, flt, None, 1, 1, 0.1, 0.1, 2.0, "RELU")
    assert (a == b).all()


def test_rounding_ties_and_saturation(oracle):
    """1x1 conv with unit weight: acc = src, x = acc * 0.5 -> ties round away from zero
    (roundf, compiler/lib/KernelGen/BareMetal/Activation.cpp:50-56) and clamp to int8."""
    src = np.arange(-128, 128, dtype=np.int8).reshape(1, 1, 16, 16)
    flt = np.ones((1, 1, 1, 1), np.int8)
    out = oracle.conv_bias_qs8(src, flt, None, 1, 0, 1.0, 1.0, 2.0).reshape(-1)
    x = src.reshape(-1).astype(np.float64) / 2
    want = np.clip(np.sign(x) * np.floor(np.abs(x) + 0.5), -128, 127).astype(np.int8)
    assert (out == want).all()
    sat = oracle.conv_bias_qs8(src, flt, None, 1, 0, 4.0, 1.0, 1.0).reshape(-1)
    assert sat.max() == 127 and sat.min() == -128


def test_accumulator_linearity(oracle):
    """int32 accumulators are linear in the source: acc(a + b) = acc(a) + acc(b) (no bias)."""
    r = cases.rng_for("linearity")
    a = r.integers(-60, 60, (1, 16, 12, 12), dtype=np.int8)
    b = r.integers(-60, 60, (1, 16, 12, 12), dtype=np.int8)
    flt = r.integers(-127, 128, (8, 16, 3, 3), dtype=np.int8)
    acc = lambda s: oracle.conv_bias_qs8(s, flt, None, 1, 1, 1, 1, 1, return_acc=True)[1]
    assert (acc((a + b).astype(np.int8)) == acc(a) + acc(b)).all()


def test_per_channel_scale_extension(oracle):
    """Per-channel filter scales use the per-tensor formula channel by channel."""
    r = cases.rng_for("perchannel")
    src = r.integers(-128, 128, (1, 8, 10, 10), dtype=np.int8)
    flt = r.integers(-127, 128, (6, 8, 3, 3), dtype=np.int8)
    bias = r.integers(-500, 500, (6,), dtype=np.int32)
    sf = r.uniform(0.005, 0.02, 6).astype(np.float32)
    full = oracle.conv_bias_qs8(src, flt, bias, 1, 1, 0.05, sf, 0.2, "RELU")
    for o in range(6):
        one = oracle.conv_bias_qs8(src, flt[o:o + 1], bias[o:o + 1], 1, 1, 0.05, float(sf[o]),
                                   0.2, "RELU")
        assert (full[:, o] == one[:, 0]).all()
