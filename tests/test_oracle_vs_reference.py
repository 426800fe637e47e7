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


def test_nchw44_convs_match_reference(reference):
    """The NCHW44 restatement (layout conversions around the NCHW one) against the
    reference's ConvGeneral generated for NCHW44 / NCHW_NCHW44, at odd sizes."""
    O = reference
    r = cases.rng_for("random_nchw44")
    for form, k, stride, pad, act, with_bias in [
            ("dense", 1, 1, 0, "RELU", True), ("dense", 3, 1, 1, "RELU", True),
            ("dense", 3, 2, 1, "IDENTITY", True), ("dense", 3, 1, 1, "H_SWISH", False),
            ("channel_wise", 3, 1, 1, "RELU", True), ("channel_wise", 3, 2, 1, "IDENTITY", True),
            ("channel_wise", 5, 1, 2, "H_SWISH", True), ("first_layer", 3, 2, 1, "RELU", True),
            ("first_layer", 7, 2, 3, "RELU", True), ("first_layer", 3, 1, 1, "IDENTITY", False)]:
        for _ in range(3):
            oc = 4 * int(r.integers(1, 6))
            ic = (int(r.integers(1, 5)) if form == "first_layer"
                  else oc if form == "channel_wise" else 4 * int(r.integers(1, 6)))
            n, h, w = int(r.integers(1, 3)), int(r.integers(k, 20)), int(r.integers(k, 20))
            src = r.integers(-128, 128, (n, ic, h, w), dtype=np.int8)
            flt = (r.integers(-127, 128, (oc, 1, 1, k, k), dtype=np.int8)
                   if form == "channel_wise"
                   else r.integers(-127, 128, (oc, ic, k, k), dtype=np.int8))
            bias = r.integers(-2000, 2001, (oc,), dtype=np.int32) if with_bias else None
            if form != "first_layer":
                src = O.nchw_to_nchw44(src)
            flt44 = O.filter_to_nchw44(flt, form)
            s = (float(r.uniform(0.01, 0.1)), float(r.uniform(0.005, 0.02)),
                 float(r.uniform(0.05, 3)))
            a = O.conv_bias_qs8_nchw44(src, flt44, bias, stride, pad, *s, form, act)
            b = O.ref_conv_bias_qs8_nchw44(src, flt44, bias, stride, pad, *s, form, act)
            assert (a == b).all(), (form, k, stride, act, oc, ic, h, w)


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


# ---- fp32 path: the restated checker against the reference's own fp32 kernels ----------------
def _close(a, b, rtol=2e-5, atol=2e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    assert (np.abs(a - b) <= atol + rtol * np.abs(b)).all(), float(np.abs(a - b).max())


def test_fp32_conv_matches_reference_im2col_kernel(reference):
    """GI_kernel_conv2d_im2col_* (weight packing through its init function, workspace through
    its workspace function) against the double-accumulating restatement: the two differ by
    fp32 summation noise only."""
    O = reference
    r = cases.rng_for("f32_conv_ref")
    for k, stride, pad, act, bias in ((3, 1, 1, "IDENTITY", True), (3, 2, 1, "IDENTITY", True),
                                      (1, 1, 0, "IDENTITY", True), (3, 1, 1, "RELU", True),
                                      (1, 1, 0, "SIGMOID", True), (3, 1, 1, "IDENTITY", False)):
        for n, ic, oc, h, w in ((1, 16, 32, 16, 16), (2, 24, 40, 13, 17), (1, 64, 12, 9, 9)):
            src = r.standard_normal((n, ic, h, w)).astype(np.float32)
            flt = (r.standard_normal((oc, ic, k, k)) / np.sqrt(ic * k * k)).astype(np.float32)
            b = r.standard_normal(oc).astype(np.float32) if bias else None
            _close(O.conv_bias_f32(src, flt, b, stride, pad, act),
                   O.ref_conv_bias_f32(src, flt, b, stride, pad, act))


def test_fp32_matmul_matches_reference_4x12_kernel(reference):
    O = reference
    r = cases.rng_for("f32_matmul_ref")
    for m, n, k in ((64, 64, 64), (37, 50, 129), (5, 12, 300), (128, 1, 64)):
        a = r.standard_normal((m, k)).astype(np.float32)
        b = r.standard_normal((k, n)).astype(np.float32)
        _close(O.matmul_f32(a, b), O.ref_matmul_f32(a, b), 2e-5, 2e-6 * np.sqrt(k))


@pytest.mark.parametrize("mode", ["SILU", "SIGMOID", "RELU", "H_SWISH", "EXP", "ADD", "SUB", "MUL",
                                  "MAX", "FUSE_ADD_RELU"])
def test_fp32_elemwise_matches_reference(reference, mode):
    """SILU resolves to the BareMetal kernel (x / (1 + expf(-x))), the others to the
    GeneralIntrinsic ones, whose exp is a polynomial: agreement to a few ulp."""
    O = reference
    r = cases.rng_for("f32_elem_ref_" + mode)
    a = (3 * r.standard_normal((2, 5, 9, 13))).astype(np.float32)
    b = (3 * r.standard_normal((2, 5, 9, 13))).astype(np.float32)
    binary = mode in ("ADD", "SUB", "MUL", "MAX", "FUSE_ADD_RELU")
    _close(O.elemwise_f32(mode, a, b if binary else None),
           O.ref_elemwise_f32(mode, a, b if binary else None), 1e-5, 1e-6)


def test_fp32_data_movement_and_pooling_match_reference_exactly(reference):
    O = reference
    r = cases.rng_for("f32_move_ref")
    xs = [r.standard_normal((2, c, 7, 9)).astype(np.float32) for c in (8, 3, 16)]
    assert (O.concat_f32(xs) == O.ref_concat_f32(xs)).all()
    x = r.standard_normal((2, 6, 10, 13)).astype(np.float32)
    for oh, ow in ((20, 26), (17, 31), (5, 7)):
        assert (O.resize_nearest_f32(x, oh, ow) == O.ref_resize_nearest_f32(x, oh, ow)).all()
    x = r.standard_normal((2, 8, 20, 20)).astype(np.float32)
    for window in (5, 9, 13):
        assert (O.pooling_f32(x, "MAX", window, 1, window // 2)
                == O.ref_pooling_f32(x, "MAX", window, 1, window // 2)).all()
    for mode in ("AVERAGE", "AVERAGE_COUNT_EXCLUDE_PADDING"):
        _close(O.pooling_f32(x, mode, 3, 2, 1), O.ref_pooling_f32(x, mode, 3, 2, 1), 1e-6, 1e-7)


def test_fp32_qsi8_typecvt_matches_reference_gi_kernel(reference):
    """fp32 <-> qsi8 resolve to the GeneralIntrinsic TypeCvt on x86, not the BareMetal one:
    values next to ties, in the SIMD groups and in the trailing elements alike."""
    O = reference
    r = cases.rng_for("typecvt_gi")
    for n in (16, 37, 1000, 5, 4099):
        x = (r.standard_normal(n) * 60).astype(np.float32)
        ties = (np.arange(-130, 131, dtype=np.float32) + np.float32(0.5)) * np.float32(0.7)
        x[:min(n, ties.size)] = ties[:min(n, ties.size)]
        x[-3:] = np.float32([0.49999997 * 0.7, -0.49999997 * 0.7, 0.35])[:min(3, n)]
        assert (O.typecvt_f32_qs8(x, 0.3, 0.7) == O.ref_typecvt_f32_qs8(x, 0.3, 0.7)).all()
        q = r.integers(-128, 128, n, dtype=np.int8)
        assert (O.typecvt_qs8_f32(q, 0.3, 0.7) == O.ref_typecvt_qs8_f32(q, 0.3, 0.7)).all()
