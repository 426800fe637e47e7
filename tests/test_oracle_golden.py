"""The CPU restatement (oracle/megcc_oracle.c) against the committed golden vectors, which
were produced by the reference's own generated x86 kernels (tests/golden/make_golden.py)."""
import numpy as np
import pytest

import cases
import golden_util as G


def _conv(oracle, c):
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    dst = oracle.conv_bias_qs8(src, flt, bias, c["stride"], c["pad"], s0, s1, s2, c["act"],
                               c["groups"])
    G.check("conv_bias_qs8", c["name"], dst, src, flt, bias)


def test_conv_naive_catalogue(oracle):
    for c in cases.conv_naive_catalogue():
        _conv(oracle, c)


def test_conv_im2col_catalogue(oracle):
    for c in cases.conv_im2col_catalogue():
        _conv(oracle, c)


@pytest.mark.parametrize("dst_scale", [0.1, 5.0])
def test_conv_cfg1(oracle, dst_scale):
    _conv(oracle, cases.conv_cfg1(dst_scale))


def test_conv_model_shapes(oracle):
    for c in cases.conv_model_shapes():
        _conv(oracle, c)


def test_conv_nchw44_catalogue(oracle):
    """Dense, channel-wise and first-layer NCHW44 filters against the reference's NCHW44
    kernels' outputs."""
    for c in cases.conv_nchw44_catalogue():
        src, flt44, bias = cases.conv_nchw44_inputs(c, oracle)
        s0, s1, s2 = c["scales"]
        dst = oracle.conv_bias_qs8_nchw44(src, flt44, bias, c["stride"], c["pad"], s0, s1, s2,
                                          c["form"], c["act"])
        G.check("conv_bias_nchw44", c["name"], dst, src, flt44, bias)


def test_pooling(oracle):
    for c in cases.pool_catalogue():
        x = cases.pool_input(c)
        G.check("pooling_qs8", c["name"],
                oracle.pooling_qs8(x, c["mode"], c["window"], c["stride"], c["pad"]), x)


def test_qelemwise(oracle):
    for c in cases.qelem_catalogue():
        a, b = cases.qelem_inputs(c)
        s0, s1, s2 = c["scales"]
        G.check("qelemwise", c["name"], oracle.qelemwise(c["mode"], a, b, s0, s1, s2), a, b)


def test_typecvt(oracle):
    for c in cases.typecvt_catalogue():
        x = cases.typecvt_input(c)
        G.check("typecvt_qs32_qs8", c["name"],
                oracle.typecvt_qs32_qs8(x, c["s_src"], c["s_dst"]), x)


def test_matmul_is_exact_integer_gemm(oracle):
    r = cases.rng_for("matmul")
    for m, n, k in ((4, 3, 4), (16, 15, 16), (64, 56, 64), (33, 17, 129)):
        a = r.integers(-127, 128, (m, k), dtype=np.int8)
        b = r.integers(-127, 128, (k, n), dtype=np.int8)
        want = a.astype(np.int64) @ b.astype(np.int64)
        assert (oracle.matmul_s8_s32(a, b) == want).all()


def test_fp32_conv_and_matmul_against_reference_vectors(oracle):
    """The fp32 restatement against outputs of the reference's GeneralIntrinsic kernels
    (fp32 summation order differs: 2e-5 relative / 2e-6 absolute)."""
    for c in cases.f32_conv_catalogue():
        src, flt, bias = cases.f32_conv_inputs(c)
        out = oracle.conv_bias_f32(src, flt, bias, c["stride"], c["pad"], c["act"])
        G.check_close("f32_ops", c["name"], out, 2e-5, 2e-6, src, flt, bias)
    for c in cases.f32_matmul_catalogue():
        a, b = cases.f32_matmul_inputs(c)
        G.check_close("f32_ops", c["name"], oracle.matmul_f32(a, b), 2e-5,
                      2e-6 * np.sqrt(c["k"]), a, b)
