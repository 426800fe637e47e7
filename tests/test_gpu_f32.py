"""fp32 operators through the C ABI against the CPU checker: 1e-4 relative / 1e-5 absolute
for the contractions (fp32 sums in another order), exact for the data-movement operators."""
import numpy as np
import pytest

import cases
import golden_util as G

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from megcc_b200 import ops as O
    return O


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, rtol=RTOL, atol=ATOL):
    """|got - want| <= atol + rtol * |want| elementwise, and no NaN."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    err = np.abs(got - want) - (atol + rtol * np.abs(want))
    worst = float(err.max())
    assert worst <= 0, f"worst excess {worst:.3e} at {np.unravel_index(err.argmax(), err.shape)}"


def to_nchw(t):
    return t.cpu().numpy().transpose(0, 3, 1, 2)


CONV_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act, algo
    ("umma_3x3_32_64", 2, 32, 64, 40, 40, 3, 1, 1, "SILU", "umma"),
    ("umma_3x3_s2_64_128", 2, 64, 128, 40, 40, 3, 2, 1, "SILU", "umma"),
    ("umma_1x1_128_64", 2, 128, 64, 24, 24, 1, 1, 0, "SILU", "umma"),
    ("umma_1x1_1024_512", 8, 1024, 512, 10, 10, 1, 1, 0, "IDENTITY", "umma"),
    ("umma_stem_16_32", 1, 16, 32, 64, 64, 3, 1, 1, "SILU", "umma"),
    ("umma_3x3_256_256", 4, 256, 256, 20, 20, 3, 1, 1, "RELU", "umma"),
    ("umma_ragged_oc80", 2, 128, 80, 20, 20, 1, 1, 0, "SIGMOID", "umma"),
    ("umma_ragged_m", 3, 32, 48, 27, 29, 3, 1, 1, "H_SWISH", "umma"),
    ("direct_head_oc4", 2, 128, 4, 20, 20, 1, 1, 0, "IDENTITY", "direct"),
    ("direct_head_oc1", 2, 128, 1, 20, 20, 1, 1, 0, "SIGMOID", "direct"),
    ("direct_odd", 2, 12, 20, 17, 19, 3, 2, 1, "SILU", "auto"),
    ("direct_grouped", 2, 24, 36, 15, 15, 3, 1, 1, "RELU", "auto"),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=[c[0] for c in CONV_CASES])
def test_conv_bias_f32_matches_oracle(ops, oracle, case):
    name, n, ic, oc, h, w, k, stride, pad, act, algo = case
    groups = 6 if name == "direct_grouped" else 1
    r = cases.rng_for("f32_" + name)
    src = r.standard_normal((n, ic, h, w)).astype(np.float32)
    flt = (r.standard_normal((oc, ic // groups, k, k)) / np.sqrt(ic // groups * k * k)).astype(np.float32)
    bias = r.standard_normal(oc).astype(np.float32)
    p = ops.conv_f32_param(n, ic, h, w, oc, k, k, stride, pad, groups, act)
    packed = ops.pack_filter_f32(p, dev(flt))
    out = ops.conv_bias_f32_nhwc(p, ops.nchw_to_nhwc_f32(dev(src)), packed, dev(bias), algo=algo)
    want = oracle.conv_bias_f32(src, flt, bias, stride, pad, act, groups)
    close(to_nchw(out), want)
    assert ops.device_status() == 0


def test_conv_and_matmul_f32_against_reference_vectors(ops):
    """Outputs of the reference's own fp32 kernels (GI im2col ConvBias, GI 4x12 MatrixMul),
    committed under tests/golden/: 1e-4 relative / 1e-5 absolute."""
    for c in cases.f32_conv_catalogue():
        src, flt, bias = cases.f32_conv_inputs(c)
        p = ops.conv_f32_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                               c["pad"], 1, c["act"])
        out = ops.conv_bias_f32_nhwc(p, ops.nchw_to_nhwc_f32(dev(src)),
                                     ops.pack_filter_f32(p, dev(flt)),
                                     None if bias is None else dev(bias))
        G.check_close("f32_ops", c["name"], to_nchw(out), RTOL, ATOL, src, flt, bias)
    for c in cases.f32_matmul_catalogue():
        a, b = cases.f32_matmul_inputs(c)
        G.check_close("f32_ops", c["name"], ops.matmul_f32(dev(a), dev(b)).cpu().numpy(), RTOL,
                      ATOL * np.sqrt(c["k"]), a, b)
    assert ops.device_status() == 0


def test_conv_f32_residual_and_channel_slice_of_a_wider_buffer(ops, oracle):
    """+ z after the activation (bottleneck shortcut), written into channels 32..95 of a
    128-channel buffer (a Concat without the copy)."""
    r = cases.rng_for("f32_residual_slice")
    n, ic, oc, hw = 2, 64, 64, 24
    src = r.standard_normal((n, ic, hw, hw)).astype(np.float32)
    flt = (r.standard_normal((oc, ic, 3, 3)) / 24).astype(np.float32)
    bias = r.standard_normal(oc).astype(np.float32)
    z = r.standard_normal((n, oc, hw, hw)).astype(np.float32)
    p = ops.conv_f32_param(n, ic, hw, hw, oc, 3, 3, 1, 1, 1, "SILU")
    wide = torch.full((n, hw, hw, 128), 7.0, dtype=torch.float32, device="cuda")
    ops.conv_bias_f32_nhwc(p, ops.nchw_to_nhwc_f32(dev(src)), ops.pack_filter_f32(p, dev(flt)),
                           dev(bias), z=ops.nchw_to_nhwc_f32(dev(z)), dst=wide[:, :, :, 32:],
                           dst_pitch=128, algo="umma")
    got = wide.cpu().numpy()
    want = oracle.conv_bias_f32(src, flt, bias, 1, 1, "SILU", z=z)
    close(got[:, :, :, 32:96].transpose(0, 3, 1, 2), want)
    assert (got[:, :, :, :32] == 7.0).all() and (got[:, :, :, 96:] == 7.0).all()


MATMUL_SHAPES = [(512, 512, 512), (300, 72, 640), (1024, 1000, 2048), (64, 15, 48), (2048, 2048, 2048)]


@pytest.mark.parametrize("shape", MATMUL_SHAPES, ids=["x".join(map(str, s)) for s in MATMUL_SHAPES])
def test_matmul_f32_matches_oracle(ops, oracle, shape):
    m, n, k = shape
    r = cases.rng_for("f32_matmul_%dx%dx%d" % shape)
    a = r.standard_normal((m, k)).astype(np.float32)
    b = r.standard_normal((k, n)).astype(np.float32)
    got = ops.matmul_f32(dev(a), dev(b)).cpu().numpy()
    want = oracle.matmul_f32(a, b)
    # N(0,1) operands: the sum has magnitude ~sqrt(k), and the tolerance is relative to the
    # result with the absolute part scaled likewise
    close(got, want, RTOL, ATOL * np.sqrt(k))
    assert ops.device_status() == 0


@pytest.mark.parametrize("mode", ["RELU", "SIGMOID", "SILU", "H_SWISH", "EXP", "ADD", "SUB",
                                  "MUL", "MAX", "FUSE_ADD_RELU"])
def test_elemwise_f32_matches_oracle(ops, oracle, mode):
    r = cases.rng_for("f32_elem_" + mode)
    a = (3 * r.standard_normal((3, 5, 7, 11))).astype(np.float32)
    b = (3 * r.standard_normal((3, 5, 7, 11))).astype(np.float32)
    binary = mode in ("ADD", "SUB", "MUL", "MAX", "FUSE_ADD_RELU")
    got = ops.elemwise_f32(mode, dev(a), dev(b) if binary else None).cpu().numpy()
    want = oracle.elemwise_f32(mode, a, b if binary else None)
    close(got, want, 1e-5, 1e-6)


def test_concat_resize_pool_focus_relayout_are_exact(ops, oracle):
    r = cases.rng_for("f32_movement")
    xs = [r.standard_normal((2, c, 9, 11)).astype(np.float32) for c in (16, 32, 8, 12)]
    got = ops.concat_f32_nhwc([ops.nchw_to_nhwc_f32(dev(x)) for x in xs])
    assert (to_nchw(got) == oracle.concat_f32(xs)).all()
    odd = [r.standard_normal((1, c, 5, 5)).astype(np.float32) for c in (3, 5)]
    got = ops.concat_f32_nhwc([ops.nchw_to_nhwc_f32(dev(x)) for x in odd])
    assert (to_nchw(got) == oracle.concat_f32(odd)).all()
    x = r.standard_normal((2, 24, 10, 13)).astype(np.float32)
    got = ops.resize_nearest_f32_nhwc(ops.nchw_to_nhwc_f32(dev(x)), 20, 26)
    assert (to_nchw(got) == oracle.resize_nearest_f32(x, 20, 26)).all()
    got = ops.resize_nearest_f32_nhwc(ops.nchw_to_nhwc_f32(dev(x)), 17, 31)
    assert (to_nchw(got) == oracle.resize_nearest_f32(x, 17, 31)).all()
    for window in (5, 9, 13):
        x = r.standard_normal((2, 32, 20, 20)).astype(np.float32)
        got = ops.pooling_f32_nhwc(ops.nchw_to_nhwc_f32(dev(x)), "MAX", window, 1, window // 2)
        assert (to_nchw(got) == oracle.pooling_f32(x, "MAX", window, 1, window // 2)).all()
    x = r.standard_normal((2, 6, 12, 12)).astype(np.float32)
    for mode in ("AVERAGE", "AVERAGE_COUNT_EXCLUDE_PADDING"):
        got = ops.pooling_f32_nhwc(ops.nchw_to_nhwc_f32(dev(x)), mode, 3, 2, 1)
        close(to_nchw(got), oracle.pooling_f32(x, mode, 3, 2, 1), 1e-6, 1e-7)
    img = r.uniform(0, 1, (2, 3, 32, 48)).astype(np.float32)
    got = ops.focus_f32(dev(img), 16)
    assert (to_nchw(got) == oracle.focus_f32(img, 16)).all()
    y = ops.nchw_to_nhwc_f32(dev(x))
    assert (ops.nhwc_to_nchw_f32(y).cpu().numpy() == x).all()


# ---- whole fp32 models through the compiler and the LITE_* runtime -------------------------
def run_f32_model(spec, x, forwards=3):
    from megcc_b200 import lite
    from oracle import netwalk, oracle as O
    want = netwalk.run_f32(spec, x, O)
    net = lite.Network(spec.to_graph().compile([x.shape[0]]))
    outs = []
    for _ in range(forwards):  # eager, capture, replay
        net.set_input("data", x)
        net.forward()
        net.wait()
        outs.append([net.output(n, dtype=np.float32).reshape(w.shape)
                     for n, w in zip(net.output_names(), want)])
    net.close()
    return outs, want


@pytest.mark.parametrize("hw,batch", [(128, 4), (64, 2), (224, 1)])
def test_yolox_s_matches_oracle(ops, hw, batch):
    """YOLOX-s-style detector (83 ConvBias layers, SPP, PAFPN, three decoupled heads) against
    the CPU checker walking the same layer list. 128 x 128 at batch 4 runs nearly every
    ConvBias on the tensor cores; 64 x 64 at batch 2 leaves the deep, small maps to the
    general kernel."""
    from megcc_b200 import zoo
    spec = zoo.yolox_s(hw=hw)
    x = cases.rng_for(f"yolox_{hw}").uniform(0, 1, (batch, 3, hw, hw)).astype(np.float32)
    outs, want = run_f32_model(spec, x)
    for i, got in enumerate(outs):
        for g, w in zip(got, want):
            close(g, w)
    # the outputs must exercise the arithmetic: regressions and scores spread, nothing
    # collapsed to a constant or saturated
    assert all(w[:, :4].std() > 0.1 and 0.02 < w[:, 5:].std() < 0.45 for w in want)
    assert ops.device_status() == 0


def test_fp32_matmul_model_matches_oracle(ops, oracle):
    """conv -> global average pool -> MatrixMul (fp32) through the compiler and the runtime."""
    from megcc_b200 import lite
    from megcc_b200.compiler import Graph
    r = cases.rng_for("f32_gap_matmul")
    n = 256
    g = Graph("gap_matmul_f32")
    x = g.input_f32("data", 32, 8, 8)
    f = (r.standard_normal((64, 32, 3, 3)) / 17).astype(np.float32)
    y = g.conv_f32("conv", x, f, None, 1, 1, "RELU")
    y = g.pooling("gap", y, "AVERAGE", 8, 8, 0)
    b = r.standard_normal((64, 200)).astype(np.float32)
    y = g.matmul_f32("fc", y, b)
    g.mark_output(y)
    src = r.standard_normal((n, 32, 8, 8)).astype(np.float32)
    conv = oracle.conv_bias_f32(src, f, None, 1, 1, "RELU")
    pooled = oracle.pooling_f32(conv, "AVERAGE", 8, 8, 0).reshape(n, 64)
    want = oracle.matmul_f32(pooled, b)
    net = lite.Network(g.compile([n]))
    for _ in range(3):
        net.set_input("data", src)
        net.forward()
        net.wait()
        got = net.output(net.output_names()[0], dtype=np.float32).reshape(n, 200)
        close(got, want, RTOL, 3 * ATOL)
    net.close()
