"""Parity of the CUDA operators, called through the C ABI, with the CPU oracle and with the
golden vectors produced by the reference's own x86 kernels. Bit-exact everywhere."""
import numpy as np
import pytest

import cases
import golden_util as G

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from megcc_b200 import ops as O
    return O


@pytest.fixture
def tune(ops):
    """Sets kernel-selection switches for one test and puts the old values back."""
    saved = []

    def set_(name, value):
        saved.append((name, ops.set_option(name, value)))

    yield set_
    for name, old in reversed(saved):
        ops.set_option(name, old)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_conv_nchw(ops, c, algo="auto", flt_scales=None):
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    p = ops.conv_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                       c["pad"], c["groups"], c["act"], s0, s1, s2)
    out = ops.conv_bias_qs8_nchw(p, dev(src), dev(flt), None if bias is None else dev(bias),
                                 None if flt_scales is None else dev(flt_scales), algo=algo)
    torch.cuda.synchronize()
    return out.cpu().numpy(), (src, flt, bias)


def test_conv_naive_catalogue_golden(ops):
    for c in cases.conv_naive_catalogue():
        out, ins = run_conv_nchw(ops, c)
        G.check("conv_bias_qs8", c["name"], out, *ins)


def test_conv_im2col_catalogue_golden(ops):
    for c in cases.conv_im2col_catalogue():
        out, ins = run_conv_nchw(ops, c)
        G.check("conv_bias_qs8", c["name"], out, *ins)


def test_conv_model_shapes_golden(ops):
    for c in cases.conv_model_shapes():
        out, ins = run_conv_nchw(ops, c)
        G.check("conv_bias_qs8", c["name"], out, *ins)


def test_conv_nchw44_catalogue_golden(ops, oracle):
    """Tensors and filters in the NCHW44 layouts: relayout to NHWC, filter repacked straight
    from its NCHW44 form, ConvBias, relayout back; against the outputs of the reference's
    NCHW44 kernels."""
    for c in cases.conv_nchw44_catalogue():
        src, flt44, bias = cases.conv_nchw44_inputs(c, oracle)
        s0, s1, s2 = c["scales"]
        p = ops.conv_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                           c["pad"], c["groups"], c["act"], s0, s1, s2)
        first = c["form"] == "first_layer"
        x = dev(src) if first else ops.nchw44_to_nhwc(dev(src))
        packed = ops.pack_filter_nchw44(p, dev(flt44), c["form"])
        b = None if bias is None else dev(bias)
        if ops.conv_s2d_supported(p):
            y = ops.conv_bias_qs8_s2d(p, x, packed, b, src_is_nchw=first)
        else:
            y = ops.conv_bias_qs8_nhwc(p, x, packed, b, src_is_nchw=first)
        out = ops.nhwc_to_nchw44(y).cpu().numpy()
        G.check("conv_bias_nchw44", c["name"], out, src, flt44, bias)


def test_nchw44_relayouts_are_inverse_and_match_numpy(ops, oracle):
    r = cases.rng_for("nchw44_relayout")
    for n, c, h, w in [(1, 4, 1, 1), (3, 20, 7, 5), (2, 64, 33, 31), (5, 8, 1, 130)]:
        x = r.integers(-128, 128, (n, c, h, w), dtype=np.int8)
        x44 = oracle.nchw_to_nchw44(x)
        nhwc = ops.nchw44_to_nhwc(dev(x44))
        assert (nhwc.cpu().numpy() == x.transpose(0, 2, 3, 1)).all()
        assert (ops.nhwc_to_nchw44(nhwc).cpu().numpy() == x44).all()


@pytest.mark.parametrize("algo", ["direct", "umma"])
@pytest.mark.parametrize("dst_scale", [0.1, 5.0])
def test_conv_cfg1_golden(ops, algo, dst_scale):
    c = cases.conv_cfg1(dst_scale)
    out, ins = run_conv_nchw(ops, c, algo=algo)
    G.check("conv_bias_qs8", c["name"], out, *ins)
    assert ops.device_status() == 0


UMMA_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act
    ("s1_64", 2, 64, 64, 32, 32, 3, 1, 1, "RELU"),
    ("s1_64_identity", 1, 64, 64, 56, 56, 3, 1, 1, "IDENTITY"),
    ("s1_64_hswish", 1, 64, 64, 56, 56, 3, 1, 1, "H_SWISH"),
    ("ragged_m", 3, 64, 64, 27, 29, 3, 1, 1, "RELU"),
    ("s2_64_128", 2, 64, 128, 56, 56, 3, 2, 1, "RELU"),
    ("proj_64_128", 2, 64, 128, 56, 56, 1, 2, 0, "IDENTITY"),
    ("s1_128", 2, 128, 128, 28, 28, 3, 1, 1, "RELU"),
    ("s2_128_256", 2, 128, 256, 28, 28, 3, 2, 1, "RELU"),
    ("s1_256", 4, 256, 256, 14, 14, 3, 1, 1, "RELU"),
    ("s1_512", 6, 512, 512, 7, 7, 3, 1, 1, "RELU"),
    ("fc_512_1000", 256, 512, 1000, 1, 1, 1, 1, 0, "IDENTITY"),
    ("pw_1024", 3, 1024, 1024, 7, 7, 1, 1, 0, "RELU"),
    ("k5_s1", 2, 64, 72, 40, 40, 5, 1, 2, "RELU"),
    ("k7_s2_p3", 1, 64, 64, 48, 48, 7, 2, 3, "RELU"),
    ("nopad_k3", 1, 64, 64, 50, 50, 3, 1, 0, "RELU"),
    ("s3", 1, 64, 64, 50, 47, 3, 3, 1, "RELU"),
    ("oc76_bytes", 2, 64, 76, 40, 40, 3, 1, 1, "RELU"),
    ("oc1000_8byte", 300, 512, 1000, 1, 1, 1, 1, 0, "RELU"),
]


@pytest.mark.parametrize("case", UMMA_CASES, ids=[c[0] for c in UMMA_CASES])
def test_conv_umma_matches_oracle(ops, oracle, case):
    name, n, ic, oc, h, w, k, stride, pad, act = case
    c = dict(name="umma_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    out, (src, flt, bias) = run_conv_nchw(ops, c, algo="umma")
    s0, s1, s2 = c["scales"]
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, act)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0
    # the result must exercise the requantisation, not sit on the clamps
    assert (np.abs(want.astype(int)) < 127).mean() > 0.3


@pytest.mark.parametrize("algo", ["umma", "patch"])
@pytest.mark.parametrize("act", ["RELU", "IDENTITY"])
def test_conv_reference_operation_order_without_verified_forms(ops, oracle, algo, act,
                                                               tune):
    """The epilogue with the reference's own six float operations (the verified short forms
    switched off), and the same case with them on: both bit-exact."""
    c = dict(name="exact_chain_" + act, n=2, ic=64, oc=64, h=40, w=40, k=3, stride=1, pad=1,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.9))
    s0, s1, s2 = c["scales"]
    src, flt, bias = cases.conv_inputs(c)
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 1, s0, s1, s2, act)
    out, _ = run_conv_nchw(ops, c, algo=algo)
    assert (out == want).all()
    tune("fast_requant", 0)
    out, _ = run_conv_nchw(ops, c, algo=algo)
    assert (out == want).all()
    assert ops.device_status() == 0


BN256_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act, forced
    ("s1_256", 4, 256, 256, 14, 14, 3, 1, 1, "RELU", True),
    ("s1_512", 6, 512, 512, 7, 7, 3, 1, 1, "RELU", True),
    ("s2_128_256", 2, 128, 256, 28, 28, 3, 2, 1, "IDENTITY", True),
    ("ragged_oc320", 4, 128, 320, 20, 20, 3, 1, 1, "RELU", True),
    ("pw_1024", 3, 1024, 1024, 7, 7, 1, 1, 0, "H_SWISH", True),
    ("auto_256_n100", 100, 256, 256, 14, 14, 3, 1, 1, "RELU", False),
]


@pytest.mark.parametrize("case", BN256_CASES, ids=[c[0] for c in BN256_CASES])
def test_conv_umma_256_wide_tiles_match_oracle(ops, oracle, case, tune):
    """The 128 x 256 output tile (one CTA per SM, sixteen epilogue warps): forced through the
    tuning variable on small shapes, and chosen by the launcher itself on one large enough."""
    name, n, ic, oc, h, w, k, stride, pad, act, forced = case
    if forced:
        tune("conv_bn", 256)
    c = dict(name="bn256_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    out, (src, flt, bias) = run_conv_nchw(ops, c, algo="umma")
    s0, s1, s2 = c["scales"]
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, act)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0


SMALL_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act, algo: activations below 128 KiB
    ("b1_128_28", 1, 128, 128, 28, 28, 3, 1, 1, "RELU", "umma"),
    ("b1_256_14", 1, 256, 256, 14, 14, 3, 1, 1, "RELU", "umma"),
    ("b1_512_7", 1, 512, 512, 7, 7, 3, 1, 1, "IDENTITY", "umma"),
    ("b1_256_512_s2", 1, 256, 512, 14, 14, 3, 2, 1, "RELU", "umma"),
    ("b1_proj_s2", 1, 128, 256, 28, 28, 1, 2, 0, "IDENTITY", "umma"),
    ("b3_512_7", 3, 512, 512, 7, 7, 3, 1, 1, "RELU", "umma"),
    ("b1_128_28_patch", 1, 128, 128, 28, 28, 3, 1, 1, "RELU", "patch"),
    ("b1_64_20_patch", 1, 64, 64, 20, 20, 3, 1, 1, "RELU", "patch"),
]


@pytest.mark.parametrize("case", SMALL_CASES, ids=[c[0] for c in SMALL_CASES])
def test_conv_small_activation_in_registered_range(ops, oracle, case):
    """Batch 1 of the late ResNet layers: the activation is smaller than the 128 KiB a TMA map
    is built over. Inside a registered readable range (what the runtime does with its arena)
    the tensor-core kernels take it; the same call outside such a range is refused by the
    forced algorithm and served by the general kernel under "auto"."""
    import ctypes
    from megcc_b200._lib import check, lib
    name, n, ic, oc, h, w, k, stride, pad, act, algo = case
    c = dict(name="small_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    s0, s1, s2 = c["scales"]
    src, flt, bias = cases.conv_inputs(c)
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, act)
    p = ops.conv_param(n, ic, h, w, oc, k, k, stride, pad, 1, act, s0, s1, s2)
    packed = ops.pack_filter(p, dev(flt))
    nhwc = np.ascontiguousarray(src.transpose(0, 2, 3, 1))
    assert nhwc.size < 131072
    # an "arena": the activation sits at an odd 256-byte offset, 192 KiB of bytes follow it
    arena = torch.randint(-128, 128, (nhwc.size + 256 * 3 + 192 * 1024,), dtype=torch.int8,
                          device="cuda")
    view = arena[768:768 + nhwc.size].view(n, h, w, ic)
    view.copy_(torch.from_numpy(nhwc))
    check(lib().mb200_register_readable_range(ctypes.c_void_p(arena.data_ptr()), arena.numel()))
    try:
        out = ops.conv_bias_qs8_nhwc(p, view, packed, dev(bias), algo=algo)
        torch.cuda.synchronize()
    finally:
        check(lib().mb200_unregister_readable_range(ctypes.c_void_p(arena.data_ptr())))
    got = out.cpu().numpy().transpose(0, 3, 1, 2)
    bad = int((got != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(got != want)[:4].tolist()}"
    assert ops.device_status() == 0
    # not registered any more: the tensor-core kernels decline, "auto" still answers
    with pytest.raises(Exception):
        ops.conv_bias_qs8_nhwc(p, view, packed, dev(bias), algo=algo)
    out = ops.conv_bias_qs8_nhwc(p, view, packed, dev(bias), algo="auto")
    assert (out.cpu().numpy().transpose(0, 3, 1, 2) == want).all()


SPLITK_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act, split
    ("s1_256_x2", 4, 256, 256, 14, 14, 3, 1, 1, "RELU", 2),
    ("s1_256_x3", 4, 256, 256, 14, 14, 3, 1, 1, "IDENTITY", 3),
    ("s1_256_x4", 4, 256, 256, 14, 14, 3, 1, 1, "RELU", 4),
    ("s1_512_x3", 6, 512, 512, 7, 7, 3, 1, 1, "RELU", 3),          # two channel tiles
    ("s2_128_256_x2", 2, 128, 256, 28, 28, 3, 2, 1, "IDENTITY", 2),  # 9 K steps: 5 + 4
    ("ragged_oc320_x3", 4, 128, 320, 20, 20, 3, 1, 1, "RELU", 3),
    ("pw_1024_x2", 3, 1024, 1024, 7, 7, 1, 1, 0, "H_SWISH", 2),     # tiled A map
]


@pytest.mark.parametrize("case", SPLITK_CASES, ids=[c[0] for c in SPLITK_CASES])
def test_conv_umma_split_k_matches_oracle(ops, oracle, case, tune):
    """128 x 256 tiles cut along K: every part leaves its accumulators in scratch and the last
    one to finish sums and requantises. Forced on small shapes (all tiles split), run twice:
    the second launch finds the counters as the first one left them."""
    name, n, ic, oc, h, w, k, stride, pad, act, split = case
    tune("conv_bn", 256)
    tune("conv_splitk", split)
    c = dict(name="splitk_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    s0, s1, s2 = c["scales"]
    want = None
    for _ in range(2):
        out, (src, flt, bias) = run_conv_nchw(ops, c, algo="umma")
        if want is None:
            want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, act)
        bad = int((out != want).sum())
        assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0


@pytest.mark.parametrize("mode", [None, "QFUSE_ADD_RELU"])
def test_conv_umma_split_k_last_wave_equals_unsplit(ops, mode, tune):
    """A ResNet stage-4 shape at batch 256 (196 tiles on 148 SMs: 148 whole tiles, 48 tiles
    in three parts each), with and without the fused residual step, against the same kernel
    without the split (itself checked against the oracle on smaller shapes)."""
    n, ic, oc, hw = 256, 512, 512, 7
    rng = cases.rng_for("splitk_auto_%s" % mode)
    src = dev(rng.integers(-128, 128, (n, hw, hw, ic), dtype=np.int8))
    flt = rng.integers(-127, 128, (oc, ic, 3, 3), dtype=np.int8)
    bias = dev(rng.integers(-1000, 1000, (oc,), dtype=np.int32))
    z = dev(rng.integers(-128, 128, (n, hw, hw, oc), dtype=np.int8))
    p = ops.conv_param(n, ic, hw, hw, oc, 3, 3, 1, 1, 1, "IDENTITY" if mode else "RELU",
                       0.05, 0.01, 1.6)
    packed = ops.pack_filter(p, dev(flt))

    def run():
        if mode:
            return ops.conv_bias_qs8_nhwc_fused(p, src, packed, bias, z, mode, 0.7, 1.3,
                                                algo="umma").cpu().numpy()
        return ops.conv_bias_qs8_nhwc(p, src, packed, bias, algo="umma").cpu().numpy()

    whole = run()
    assert (np.abs(whole.astype(int)) < 127).mean() > 0.3
    tune("conv_splitk", 3)
    for _ in range(2):
        assert (run() == whole).all()
    assert ops.device_status() == 0


PAIR_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, act
    ("s1_256", 4, 256, 256, 14, 14, 3, 1, 1, "RELU"),            # 784 pixels: 3 full pairs + tail
    ("s1_512", 6, 512, 512, 7, 7, 3, 1, 1, "RELU"),              # 294 pixels, two channel tiles
    ("s2_128_256", 2, 128, 256, 28, 28, 3, 2, 1, "IDENTITY"),
    ("ragged_oc320", 4, 128, 320, 20, 20, 3, 1, 1, "RELU"),      # second channel tile: 64 of 256
    ("peer_empty", 11, 128, 256, 10, 10, 3, 1, 1, "H_SWISH"),    # 1100 pixels: the last pair's peer is idle
    ("pw_1024", 3, 1024, 1024, 7, 7, 1, 1, 0, "RELU"),
]


@pytest.mark.parametrize("case", PAIR_CASES, ids=[c[0] for c in PAIR_CASES])
def test_conv_pair_of_sms_matches_oracle(ops, oracle, case, tune):
    """256 x 256 tiles computed by two CTAs on two SMs (tcgen05 cta_group::2)."""
    name, n, ic, oc, h, w, k, stride, pad, act = case
    tune("conv_pair", 1)
    c = dict(name="pair_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=1, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    out, (src, flt, bias) = run_conv_nchw(ops, c, algo="umma")
    s0, s1, s2 = c["scales"]
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, act)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0


DW_CASES = [
    # name, n, c, h, w, stride, pad, act, per_channel
    ("mbv1_112_c32", 2, 32, 112, 112, 1, 1, "RELU", False),
    ("mbv1_112_c64_s2", 2, 64, 112, 112, 2, 1, "RELU", True),
    ("mbv1_14_c512", 3, 512, 14, 14, 1, 1, "RELU", True),
    ("mbv1_7_c1024", 2, 1024, 7, 7, 1, 1, "IDENTITY", True),
    ("odd_hw_nopad", 2, 48, 13, 17, 1, 0, "H_SWISH", False),
    ("odd_hw_s2_pad2", 1, 16, 15, 11, 2, 2, "RELU", False),
    # stride 1 over whole 64-channel slices: the tensor-core form (block-diagonal filter)
    ("tc_56_c128", 2, 128, 56, 56, 1, 1, "RELU", False),
    ("tc_28_c256_identity", 2, 256, 28, 28, 1, 1, "IDENTITY", False),
    ("tc_30x24_c64_nopad", 3, 64, 30, 24, 1, 0, "H_SWISH", True),
    ("tc_partial_patches_c192", 2, 192, 27, 23, 1, 1, "RELU", True),
    # 32 channels: pixel pairs as 64-byte rows, two diagonals in the filter tile
    ("tc_pairs_112_c32", 2, 32, 112, 112, 1, 1, "RELU", True),
    ("tc_pairs_c32_20x36_identity", 8, 32, 20, 36, 1, 1, "IDENTITY", False),
    ("auto_tc_14_c512", 64, 512, 14, 14, 1, 1, "RELU", False),   # 1024 patches on 148 SMs: "auto" takes it
]


@pytest.mark.parametrize("form", ["one", "2", "4"])
@pytest.mark.parametrize("case", [DW_CASES[1], DW_CASES[4], DW_CASES[5]],
                         ids=["c64_s2", "odd_hw_nopad", "odd_hw_s2_pad2"])
def test_depthwise_kernel_forms(ops, oracle, case, form, tune):
    """Every form of the depthwise kernel at both strides, chosen by its tuning variable: one
    output per thread (it also serves the fused residual step), two and four outputs."""
    if form == "one":
        tune("dw_one_output", 1)
    else:
        tune("dw_out", int(form))
    name, n, ch, h, w, stride, pad, act, per_channel = case
    c = dict(name="dw_" + name, n=n, ic=ch, oc=ch, h=h, w=w, k=3, stride=stride, pad=pad,
             groups=ch, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.06))
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    scales = None
    if per_channel:
        scales = cases.rng_for("dw_scales_" + name).uniform(0.005, 0.02, ch).astype(np.float32)
    out, _ = run_conv_nchw(ops, c, algo="auto", flt_scales=scales)
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, scales if per_channel else s1,
                                s2, act, groups=ch)
    assert (out == want).all()


@pytest.mark.parametrize("case", DW_CASES, ids=[c[0] for c in DW_CASES])
def test_depthwise_3x3_matches_oracle(ops, oracle, case):
    """The vectorised depthwise kernel (auto) against the oracle, and against the general
    kernel (direct) on the same inputs."""
    name, n, ch, h, w, stride, pad, act, per_channel = case
    c = dict(name="dw_" + name, n=n, ic=ch, oc=ch, h=h, w=w, k=3, stride=stride, pad=pad,
             groups=ch, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.06))
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    scales = None
    if per_channel:
        scales = cases.rng_for("dw_scales_" + name).uniform(0.005, 0.02, ch).astype(np.float32)
    # "tc_" cases: the tensor-core form by name ("auto" takes it only from four patches of real outputs per SM up)
    out, _ = run_conv_nchw(ops, c, algo="patch" if name.startswith("tc_") else "auto",
                           flt_scales=scales)
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, scales if per_channel else s1,
                                s2, act, groups=ch)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    ref, _ = run_conv_nchw(ops, c, algo="direct", flt_scales=scales)
    assert (ref == want).all()
    assert (np.abs(want.astype(int)) < 127).mean() > 0.3


@pytest.mark.parametrize("case", [DW_CASES[2], DW_CASES[6]], ids=["c512_14", "c128_56"])
def test_depthwise_stride1_on_cuda_cores(ops, oracle, case, tune):
    """The shapes the tensor-core depthwise form takes by default, through the CUDA-core
    kernel (dw_tensor = 0): both stay bit-exact against the oracle."""
    tune("dw_tensor", 0)
    name, n, ch, h, w, stride, pad, act, per_channel = case
    c = dict(name="dw_" + name, n=n, ic=ch, oc=ch, h=h, w=w, k=3, stride=stride, pad=pad,
             groups=ch, act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.06))
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    scales = None
    if per_channel:
        scales = cases.rng_for("dw_scales_" + name).uniform(0.005, 0.02, ch).astype(np.float32)
    out, _ = run_conv_nchw(ops, c, algo="auto", flt_scales=scales)
    want = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, scales if per_channel else s1,
                                s2, act, groups=ch)
    assert (out == want).all()


FUSED_CASES = [
    # name, n, ic, oc, h, w, k, stride, pad, algo
    ("patch_64", 2, 64, 64, 40, 40, 3, 1, 1, "patch"),
    ("umma_128", 2, 128, 128, 28, 28, 3, 1, 1, "umma"),
    ("umma_oc72", 2, 64, 72, 40, 40, 3, 1, 1, "umma"),    # 8-byte vectors
    ("umma_oc76", 2, 64, 76, 40, 40, 3, 1, 1, "umma"),    # byte stores
    ("umma_256_wide", 4, 256, 256, 14, 14, 3, 1, 1, "umma"),
    ("direct_dw", 2, 32, 32, 20, 20, 3, 1, 1, "direct"),
    ("patch_dw", 2, 128, 128, 40, 36, 3, 1, 1, "patch"),   # depthwise, block-diagonal form
    ("patch_pairs_dw", 4, 32, 32, 40, 36, 3, 1, 1, "patch"),   # ... 32 channels as pixel pairs
]


@pytest.mark.parametrize("mode", ["QADD", "QFUSE_ADD_RELU"])
@pytest.mark.parametrize("case", FUSED_CASES, ids=[c[0] for c in FUSED_CASES])
def test_conv_with_fused_residual_step_matches_two_oracle_kernels(ops, oracle, case, mode,
                                                                  tune):
    """ConvBias + QADD / QFUSE_ADD_RELU in one launch == the reference's two kernels run one
    after the other (ConvBias to int8 at its own scale, then ElemwiseMultiType)."""
    name, n, ic, oc, h, w, k, stride, pad, algo = case
    if name == "umma_256_wide":
        tune("conv_bn", 256)
    groups = ic if name.endswith("_dw") else 1
    c = dict(name="fused_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=groups, act="IDENTITY", range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.3 * (ic // groups * k * k / 576.0) ** 0.5 + 0.1))
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    p = ops.conv_param(n, ic, h, w, oc, k, k, stride, pad, groups, "IDENTITY", s0, s1, s2)
    conv = oracle.conv_bias_qs8(src, flt, bias, stride, pad, s0, s1, s2, "IDENTITY",
                                groups=groups)
    z = cases.rng_for("fused_z_" + name).integers(-128, 128, conv.shape, dtype=np.int8)
    z_scale, out_scale = 0.7, 1.3
    want = oracle.qelemwise(mode, conv, z, s2, z_scale, out_scale)
    packed = ops.pack_filter(p, dev(flt))
    out = ops.conv_bias_qs8_nhwc_fused(
        p, ops.nchw_to_nhwc(dev(src)), packed, dev(bias), ops.nchw_to_nhwc(dev(z)), mode,
        z_scale, out_scale, algo=algo)
    got = ops.nhwc_to_nchw(out).cpu().numpy()
    bad = int((got != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(got != want)[:4].tolist()}"
    assert ops.device_status() == 0


PATCH_CASES = [
    # name, n, ic, oc, h, w, k, pad, act  (all stride 1)
    ("c64_56", 2, 64, 64, 56, 56, 3, 1, "RELU"),
    ("c64_ragged", 3, 64, 64, 27, 29, 3, 1, "IDENTITY"),
    ("c64_oc128", 2, 64, 128, 40, 40, 3, 1, "RELU"),
    ("c128_oc64", 2, 128, 64, 28, 28, 3, 1, "RELU"),
    ("c128_28", 2, 128, 128, 28, 28, 3, 1, "RELU"),
    ("c128_28_many_tiles", 80, 128, 128, 28, 28, 3, 1, "RELU"),   # 640 patches: 4-5 per CTA
    ("c128_oc64_many_tiles", 80, 128, 64, 28, 28, 3, 1, "IDENTITY"),
    ("c96_oc128_k3", 2, 96, 128, 30, 30, 3, 1, "IDENTITY"),
    ("c32_k5", 2, 32, 72, 50, 50, 5, 2, "H_SWISH"),
    ("c16_k2x4", 8, 16, 64, 40, 40, 4, 2, "RELU"),
    ("c96_k1", 4, 96, 200, 33, 31, 1, 0, "RELU"),
    ("c64_nopad", 2, 64, 64, 40, 44, 3, 0, "RELU"),
]


@pytest.mark.parametrize("case", PATCH_CASES, ids=[c[0] for c in PATCH_CASES])
def test_conv_patch_matches_oracle(ops, oracle, case):
    name, n, ic, oc, h, w, k, pad, act = case
    c = dict(name="patch_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=1, pad=pad, groups=1,
             act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.37 * (ic * k * k / 576.0) ** 0.5 + 0.4))
    out, (src, flt, bias) = run_conv_nchw(ops, c, algo="patch")
    s0, s1, s2 = c["scales"]
    want = oracle.conv_bias_qs8(src, flt, bias, 1, pad, s0, s1, s2, act)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0
    assert (np.abs(want.astype(int)) < 127).mean() > 0.3


S2D_CASES = [
    # name, n, ic, oc, h, w, k, pad, act  (all stride 2)
    ("r18_stem", 2, 3, 64, 224, 224, 7, 3, "RELU"),
    ("mbv1_stem", 2, 3, 32, 224, 224, 3, 1, "RELU"),
    ("odd_hw", 3, 3, 64, 225, 223, 7, 3, "IDENTITY"),
    ("odd_h_w8", 4, 3, 48, 97, 104, 3, 1, "RELU"),
    ("odd_h_w8_k7", 8, 3, 64, 61, 72, 7, 3, "IDENTITY"),
    ("ic1_k5", 4, 1, 40, 120, 120, 5, 2, "RELU"),
    ("ic4_k3_nopad", 4, 4, 136, 96, 100, 3, 0, "H_SWISH"),
    ("ic2_k2", 4, 2, 64, 128, 128, 2, 0, "RELU"),
    ("k1", 8, 3, 64, 128, 128, 1, 0, "RELU"),
]


@pytest.mark.parametrize("case", S2D_CASES, ids=[c[0] for c in S2D_CASES])
def test_conv_first_layer_space_to_depth_matches_oracle(ops, oracle, case):
    import ctypes
    from megcc_b200._lib import lib
    name, n, ic, oc, h, w, k, pad, act = case
    c = dict(name="s2d_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=2, pad=pad, groups=1,
             act=act, range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.05 * (ic * k * k) ** 0.5 + 0.05))
    s0, s1, s2 = c["scales"]
    p = ops.conv_param(n, ic, h, w, oc, k, k, 2, pad, 1, act, s0, s1, s2)
    assert lib().mb200_conv_s2d_supported(ctypes.byref(p)) == 1
    out, (src, flt, bias) = run_conv_nchw(ops, c)  # auto: takes the space-to-depth path
    want = oracle.conv_bias_qs8(src, flt, bias, 2, pad, s0, s1, s2, act)
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert ops.device_status() == 0
    assert (np.abs(want.astype(int)) < 127).mean() > 0.3
    direct, _ = run_conv_nchw(ops, c, algo="direct")
    assert (direct == want).all()


POOL_CASES = [
    # name, n, ic, oc, h, w, k, pad, act, per_channel, bias  (stride 2, then MAX 3x3 / 2 / pad 1)
    ("r18_stem", 2, 3, 64, 224, 224, 7, 3, "RELU", False, True),
    ("odd_hw", 3, 3, 64, 225, 223, 7, 3, "IDENTITY", False, True),
    ("k3_oc32", 4, 3, 32, 97, 104, 3, 1, "RELU", False, True),
    ("k5_ic1_oc48", 4, 1, 48, 120, 120, 5, 2, "RELU", True, True),
    ("k3_nopad_oc16", 4, 4, 16, 96, 100, 3, 0, "IDENTITY", False, False),
    ("tiny_maps", 32, 3, 64, 33, 35, 7, 3, "RELU", False, True),
    ("one_tile_row", 48, 2, 64, 26, 30, 3, 1, "RELU", True, True),
]


@pytest.mark.parametrize("case", POOL_CASES, ids=[c[0] for c in POOL_CASES])
def test_first_layer_conv_with_fused_max_pool_matches_two_oracle_kernels(ops, oracle, case):
    """ConvBias + Pooling MAX 3x3 / 2 / pad 1 as one kernel (the window maximum is taken on the
    int32 accumulators, one output in four is requantised) against the two CPU kernels run one
    after the other."""
    name, n, ic, oc, h, w, k, pad, act, per_channel, with_bias = case
    c = dict(name="pool_" + name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=2, pad=pad, groups=1,
             act=act, range=(-128, 127), bias_range=(-1000, 1000), bias=with_bias,
             scales=(0.05, 0.01, 0.05 * (ic * k * k) ** 0.5 + 0.05))
    src, flt, bias = cases.conv_inputs(c)
    s0, s1, s2 = c["scales"]
    sf = (cases.rng_for(c["name"] + "_pc").uniform(0.005, 0.02, oc).astype(np.float32)
          if per_channel else None)
    p = ops.conv_param(n, ic, h, w, oc, k, k, 2, pad, 1, act, s0, s1, s2)
    assert ops.conv_s2d_pool_supported(p)
    packed = ops.pack_filter_s2d(p, dev(flt))
    got = ops.conv_bias_pool_qs8_s2d(p, dev(src), packed, None if bias is None else dev(bias),
                                     None if sf is None else dev(sf))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    conv = oracle.conv_bias_qs8(src, flt, bias, 2, pad, s0, s1 if sf is None else sf, s2, act)
    want = oracle.pooling_qs8(conv, "MAX", 3, 2, 1)
    out = got.cpu().numpy().transpose(0, 3, 1, 2)
    assert out.shape == want.shape
    bad = int((out != want).sum())
    assert bad == 0, f"{bad}/{want.size} differ; first at {np.argwhere(out != want)[:4].tolist()}"
    assert len(np.unique(want)) > 8


def test_fused_max_pool_is_refused_where_it_does_not_commute(ops):
    # H_SWISH is not monotonic; more than 64 output channels have no pooled epilogue
    assert not ops.conv_s2d_pool_supported(
        ops.conv_param(2, 3, 224, 224, 64, 7, 7, 2, 3, 1, "H_SWISH", 0.05, 0.01, 0.5))
    assert not ops.conv_s2d_pool_supported(
        ops.conv_param(2, 3, 224, 224, 128, 7, 7, 2, 3, 1, "RELU", 0.05, 0.01, 0.5))
    assert not ops.conv_s2d_pool_supported(
        ops.conv_param(2, 64, 56, 56, 64, 3, 3, 2, 1, 1, "RELU", 0.05, 0.01, 0.5))


def test_conv_umma_per_channel_scales(ops, oracle):
    c = dict(name="umma_perchannel", n=2, ic=64, oc=128, h=32, w=32, k=3, stride=1, pad=1,
             groups=1, act="RELU", range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.8))
    sf = cases.rng_for("umma_perchannel_scales").uniform(0.005, 0.02, 128).astype(np.float32)
    out, (src, flt, bias) = run_conv_nchw(ops, c, algo="umma", flt_scales=sf)
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 1, 0.05, sf, 0.8, "RELU")
    assert (out == want).all()


def test_conv_accumulators_match_oracle(ops, oracle):
    c = dict(name="acc_parity", n=1, ic=20, oc=20, h=10, w=10, k=3, stride=1, pad=0, groups=1,
             act="IDENTITY", range=(30, 50), scales=(1.0, 2.0, 4.0))
    src, flt, bias = cases.conv_inputs(c)
    p = ops.conv_param(1, 20, 10, 10, 20, 3, 3, 1, 0, 1, "IDENTITY", 1.0, 2.0, 4.0)
    packed = ops.pack_filter(p, dev(flt))
    acc = ops.conv_acc_qs8_nhwc(p, ops.nchw_to_nhwc(dev(src)), packed, dev(bias))
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 0, 1.0, 2.0, 4.0, return_acc=True)[1]
    assert (acc.cpu().numpy().transpose(0, 3, 1, 2) == want).all()


@pytest.mark.parametrize("ic,oc,groups", [(64, 64, 1), (20, 12, 1), (32, 32, 32), (6, 6, 1)])
def test_conv_on_tensors_that_start_at_an_odd_byte(ops, oracle, ic, oc, groups):
    """int8 tensors sliced out of a larger buffer at byte offset 1: no vector or TMA path may
    take them, and the byte-wise kernel gives the same result."""
    c = dict(name=f"odd_offset_{ic}_{oc}_{groups}", n=2, ic=ic, oc=oc, h=19, w=17, k=3, stride=1,
             pad=1, groups=groups, act="RELU", range=(-128, 127), bias_range=(-1000, 1000),
             scales=(0.05, 0.01, 0.4))
    src, flt, bias = cases.conv_inputs(c)
    p = ops.conv_param(2, ic, 19, 17, oc, 3, 3, 1, 1, groups, "RELU", 0.05, 0.01, 0.4)

    def at_offset_one(t):
        buf = torch.empty(t.numel() + 64, dtype=torch.int8, device="cuda")
        off = 1 + (-buf.data_ptr()) % 16  # one past a 16-byte boundary
        view = buf[off:off + t.numel()].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 == 1
        return view

    nhwc = at_offset_one(ops.nchw_to_nhwc(dev(src)))
    packed = at_offset_one(ops.pack_filter(p, dev(flt)))
    dst = at_offset_one(torch.zeros((2, 19, 17, oc), dtype=torch.int8, device="cuda"))
    ops.conv_bias_qs8_nhwc(p, nhwc, packed, dev(bias), dst=dst)
    torch.cuda.synchronize()
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 1, 0.05, 0.01, 0.4, "RELU", groups=groups)
    assert (dst.cpu().numpy().transpose(0, 3, 1, 2) == want).all()
    acc = ops.conv_acc_qs8_nhwc(p, nhwc, packed, dev(bias))
    want_acc = oracle.conv_bias_qs8(src, flt, bias, 1, 1, 0.05, 0.01, 0.4, "RELU", groups=groups,
                                    return_acc=True)[1]
    assert (acc.cpu().numpy().transpose(0, 3, 1, 2) == want_acc).all()
    assert ops.device_status() == 0


@pytest.mark.parametrize("scales", [(1e-18, 1e-18, 1e-32), (3e12, 2e12, 6e28), (0.05, 0.01, 1e-21)])
def test_conv_with_scales_outside_the_fast_division_range(ops, oracle, scales):
    """Scale triples for which the three-instruction division is not proven exact take the
    general kernel with the true division: still bit-exact."""
    c = dict(name="extreme_scales", n=2, ic=64, oc=64, h=24, w=24, k=3, stride=1, pad=1, groups=1,
             act="IDENTITY", range=(-128, 127), bias_range=(-1000, 1000), scales=scales)
    out, (src, flt, bias) = run_conv_nchw(ops, c)
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 1, *scales, "IDENTITY")
    assert (out == want).all()


def test_first_layer_reads_nchw_in_place(ops, oracle):
    c = dict(name="stem_nchw", n=2, ic=3, oc=64, h=64, w=64, k=7, stride=2, pad=3, groups=1,
             act="RELU", range=(-128, 127), bias_range=(-1000, 1000), scales=(0.05, 0.01, 0.9))
    src, flt, bias = cases.conv_inputs(c)
    p = ops.conv_param(2, 3, 64, 64, 64, 7, 7, 2, 3, 1, "RELU", 0.05, 0.01, 0.9)
    packed = ops.pack_filter(p, dev(flt))
    out = ops.conv_bias_qs8_nhwc(p, dev(src), packed, dev(bias), src_is_nchw=True)
    want = oracle.conv_bias_qs8(src, flt, bias, 2, 3, 0.05, 0.01, 0.9, "RELU")
    assert (out.cpu().numpy().transpose(0, 3, 1, 2) == want).all()


MATMUL_SHAPES = [(512, 512, 512), (1024, 1000, 2048), (300, 72, 640), (64, 15, 64),
                 (16, 56, 16), (2048, 2048, 2048)]


@pytest.mark.parametrize("shape", MATMUL_SHAPES, ids=["x".join(map(str, s)) for s in MATMUL_SHAPES])
def test_matmul_int8_matches_oracle(ops, oracle, shape):
    """int8 x int8 -> int32 exactly, and requantised to int8 (x 0.002) by the TypeCvt rule.
    Small shapes are the reference's Arm int8 GEMM test family (m, n, k in 4..64)."""
    m, n, k = shape
    r = cases.rng_for("matmul_%dx%dx%d" % shape)
    a = r.integers(-127, 128, (m, k), dtype=np.int8)
    b = r.integers(-127, 128, (k, n), dtype=np.int8)
    want = oracle.matmul_s8_s32(a, b)
    bp = ops.matmul_pack_b(dev(b))
    got = ops.matmul_s8_s32(dev(a), bp).cpu().numpy()
    assert (got == want).all()
    scale = 0.002 if k <= 512 else 0.0002
    q = ops.matmul_s8_qs8(dev(a), bp, scale, 1.0).cpu().numpy()
    want_q = oracle.typecvt_qs32_qs8(want, scale, 1.0)
    assert (q == want_q).all()
    assert ops.device_status() == 0


SWEEP = [(512, 512, 512), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
         (4096, 1000, 2048)]


@pytest.mark.parametrize("shape", SWEEP, ids=["x".join(map(str, s)) for s in SWEEP])
def test_matmul_sweep_shapes_requantised(ops, oracle, shape):
    """The MatMul sweep: int8 x int8 -> int32 -> qint8 with scale 0.002, values in [-127, 127].
    The oracle computes 48 sampled rows of A against the whole of B (the full product of
    the largest shape would take the CPU minutes); a 32-bit checksum of the whole int8
    result is compared between the int32 path + stand-alone TypeCvt and the fused path."""
    m, n, k = shape
    r = cases.rng_for("matmul_sweep_%dx%dx%d" % shape)
    a = r.integers(-127, 128, (m, k), dtype=np.int8)
    b = r.integers(-127, 128, (k, n), dtype=np.int8)
    bp = ops.matmul_pack_b(dev(b))
    a_dev = dev(a)
    c32 = ops.matmul_s8_s32(a_dev, bp)
    q = ops.matmul_s8_qs8(a_dev, bp, 0.002, 1.0)
    rows = np.sort(r.choice(m, size=min(48, m), replace=False))
    want32 = oracle.matmul_s8_s32(a[rows], b)
    assert (c32[torch.from_numpy(rows).cuda()].cpu().numpy() == want32).all()
    want_q = oracle.typecvt_qs32_qs8(want32, 0.002, 1.0)
    assert (q[torch.from_numpy(rows).cuda()].cpu().numpy() == want_q).all()
    # fused requantisation == int32 product followed by the stand-alone TypeCvt kernel
    q2 = ops.typecvt_qs32_qs8(c32, 0.002, 1.0)
    assert bool((q == q2).all())
    assert ops.device_status() == 0


def test_pooling_golden(ops):
    for c in cases.pool_catalogue():
        x = cases.pool_input(c)
        y = ops.pooling_qs8_nhwc(ops.nchw_to_nhwc(dev(x)), c["mode"], c["window"], c["stride"],
                                 c["pad"])
        out = ops.nhwc_to_nchw(y).cpu().numpy()
        G.check("pooling_qs8", c["name"], out, x)


@pytest.mark.parametrize("shape", [(3, 32, 13, 13, 1), (2, 16, 15, 9, 0), (1, 48, 6, 31, 1),
                                   (2, 64, 112, 112, 1)],
                         ids=["odd_out_pad1", "nopad", "wide_row", "stem"])
def test_max_pool_3x3_stride2_matches_oracle(ops, oracle, shape):
    """The two-outputs-per-thread kernel of the ResNet stem's pool: odd output widths (a last
    pair with one output), windows that hang over every border."""
    n, c, h, w, pad = shape
    x = cases.rng_for("pool3x3s2_%d_%d_%d_%d_%d" % shape).integers(-128, 128, (n, c, h, w),
                                                                  dtype=np.int8)
    y = ops.pooling_qs8_nhwc(ops.nchw_to_nhwc(dev(x)), "MAX", 3, 2, pad)
    out = ops.nhwc_to_nchw(y).cpu().numpy()
    assert (out == oracle.pooling_qs8(x, "MAX", 3, 2, pad)).all()


@pytest.mark.parametrize("mode", ["AVERAGE", "AVERAGE_COUNT_EXCLUDE_PADDING"])
def test_global_average_pool_matches_oracle(ops, oracle, mode):
    """One window per image (the classifier's pool): sums of 25 int8 values whose mean hits
    many .5 ties, which must round away from zero as the reference's roundf does."""
    x = cases.rng_for("gap_" + mode).integers(-128, 128, (5, 48, 5, 5), dtype=np.int8)
    x[0, :, :, :] = 127
    x[1, :, :, :] = -128
    y = ops.pooling_qs8_nhwc(ops.nchw_to_nhwc(dev(x)), mode, 5, 5, 0)
    out = ops.nhwc_to_nchw(y).cpu().numpy()
    assert (out == oracle.pooling_qs8(x, mode, 5, 5, 0)).all()


@pytest.mark.parametrize("shape", [(16, 512, 7, 7), (3, 1040, 5, 5), (2, 16, 3, 3), (4, 32, 2, 2),
                                   (2, 528, 14, 14)],
                         ids=lambda s: "x".join(map(str, s)))
def test_global_average_pool_shapes(ops, oracle, shape):
    """The CTA-per-image kernel (pixels split over four warps, partial sums in shared memory):
    fewer and more than 32 channel vectors per image, pixel counts that are no multiple of
    four, and a 2x2 image that stays on the one-thread-per-output kernel."""
    n, c, h, w = shape
    x = cases.rng_for("gap_shape_%d_%d_%d_%d" % shape).integers(-128, 128, shape, dtype=np.int8)
    x[0, : c // 2] = 127
    y = ops.pooling_qs8_nhwc(ops.nchw_to_nhwc(dev(x)), "AVERAGE", h, h, 0)
    out = ops.nhwc_to_nchw(y).cpu().numpy()
    assert (out == oracle.pooling_qs8(x, "AVERAGE", h, h, 0)).all()


def test_qelemwise_golden(ops):
    """Same-shape operands and the broadcast forms of the reference's fixture catalogue
    ({2,3,4,5} with {1,3,1,1}: one value per channel of an NCHW tensor; with a scalar)."""
    for c in cases.qelem_catalogue():
        a, b = cases.qelem_inputs(c)
        s0, s1, s2 = c["scales"]
        if c["a"] == c["b"]:
            out = ops.qelemwise_qs8(c["mode"], dev(a), dev(b), s0, s1, s2)
        elif b.size == 1:
            out = ops.qelemwise_qs8_bcast(c["mode"], dev(a), dev(b), s0, s1, s2, 0, 1)
        else:
            assert b.size == a.shape[1]
            out = ops.qelemwise_qs8_bcast(c["mode"], dev(a), dev(b), s0, s1, s2, a.shape[1],
                                          int(np.prod(a.shape[2:])))
        G.check("qelemwise", c["name"], out.cpu().numpy(), a, b)


def test_typecvt_between_fp32_and_qsi8_follows_the_gi_rule(ops, oracle):
    r = cases.rng_for("typecvt_gi_gpu")
    for n in (16, 37, 4099):
        x = (r.standard_normal(n) * 60).astype(np.float32)
        ties = (np.arange(-130, 131, dtype=np.float32) + np.float32(0.5)) * np.float32(0.7)
        x[:min(n, ties.size)] = ties[:min(n, ties.size)]
        x[-3:] = np.float32([0.49999997 * 0.7, -0.49999997 * 0.7, 0.35])
        got = ops.typecvt_f32_qs8(dev(x), 0.3, 0.7).cpu().numpy()
        assert (got == oracle.typecvt_f32_qs8(x, 0.3, 0.7)).all()
        q = r.integers(-128, 128, n, dtype=np.int8)
        got = ops.typecvt_qs8_f32(dev(q), 0.3, 0.7).cpu().numpy()
        assert (got == oracle.typecvt_qs8_f32(q, 0.3, 0.7)).all()


def test_qrelu_matches_oracle(ops, oracle):
    a = cases.rng_for("qrelu").integers(-128, 128, (3, 5, 7, 11), dtype=np.int8)
    out = ops.qelemwise_qs8("QRELU", dev(a), None, 0.3, 1.0, 0.7).cpu().numpy()
    assert (out == oracle.qelemwise("QRELU", a, None, 0.3, 1.0, 0.7)).all()


def test_typecvt_golden(ops):
    for c in cases.typecvt_catalogue():
        x = cases.typecvt_input(c)
        out = ops.typecvt_qs32_qs8(dev(x), c["s_src"], c["s_dst"]).cpu().numpy()
        G.check("typecvt_qs32_qs8", c["name"], out, x)


def test_relayout_round_trip(ops):
    x = cases.rng_for("relayout").integers(-128, 128, (3, 37, 19, 23), dtype=np.int8)
    y = ops.nchw_to_nhwc(dev(x))
    assert (y.cpu().numpy() == x.transpose(0, 2, 3, 1)).all()
    assert (ops.nhwc_to_nchw(y).cpu().numpy() == x).all()


def test_bad_arguments_return_status_not_trap(ops):
    from megcc_b200._lib import MegccError
    p = ops.conv_param(1, 6, 8, 8, 4, 3, 3, 1, 1, 4, "RELU", 1, 1, 1)  # 6 % 4 != 0
    with pytest.raises(MegccError) as e:
        ops.pack_filter(p, torch.zeros(10, dtype=torch.int8, device="cuda"))
    assert e.value.status == 12
    p = ops.conv_param(1, 3, 8, 8, 8, 3, 3, 1, 1, 1, "RELU", 1, 1, 1)
    with pytest.raises(MegccError) as e:
        ops.conv_bias_qs8_nhwc(p, torch.zeros(192, dtype=torch.int8, device="cuda"),
                               torch.zeros(216, dtype=torch.int8, device="cuda"), None,
                               algo="umma")
    assert e.value.status == 6
