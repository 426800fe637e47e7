"""Seeded test cases shared by the golden-vector generator and the parity tests.

The shapes, value ranges and scales restate the fixture catalogue of the reference's own
kernel unit tests (compiler/test/kernel/opr/naive/conv.cpp:53-131, pool.cpp:41-67,
elemwise_multitype.cpp:33-62, typecvt.cpp:39-70, compiler/test/kernel/opr/arm/conv.cpp:453-584)
plus the single-op benchmark configuration. Inputs come from numpy's PCG64 with a seed
derived from the case name, so a case is reproducible from its name alone.
"""
import zlib

import numpy as np


def rng_for(name):
    return np.random.Generator(np.random.PCG64(0x5EED0000 + zlib.crc32(name.encode())))


def conv_inputs(c):
    r = rng_for(c["name"])
    lo, hi = c["range"]
    g = c["groups"]
    src = r.integers(lo, hi + 1, (c["n"], c["ic"], c["h"], c["w"]), dtype=np.int8)
    fshape = ((c["oc"], c["ic"], c["k"], c["k"]) if g == 1
              else (g, c["oc"] // g, c["ic"] // g, c["k"], c["k"]))
    flt = r.integers(max(lo, -127), hi + 1, fshape, dtype=np.int8)
    blo, bhi = c.get("bias_range", c["range"])
    bias = r.integers(blo, bhi + 1, (c["oc"],), dtype=np.int32) if c.get("bias", True) else None
    return src, flt, bias


def _conv(name, n, ic, oc, h, w, k, stride, pad, groups, act, rng, scales, **kw):
    d = dict(name=name, n=n, ic=ic, oc=oc, h=h, w=w, k=k, stride=stride, pad=pad,
             groups=groups, act=act, range=rng, scales=scales)
    d.update(kw)
    return d


def conv_naive_catalogue():
    """TEST(NAIVE, ConvBiasNCHWQS8) + ConvBiasNCHWQS8Overflow."""
    out = []
    for act in ("IDENTITY", "RELU"):
        for oc in (1, 4):
            for ic in (1, 4):
                for hw in (7, 12):
                    for k in (1, 3):
                        for pad in sorted({0, k // 2}):
                            for stride in (1, 2):
                                base = f"naive_{act}_oc{oc}_ic{ic}_hw{hw}_k{k}_p{pad}_s{stride}"
                                out.append(_conv(base + "_dense", 2, ic, oc, hw, hw, k, stride,
                                                 pad, 1, act, (-3, 3), (1.0, 2.0, 4.0)))
                                if ic == oc:
                                    out.append(_conv(base + "_dw", 2, ic, oc, hw, hw, k, stride,
                                                     pad, oc, act, (-3, 3), (1.0, 2.0, 4.0)))
    out.append(_conv("overflow_pos", 1, 20, 20, 10, 10, 3, 1, 0, 1, "IDENTITY", (30, 50),
                     (1.0, 2.0, 4.0)))
    out.append(_conv("overflow_neg", 1, 20, 20, 10, 10, 3, 1, 0, 1, "IDENTITY", (-50, -30),
                     (1.0, 2.0, 4.0)))
    return out


def conv_im2col_catalogue():
    """Shape family of the Arm ConvBiasIm2colDot test, run here through the x86 kernel:
    values U[-50,50], scales 2.5 * 2.5 -> 40.25, RELU / IDENTITY / H_SWISH."""
    out = []
    sc = (2.5, 2.5, 40.25)
    for act in ("IDENTITY", "RELU", "H_SWISH"):
        for n, oc, ic in ((1, 3, 4), (3, 7, 21), (1, 21, 4)):
            for stride in (1, 2, 3):
                for k in (2, 3, 5):
                    for hw in (7, 13, 23):
                        if hw < k:
                            continue
                        name = f"im2col_{act}_n{n}_oc{oc}_ic{ic}_s{stride}_k{k}_hw{hw}"
                        out.append(_conv(name, n, ic, oc, hw, hw, k, stride, k // 2, 1, act,
                                         (-50, 50), sc))
    for act in ("IDENTITY", "RELU"):
        out.append(_conv(f"im2col_{act}_22x33", 1, 21, 7, 22, 33, 3, 1, 1, 1, act, (-50, 50),
                         sc))
        for g, icpg in ((3, 4), (7, 9)):
            out.append(_conv(f"im2col_{act}_g{g}_icpg{icpg}", 2, g * icpg, g * 5, 13, 13, 3, 1,
                             1, g, act, (-50, 50), sc))
    return out


def conv_cfg1(dst_scale):
    """Single-op benchmark configuration: N=1, IC=OC=64, 56x56, 3x3 s1 p1, fused ReLU."""
    return _conv(f"cfg1_dst{dst_scale}", 1, 64, 64, 56, 56, 3, 1, 1, 1, "RELU", (-128, 127),
                 (0.05, 0.01, dst_scale), bias_range=(-1000, 1000))


def conv_model_shapes():
    """One small-batch instance of every distinct conv shape of the two int8 models."""
    out = []
    sc = (0.05, 0.01, 2.0)
    r18 = [(3, 64, 224, 7, 2, 3), (64, 64, 56, 3, 1, 1), (64, 128, 56, 3, 2, 1),
           (64, 128, 56, 1, 2, 0), (128, 128, 28, 3, 1, 1), (128, 256, 28, 3, 2, 1),
           (128, 256, 28, 1, 2, 0), (256, 256, 14, 3, 1, 1), (256, 512, 14, 3, 2, 1),
           (256, 512, 14, 1, 2, 0), (512, 512, 7, 3, 1, 1), (512, 1000, 1, 1, 1, 0)]
    for ic, oc, hw, k, s, p in r18:
        out.append(_conv(f"r18_ic{ic}_oc{oc}_hw{hw}_k{k}_s{s}", 2, ic, oc, hw, hw, k, s, p, 1,
                         "RELU", (-128, 127), sc, bias_range=(-1000, 1000)))
    mb = [(3, 32, 224, 3, 2, 1, 1), (32, 32, 112, 3, 1, 1, 32), (32, 64, 112, 1, 1, 0, 1),
          (64, 64, 112, 3, 2, 1, 64), (128, 128, 56, 3, 1, 1, 128), (256, 256, 28, 3, 2, 1, 256),
          (512, 512, 14, 3, 1, 1, 512), (512, 1024, 7, 1, 1, 0, 1), (1024, 1024, 7, 3, 1, 1, 1024),
          (1024, 1000, 1, 1, 1, 0, 1)]
    for ic, oc, hw, k, s, p, g in mb:
        out.append(_conv(f"mbv1_ic{ic}_oc{oc}_hw{hw}_k{k}_s{s}_g{g}", 1, ic, oc, hw, hw, k, s, p,
                         g, "RELU", (-128, 127), sc, bias_range=(-1000, 1000)))
    return out


def conv_nchw44_catalogue():
    """ConvBias as a model compiled with --enable_nchw44 carries it: dense, channel-wise and
    first-layer (NCHW input) filters, each at a toy size and at one that reaches the
    tensor-core kernels. `form` names the filter layout; inputs are built in NCHW / OIHW by
    conv_inputs and converted by conv_nchw44_inputs."""
    out = []
    forms = [
        ("dense", 1, 1, 0, "RELU", True), ("dense", 3, 1, 1, "RELU", True),
        ("dense", 3, 2, 1, "IDENTITY", True), ("dense", 3, 1, 1, "H_SWISH", False),
        ("channel_wise", 3, 1, 1, "RELU", True), ("channel_wise", 3, 2, 1, "IDENTITY", True),
        ("channel_wise", 5, 1, 2, "H_SWISH", True),
        ("first_layer", 3, 2, 1, "RELU", True), ("first_layer", 7, 2, 3, "RELU", True),
        ("first_layer", 3, 1, 1, "IDENTITY", False),
    ]
    for form, k, stride, pad, act, bias in forms:
        for size in ("toy", "wide"):
            if form == "first_layer":
                n, ic, oc, hw = (2, 3, 8, 13) if size == "toy" else (4, 3, 32, 64)
            elif form == "dense":
                n, ic, oc, hw = (2, 8, 12, 9) if size == "toy" else (4, 64, 128, 28)
            else:
                n, ic, oc, hw = (2, 8, 8, 9) if size == "toy" else (4, 96, 96, 28)
            groups = ic if form == "channel_wise" else 1
            name = f"nchw44_{form}_{size}_k{k}_s{stride}_p{pad}_{act}_b{int(bias)}"
            out.append(_conv(name, n, ic, oc, hw, hw + 2, k, stride, pad, groups, act, (-128, 127),
                             (0.05, 0.01, 0.3 if k > 1 else 0.1), bias=bias,
                             bias_range=(-3000, 3000), form=form))
    return out


def conv_nchw44_inputs(c, O):
    """(src, flt44, bias) in the layouts the NCHW44 model holds; O is the oracle module, whose
    layout helpers restate the reference's index formulas."""
    src, flt, bias = conv_inputs(c)
    if c["form"] != "first_layer":
        src = O.nchw_to_nchw44(src)
    return src, O.filter_to_nchw44(flt, c["form"]), bias


def nchw44_block_spec(seed=0):
    """A block whose input and output are both spatial NCHW44 tensors: dense 3x3, channel-wise
    3x3 / 2, dense 1x1, and a residual add around a second dense 3x3."""
    from megcc_b200 import zoo
    rng = np.random.Generator(np.random.PCG64(0x44440000 + seed))
    n = zoo.NetSpec("nchw44_block", 16, 30, 34, 0.05)
    a = n.conv(rng, "c1", "data", 64, 3, 1, 1)
    b = n.conv(rng, "dw", a, 64, 3, 2, 1, groups=64)
    c = n.conv(rng, "pw", b, 96, 1, 1, 0)
    d = n.conv(rng, "c2", c, 96, 3, 1, 1, act="IDENTITY")
    n.output = n.qelem("add", "QFUSE_ADD_RELU", d, c)
    return n


def pool_catalogue():
    """TEST(NAIVE, PoolingNCHWQuant): values U[-127,127], scale 0.7 both sides."""
    out = []
    for mode in ("MAX", "AVERAGE", "AVERAGE_COUNT_EXCLUDE_PADDING"):
        for window in (2, 3, 5):
            for stride in sorted({1, window}):
                for pad in sorted({0, window // 2}):
                    for n in (1, 3):
                        for c in (1, 3):
                            for hw in (5, 23):
                                out.append(dict(
                                    name=f"pool_{mode}_w{window}_s{stride}_p{pad}_n{n}_c{c}_hw{hw}",
                                    mode=mode, window=window, stride=stride, pad=pad, n=n, c=c,
                                    hw=hw))
    out.append(dict(name="pool_r18_max", mode="MAX", window=3, stride=2, pad=1, n=2, c=64, hw=112))
    out.append(dict(name="pool_r18_gap", mode="AVERAGE", window=7, stride=7, pad=0, n=2, c=512,
                    hw=7))
    return out


def pool_input(c):
    return rng_for(c["name"]).integers(-127, 128, (c["n"], c["c"], c["hw"], c["hw"]),
                                       dtype=np.int8)


def qelem_catalogue():
    """TEST(NAIVE, ElementwiseMultitypeBinary), qint8 operands: scales 1, 2 -> 3."""
    out = []
    for mode in ("QADD", "QFUSE_ADD_RELU", "QMUL"):
        for a, b in (((1,), (1,)), ((1, 10), (1, 10)), ((2, 3, 4, 5), (2, 3, 4, 5)),
                     ((2, 3, 4, 5), (1, 3, 1, 1)), ((2, 3, 4, 5), (1,))):
            out.append(dict(name=f"qelem_{mode}_{'x'.join(map(str, a))}_{'x'.join(map(str, b))}",
                            mode=mode, a=a, b=b, scales=(1.0, 2.0, 3.0)))
        out.append(dict(name=f"qelem_{mode}_residual", mode=mode, a=(2, 64, 56, 56),
                        b=(2, 64, 56, 56), scales=(0.031, 0.047, 0.052)))
    return out


def qelem_inputs(c):
    r = rng_for(c["name"])
    return (r.integers(-128, 128, c["a"], dtype=np.int8),
            r.integers(-128, 128, c["b"], dtype=np.int8))


def typecvt_catalogue():
    """qsi32 -> qsi8 part of TEST(NAIVE, TypecvtQuant) plus the GEMM requant scale."""
    out = []
    for shape in ((2, 10), (2, 10, 4), (3, 4, 5, 6)):
        for s_src, s_dst in ((0.3, 0.7), (0.3, 0.5)):
            out.append(dict(name=f"cvt_{'x'.join(map(str, shape))}_{s_src}_{s_dst}", shape=shape,
                            range=(-300, 300), s_src=s_src, s_dst=s_dst))
    out.append(dict(name="cvt_gemm_requant", shape=(64, 100), range=(-130000, 130000), s_src=0.002,
                    s_dst=1.0))
    return out


def typecvt_input(c):
    lo, hi = c["range"]
    return rng_for(c["name"]).integers(lo, hi + 1, c["shape"], dtype=np.int32)


def f32_conv_catalogue():
    """fp32 ConvBias cases in the nonlinearities the reference's own fp32 kernels take."""
    out = []
    for k, stride, pad, act, bias in ((3, 1, 1, "IDENTITY", True), (3, 2, 1, "IDENTITY", True),
                                      (1, 1, 0, "IDENTITY", True), (3, 1, 1, "RELU", True),
                                      (1, 1, 0, "SIGMOID", True), (3, 1, 1, "IDENTITY", False)):
        for n, ic, oc, h, w in ((2, 32, 64, 40, 40), (2, 64, 48, 24, 20), (3, 16, 32, 48, 48)):
            out.append(dict(name=f"f32conv_k{k}_s{stride}_p{pad}_{act}_b{int(bias)}_{n}x{ic}x{oc}x{h}x{w}",
                            k=k, stride=stride, pad=pad, act=act, bias=bias, n=n, ic=ic, oc=oc,
                            h=h, w=w))
    return out


def f32_conv_inputs(c):
    r = rng_for(c["name"])
    src = r.standard_normal((c["n"], c["ic"], c["h"], c["w"])).astype(np.float32)
    flt = (r.standard_normal((c["oc"], c["ic"], c["k"], c["k"]))
           / np.sqrt(c["ic"] * c["k"] * c["k"])).astype(np.float32)
    bias = r.standard_normal(c["oc"]).astype(np.float32) if c["bias"] else None
    return src, flt, bias


def f32_matmul_catalogue():
    return [dict(name=f"f32mm_{m}x{n}x{k}", m=m, n=n, k=k)
            for m, n, k in ((512, 512, 512), (300, 72, 640), (64, 15, 48), (1024, 1000, 2048))]


def f32_matmul_inputs(c):
    r = rng_for(c["name"])
    return (r.standard_normal((c["m"], c["k"])).astype(np.float32),
            r.standard_normal((c["k"], c["n"])).astype(np.float32))
