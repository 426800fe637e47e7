"""Random-init int8 networks of the benchmark configurations, as plain layer lists.

A network is a ``NetSpec``: the input description plus an ordered list of layer dicts
(``conv`` / ``pool`` / ``qelem``) holding the seeded weights and quantisation scales. The
same list is turned into a compiled model by ``NetSpec.to_graph`` and can be walked by any
other executor (the tests walk it with the CPU checker).

Weights are uniform int8 in [-127, 127]; filter scales are drawn uniform in [0.005, 0.02]
(one per tensor, or one per output channel with ``per_channel=True``); biases are uniform
int32 in [-1000, 1000]. Output scales are set analytically from the fan-in so that the
int8 activations neither vanish nor sit on the clamps.
"""
import math

import numpy as np

from .compiler import Graph


class NetSpec:
    def __init__(self, name, in_c, in_h, in_w, in_scale):
        self.name = name
        self.input = dict(name="data", c=in_c, h=in_h, w=in_w, scale=in_scale)
        self.layers = []
        self.shapes = {"data": (in_c, in_h, in_w)}
        self.scales = {"data": in_scale}
        self.rms = {"data": 74.0}
        self.output = None

    # -- construction helpers ---------------------------------------------------------
    def conv(self, rng, name, src, oc, k, stride, pad, act="RELU", groups=1,
             per_channel=False):
        ic, h, w = self.shapes[src]
        icpg = ic // groups
        flt = rng.integers(-127, 128, (oc, icpg, k, k), dtype=np.int8)
        if groups > 1:
            flt = flt.reshape(groups, oc // groups, icpg, k, k)
        bias = rng.integers(-1000, 1001, (oc,), dtype=np.int32)
        if per_channel:
            s_flt = rng.uniform(0.005, 0.02, oc).astype(np.float32)
            s_mean = float(s_flt.mean())
        else:
            s_flt = float(np.float32(rng.uniform(0.005, 0.02)))
            s_mean = s_flt
        fan_in = icpg * k * k
        acc_rms = self.rms[src] * 73.3 * math.sqrt(fan_in)
        s_dst = float(np.float32(acc_rms * self.scales[src] * s_mean / 40.0))
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        self.layers.append(dict(op="conv", name=name, src=src, flt=flt, bias=bias, stride=stride,
                                pad=pad, groups=groups, act=act, s_flt=s_flt, s_dst=s_dst))
        self.shapes[name] = (oc, oh, ow)
        self.scales[name] = s_dst
        self.rms[name] = 28.0 if act == "RELU" else 40.0
        return name

    def pool(self, name, src, mode, window, stride, pad):
        c, h, w = self.shapes[src]
        self.layers.append(dict(op="pool", name=name, src=src, mode=mode, window=window,
                                stride=stride, pad=pad))
        self.shapes[name] = (c, (h + 2 * pad - window) // stride + 1,
                             (w + 2 * pad - window) // stride + 1)
        self.scales[name] = self.scales[src]
        # a max over a window of post-ReLU values is larger, a mean smaller
        self.rms[name] = self.rms[src] * (2.2 if mode == "MAX" else 0.65)
        return name

    def qelem(self, name, mode, a, b):
        s_dst = float(np.float32(1.0 * max(self.scales[a], self.scales[b])))
        self.layers.append(dict(op="qelem", name=name, mode=mode, a=a, b=b, s_dst=s_dst))
        self.shapes[name] = self.shapes[a]
        self.scales[name] = s_dst
        self.rms[name] = 38.0
        return name

    # -- derived quantities -------------------------------------------------------------
    def macs_per_image(self):
        total = 0
        for l in self.layers:
            if l["op"] == "conv":
                oc, oh, ow = self.shapes[l["name"]]
                ic = self.shapes[l["src"]][0]
                k = l["flt"].shape[-1]
                total += oc * oh * ow * (ic // l["groups"]) * k * k
        return total

    def to_graph(self, nchw44=False):
        """nchw44: build the model as MegCC's --enable_nchw44 would hand it over: filters in
        the NCHW44 layouts (first-layer form on the NCHW input, dense, channel-wise), outputs
        handed back as [N, C/4, H, W, 4]. Operators whose channel counts are not multiples
        of 4 (other than the first layer's input) have no NCHW44 form."""
        g = Graph(self.name + ("_nchw44" if nchw44 else ""))
        # an NCHW44 model's input is NCHW44 itself unless its channels do not fill blocks of
        # four (the image input of a first layer)
        in44 = nchw44 and self.input["c"] % 4 == 0
        ids = {"data": (g.input_nchw44 if in44 else g.input)(
            "data", self.input["c"], self.input["h"], self.input["w"], self.input["scale"])}
        for l in self.layers:
            if l["op"] == "conv":
                pc = np.ndim(l["s_flt"]) > 0
                s_flt = float(np.mean(l["s_flt"])) if pc else l["s_flt"]
                if nchw44:
                    form = ("first_layer" if l["src"] == "data" and not in44
                            else "dense" if l["groups"] == 1 else "channel_wise")
                    ids[l["name"]] = g.conv_bias_nchw44(
                        l["name"], ids[l["src"]], filter_to_nchw44(l["flt"], form), l["bias"],
                        l["stride"], l["pad"], s_flt, l["s_dst"], form, l["act"],
                        l["s_flt"] if pc else None)
                    continue
                ids[l["name"]] = g.conv_bias(
                    l["name"], ids[l["src"]], l["flt"], l["bias"], l["stride"], l["pad"],
                    s_flt, l["s_dst"], l["act"], l["groups"], l["s_flt"] if pc else None)
            elif l["op"] == "pool":
                ids[l["name"]] = g.pooling(l["name"], ids[l["src"]], l["mode"], l["window"],
                                           l["stride"], l["pad"])
            else:
                ids[l["name"]] = g.qelemwise(l["name"], l["mode"], ids[l["a"]],
                                             None if l["b"] is None else ids[l["b"]], l["s_dst"])
        g.mark_output(ids[self.output])
        return g


def filter_to_nchw44(flt, form):
    """OIHW or [G, 1, 1, KH, KW] int8 -> the NCHW44 filter layouts MegEngine's layout
    transform produces (index formulas: compiler/lib/KernelGen/BareMetal/ConvKernel.cpp
    :48-62,88-101): dense [OC/4, IC/4, KH, KW, 4 ic, 4 oc], channel_wise
    [G/4, 1, 1, KH, KW, 4], first_layer [OC/4, KH, KW, IC, 4 oc]."""
    flt = np.asarray(flt)
    kh, kw = flt.shape[-2:]
    if form == "dense":
        oc, ic = flt.shape[:2]
        return np.ascontiguousarray(
            flt.reshape(oc // 4, 4, ic // 4, 4, kh, kw).transpose(0, 2, 4, 5, 3, 1))
    if form == "channel_wise":
        g = flt.shape[0]
        return np.ascontiguousarray(
            flt.reshape(g // 4, 4, kh, kw).transpose(0, 2, 3, 1).reshape(g // 4, 1, 1, kh, kw, 4))
    if form == "first_layer":
        oc, ic = flt.shape[:2]
        return np.ascontiguousarray(flt.reshape(oc // 4, 4, ic, kh, kw).transpose(0, 3, 4, 2, 1))
    raise ValueError(f"unknown NCHW44 filter form {form!r}")


def resnet18(seed=0, classes=1000, hw=224, per_channel=False):
    """ResNet-18: 7x7/2 stem, 3x3/2 max-pool, four stages of two basic blocks
    (64/128/256/512 channels, 1x1/2 projection on the first block of stages 2-4), global
    average pool, FC as a 1x1 ConvBias. Residual adds are QFUSE_ADD_RELU."""
    rng = np.random.Generator(np.random.PCG64(0x5EED1800 + seed))
    n = NetSpec("resnet18_int8", 3, hw, hw, 0.02)
    x = n.conv(rng, "stem", "data", 64, 7, 2, 3, per_channel=per_channel)
    x = n.pool("maxpool", x, "MAX", 3, 2, 1)
    for stage, ch in enumerate((64, 128, 256, 512)):
        for block in range(2):
            stride = 2 if (stage > 0 and block == 0) else 1
            p = f"s{stage + 1}b{block}"
            y = n.conv(rng, p + "_conv1", x, ch, 3, stride, 1, per_channel=per_channel)
            y = n.conv(rng, p + "_conv2", y, ch, 3, 1, 1, act="IDENTITY", per_channel=per_channel)
            sc = x
            if stride != 1:
                sc = n.conv(rng, p + "_proj", x, ch, 1, stride, 0, act="IDENTITY",
                            per_channel=per_channel)
            x = n.qelem(p + "_add", "QFUSE_ADD_RELU", y, sc)
    c, h, w = n.shapes[x]
    x = n.pool("gap", x, "AVERAGE", h, h, 0)
    x = n.conv(rng, "fc", x, classes, 1, 1, 0, act="IDENTITY", per_channel=per_channel)
    n.output = x
    return n


def mobilenet_v1(seed=0, classes=1000, hw=224, per_channel=False):
    """MobileNetV1 width 1.0: 3x3/2 stem to 32 channels, then 13 depthwise-3x3 +
    pointwise-1x1 blocks (64,128,128,256,256,512x6,1024,1024; stride 2 at blocks 2,4,6,12),
    global average pool, FC as a 1x1 ConvBias. ReLU6 is RELU plus the int8 clamp."""
    rng = np.random.Generator(np.random.PCG64(0x5EED3100 + seed))
    n = NetSpec("mobilenet_v1_int8", 3, hw, hw, 0.02)
    x = n.conv(rng, "stem", "data", 32, 3, 2, 1, per_channel=per_channel)
    chans = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
    for i, oc in enumerate(chans, start=1):
        stride = 2 if i in (2, 4, 6, 12) else 1
        ic = n.shapes[x][0]
        x = n.conv(rng, f"dw{i}", x, ic, 3, stride, 1, groups=ic, per_channel=per_channel)
        x = n.conv(rng, f"pw{i}", x, oc, 1, 1, 0, per_channel=per_channel)
    c, h, w = n.shapes[x]
    x = n.pool("gap", x, "AVERAGE", h, h, 0)
    x = n.conv(rng, "fc", x, classes, 1, 1, 0, act="IDENTITY", per_channel=per_channel)
    n.output = x
    return n


def single_conv(n_unused=None, ic=64, oc=64, hw=56, k=3, stride=1, pad=1, seed=0,
                s_src=0.05, s_flt=0.01, s_dst=0.1, act="RELU"):
    """The single-operator configuration: one qint8 ConvBias with the given scales."""
    rng = np.random.Generator(np.random.PCG64(0x5EED0100 + seed))
    n = NetSpec("conv_bias_qs8", ic, hw, hw, s_src)
    flt = rng.integers(-127, 128, (oc, ic, k, k), dtype=np.int8)
    bias = rng.integers(-1000, 1001, (oc,), dtype=np.int32)
    n.layers.append(dict(op="conv", name="conv", src="data", flt=flt, bias=bias, stride=stride,
                         pad=pad, groups=1, act=act, s_flt=s_flt, s_dst=s_dst))
    n.shapes["conv"] = (oc, (hw + 2 * pad - k) // stride + 1, (hw + 2 * pad - k) // stride + 1)
    n.scales["conv"] = s_dst
    n.output = "conv"
    return n


# ----------------------------------------------------------------------------------------
# fp32 detector (YOLOX-style)
# ----------------------------------------------------------------------------------------
def _np_conv(x, flt, stride, pad):
    """Plain numpy cross-correlation (NCHW, OIHW) for the small calibration pass below."""
    n, c, h, w = x.shape
    oc, _, k, _ = flt.shape
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    win = np.lib.stride_tricks.sliding_window_view(xp, (k, k), axis=(2, 3))[:, :, ::stride, ::stride]
    return np.einsum("nchwij,ocij->nohw", win, flt, optimize=True).astype(np.float32)


def _np_act(act, x):
    if act == "SILU":
        return (x / (1 + np.exp(-x))).astype(np.float32)
    if act == "SIGMOID":
        return (1 / (1 + np.exp(-x))).astype(np.float32)
    if act == "RELU":
        return np.maximum(x, 0)
    return x


class F32Spec:
    """An fp32 network as an ordered list of layer dicts over named tensors (NCHW shapes):
    ``focus`` / ``conv`` / ``concat`` / ``resize`` / ``pool`` / ``elem``. ``outputs`` lists the
    model outputs. ``to_graph`` compiles it; oracle/netwalk.py walks it on the CPU.

    Random weights are calibrated while the network is described: a 256 x 256 image runs along
    in numpy, and every ConvBias filter is rescaled so that its pre-activation output has a
    standard deviation of CALIB_STD on it. With SiLU no fixed initialisation gain keeps a
    60-layer network's activations away from zero or overflow, hence the calibration. The
    target is 0.25, not 1: a random SiLU network with unit-variance pre-activations is chaotic
    (scaling every ConvBias output by 1 - 1e-7 moved the outputs of this detector by 2e-3 in
    float64 arithmetic), so that no two fp32 implementations, CPU ones included, agree on it
    to 1e-4. At 0.25 the network is contractive, as trained networks are: the same
    perturbation moves the outputs by 5e-6 and the activation statistics no longer depend on
    the image size, while all values stay of order 0.1 to 1."""

    CALIB_HW = 256
    CALIB_STD = 0.25

    def __init__(self, name, in_c, in_h, in_w, seed=0):
        self.name = name
        self.input = dict(name="data", c=in_c, h=in_h, w=in_w)
        self.layers = []
        self.shapes = {"data": (in_c, in_h, in_w)}
        self.outputs = []
        cal = np.random.Generator(np.random.PCG64(0x5EEDCA1 + seed))
        self.cal = {"data": cal.uniform(0, 1, (1, in_c, self.CALIB_HW, self.CALIB_HW)).astype(np.float32)}

    def focus(self, name, src, c_out):
        c, h, w = self.shapes[src]
        self.layers.append(dict(op="focus", name=name, src=src, c_out=c_out))
        self.shapes[name] = (c_out, h // 2, w // 2)
        x = self.cal[src]
        parts = [x[:, :, 0::2, 0::2], x[:, :, 1::2, 0::2], x[:, :, 0::2, 1::2], x[:, :, 1::2, 1::2]]
        out = np.concatenate(parts, axis=1)
        pad = np.zeros((out.shape[0], c_out - out.shape[1]) + out.shape[2:], np.float32)
        self.cal[name] = np.concatenate([out, pad], axis=1)
        return name

    def conv(self, rng, name, src, oc, k, stride, act="SILU", z=None, real_ic=None):
        """ConvBias with random weights (batch norm folded into the bias); real_ic: input
        channels that carry data (the rest are zero padding and get zero weights)."""
        ic, h, w = self.shapes[src]
        flt = rng.standard_normal((oc, ic, k, k)).astype(np.float32)
        if real_ic is not None:
            flt[:, real_ic:] = 0
        pad = k // 2
        pre = _np_conv(self.cal[src], flt, stride, pad)
        gain = self.CALIB_STD / max(float(pre.std()), 1e-6)
        flt = (flt * gain).astype(np.float32)
        bias = rng.uniform(-0.1, 0.1, oc).astype(np.float32)
        out = _np_act(act, pre * gain + bias.reshape(1, -1, 1, 1))
        if z is not None:
            out = out + self.cal[z]
        self.cal[name] = out.astype(np.float32)
        self.layers.append(dict(op="conv", name=name, src=src, flt=flt, bias=bias, stride=stride,
                                pad=pad, act=act, z=z))
        self.shapes[name] = (oc, (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1)
        return name

    def concat(self, name, srcs):
        c = sum(self.shapes[s][0] for s in srcs)
        self.layers.append(dict(op="concat", name=name, srcs=list(srcs)))
        self.shapes[name] = (c,) + self.shapes[srcs[0]][1:]
        self.cal[name] = np.concatenate([self.cal[s] for s in srcs], axis=1)
        return name

    def resize_like(self, name, src, like):
        """Nearest-neighbour resize of src to the spatial extent of the tensor `like`."""
        oh, ow = self.shapes[like][1:]
        self.layers.append(dict(op="resize", name=name, src=src, oh=oh, ow=ow))
        self.shapes[name] = (self.shapes[src][0], oh, ow)
        x, ch, cw = self.cal[src], self.cal[like].shape[2], self.cal[like].shape[3]
        iy = np.minimum((np.arange(ch) * x.shape[2]) // ch, x.shape[2] - 1)
        ix = np.minimum((np.arange(cw) * x.shape[3]) // cw, x.shape[3] - 1)
        self.cal[name] = x[:, :, iy][:, :, :, ix]
        return name

    def pool(self, name, src, mode, window, stride, pad):
        assert mode == "MAX"
        c, h, w = self.shapes[src]
        self.layers.append(dict(op="pool", name=name, src=src, mode=mode, window=window,
                                stride=stride, pad=pad))
        self.shapes[name] = (c, (h + 2 * pad - window) // stride + 1,
                             (w + 2 * pad - window) // stride + 1)
        x = np.pad(self.cal[src], ((0, 0), (0, 0), (pad, pad), (pad, pad)), constant_values=-np.inf)
        win = np.lib.stride_tricks.sliding_window_view(x, (window, window), axis=(2, 3))
        self.cal[name] = win[:, :, ::stride, ::stride].max(axis=(4, 5)).astype(np.float32)
        return name

    def elem(self, name, mode, a, b=None):
        self.layers.append(dict(op="elem", name=name, mode=mode, a=a, b=b))
        self.shapes[name] = self.shapes[a]
        x = self.cal[a]
        self.cal[name] = _np_act(mode, x) if b is None else {
            "ADD": x + self.cal[b], "MUL": x * self.cal[b]}.get(mode, x)
        return name

    def macs_per_image(self):
        """Multiply-accumulates of the ConvBias layers, zero padding channels not counted."""
        total = 0
        for l in self.layers:
            if l["op"] == "conv":
                oc, oh, ow = self.shapes[l["name"]]
                real_ic = int((np.abs(l["flt"]).sum(axis=(0, 2, 3)) > 0).sum())
                total += oc * oh * ow * real_ic * l["flt"].shape[2] * l["flt"].shape[3]
        return total

    def to_graph(self):
        g = Graph(self.name)
        ids = {"data": g.input_f32("data", self.input["c"], self.input["h"], self.input["w"])}
        for l in self.layers:
            op = l["op"]
            if op == "focus":
                ids[l["name"]] = g.focus(l["name"], ids[l["src"]], l["c_out"])
            elif op == "conv":
                ids[l["name"]] = g.conv_f32(l["name"], ids[l["src"]], l["flt"], l["bias"],
                                            l["stride"], l["pad"], l["act"],
                                            z=None if l["z"] is None else ids[l["z"]])
            elif op == "concat":
                ids[l["name"]] = g.concat(l["name"], [ids[s] for s in l["srcs"]])
            elif op == "resize":
                ids[l["name"]] = g.resize_nearest(l["name"], ids[l["src"]], l["oh"], l["ow"])
            elif op == "pool":
                ids[l["name"]] = g.pooling(l["name"], ids[l["src"]], l["mode"], l["window"],
                                           l["stride"], l["pad"])
            else:
                ids[l["name"]] = g.elemwise_f32(l["name"], l["mode"], ids[l["a"]],
                                                None if l["b"] is None else ids[l["b"]])
        for o in self.outputs:
            g.mark_output(ids[o])
        return g


def yolox_s(seed=0, hw=640, classes=80, width=0.5, depth=0.33):
    """YOLOX-s-style detector: Focus stem, CSPDarknet backbone (width 0.5, depth 0.33) with
    SiLU and an SPP block of 5/9/13 max-pools, PAFPN neck with nearest 2x upsampling and
    channel concats, decoupled heads at strides 8/16/32 whose outputs are
    [box regression (4), sigmoid(objectness) (1), sigmoid(class scores)] per position.
    Batch norm is folded into the ConvBias biases; weights are random, calibrated to unit-scale
    activations (see F32Spec).
    The Focus output is padded from 12 to 16 channels (zeros, with zero filter weights) so
    that the stem's ConvBias reads whole 64-byte rows."""
    rng = np.random.Generator(np.random.PCG64(0x5EED5000 + seed))
    n = F32Spec("yolox_s_f32", 3, hw, hw, seed)
    ch = lambda c: int(c * width)
    nb = max(round(3 * depth), 1)

    def csp(prefix, x, out_c, blocks, shortcut):
        hidden = out_c // 2
        a = n.conv(rng, prefix + "_conv1", x, hidden, 1, 1)
        b = n.conv(rng, prefix + "_conv2", x, hidden, 1, 1)
        for i in range(blocks):
            y = n.conv(rng, f"{prefix}_m{i}_conv1", a, hidden, 1, 1)
            a = n.conv(rng, f"{prefix}_m{i}_conv2", y, hidden, 3, 1, z=a if shortcut else None)
        cat = n.concat(prefix + "_cat", [a, b])
        return n.conv(rng, prefix + "_conv3", cat, out_c, 1, 1)

    x = n.focus("focus", "data", 16)
    x = n.conv(rng, "stem", x, ch(64), 3, 1, real_ic=12)
    x = n.conv(rng, "dark2_conv", x, ch(128), 3, 2)
    x = csp("dark2_csp", x, ch(128), nb, True)
    x = n.conv(rng, "dark3_conv", x, ch(256), 3, 2)
    c3 = csp("dark3_csp", x, ch(256), nb * 3, True)
    x = n.conv(rng, "dark4_conv", c3, ch(512), 3, 2)
    c4 = csp("dark4_csp", x, ch(512), nb * 3, True)
    x = n.conv(rng, "dark5_conv", c4, ch(1024), 3, 2)
    s = n.conv(rng, "spp_conv1", x, ch(1024) // 2, 1, 1)
    pools = [n.pool(f"spp_pool{k}", s, "MAX", k, 1, k // 2) for k in (5, 9, 13)]
    x = n.concat("spp_cat", [s] + pools)
    x = n.conv(rng, "spp_conv2", x, ch(1024), 1, 1)
    c5 = csp("dark5_csp", x, ch(1024), nb, False)

    # PAFPN
    fpn0 = n.conv(rng, "lateral_conv0", c5, ch(512), 1, 1)
    up = n.resize_like("up0", fpn0, c4)
    x = n.concat("fpn_cat0", [up, c4])
    x = csp("c3_p4", x, ch(512), nb, False)
    fpn1 = n.conv(rng, "reduce_conv1", x, ch(256), 1, 1)
    up = n.resize_like("up1", fpn1, c3)
    x = n.concat("fpn_cat1", [up, c3])
    p3 = csp("c3_p3", x, ch(256), nb, False)
    d = n.conv(rng, "bu_conv2", p3, ch(256), 3, 2)
    x = n.concat("pan_cat1", [d, fpn1])
    p4 = csp("c3_n3", x, ch(512), nb, False)
    d = n.conv(rng, "bu_conv1", p4, ch(512), 3, 2)
    x = n.concat("pan_cat0", [d, fpn0])
    p5 = csp("c3_n4", x, ch(1024), nb, False)

    # decoupled heads
    hc = ch(256)
    for lvl, feat in enumerate((p3, p4, p5)):
        t = n.conv(rng, f"head{lvl}_stem", feat, hc, 1, 1)
        c = n.conv(rng, f"head{lvl}_cls0", t, hc, 3, 1)
        c = n.conv(rng, f"head{lvl}_cls1", c, hc, 3, 1)
        r = n.conv(rng, f"head{lvl}_reg0", t, hc, 3, 1)
        r = n.conv(rng, f"head{lvl}_reg1", r, hc, 3, 1)
        cls = n.conv(rng, f"head{lvl}_cls_pred", c, classes, 1, 1, act="SIGMOID")
        reg = n.conv(rng, f"head{lvl}_reg_pred", r, 4, 1, 1, act="IDENTITY")
        obj = n.conv(rng, f"head{lvl}_obj_pred", r, 1, 1, 1, act="SIGMOID")
        n.outputs.append(n.concat(f"head{lvl}_out", [reg, obj, cls]))
    return n
