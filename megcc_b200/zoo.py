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

    def to_graph(self):
        g = Graph(self.name)
        ids = {"data": g.input("data", self.input["c"], self.input["h"], self.input["w"],
                               self.input["scale"])}
        for l in self.layers:
            if l["op"] == "conv":
                pc = np.ndim(l["s_flt"]) > 0
                ids[l["name"]] = g.conv_bias(
                    l["name"], ids[l["src"]], l["flt"], l["bias"], l["stride"], l["pad"],
                    float(np.mean(l["s_flt"])) if pc else l["s_flt"], l["s_dst"], l["act"],
                    l["groups"], l["s_flt"] if pc else None)
            elif l["op"] == "pool":
                ids[l["name"]] = g.pooling(l["name"], ids[l["src"]], l["mode"], l["window"],
                                           l["stride"], l["pad"])
            else:
                ids[l["name"]] = g.qelemwise(l["name"], l["mode"], ids[l["a"]],
                                             None if l["b"] is None else ids[l["b"]], l["s_dst"])
        g.mark_output(ids[self.output])
        return g


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
