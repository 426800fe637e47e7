"""Launches the bandwidth-bound kernels of the hot path at the sizes they have in the bench
workloads (ResNet-18 at batch 256, MobileNetV1 at batch 64): the 3x3/2 max-pool of the stem,
the global average pool, depthwise 3x3 at stride 1 and 2, and the stand-alone residual add.
Once each, then ten times each between two events; prints the mean time of the ten and the
algorithmic bandwidth (each input read once, the output written once).

Meant to be run under a profiler, capturing the first launches:

    ncu --set full --clock-control none -k regex:"pooling|conv_dw|qelemwise" -c 5 \
        python -m megcc_b200.profile_ops
"""
import numpy as np
import torch

from . import ops


def main():
    rng = np.random.default_rng(0)
    dev = lambda a: torch.from_numpy(a).cuda()
    i8 = lambda *shape: dev(rng.integers(-128, 128, shape, dtype=np.int8))
    cases = []

    x = i8(256, 112, 112, 64)
    cases.append(("max_pool_3x3s2_64ch_112", lambda: ops.pooling_qs8_nhwc(x, "MAX", 3, 2, 1),
                  x.numel() * 1.25))
    g = i8(256, 7, 7, 512)
    cases.append(("global_avg_pool_512ch_7", lambda: ops.pooling_qs8_nhwc(g, "AVERAGE", 7, 7, 0),
                  g.numel() * (1 + 1 / 49)))
    for name, c, hw, stride in (("depthwise_3x3s1_32ch_112", 32, 112, 1),
                                ("depthwise_3x3s2_64ch_112", 64, 112, 2),
                                ("depthwise_3x3s1_512ch_14", 512, 14, 1)):
        p = ops.conv_param(64, c, hw, hw, c, 3, 3, stride, 1, c, "RELU", 0.05, 0.01, 0.06)
        s = i8(64, hw, hw, c)
        f = ops.pack_filter(p, dev(rng.integers(-127, 128, (c, 1, 1, 3, 3), dtype=np.int8)))
        b = dev(rng.integers(-1000, 1000, (c,), dtype=np.int32))
        d = torch.empty((64, hw // stride, hw // stride, c), dtype=torch.int8, device="cuda")
        cases.append((name, (lambda p=p, s=s, f=f, b=b, d=d: ops.conv_bias_qs8_nhwc(
            p, s, f, b, dst=d, algo="auto")), s.numel() + d.numel()))
    a, b2 = i8(256, 56, 56, 64), i8(256, 56, 56, 64)
    cases.append(("residual_add_relu_64ch_56",
                  lambda: ops.qelemwise_qs8("QFUSE_ADD_RELU", a, b2, 0.5, 0.7, 0.9),
                  3.0 * a.numel()))
    for rnd in range(2):
        for name, fn, nbytes in cases:
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            reps = 10 if rnd else 1
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            if rnd:
                ms = e0.elapsed_time(e1) / reps
                print(f"{name}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s")
    print("device status", ops.device_status())


if __name__ == "__main__":
    main()
