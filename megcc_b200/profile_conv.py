"""Launches representative qint8 ConvBias kernels (first layer 3->64 7x7/2, and the 3x3
convolutions of the four ResNet-18 stages: 64 channels at 56x56, 128 at 28x28, 256 at 14x14,
512 at 7x7) on a small batch: once each, then ten times each between
two events, and prints the mean time of the ten.

Meant to be run under a profiler, capturing the first launches:

    ncu --set full --clock-control none -k regex:conv_ -c 3 \
        python -m megcc_b200.profile_conv 32

A second argument keeps only the cases whose name contains it, e.g. the first layer with the
max-pool behind it folded in:

    ncu --set full --clock-control none -k regex:conv_patch -c 1 \
        python -m megcc_b200.profile_conv 32 first_layer_pool
"""
import ctypes
import sys

import numpy as np
import torch

from . import ops
from ._lib import check, lib


def main(batch=32, only=""):
    rng = np.random.default_rng(0)
    dev = lambda a: torch.from_numpy(a).cuda()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    cases = []

    p = ops.conv_param(batch, 3, 224, 224, 64, 7, 7, 2, 3, 1, "RELU", 0.02, 0.01, 0.5)
    src = dev(rng.integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8))
    flt = dev(rng.integers(-127, 128, (64, 3, 7, 7), dtype=np.int8))
    bias = dev(rng.integers(-1000, 1000, (64,), dtype=np.int32))
    packed = torch.empty(lib().mb200_conv_s2d_filter_bytes(ctypes.byref(p)), dtype=torch.int8,
                         device="cuda")
    check(lib().mb200_conv_s2d_pack_filter(ctypes.byref(p), ptr(flt), ptr(packed), st))
    ws = torch.empty(lib().mb200_conv_s2d_workspace_bytes(ctypes.byref(p)), dtype=torch.int8,
                     device="cuda")
    dst = torch.empty((batch, 112, 112, 64), dtype=torch.int8, device="cuda")

    def first_layer():
        check(lib().mb200_conv_bias_qs8_s2d(ctypes.byref(p), ptr(src), 1, ptr(packed), ptr(bias),
                                            None, ptr(dst), ptr(ws), ws.numel(), st))

    cases.append(("first_layer_3_64_7x7s2", first_layer, 2.0 * batch * 64 * 112 * 112 * 147))
    pooled = torch.empty((batch, 56, 56, 64), dtype=torch.int8, device="cuda")

    def first_layer_pool():
        check(lib().mb200_conv_bias_pool_qs8_s2d(
            ctypes.byref(p), ptr(src), 1, ptr(packed), ptr(bias), None, ptr(pooled), ptr(ws),
            ws.numel(), st))

    cases.append(("first_layer_pool_3_64_7x7s2_max3x3s2", first_layer_pool,
                  2.0 * batch * 64 * 112 * 112 * 147))
    for name, c, hw in (("conv_64_64_3x3_56", 64, 56), ("conv_128_128_3x3_28", 128, 28),
                        ("conv_256_256_3x3_14", 256, 14), ("conv_512_512_3x3_7", 512, 7)):
        pp = ops.conv_param(batch, c, hw, hw, c, 3, 3, 1, 1, 1, "RELU", 0.05, 0.01, 2.0)
        s = dev(rng.integers(-128, 128, (batch, hw, hw, c), dtype=np.int8))
        f = ops.pack_filter(pp, dev(rng.integers(-127, 128, (c, c, 3, 3), dtype=np.int8)))
        b = dev(rng.integers(-1000, 1000, (c,), dtype=np.int32))
        d = torch.empty((batch, hw, hw, c), dtype=torch.int8, device="cuda")
        cases.append((name, (lambda pp=pp, s=s, f=f, b=b, d=d: ops.conv_bias_qs8_nhwc(
            pp, s, f, b, dst=d, algo="auto")), 2.0 * batch * c * hw * hw * c * 9))
    # the 1x1 / stride 2 projection of the first block of a ResNet stage (64 -> 128 at 56 x 56)
    pp = ops.conv_param(batch, 64, 56, 56, 128, 1, 1, 2, 0, 1, "IDENTITY", 0.05, 0.01, 0.5)
    s = dev(rng.integers(-128, 128, (batch, 56, 56, 64), dtype=np.int8))
    f = ops.pack_filter(pp, dev(rng.integers(-127, 128, (128, 64, 1, 1), dtype=np.int8)))
    b = dev(rng.integers(-1000, 1000, (128,), dtype=np.int32))
    d = torch.empty((batch, 28, 28, 128), dtype=torch.int8, device="cuda")
    cases.append(("proj_64_128_1x1s2_56", (lambda: ops.conv_bias_qs8_nhwc(pp, s, f, b, dst=d,
                                                                         algo="auto")),
                  2.0 * batch * 128 * 28 * 28 * 64))
    cases = [c for c in cases if only in c[0]]
    for rnd in range(2):
        for name, fn, work in cases:
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            reps = 10 if rnd else 1
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            if rnd:
                ms = e0.elapsed_time(e1) / reps
                print(f"{name}: {ms * 1e3:.1f} us, {work / ms / 1e9:.0f} TOP/s")
    print("device status", ops.device_status())


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 32, sys.argv[2] if len(sys.argv) > 2 else "")
