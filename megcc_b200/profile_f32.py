"""Launches the fp32 (split-tf32) tensor-core kernels on small cases: one YOLOX-style ConvBias
(128 -> 128 channels, 3x3, 80 x 80, SiLU; the batch is the first argument) and the fp32
MatrixMul at 2048^3; once each, then ten times each between two events.

Meant to be run under a profiler, capturing the first launch of the kernel:

    ncu --section SpeedOfLight --section MemoryWorkloadAnalysis --clock-control none \
        -k regex:conv_f32_umma -c 1 python -m megcc_b200.profile_f32 8 conv
"""
import sys

import numpy as np
import torch

from . import ops


def main(batch=8, only=""):
    rng = np.random.default_rng(0)
    dev = lambda a: torch.from_numpy(a).cuda()
    cases = []
    c, hw = 128, 80
    p = ops.conv_f32_param(batch, c, hw, hw, c, 3, 3, 1, 1, 1, "SILU")
    src = dev(rng.standard_normal((batch, hw, hw, c)).astype(np.float32))
    flt = ops.pack_filter_f32(p, dev((rng.standard_normal((c, c, 3, 3)) / 34).astype(np.float32)))
    bias = dev(rng.standard_normal(c).astype(np.float32))
    dst = torch.empty((batch, hw, hw, c), dtype=torch.float32, device="cuda")
    cases.append(("conv_f32_128_128_3x3_80", lambda: ops.conv_bias_f32_nhwc(p, src, flt, bias, dst=dst),
                  2.0 * batch * c * hw * hw * c * 9))
    m = 2048
    a = dev(rng.standard_normal((m, m)).astype(np.float32))
    b = dev(rng.standard_normal((m, m)).astype(np.float32))
    cases.append(("matmul_f32_2048", lambda: ops.matmul_f32(a, b), 2.0 * m * m * m))
    cases = [x for x in cases if only in x[0]]
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
                print(f"{name}: {ms * 1e3:.1f} us, {work / ms / 1e9:.1f} fp32-TFLOP/s")
    print("device status", ops.device_status())


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 8, sys.argv[2] if len(sys.argv) > 2 else "")
