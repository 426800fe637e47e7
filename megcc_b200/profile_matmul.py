"""Times the int8 matrix product (int32 output, and requantised int8 output) on the shapes of
the MatMul sweep: M = N = K in {512, 2048, 4096, 8192} and M=4096, N=1000, K=2048. Ten
launches between two events after one warm-up launch; prints the mean and TOP/s.

    python -m megcc_b200.profile_matmul
"""
import numpy as np
import torch

from . import ops

SHAPES = [(512, 512, 512), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
          (4096, 1000, 2048)]


def main():
    rng = np.random.default_rng(0)
    for m, n, k in SHAPES:
        a = torch.from_numpy(rng.integers(-127, 128, (m, k), dtype=np.int8)).cuda()
        b = torch.from_numpy(rng.integers(-127, 128, (k, n), dtype=np.int8)).cuda()
        bp = ops.matmul_pack_b(b)
        for name, fn in (("int32", lambda: ops.matmul_s8_s32(a, bp)),
                         ("qint8", lambda: ops.matmul_s8_qs8(a, bp, 0.002, 1.0))):
            fn()
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            print(f"matmul {m}x{n}x{k} -> {name}: {ms * 1e3:.1f} us, "
                  f"{2.0 * m * n * k / ms / 1e9:.0f} TOP/s")
    print("device status", ops.device_status())


if __name__ == "__main__":
    main()
