"""TEST / BENCHMARK INFRASTRUCTURE: one pinned host process of the CPU baseline.

    python -m oracle.cpu_worker <cpu> <steps> <warmup> <start_epoch_seconds>

The reference's runtime is single-threaded C, so its throughput on a many-core host is
measured the way a user would deploy it: one process per core, each walking the whole network
on its own image with the reference's generated x86 kernels (oracle/_ref; the restated C
checker when those were never built). The worker pins itself to <cpu>, warms up, waits for
the common start time, runs <steps> forwards and prints one JSON line with its own begin and
end times (time.time()), which the parent combines into images per second."""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    cpu, steps, warmup = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    start = float(sys.argv[4])
    try:
        os.sched_setaffinity(0, {cpu})
    except OSError:
        pass
    os.environ["OMP_NUM_THREADS"] = "1"  # the restated checker may use OpenMP; one core each
    import numpy as np

    from megcc_b200 import zoo
    from oracle import netwalk
    from oracle import oracle as O
    use_ref = O.ref_lib() is not None
    if not use_ref:
        O.lib()
    spec = zoo.resnet18()
    x = np.random.default_rng(1234 + cpu).integers(-128, 128, (1, 3, 224, 224), dtype=np.int8)
    for _ in range(warmup):
        netwalk.run(spec, x, O, use_ref)
    while time.time() < start:
        time.sleep(0.001)
    t0 = time.time()
    for _ in range(steps):
        netwalk.run(spec, x, O, use_ref)
    t1 = time.time()
    print(json.dumps(dict(cpu=cpu, t0=t0, t1=t1, steps=steps,
                          kind="reference" if use_ref else "port")))


if __name__ == "__main__":
    main()
