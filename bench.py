#!/usr/bin/env python
"""Headline benchmark: ResNet-18 int8, batch 256 per GPU, img/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One process per GPU (the driver starts N of them with torch.distributed.run). A step is
one forward of a 256-image batch through the compiled model:

  value     img/s with the input batch already in device memory and the logits left there
            (CUDA-graph replay through LITE_forward / LITE_wait), timed with CUDA events on
            the network's stream, max over ranks
  e2e       the same through the host-buffer boundary a LITE_* user sees: pinned host input
            copied in and logits copied out inside every timed step; three LiteNetworks
            take turns so that a step's input copy overlaps the compute of earlier steps
  roofline  the tcgen05 ConvBias kernel: algorithmic int8 ops of every launch / its CUDA
            event time, against 2 x the measured bf16 tensor peak
  cpu_baseline  the reference's own generated x86 kernels (oracle/_ref) walking the same
            network on the host cores, one image per thread (a bounded sample)

--impl reference times only that CPU path and prints it in the same JSON shape.
All data is synthetic (seeded uniform int8) and weights are random-init.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 256
METRIC = "resnet18_int8_images_per_second"
UNIT = "img/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_burst=p["bf16_tflops"],
                    bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi SM clock and throttle reasons, sampled every 20 ms from before the warm-up
    until after the timed regions. Samples are time-stamped on arrival so that the ones
    that fall inside the timed region can be told apart from the rest of the run."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.samples = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True, bufsize=1)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def wait_first(self, timeout=5.0):
        t0 = time.perf_counter()
        while self.proc and not self.samples and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def stop(self, windows):
        """windows: [(t_begin, t_end)] of the timed regions (perf_counter seconds)."""
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def digest(rows):
            sm, mx, reasons = [], [], set()
            for _, l in rows:
                f = [x.strip() for x in l.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, v in zip(names, f[5:9]):
                    if v.lower() == "active":
                        reasons.add(n)
            sm.sort()
            return sm, mx, sorted(reasons)

        inside = [r for r in self.samples
                  if any(b - 0.02 <= r[0] <= e + 0.02 for b, e in windows)]
        window = "timed regions"
        if len(inside) < 3:  # a very short timed region: fall back to the loaded run around it
            lo = min(b for b, _ in windows) - 1.0
            hi = max(e for _, e in windows) + 0.2
            inside = [r for r in self.samples if lo <= r[0] <= hi]
            window = "timed regions and the warm-up before them"
        sm, mx, reasons = digest(inside)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    samples=len(sm), window=window, reasons=reasons)


def cpu_reference_run(spec, steps, warmup, threads):
    """The reference's own x86 kernels on the host: each step walks the network once per
    thread on one image, all threads in parallel. Returns (img/s, seconds per step)."""
    import numpy as np
    from oracle import netwalk
    from oracle import oracle as O

    if O.ref_lib() is None:
        kind, use_ref = "port", False
        O.lib()
    else:
        kind, use_ref = "reference", True
    rng = np.random.default_rng(1234)
    xs = [rng.integers(-128, 128, (1, 3, 224, 224), dtype=np.int8) for _ in range(threads)]

    def one_step():
        ts = [threading.Thread(target=netwalk.run, args=(spec, xs[i], O, use_ref))
              for i in range(threads)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = time.perf_counter() - t0
    return threads * steps / dt, dt / steps, kind


def other_configs(local_rank):
    """The figures BASELINE's metric names besides the headline: batch-1 latency (p50 / p95 of
    50 CUDA-graph forwards after 10 warm-ups, input resident in HBM, one event pair per
    forward; `e2e_p50_ms` = wall clock of LITE_forward + LITE_wait from a pinned host input,
    logits back on the host), MobileNetV1 at batch 64, and ResNet-18 at batch 256 with one
    filter scale per output channel (the reference has one per tensor, so that variant has
    no reference arm). Short runs on rank 0 only; none of them is the `value`."""
    import numpy as np
    import torch

    from megcc_b200 import lite, zoo
    dev = torch.device("cuda", local_rank)

    def forwards(spec, batch, host_input):
        model = spec.to_graph().compile([batch])
        rng = np.random.default_rng(7)
        x = torch.from_numpy(rng.integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8))
        x = x.pin_memory() if host_input else x.to(dev)
        net = (lite.Network(model, device_id=local_rank) if host_input else
               lite.Network(model, device_id=local_rank, device_io=("fc:out",)))
        net.set_input_ptr("data", x.data_ptr(), x.numel())
        stream = torch.cuda.ExternalStream(net.stream())
        for _ in range(10):
            net.forward()
        net.wait()
        times = []
        for _ in range(50):
            if host_input:
                t0 = time.perf_counter()
                net.forward()
                net.wait()
                times.append((time.perf_counter() - t0) * 1e3)
            else:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                net.forward()
                e1.record(stream)
                net.wait()
                times.append(e0.elapsed_time(e1))
        net.close()
        times.sort()
        return times[len(times) // 2], times[int(len(times) * 0.95)]

    out = {}
    for name, make in (("resnet18", zoo.resnet18), ("mobilenetv1", zoo.mobilenet_v1)):
        p50, p95 = forwards(make(), 1, False)
        e2e50, _ = forwards(make(), 1, True)
        out[name + "_b1"] = dict(p50_ms=round(p50, 4), p95_ms=round(p95, 4),
                                 e2e_p50_ms=round(e2e50, 4))
    p50, _ = forwards(zoo.mobilenet_v1(), 64, False)
    out["mobilenetv1_b64"] = dict(ms_per_forward=round(p50, 4), img_s=round(64 / (p50 * 1e-3)))
    p50, _ = forwards(zoo.resnet18(per_channel=True), BATCH, False)
    out["resnet18_b256_per_channel_scales"] = dict(ms_per_forward=round(p50, 4),
                                                   img_s=round(BATCH / (p50 * 1e-3)))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="megcc_b200", choices=["megcc_b200", "reference"])
    ap.add_argument("--cpu-threads", type=int, default=0)
    args = ap.parse_args()

    from megcc_b200 import shard
    rank, local_rank, world = shard.env_rank()

    from megcc_b200 import zoo
    spec = zoo.resnet18()
    threads = args.cpu_threads or min(os.cpu_count() or 1, 64)
    config = dict(workload="resnet18_int8_b256", per_gpu_batch=BATCH, global_batch=BATCH * world,
                  input="3x224x224 int8", classes=1000, scales="per-tensor",
                  parallelism=f"batch-sharded x{world}, no collective",
                  l2="working set per step 1.7 GB, far larger than the 126 MB L2",
                  macs_per_image=spec.macs_per_image())

    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
        ips, sec, kind = cpu_reference_run(spec, steps, warmup, threads)
        sample = (f"{steps} steps x {threads} images (one per thread) of the same network, "
                  f"{warmup} warm-up; the {BATCH}-image batch is not run in full on the CPU")
        print(json.dumps(dict(
            impl="reference", metric=METRIC, value=ips, unit=UNIT, n_gpus=args.gpus,
            steps=steps, warmup=warmup, ms_per_step=sec * 1e3, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="int8", data="synthetic", config=config,
            cpu_baseline=dict(value=ips, unit=UNIT, cores=threads, kind=kind, sample=sample),
            e2e=dict(value=ips, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))))
        return

    import numpy as np
    import torch

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    # host staging next to the GPU: the end-to-end arm is bound by the input copy
    affinity_before = shard.bind_to_gpu_cpus(local_rank)
    group = shard.Group("nccl", torch.device("cuda", local_rank))

    def barrier():
        group.barrier()
        torch.cuda.synchronize()

    max_over_ranks = group.max

    from megcc_b200 import lite

    model = spec.to_graph().compile([BATCH])
    rng = np.random.default_rng(1000 + rank)
    x_host = torch.from_numpy(
        rng.integers(-128, 128, (BATCH, 3, 224, 224), dtype=np.int8)).pin_memory()
    x_dev = x_host.cuda()
    in_bytes = x_host.numel()

    # ---- device-resident arm: input in HBM, logits stay in HBM ----
    net = lite.Network(model, device_id=local_rank, device_io=("fc:out",))
    stream = torch.cuda.ExternalStream(net.stream())
    ops_per_step = None  # counted from the loaded model below
    net.set_input_ptr("data", x_dev.data_ptr(), in_bytes)
    # kernel launches per step = instructions of the model (+1: the first layer's
    # space-to-depth kernel), all inside one CUDA graph launch
    ops_per_step = len(net.profile()) + 1
    sampler = ClockSampler(local_rank).start()
    sampler.wait_first()
    for _ in range(max(args.warmup, 3)):
        net.forward()
    net.wait()
    # keep the GPU under the same load for a moment so the clock samples mean something
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.3:
        net.forward()
        net.wait()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    w0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.steps):
        net.forward()
    e1.record(stream)
    net.wait()
    w1 = time.perf_counter()
    barrier()
    ms_dev = max_over_ranks(e0.elapsed_time(e1))

    # ---- end-to-end arm: pinned host input in, logits out, every step ----
    # Three LiteNetworks of the same model take turns, each with its own stream, arena and
    # pinned input buffer: LITE_forward only enqueues (copy in, graph, copy out), so the
    # host-to-device copy of a step runs while earlier steps compute, and with three in flight
    # a copy is always queued when the link falls idle (with two, both copies and then both
    # graphs tended to run side by side and the link idled during the graphs). Every step
    # still copies its 38.5 MB in and its logits out inside the timed region, and the host
    # reads each step's result.
    depth = 3
    nets = [lite.Network(model, device_id=local_rank) for _ in range(depth)]
    out_bytes = nets[0].tensor_bytes("fc:out", lite.LITE_OUTPUT)
    x_hosts = [x_host] + [x_host.clone().pin_memory() for _ in range(depth - 1)]
    for n, xh in zip(nets, x_hosts):
        n.set_input_ptr("data", xh.data_ptr(), in_bytes)
    streams2 = [torch.cuda.ExternalStream(n.stream()) for n in nets]
    checksum = 0

    def collect(n):
        n.wait()
        return int(np.frombuffer(
            (lite.C.c_int8 * 8).from_address(n.output_ptr("fc:out")), dtype=np.int8)[0])

    def pipelined(steps, first_event=None, end_events=None):
        """`steps` forwards, `depth` of them in flight; the host reads every result."""
        x = 0
        if first_event is not None:
            first_event.record(streams2[0])
        in_flight = []
        for i in range(steps):
            n = nets[i % depth]
            n.forward()
            in_flight.append(n)
            if len(in_flight) == depth:
                x ^= collect(in_flight.pop(0))
        if end_events is not None:
            for ev, st in zip(end_events, streams2):
                ev.record(st)
        while in_flight:
            x ^= collect(in_flight.pop(0))
        return x

    for n in nets:  # first pass of each network: eager, then graph capture
        for _ in range(2):
            n.forward()
            n.wait()
    # warm-up in the timed loop's own form, and long enough (0.3 s) that link and clocks are
    # in their loaded state when the timed region starts
    pipelined(max(args.warmup, 3) * depth)
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.3:
        pipelined(2 * depth)
    barrier()
    f0 = torch.cuda.Event(enable_timing=True)
    f_end = [torch.cuda.Event(enable_timing=True) for _ in nets]
    w2 = time.perf_counter()
    checksum ^= pipelined(args.steps, f0, f_end)
    for ev in f_end:
        ev.synchronize()
    w3 = time.perf_counter()
    barrier()
    f1_ms = max(f0.elapsed_time(ev) for ev in f_end)
    ms_e2e = max_over_ranks(f1_ms)
    clocks = sampler.stop([(w0, w1), (w2, w3)])

    # ---- per-kernel pass for the roofline of the dominant kernel ----
    roofline = None
    cpu_baseline = None
    extra = None
    if rank == 0:
        peaks = load_peaks()
        net.set_profile(True)
        for _ in range(5):
            net.forward()
            net.wait()
        rows = net.profile()
        net.set_profile(False)
        shapes = spec.shapes
        conv_ops = {}
        for l in spec.layers:
            if l["op"] == "conv":
                oc, oh, ow = shapes[l["name"]]
                ic = shapes[l["src"]][0]
                k = l["flt"].shape[-1]
                conv_ops[l["name"]] = 2.0 * BATCH * oc * oh * ow * (ic // l["groups"]) * k * k
        total_ms = sum(r[2] for r in rows)
        # every ConvBias of this network runs on the tcgen05 kernels (the 3-channel first layer
        # after its space-to-depth step)
        # an instruction named "a+b" is ConvBias a with the elementwise b fused behind it
        conv_of = lambda n: n.split("+")[0]
        umma = [(conv_of(n), ms) for n, s, ms, c in rows if conv_of(n) in conv_ops and c]
        umma_ops = sum(conv_ops[n] for n, _ in umma)
        umma_ms = sum(ms for _, ms in umma)
        peak = 2.0 * peaks["bf16_sustained"]
        achieved = umma_ops / (umma_ms * 1e-3) / 1e12 if umma_ms > 0 else 0.0
        roofline = dict(
            bound="tensor",
            kernel="conv_umma_kernel / conv_patch_kernel (tcgen05 kind::i8 implicit GEMM)",
            achieved=achieved, peak=peak, unit="TOP/s", frac=achieved / peak, traffic=None,
            launches_per_step=len(umma), share_of_step=umma_ms / total_ms if total_ms else None,
            peak_note=f"2 x bf16 sustained ({peaks['source']}); int8 dense peak is not in "
                      "MEASURED_PEAKS.json",
            per_kernel_ms={n: round(ms, 4) for n, s, ms, c in rows})
        try:
            extra = other_configs(local_rank)
        except Exception as e:  # never lose the headline line to a side measurement
            extra = dict(error=repr(e))
        if affinity_before is not None:
            os.sched_setaffinity(0, affinity_before)  # the CPU leg uses every host core
        ips_cpu, sec, kind = cpu_reference_run(spec, 2, 1, threads)
        cpu_baseline = dict(
            value=ips_cpu, unit=UNIT, cores=threads, kind=kind,
            sample=f"2 steps x {threads} images (one per thread), 1 warm-up step")
    net.close()
    for n in nets:
        n.close()
    group.close()
    if rank != 0:
        return
    images = BATCH * world * args.steps
    value = images / (ms_dev * 1e-3)
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps,
        warmup=max(args.warmup, 3), ms_per_step=ms_dev / args.steps, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="int8", data="synthetic", config=config,
        clocks=clocks, gpu_launches=ops_per_step * args.steps,
        e2e=dict(value=images / (ms_e2e * 1e-3), unit=UNIT, ms_per_step=ms_e2e / args.steps,
                 h2d_bytes_per_step=in_bytes, d2h_bytes_per_step=out_bytes),
        roofline=roofline, cpu_baseline=cpu_baseline, other_configs=extra)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
