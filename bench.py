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
            event time, against 2 x the measured bf16 tensor peak, with the fractions against
            the other candidate denominators (2 x bf16 burst, the int8 MMA issue rate measured
            in this run, nominal dense int8) and the step-level figure beside it
  cpu_baseline  the reference's own generated x86 kernels (oracle/_ref) walking the same
            network on the host cores, one pinned process per core (a bounded sample)
  parity_checked  images of the timed batch whose logits, from the very networks that were
            timed, equal the CPU checker's bit for bit (checked outside the timed regions)
  strong_scaling  (N > 1) the same 256 images split over the ranks
  h2d_probe (N > 1) host-to-device bandwidth per rank, alone and all ranks together

The timed region of --steps steps is repeated --regions times; value and e2e come from the
median region.

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
# DRAM bytes moved by the tensor-core ConvBias launches of one batch-256 forward, measured
# once under ncu (the capture cannot run inside a timed benchmark)
CONV_DRAM_BYTES_PER_STEP = 934.4e6
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


def cpu_reference_run(steps, warmup, procs):
    """The reference's own x86 kernels on the host, deployed as a user of its single-threaded
    runtime would on a many-core box: `procs` processes, each pinned to one core, each
    walking the whole network on its own image (oracle/cpu_worker.py). All start at a common
    time after their warm-up. Returns (img/s, seconds per step, kind)."""
    cpus = sorted(os.sched_getaffinity(0))[:procs]
    runner = os.path.join(ROOT, "oracle", "_ref", "ref_lite_runner")
    if os.path.exists(runner):
        # the reference's C runtime itself: the BARE_METAL DeviceModel of the same network,
        # compiled by this repository's compile side, through the reference's LITE_forward
        # with the reference's generated kernels (oracle/ref_lite_runner.c). The runner does
        # one untimed forward, then `steps` timed ones, and reports its own mean.
        import tempfile

        import numpy as np

        from megcc_b200 import zoo
        g = zoo.resnet18().to_graph()
        g.set_option("bare_metal_model", 2)
        model = g.compile([1])
        with tempfile.TemporaryDirectory() as d:
            with open(os.path.join(d, "resnet18_b1.tiny"), "wb") as f:
                f.write(model)
            for c in cpus:
                np.random.default_rng(1234 + c).integers(
                    -128, 128, (1, 3, 224, 224), dtype=np.int8).tofile(
                    os.path.join(d, f"in{c}.bin"))
            ps = [subprocess.Popen(
                [runner, os.path.join(d, "resnet18_b1.tiny"), os.path.join(d, f"in{c}.bin"),
                 os.path.join(d, f"out{c}.bin"), str(steps), str(c)],
                stdout=subprocess.PIPE, text=True) for c in cpus]
            ms = []
            for p in ps:
                out, _ = p.communicate()
                if p.returncode != 0 or "forward_ms" not in out:
                    raise RuntimeError("a reference runtime process failed")
                ms.append(float(out.split("forward_ms")[1].split()[0]))
        span = max(ms) * 1e-3 * steps
        return len(cpus) * steps / span, span / steps, "reference"
    start = time.time() + 8.0 + 2.5 * warmup  # imports + model construction + warm-up
    ps = [subprocess.Popen([sys.executable, "-m", "oracle.cpu_worker", str(c), str(steps),
                            str(warmup), repr(start)], stdout=subprocess.PIPE, text=True,
                           cwd=ROOT) for c in cpus]
    rows = []
    for p in ps:
        out, _ = p.communicate()
        if p.returncode != 0 or not out.strip():
            raise RuntimeError("a CPU baseline worker failed")
        rows.append(json.loads(out.strip().splitlines()[-1]))
    span = max(r["t1"] for r in rows) - min(r["t0"] for r in rows)
    late = max(r["t0"] for r in rows) - start
    if late > 0.5:  # a worker missed the common start: its warm-up took longer than allowed
        span = max(r["t1"] - r["t0"] for r in rows)
    return len(rows) * steps / span, span / steps, rows[0]["kind"]


def other_configs(local_rank, rates):
    """The figures BASELINE's metric names besides the headline: batch-1 latency (p50 / p95 of
    50 CUDA-graph forwards after 10 warm-ups, input resident in HBM, one event pair per
    forward; `e2e_p50_ms` = wall clock of LITE_forward + LITE_wait from a pinned host input,
    logits back on the host), MobileNetV1 at batch 64, ResNet-18 at batch 256 with one filter
    scale per output channel (the reference has one per tensor, so that variant has no
    reference arm), the fp32 detector at batch 32 and the int8 / fp32 MatrixMul sweeps.
    Short runs on rank 0 only; none of them is the `value`."""
    import numpy as np
    import torch

    from megcc_b200 import lite, ops, zoo
    dev = torch.device("cuda", local_rank)

    def forwards(model, x, host_input, out_names, reps=50, warm=10):
        x = x.pin_memory() if host_input else x.to(dev)
        net = (lite.Network(model, device_id=local_rank) if host_input else
               lite.Network(model, device_id=local_rank, device_io=tuple(out_names)))
        net.set_input_ptr("data", x.data_ptr(), x.numel() * x.element_size())
        stream = torch.cuda.ExternalStream(net.stream())
        for _ in range(warm):
            net.forward()
        net.wait()
        times = []
        for _ in range(reps):
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

    def int8_net(spec, batch, host_input):
        rng = np.random.default_rng(7)
        x = torch.from_numpy(rng.integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8))
        return forwards(spec.to_graph().compile([batch]), x, host_input, ("fc:out",))

    out = {}
    for name, make in (("resnet18", zoo.resnet18), ("mobilenetv1", zoo.mobilenet_v1)):
        p50, p95 = int8_net(make(), 1, False)
        e2e50, _ = int8_net(make(), 1, True)
        out[name + "_b1"] = dict(p50_ms=round(p50, 4), p95_ms=round(p95, 4),
                                 e2e_p50_ms=round(e2e50, 4))
    for b in (64, BATCH):
        p50, _ = int8_net(zoo.mobilenet_v1(), b, False)
        out[f"mobilenetv1_b{b}"] = dict(ms_per_forward=round(p50, 4), img_s=round(b / (p50 * 1e-3)))
    p50, _ = int8_net(zoo.resnet18(per_channel=True), BATCH, False)
    out["resnet18_b256_per_channel_scales"] = dict(ms_per_forward=round(p50, 4),
                                                   img_s=round(BATCH / (p50 * 1e-3)))

    # fp32 detector, batch 32 at 640 x 640: three tf32 passes per product on the tensor cores
    spec = zoo.yolox_s()
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.uniform(0, 1, (32, 3, 640, 640)).astype(np.float32))
    g = spec.to_graph()
    model = g.compile([32])
    names = [o + ":out" for o in spec.outputs]
    p50, _ = forwards(model, x, False, names, reps=10, warm=3)
    flops = 2.0 * spec.macs_per_image() * 32
    out["yolox_s_fp32_b32"] = dict(
        ms_per_forward=round(p50, 3), img_s=round(32 / (p50 * 1e-3), 1),
        fp32_tflops=round(flops / (p50 * 1e-3) / 1e12, 1),
        tf32_pass_tflops=round(3 * flops / (p50 * 1e-3) / 1e12, 1),
        frac_of_measured_tf32_mma_rate=round(3 * flops / (p50 * 1e-3) / 1e12 / rates["tf32"], 3),
        arena_gb=round(g.arena_bytes(0) / 1e9, 2), gmac_per_image=round(spec.macs_per_image() / 1e9, 2),
        note="whole forward (83 ConvBias + concat / resize / pooling kernels; operands are split "
             "into their tf32 planes on chip); fp32_tflops counts 2 x MAC once, tf32_pass_tflops the three tensor-core "
             "passes that fp32 accuracy costs")

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    import ctypes as C
    from megcc_b200._lib import check, lib
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sweep_i8, sweep_f32 = {}, {}
    with torch.cuda.device(dev):
        for m, n, k in ((512, 512, 512), (2048, 2048, 2048), (4096, 4096, 4096),
                        (8192, 8192, 8192), (4096, 1000, 2048)):
            a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
            b = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev)
            bp = ops.matmul_pack_b(b)
            c = torch.empty((m, n), dtype=torch.int8, device=dev)
            ms = timed(lambda: check(lib().mb200_matmul_s8_qs8(
                m, n, k, C.c_void_p(a.data_ptr()), C.c_void_p(bp.data_ptr()),
                C.c_void_p(c.data_ptr()), 1.0, 500.0, st)))
            tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            sweep_i8[f"{m}x{n}x{k}"] = dict(ms=round(ms, 4), tops=round(tops, 1),
                                            frac_of_measured_i8_mma_rate=round(tops / rates["i8"], 3))
            af = torch.randn((m, k), dtype=torch.float32, device=dev)
            bf = torch.randn((k, n), dtype=torch.float32, device=dev)
            packed = torch.empty(lib().mb200_matmul_f32_packed_b_bytes(k, n) // 4,
                                 dtype=torch.float32, device=dev)
            check(lib().mb200_matmul_f32_pack_b(k, n, C.c_void_p(bf.data_ptr()),
                                                C.c_void_p(packed.data_ptr()), st))
            nb = lib().mb200_matmul_f32_workspace_bytes(m, k)
            ws = torch.empty(nb + 256, dtype=torch.int8, device=dev)
            wp = ws.data_ptr() + (-ws.data_ptr()) % 256
            cf = torch.empty((m, n), dtype=torch.float32, device=dev)
            ms = timed(lambda: check(lib().mb200_matmul_f32(
                m, n, k, C.c_void_p(af.data_ptr()), C.c_void_p(packed.data_ptr()),
                C.c_void_p(cf.data_ptr()), C.c_void_p(wp), nb, st)))
            tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            sweep_f32[f"{m}x{n}x{k}"] = dict(
                ms=round(ms, 4), fp32_tflops=round(tf, 1),
                frac_of_measured_tf32_mma_rate=round(3 * tf / rates["tf32"], 3))
            del a, b, bp, c, af, bf, packed, ws, cf
    out["matmul_int8_requant_sweep"] = sweep_i8
    out["matmul_fp32_sweep"] = sweep_f32
    return out


class HostBuffer:
    """Page-locked host memory from cudaHostAlloc, optionally write-combined (the CPU writes it
    once, the GPU's copy engine reads it without snooping the CPU caches)."""

    def __init__(self, nbytes, write_combined):
        import ctypes as C
        self._rt = C.CDLL("libcudart.so.12")
        self._rt.cudaHostAlloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_uint]
        self._rt.cudaFreeHost.argtypes = [C.c_void_p]
        p = C.c_void_p()
        rc = self._rt.cudaHostAlloc(C.byref(p), nbytes, 0x04 if write_combined else 0)
        if rc != 0 or not p.value:
            raise RuntimeError(f"cudaHostAlloc failed: {rc}")
        self.ptr, self.nbytes = p.value, nbytes

    def fill(self, array):
        import ctypes as C
        C.memmove(self.ptr, array.ctypes.data, min(self.nbytes, array.nbytes))

    def close(self):
        if self.ptr:
            self._rt.cudaFreeHost(self.ptr)
            self.ptr = None


def h2d_probe(group, local_rank, nbytes):
    """Host-to-device copy bandwidth of a rank's pinned staging buffer, every rank alone (the
    others idle) and all ranks together: the end-to-end arm is bound by it at 4 and 8 GPUs.
    The same with write-combined pinned memory. GB/s per rank."""
    import ctypes as C

    import torch
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    dst = torch.empty(nbytes, dtype=torch.int8, device=f"cuda:{local_rank}")
    stream = torch.cuda.current_stream()

    def rate(buf):
        def copy():
            rt.cudaMemcpyAsync(dst.data_ptr(), buf.ptr, nbytes, 1, stream.cuda_stream)
        for _ in range(2):
            copy()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(8):
            copy()
        e1.record()
        torch.cuda.synchronize()
        return 8 * nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9

    out = dict(bytes=nbytes)
    for tag, wc in (("", False), ("wc_", True)):
        buf = HostBuffer(nbytes, wc)
        alone = 0.0
        for r in range(group.world):
            group.barrier()
            if r == group.rank:
                alone = rate(buf)
        group.barrier()
        together = rate(buf)
        out.update({f"alone_{tag}gbs_min": -group.max(-alone), f"alone_{tag}gbs_max": group.max(alone),
                    f"together_{tag}gbs_min": -group.max(-together),
                    f"together_{tag}gbs_sum": group.sum(together)})
        buf.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="megcc_b200", choices=["megcc_b200", "reference"])
    ap.add_argument("--cpu-threads", type=int, default=0)
    ap.add_argument("--regions", type=int, default=11,
                    help="how often the timed region of --steps steps is repeated")
    ap.add_argument("--skip-extras", action="store_true",
                    help="headline line only: no other_configs, no CPU baseline")
    args = ap.parse_args()

    from megcc_b200 import shard
    rank, local_rank, world = shard.env_rank()

    from megcc_b200 import zoo
    spec = zoo.resnet18()
    threads = args.cpu_threads or min(len(os.sched_getaffinity(0)), 64)
    config = dict(workload="resnet18_int8_b256", per_gpu_batch=BATCH, global_batch=BATCH * world,
                  input="3x224x224 int8", classes=1000, scales="per-tensor",
                  parallelism=f"batch-sharded x{world}, no collective",
                  l2="working set per step 1.7 GB, far larger than the 126 MB L2",
                  macs_per_image=spec.macs_per_image())

    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
        ips, sec, kind = cpu_reference_run(steps, warmup, threads)
        sample = (f"{steps} steps x {threads} images (one pinned process of the reference's "
                  f"single-threaded C runtime per host core, LITE_forward on the BARE_METAL "
                  f"DeviceModel of the same network at batch 1, one image each), 1 warm-up "
                  f"forward; the {BATCH}-image batch is not run in full on the CPU")
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

    def median(v):
        v = sorted(v)
        return v[len(v) // 2]

    class Arms:
        """The two timed arms for one per-GPU batch size: device-resident (input in HBM, logits
        stay there) and end to end (pinned host input in, logits out, every step)."""

        def __init__(self, batch, seed):
            self.batch = batch
            self.model = spec.to_graph().compile([batch])
            rng = np.random.default_rng(seed)
            self.x_np = rng.integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8)
            self.x_host = torch.from_numpy(self.x_np).pin_memory()
            self.x_dev = self.x_host.cuda()
            self.in_bytes = self.x_host.numel()
            self.net = lite.Network(self.model, device_id=local_rank, device_io=("fc:out",))
            self.stream = torch.cuda.ExternalStream(self.net.stream())
            self.net.set_input_ptr("data", self.x_dev.data_ptr(), self.in_bytes)
            # Three LiteNetworks of the same model take turns in the end-to-end arm, each with
            # its own stream, arena and pinned input buffer: LITE_forward only enqueues (copy
            # in, graph, copy out), so a step's input copy runs while earlier steps compute.
            self.depth = 3
            self.nets = [lite.Network(self.model, device_id=local_rank) for _ in range(self.depth)]
            self.out_bytes = self.nets[0].tensor_bytes("fc:out", lite.LITE_OUTPUT)
            self.x_hosts = [self.x_host] + [self.x_host.clone().pin_memory()
                                            for _ in range(self.depth - 1)]
            for n, xh in zip(self.nets, self.x_hosts):
                n.set_input_ptr("data", xh.data_ptr(), self.in_bytes)
            self.streams2 = [torch.cuda.ExternalStream(n.stream()) for n in self.nets]

        def warm(self, steps):
            for _ in range(max(steps, 3)):
                self.net.forward()
            self.net.wait()
            for n in self.nets:  # eager pass, then graph capture
                for _ in range(2):
                    n.forward()
                    n.wait()
            self.pipelined(max(steps, 3) * self.depth)

        def load(self, seconds):
            t = time.perf_counter()
            while time.perf_counter() - t < seconds:
                self.net.forward()
                self.net.wait()

        def resident_region(self, steps):
            """ms of `steps` forwards, CUDA events on the network's stream, max over ranks."""
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            w0 = time.perf_counter()
            e0.record(self.stream)
            for _ in range(steps):
                self.net.forward()
            e1.record(self.stream)
            self.net.wait()
            w1 = time.perf_counter()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)), (w0, w1)

        def collect(self, n):
            n.wait()
            return int(np.frombuffer(
                (lite.C.c_int8 * 8).from_address(n.output_ptr("fc:out")), dtype=np.int8)[0])

        def pipelined(self, steps, first_event=None, end_events=None):
            """`steps` forwards, `depth` of them in flight; the host reads every result."""
            x = 0
            if first_event is not None:
                first_event.record(self.streams2[0])
            in_flight = []
            for i in range(steps):
                n = self.nets[i % self.depth]
                n.forward()
                in_flight.append(n)
                if len(in_flight) == self.depth:
                    x ^= self.collect(in_flight.pop(0))
            if end_events is not None:
                for ev, st in zip(end_events, self.streams2):
                    ev.record(st)
            while in_flight:
                x ^= self.collect(in_flight.pop(0))
            return x

        def e2e_region(self, steps):
            barrier()
            f0 = torch.cuda.Event(enable_timing=True)
            f_end = [torch.cuda.Event(enable_timing=True) for _ in self.nets]
            w0 = time.perf_counter()
            self.pipelined(steps, f0, f_end)
            for ev in f_end:
                ev.synchronize()
            w1 = time.perf_counter()
            barrier()
            return max_over_ranks(max(f0.elapsed_time(ev) for ev in f_end)), (w0, w1)

        def close(self):
            self.net.close()
            for n in self.nets:
                n.close()

    # ---- headline: 256 images per GPU (weak scaling) ----
    arms = Arms(BATCH, 1000 + rank)
    ops_per_step = len(arms.net.profile()) + 1  # instructions (+1: the first layer's s2d kernel)
    sampler = ClockSampler(local_rank).start()
    sampler.wait_first()
    arms.warm(args.warmup)
    arms.load(0.3)  # clocks and link in their loaded state before the timed regions
    windows, dev_ms, e2e_ms = [], [], []
    for _ in range(max(args.regions, 1)):
        ms, w = arms.resident_region(args.steps)
        dev_ms.append(ms)
        windows.append(w)
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.3:
        arms.pipelined(2 * arms.depth)
    for _ in range(max(args.regions, 1)):
        ms, w = arms.e2e_region(args.steps)
        e2e_ms.append(ms)
        windows.append(w)
    clocks = sampler.stop(windows)
    ms_dev, ms_e2e = median(dev_ms), median(e2e_ms)

    # ---- strong scaling: the SAME 256 images split over the ranks (BASELINE config 3) ----
    strong = None
    if world > 1:
        b, e = shard.shard_bounds(BATCH, world, rank)
        sarms = Arms(e - b, 2000 + rank)
        sarms.warm(3)
        s_dev = median([sarms.resident_region(args.steps)[0] for _ in range(5)])
        s_e2e = median([sarms.e2e_region(args.steps)[0] for _ in range(5)])
        sarms.close()
        strong = dict(global_batch=BATCH, per_gpu_batch=e - b,
                      value=BATCH * args.steps / (s_dev * 1e-3),
                      ms_per_step=s_dev / args.steps,
                      e2e_value=BATCH * args.steps / (s_e2e * 1e-3),
                      e2e_ms_per_step=s_e2e / args.steps,
                      note="global batch 256 split contiguously over the ranks, one DeviceModel per "
                           "shard size, host-side concatenation of the logits; median of 5 regions")
    probe = h2d_probe(group, local_rank, arms.in_bytes) if world > 1 else None

    # ---- rank 0: roofline, parity of the timed network, side configurations, CPU baseline ----
    roofline = cpu_baseline = extra = None
    parity_checked = 0
    if rank == 0:
        from megcc_b200 import ops as mops
        peaks = load_peaks()
        rates = dict(i8=mops.measure_mma_rate("i8"), tf32=mops.measure_mma_rate("tf32"))
        net = arms.net
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
        # after its space-to-depth step); "a+b" is ConvBias a with the elementwise b fused in
        conv_of = lambda n: n.split("+")[0]
        umma = [(conv_of(n), ms) for n, s, ms, c in rows if conv_of(n) in conv_ops and c]
        umma_ops = sum(conv_ops[n] for n, _ in umma)
        umma_ms = sum(ms for _, ms in umma)
        achieved = umma_ops / (umma_ms * 1e-3) / 1e12 if umma_ms > 0 else 0.0
        step_tops = sum(conv_ops.values()) / (ms_dev / args.steps * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_sustained"]
        roofline = dict(
            bound="tensor",
            kernel="conv_umma_kernel / conv_patch_kernel (tcgen05 kind::i8 implicit GEMM)",
            achieved=achieved, peak=peak, unit="TOP/s", frac=achieved / peak,
            traffic=CONV_DRAM_BYTES_PER_STEP, traffic_unit="bytes per step",
            traffic_note="dram__bytes_read.sum + dram__bytes_write.sum of the 21 tensor-core "
                         "launches of one forward at batch 256, one ncu capture "
                         "(profiles/resnet18_int8_b256_dram_traffic_per_kernel.md); below the "
                         "1.4 GB of algorithmic bytes because L2 keeps the smaller feature maps",
            launches_per_step=len(umma), share_of_step=umma_ms / total_ms if total_ms else None,
            peak_note=f"2 x bf16 sustained ({peaks['source']}); MEASURED_PEAKS.json holds no int8 "
                      "figure, so the other denominators are listed beside it",
            frac_vs_2x_bf16_sustained=achieved / (2.0 * peaks["bf16_sustained"]),
            frac_vs_2x_bf16_burst=achieved / (2.0 * peaks["bf16_burst"]),
            frac_vs_int8_issue_rate=achieved / rates["i8"],
            frac_vs_nominal_dense_int8=achieved / 4500.0,
            int8_issue_rate_tops=rates["i8"], tf32_issue_rate_tflops=rates["tf32"],
            step_level=dict(
                tops=step_tops, frac_vs_2x_bf16_sustained=step_tops / peak,
                frac_vs_int8_issue_rate=step_tops / rates["i8"],
                note="all ConvBias operations / the CUDA-graph step time (launch gaps and the "
                     "three bandwidth kernels included); `achieved` divides by event times of the "
                     "tensor-core launches issued one by one, which include launch latency"),
            per_kernel_ms={n: round(ms, 4) for n, s, ms, c in rows})

        # parity of the very networks that were timed: 8 of the 256 images through the CPU
        # checker against the logits of the device-resident arm's network and of one
        # end-to-end network (outside every timed region)
        from oracle import netwalk
        from oracle import oracle as O
        idx = list(range(0, BATCH, BATCH // 8))[:8]
        want = netwalk.run(spec, arms.x_np[idx], O).reshape(len(idx), -1)
        n0 = arms.nets[0]
        n0.forward()
        n0.wait()
        got = n0.output("fc:out").reshape(BATCH, -1)[idx]
        net.forward()
        net.wait()
        dev_logits = torch.empty(arms.out_bytes, dtype=torch.int8, device=f"cuda:{local_rank}")
        # device-to-device copy of the logits through the library (a [1][bytes] relayout)
        import ctypes as C
        from megcc_b200._lib import check, lib
        check(lib().mb200_relayout_nchw_to_nhwc_s8(
            C.c_void_p(net.output_ptr("fc:out")), C.c_void_p(dev_logits.data_ptr()), 1, 1, 1,
            arms.out_bytes, C.c_void_p(net.stream())))
        torch.cuda.synchronize()
        got_dev = dev_logits.cpu().numpy().reshape(BATCH, -1)[idx]
        if not ((got == want).all() and (got_dev == want).all()):
            raise AssertionError("the benchmarked network's logits differ from the CPU checker")
        parity_checked = len(idx)

        if not args.skip_extras:
            try:
                extra = other_configs(local_rank, rates)
            except Exception as e:  # never lose the headline line to a side measurement
                extra = dict(error=repr(e))
            if affinity_before is not None:
                os.sched_setaffinity(0, affinity_before)  # the CPU leg uses every host core
            ips_cpu, sec, kind = cpu_reference_run(2, 1, threads)
            cpu_baseline = dict(
                value=ips_cpu, unit=UNIT, cores=threads, kind=kind,
                sample=f"2 steps x {threads} images (one pinned process of the reference's "
                       "single-threaded C runtime per host core, LITE_forward on the BARE_METAL "
                       "DeviceModel of the same network at batch 1), 1 warm-up forward")
    arms.close()
    group.close()
    if rank != 0:
        return
    images = BATCH * world * args.steps
    spread = lambda v: dict(regions=len(v), ms_per_step_min=min(v) / args.steps,
                            ms_per_step_median=median(v) / args.steps,
                            ms_per_step_max=max(v) / args.steps)
    line = dict(
        metric=METRIC, value=images / (ms_dev * 1e-3), unit=UNIT, n_gpus=world, steps=args.steps,
        warmup=max(args.warmup, 3), ms_per_step=ms_dev / args.steps, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="int8", data="synthetic", config=config,
        clocks=clocks, gpu_launches=ops_per_step * args.steps,
        timing=dict(note="the region of `steps` steps is repeated; value and e2e are the median "
                         "region, each region timed on the device, max over ranks",
                    resident=spread(dev_ms), e2e=spread(e2e_ms)),
        e2e=dict(value=images / (ms_e2e * 1e-3), unit=UNIT, ms_per_step=ms_e2e / args.steps,
                 h2d_bytes_per_step=arms.in_bytes, d2h_bytes_per_step=arms.out_bytes),
        parity_checked=parity_checked, strong_scaling=strong, h2d_probe=probe,
        roofline=roofline, cpu_baseline=cpu_baseline, other_configs=extra)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
