"""Batch sharding across the GPUs of one box: one process per GPU, each with its own network,
arena and CUDA graph; no data-path collective. torch.distributed carries only the barrier
and the reduction of the timings (NCCL on GPUs, gloo in the CPU tests)."""
import os


def env_rank():
    """(rank, local_rank, world_size) from the torchrun environment (1 process if unset)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def shard_bounds(global_batch, world, rank):
    """Contiguous slice [begin, end) of a global batch owned by ``rank``; the first
    ``global_batch % world`` ranks take one extra image."""
    if world <= 0 or not 0 <= rank < world or global_batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(global_batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class Group:
    """Barrier and max/sum reductions over the ranks; a no-op group for one process."""

    def __init__(self, backend=None, device=None):
        self.rank, self.local_rank, self.world = env_rank()
        self.device = device
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if not dist.is_initialized():
                kwargs = {}
                if backend == "nccl" and device is not None:
                    kwargs["device_id"] = device
                dist.init_process_group(backend or "gloo", **kwargs)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def _reduce(self, value, op):
        if not self.dist:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64,
                         device=self.device if self.device is not None else "cpu")
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, value):
        return self._reduce(value, self.dist.ReduceOp.MAX if self.dist else None)

    def sum(self, value):
        return self._reduce(value, self.dist.ReduceOp.SUM if self.dist else None)

    def gather_concat(self, array):
        """Host-side concatenation of per-rank output slices on every rank (rank order)."""
        if not self.dist:
            return array
        import numpy as np
        objs = [None] * self.world
        self.dist.all_gather_object(objs, array)
        return np.concatenate(objs, axis=0)

    def close(self):
        if self.dist and self.dist.is_initialized():
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.dist = None


def bind_to_gpu_cpus(device_index):
    """Restrict this process to the CPUs next to GPU ``device_index`` (the PCI device's
    ``local_cpulist`` in sysfs), so that pinned staging buffers allocated afterwards land on
    the GPU's NUMA node. Returns the previous affinity set for ``os.sched_setaffinity`` to
    restore, or None when nothing was changed (no sysfs entry, an empty list, no permission)."""
    import os
    try:
        import torch
        pr = torch.cuda.get_device_properties(device_index)
        bdf = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        with open("/sys/bus/pci/devices/%s/local_cpulist" % bdf) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            if not part:
                continue
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        before = os.sched_getaffinity(0)
        cpus &= before
        if not cpus or cpus == before:
            return None
        os.sched_setaffinity(0, cpus)
        return before
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None
