"""Batch sharding host logic with two gloo ranks on the CPU: every image is owned exactly
once, per-rank results concatenate back in order, and timings reduce to the slowest rank."""
import os
import socket
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import sys, os
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np
from megcc_b200 import shard, zoo
from oracle import oracle as O
from oracle import netwalk
g = shard.Group("gloo")
spec = zoo.resnet18(hw=32, classes=16)
x = np.random.default_rng(5).integers(-128, 128, (5, 3, 32, 32), dtype=np.int8)
b, e = shard.shard_bounds(len(x), g.world, g.rank)
mine = netwalk.run(spec, x[b:e], O)            # this rank's slice through the CPU checker
full = g.gather_concat(mine)
slowest = g.max(10.0 + g.rank)
total = g.sum(e - b)
g.barrier()
if g.rank == 0:
    want = netwalk.run(spec, x, O)
    assert full.shape == want.shape and (full == want).all()
    assert slowest == 10.0 + g.world - 1 and total == len(x)
    print("OK", g.world, b, e)
g.close()
"""


def test_shard_bounds_partition_every_batch():
    from megcc_b200.shard import shard_bounds
    for batch in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "OK 2 0 3" in outs[0]
