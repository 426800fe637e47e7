"""Runs whole forwards of ResNet-18 int8 (random weights, batch = first argument, default 64)
through the LITE_* runtime without a CUDA graph, so that a profiler lists every kernel of a
forward as its own launch:

    ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum \
        --clock-control none -k regex:"conv_|pooling_|space_to_depth" -s 24 -c 24 --csv \
        python -m megcc_b200.profile_net 64

(-s 24 skips the first forward's 24 launches; filter packing at load has other kernel names.)
"""
import sys

import numpy as np

from . import lite, zoo


def main(batch=64, forwards=3):
    spec = zoo.resnet18()
    model = spec.to_graph().compile([batch])
    net = lite.Network(model)
    net.set_option("use_graph", 0)
    x = np.random.default_rng(0).integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8)
    for _ in range(forwards):
        net.set_input("data", x)
        net.forward()
        net.wait()
    print("logits", net.output(net.output_names()[0])[:8])
    net.close()


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 64)
