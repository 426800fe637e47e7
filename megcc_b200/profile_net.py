"""Runs whole forwards of an int8 network of the zoo (random weights) through the LITE_*
runtime without a CUDA graph, so that a profiler lists every kernel of a forward as its own
launch:

    python -m megcc_b200.profile_net [batch=64] [resnet18|mobilenetv1|yolox_s] [times]

    ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum \
        --clock-control none -k regex:"conv_|pooling_|space_to_depth" -s 24 -c 24 --csv \
        python -m megcc_b200.profile_net 64

(-s 24 skips the first ResNet-18 forward's 24 launches; filter packing at load has other
kernel names.) With `times` the runtime's own per-instruction CUDA-event timings (mean of
five forwards) are printed instead: name, kernel symbol, microseconds.
"""
import sys

import numpy as np

from . import lite, zoo

MODELS = {"resnet18": zoo.resnet18, "mobilenetv1": zoo.mobilenet_v1, "yolox_s": zoo.yolox_s}


def main(batch=64, model_name="resnet18", times=False, forwards=3):
    spec = MODELS[model_name]()
    model = spec.to_graph().compile([batch])
    net = lite.Network(model)
    net.set_option("use_graph", 0)
    if model_name == "yolox_s":  # the fp32 detector, 640 x 640
        x = np.random.default_rng(0).uniform(0, 1, (batch, 3, 640, 640)).astype(np.float32)
    else:
        x = np.random.default_rng(0).integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8)
    net.set_input("data", x)
    for _ in range(forwards):
        net.forward()
        net.wait()
    if times:
        rounds = 5
        acc = {}
        net.set_profile(True)
        for _ in range(rounds):
            net.forward()
            net.wait()
            for name, symbol, ms, _ in net.profile():
                acc.setdefault(name, [symbol, 0.0])[1] += ms / rounds
        net.set_profile(False)
        for name, (symbol, ms) in acc.items():
            print(f"{name:24s} {symbol:84s} {ms * 1e3:8.1f} us")
        total = sum(v[1] for v in acc.values())
        print(f"total {total:.4f} ms, {batch / total * 1e3:.0f} img/s (instructions timed one by one)")
    else:
        print("first outputs", net.output(net.output_names()[0], dtype=x.dtype)[:8])
    net.close()


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 64,
         sys.argv[2] if len(sys.argv) > 2 else "resnet18",
         len(sys.argv) > 3 and sys.argv[3] == "times")
