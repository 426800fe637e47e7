"""One artefact for both runtimes: the compile side can write a BARE_METAL DeviceModel (the
network as the reference's own x86 kernels) beside the CUDA one. Here the reference's C
runtime, compiled unmodified from its sources together with the reference's generated kernels
(oracle/_ref/ref_lite_runner), loads such a model through its own LITE_* API and must produce
what the CPU checker computes layer by layer. No GPU involved."""
import os
import subprocess

import numpy as np
import pytest

import cases
from oracle import netwalk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "oracle", "_ref", "ref_lite_runner")
DUMP = os.path.join(ROOT, "oracle", "_ref", "ref_tinynn_dump")

pytestmark = pytest.mark.skipif(not os.path.exists(RUNNER),
                                reason="oracle/_ref/ref_lite_runner not built (needs the "
                                       "reference tree)")


def run_reference_runtime(model, x, tmp_path, iterations=1):
    (tmp_path / "m.tiny").write_bytes(model)
    np.ascontiguousarray(x).tofile(tmp_path / "in.bin")
    r = subprocess.run([RUNNER, str(tmp_path / "m.tiny"), str(tmp_path / "in.bin"),
                        str(tmp_path / "out.bin"), str(iterations)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "forward_ms" in r.stdout
    return np.fromfile(tmp_path / "out.bin", dtype=np.int8)


@pytest.mark.parametrize("which,batch", [("resnet18", 2), ("mobilenet_v1", 1)])
def test_reference_runtime_runs_the_bare_metal_device_model(oracle, tmp_path, which, batch):
    from megcc_b200 import zoo
    spec = getattr(zoo, which)(hw=64, classes=64)
    g = spec.to_graph()
    g.set_option("bare_metal_model", 2)
    model = g.compile([batch])
    x = cases.rng_for("bare_metal_" + which).integers(-128, 128, (batch, 3, 64, 64), dtype=np.int8)
    got = run_reference_runtime(model, x, tmp_path, iterations=2)
    want = netwalk.run(spec, x, oracle).reshape(-1)
    assert got.shape == want.shape and (got == want).all()
    assert len(np.unique(want)) > 4


def test_both_device_models_in_one_file(tmp_path):
    """Option 1: the reference's flatcc reader sees a BARE_METAL (0) and a CUDA_SM100 (7)
    DeviceModel over one weight pool; this repository's loader accepts the file (it takes the
    CUDA ones). The BARE_METAL model has one Opr per operator of the network, named as the
    reference names its kernels."""
    import ctypes as C

    from megcc_b200 import _lib, zoo
    g = zoo.resnet18(hw=64, classes=64).to_graph()
    g.set_option("bare_metal_model", 1)
    model = g.compile([1, 4])
    (tmp_path / "dual.tiny").write_bytes(model)
    out = subprocess.run([DUMP, str(tmp_path / "dual.tiny")], capture_output=True, text=True,
                         check=True).stdout
    devices = [l.split("device=")[1].split()[0] for l in out.splitlines()
               if l.startswith("device_model")]
    assert devices == ["7", "7", "0", "0"]
    bare = out[out.index("device=0"):]
    oprs = [l.split()[1] for l in bare.splitlines() if l.startswith("opr ")]
    assert len(oprs) == 2 * 31 and all(o.startswith("kernel_") for o in oprs)
    assert "kernel_conv2d_7x7_NCHW_DENSE_p3x3_s2x2_d1x1_qsi8qsi8qsi32qsi8_bias_RELU" in oprs
    assert "kernel_elementwise_multitype_QFUSE_ADD_RELU_qsi8qsi8qsi8" in oprs
    buf = C.create_string_buffer(4 << 20)
    assert _lib.lib().mb200_tinynn_describe(model, len(model), buf, len(buf)) == 0


def test_operators_without_a_reference_kernel_are_refused():
    """Per-channel filter scales are an extension the reference cannot express."""
    from megcc_b200 import zoo
    from megcc_b200.compiler import CompileError
    g = zoo.resnet18(hw=64, classes=64, per_channel=True).to_graph()
    g.set_option("bare_metal_model", 1)
    with pytest.raises(CompileError) as e:
        g.compile([1])
    assert "BARE_METAL" in str(e.value)
