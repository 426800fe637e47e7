"""The generated-code path end to end: the compile side exports kernels.h / kernels.c / one
<symbol>.c per kernel exactly as the reference's exporter lays them out
(compiler/lib/Target/TinyNN/KernelExporter.cpp:15-66), a C compiler turns them into a library,
its tables are registered with the runtime, and every Opr of the model then runs as
kernels[kernel_id](inputs, nr_input, outputs, nr_output, &workspace, &opt) with its weights
prepared by init_kernels[init_id] (runtime/src/vm/op.c:161-163, runtime/src/init.c:29-131)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import cases
from oracle import netwalk

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_kernel_library(graph, directory):
    """gcc -std=c99 over the exported stubs -> libkernels.so; returns (handle, nr_kernels)."""
    from megcc_b200 import _lib
    graph.export_kernels(directory)
    srcs = sorted(f for f in os.listdir(directory) if f.endswith(".c"))
    so = os.path.join(directory, "libkernels.so")
    subprocess.run(["gcc", "-std=c99", "-O1", "-fPIC", "-shared", "-Wall", "-Werror",
                    "-I", os.path.join(ROOT, "include"), "-I", directory, "-o", so]
                   + [os.path.join(directory, f) for f in srcs]
                   + ["-L", os.path.dirname(_lib.LIB_PATH), "-lmegcc_b200",
                      "-Wl,-rpath," + os.path.dirname(_lib.LIB_PATH),
                      # several generated libraries may live in one process (as here): each
                      # binds its own kernels[] / init_kernels[]
                      "-Wl,-Bsymbolic"], check=True)
    _lib.lib()  # the operator library is resident before the stubs that call into it
    handle = C.CDLL(so)
    handle.load_kernel_init_function()
    return handle, len(graph.kernel_symbols())


def tables(handle, n):
    k = (C.c_void_p * n).in_dll(handle, "kernels")
    i = (C.c_void_p * n).in_dll(handle, "init_kernels")
    assert all(k[j] for j in range(n)) and all(i[j] for j in range(n))
    return C.addressof(k), n, C.addressof(i), n


def test_resnet18_runs_through_the_generated_kernel_tables(oracle, tmp_path):
    from megcc_b200 import lite, zoo
    spec = zoo.resnet18(hw=64, classes=64)
    x = cases.rng_for("kernel_tables_resnet").integers(-128, 128, (8, 3, 64, 64), dtype=np.int8)
    g = spec.to_graph()
    g.set_option("fuse_conv_pooling", 1)  # the stem + max-pool stub as well
    model = g.compile([8])
    assert any(s.endswith("_pool_MAX3x3s2p1") for s in g.kernel_symbols())
    handle, n = build_kernel_library(g, str(tmp_path))
    want = netwalk.run(spec, x, oracle).reshape(-1)
    net = lite.Network(model, kernel_tables=tables(handle, n))
    for _ in range(3):  # eager, graph capture, graph replay: all through the stubs
        net.set_input("data", x)
        net.forward()
        net.wait()
        assert (net.output(net.output_names()[0]) == want).all()
    net.close()


def test_fp32_detector_runs_through_the_generated_kernel_tables(oracle, tmp_path):
    from megcc_b200 import lite, zoo
    spec = zoo.yolox_s(hw=128)
    x = cases.rng_for("kernel_tables_yolox").uniform(0, 1, (2, 3, 128, 128)).astype(np.float32)
    g = spec.to_graph()
    model = g.compile([2])
    handle, n = build_kernel_library(g, str(tmp_path))
    want = netwalk.run_f32(spec, x, oracle)
    net = lite.Network(model, kernel_tables=tables(handle, n))
    for _ in range(2):
        net.set_input("data", x)
        net.forward()
        net.wait()
        for name, w in zip(net.output_names(), want):
            got = net.output(name, dtype=np.float32).reshape(w.shape)
            assert np.abs(got - w).max() <= 1e-5 + 1e-4 * np.abs(w).max()
            assert (np.abs(got - w) <= 1e-5 + 1e-4 * np.abs(w)).all()
    net.close()


def test_a_symbol_the_library_does_not_know_runs_only_through_a_registered_table(oracle, tmp_path):
    """A third party's KernelFunc: the Opr's symbol means nothing to the runtime, dispatch is
    by kernel_id alone. Without a registered table the model is refused at load."""
    from megcc_b200 import lite
    from megcc_b200.compiler import Graph
    from megcc_b200.lite import LiteError
    r = cases.rng_for("foreign_symbol")
    g = Graph("foreign")
    t = g.input("data", 64, 20, 20, 0.05)
    f = r.integers(-127, 128, (64, 64, 3, 3), dtype=np.int8)
    b = r.integers(-1000, 1000, (64,), dtype=np.int32)
    t = g.conv_bias("conv", t, f, b, 1, 1, 0.01, 0.9, "IDENTITY")
    t = g.qelemwise("relu", "QRELU", t, None, 0.7)
    g.mark_output(t)
    model = g.compile([2])
    handle, n = build_kernel_library(g, str(tmp_path))
    old = b"cuda_sm100_elementwise_multitype_QRELU_qsi8qsi8"
    new = b"thirdparty_elementwise_multitype_QRELU_qsi8qsi8"
    assert model.count(old) == 1 and len(old) == len(new)
    foreign = model.replace(old, new)
    x = r.integers(-128, 128, (2, 64, 20, 20), dtype=np.int8)
    conv = oracle.conv_bias_qs8(x, f, b, 1, 1, 0.05, 0.01, 0.9, "IDENTITY")
    want = oracle.qelemwise("QRELU", conv, None, 0.9, 1.0, 0.7)
    with pytest.raises(LiteError) as e:
        lite.Network(foreign)
    assert e.value.status == 5 and "thirdparty" in str(e.value)  # TinyNN_ERROR_NO_FOUND
    net = lite.Network(foreign, kernel_tables=tables(handle, n))
    net.set_input("data", x)
    net.forward()
    net.wait()
    got = net.output(net.output_names()[0]).reshape(want.shape)
    # the output is NHWC -> NCHW converted by the model's last instruction, also a stub
    assert (got == want).all()
    net.close()


def test_c_program_written_against_the_reference_headers_runs_on_this_library(oracle, tmp_path):
    """oracle/_ref/lite_c_driver was compiled with -I <reference>/runtime/include and linked
    against libmegcc_b200.so where the reference tree was present; here it only runs."""
    from megcc_b200 import zoo
    exe = os.path.join(ROOT, "oracle", "_ref", "lite_c_driver")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/lite_c_driver was not built (reference tree absent at build time)")
    spec = zoo.resnet18(hw=64, classes=64, seed=7)
    x = cases.rng_for("lite_c_driver").integers(-128, 128, (4, 3, 64, 64), dtype=np.int8)
    (tmp_path / "model.tiny").write_bytes(spec.to_graph().compile([4]))
    (tmp_path / "input.bin").write_bytes(x.tobytes())
    subprocess.run([exe, str(tmp_path / "model.tiny"), str(tmp_path / "input.bin"),
                    str(tmp_path / "output.bin"), "3"], check=True, timeout=120)
    got = np.frombuffer((tmp_path / "output.bin").read_bytes(), dtype=np.int8)
    assert (got == netwalk.run(spec, x, oracle).reshape(-1)).all()
