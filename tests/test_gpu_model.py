"""Whole compiled models through the LITE_* C API on the GPU, against the CPU checker
walking the same layer list (bit-exact int8 outputs)."""
import numpy as np
import pytest

import cases
import golden_util as G
from oracle import netwalk

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lite():
    assert torch.cuda.is_available()
    from megcc_b200 import lite as L
    return L


def run_model(lite, model, x, out_shape, forwards=1, device_io=()):
    net = lite.Network(model, device_io=device_io)
    name_in, name_out = net.input_names()[0], net.output_names()[0]
    outs = []
    for _ in range(forwards):
        net.set_input(name_in, x)
        net.forward()
        net.wait()
        outs.append(net.output(name_out).reshape(out_shape))
    net.close()
    return outs


def test_single_conv_model_matches_golden(lite):
    from megcc_b200 import zoo
    for dst_scale in (0.1, 5.0):
        c = cases.conv_cfg1(dst_scale)
        src, flt, bias = cases.conv_inputs(c)
        spec = zoo.single_conv(s_dst=dst_scale)
        spec.layers[0]["flt"], spec.layers[0]["bias"] = flt, bias
        model = spec.to_graph().compile([1])
        out = run_model(lite, model, src, (1, 64, 56, 56))[0]
        G.check("conv_bias_qs8", c["name"], out, src, flt, bias)


@pytest.mark.parametrize("per_channel", [False, True])
def test_resnet18_matches_oracle(lite, oracle, per_channel):
    from megcc_b200 import zoo
    spec = zoo.resnet18(per_channel=per_channel)
    x = cases.rng_for("resnet18_input").integers(-128, 128, (4, 3, 224, 224), dtype=np.int8)
    model = spec.to_graph().compile([4])
    want = netwalk.run(spec, x, oracle)
    # three forwards: eager pass, graph capture + launch, graph replay
    outs = run_model(lite, model, x, want.shape, forwards=3)
    for i, out in enumerate(outs):
        bad = int((out != want).sum())
        assert bad == 0, f"forward {i}: {bad}/{want.size} logits differ"
    assert len(np.unique(want)) > 8


def test_resnet18_without_fusion_matches_oracle(lite, oracle):
    """One instruction per operator (the residual adds as separate kernels)."""
    from megcc_b200 import zoo
    spec = zoo.resnet18(seed=2)
    x = cases.rng_for("resnet18_nofuse").integers(-128, 128, (4, 3, 224, 224), dtype=np.int8)
    g = spec.to_graph()
    g.set_option("fuse_conv_elemwise", 0)
    g.set_option("fuse_conv_pooling", 0)
    want = netwalk.run(spec, x, oracle)
    out = run_model(lite, g.compile([4]), x, want.shape, forwards=2)[1]
    assert (out == want).all()


def test_resnet18_with_stem_and_max_pool_as_one_instruction(lite, oracle):
    """The opt-in ConvBias + MAX pooling fusion: the stem never stores its 112 x 112 result."""
    from megcc_b200 import zoo
    spec = zoo.resnet18(seed=3)
    x = cases.rng_for("resnet18_poolfuse").integers(-128, 128, (4, 3, 224, 224), dtype=np.int8)
    g = spec.to_graph()
    g.set_option("fuse_conv_pooling", 1)
    model = g.compile([4])
    assert any(s.endswith("_pool_MAX3x3s2p1") for s in g.kernel_symbols())
    assert not any("pooling_MAX" in s for s in g.kernel_symbols())
    want = netwalk.run(spec, x, oracle)
    for out in run_model(lite, model, x, want.shape, forwards=3):
        assert (out == want).all()


def test_resnet18_reference_kernels_agree(lite, reference):
    """Same check against the reference's own x86 kernels chained layer by layer."""
    from megcc_b200 import zoo
    spec = zoo.resnet18(seed=1)
    x = cases.rng_for("resnet18_ref_input").integers(-128, 128, (1, 3, 224, 224), dtype=np.int8)
    want = netwalk.run(spec, x, reference, use_reference=True)
    out = run_model(lite, spec.to_graph().compile([1]), x, want.shape)[0]
    assert (out == want).all()


def test_mobilenet_v1_matches_oracle(lite, oracle):
    from megcc_b200 import zoo
    spec = zoo.mobilenet_v1()
    x = cases.rng_for("mbv1_input").integers(-128, 128, (2, 3, 224, 224), dtype=np.int8)
    want = netwalk.run(spec, x, oracle)
    outs = run_model(lite, spec.to_graph().compile([2]), x, want.shape, forwards=2)
    assert (outs[0] == want).all() and (outs[1] == want).all()


def test_matmul_instruction_in_a_model_matches_oracle(lite, oracle):
    """conv -> global average pool -> MatrixMul + TypeCvt through the compiler and the
    runtime (graph replay on the third forward), against the oracle's exact integer product
    and the reference's TypeCvt rule. Batch 200: the product runs on the tensor cores."""
    from megcc_b200.compiler import Graph
    rng = np.random.default_rng(11)
    n = 200
    g = Graph("gap_matmul")
    x = g.input("data", 64, 8, 8, 0.05)
    f = rng.integers(-127, 128, (64, 64, 3, 3), dtype=np.int8)
    y = g.conv_bias("conv", x, f, None, 1, 1, 0.01, 0.9, "RELU")
    y = g.pooling("gap", y, "AVERAGE", 8, 8, 0)
    b = rng.integers(-127, 128, (64, 200), dtype=np.int8)
    y = g.matmul("fc", y, b, 0.01, 25.0)
    g.mark_output(y)
    model = g.compile([n])
    src = rng.integers(-128, 128, (n, 64, 8, 8), dtype=np.int8)
    conv = oracle.conv_bias_qs8(src, f, None, 1, 1, 0.05, 0.01, 0.9, "RELU")
    pooled = oracle.pooling_qs8(conv, "AVERAGE", 8, 8, 0).reshape(n, 64)
    acc = oracle.matmul_s8_s32(pooled, b)
    want = oracle.typecvt_qs32_qs8(acc, float(np.float32(0.9) * np.float32(0.01)), 25.0)
    for out in run_model(lite, model, src, (n, 200), forwards=3):
        assert (out == want).all()
    assert (np.abs(want.astype(int)) < 127).mean() > 0.3


def test_three_networks_in_flight_with_large_host_inputs(lite, oracle):
    """Three networks of one model on one GPU, each given a different 9.6 MB host input
    (large enough to be copied in four pieces on the side streams), forwards enqueued before
    any wait and collected out of order, twice: every network's output must be its own
    input's result. Exercises the split copy and the one-after-the-other ordering of the
    networks' kernel sequences."""
    from megcc_b200 import zoo
    n = 64
    spec = zoo.single_conv(ic=3, oc=64, hw=224, k=7, stride=2, pad=3, s_src=0.02, s_flt=0.01,
                           s_dst=0.5)
    flt, bias = spec.layers[0]["flt"], spec.layers[0]["bias"]
    model = spec.to_graph().compile([n])
    rng = np.random.default_rng(5)
    nets = [lite.Network(model) for _ in range(3)]
    name_in, name_out = nets[0].input_names()[0], nets[0].output_names()[0]
    for rnd in range(2):
        xs = [rng.integers(-128, 128, (n, 3, 224, 224), dtype=np.int8) for _ in nets]
        for net, x in zip(nets, xs):
            net.set_input(name_in, x)
            net.forward()
        for i in (2, 0, 1):
            nets[i].wait()
            out = nets[i].output(name_out).reshape(n, 64, 112, 112)
            want = oracle.conv_bias_qs8(xs[i], flt, bias, 2, 3, 0.02, 0.01, 0.5, "RELU")
            assert (out == want).all(), (rnd, i)
    for net in nets:
        net.close()


def test_batch_variants_and_device_io(lite, oracle):
    from megcc_b200 import zoo
    spec = zoo.resnet18(hw=64, classes=100)
    model = spec.to_graph().compile([1, 3])
    net = lite.Network(model, device_io=("fc:out",))
    x3 = cases.rng_for("variants").integers(-128, 128, (3, 3, 64, 64), dtype=np.int8)
    want3 = netwalk.run(spec, x3, oracle)
    # DeviceModel 0 is the batch-1 variant; selecting the batch-3 layout switches models
    net.select_batch("data", (3, 3, 64, 64))
    assert net.tensor_bytes("data") == x3.nbytes
    xd = torch.from_numpy(x3).cuda()
    for _ in range(3):
        net.set_input_ptr("data", xd.data_ptr(), x3.nbytes)  # device memory, used in place
        net.forward()
        net.wait()
    import ctypes
    ptr = net.output_ptr("fc:out")  # device pointer: declared with is_host = 0
    rt = ctypes.CDLL("/usr/local/cuda/lib64/libcudart.so")
    host = np.empty(want3.size, np.int8)
    # kind 2 = device to host: fails if ptr were host memory
    rc = rt.cudaMemcpy(ctypes.c_void_p(host.ctypes.data), ctypes.c_void_p(ptr),
                       ctypes.c_size_t(want3.size), 2)
    assert rc == 0
    assert (host.reshape(want3.shape) == want3).all()
    net.select_batch("data", (1, 3, 64, 64))
    net.set_input("data", x3[:1])
    net.forward()
    net.wait()
    net.close()


def test_api_errors(lite):
    from megcc_b200 import zoo
    model = zoo.single_conv(hw=16).to_graph().compile([1])
    with pytest.raises(lite.LiteError) as e:
        lite.Network(model[:100])
    assert e.value.status == 7
    net = lite.Network(model)
    with pytest.raises(lite.LiteError) as e:
        net.forward()  # no input memory yet
    assert e.value.status == 1
    with pytest.raises(lite.LiteError) as e:
        net.set_input("data", np.zeros(5, np.int8))  # wrong byte count
    assert e.value.status == 13
    with pytest.raises(lite.LiteError) as e:
        net.tensor("nonexistent")
    assert e.value.status == 5
    net.close()


def _sampled_parity(lite, oracle, spec, batch, name, samples=4, forwards=2):
    """Runs `batch` images on the GPU and checks `samples` of them, spread over the batch,
    against the CPU checker (images are independent, so a subset proves the rest of the
    batch's code path: tile tails, wave boundaries, the kernel choice made for this batch)."""
    x = cases.rng_for(name).integers(-128, 128, (batch, 3, 224, 224), dtype=np.int8)
    idx = sorted({int(i) for i in np.linspace(0, batch - 1, min(samples, batch))})
    want = netwalk.run(spec, x[idx], oracle).reshape(len(idx), -1)
    outs = run_model(lite, spec.to_graph().compile([batch]), x, (batch, want.shape[1]),
                     forwards=forwards)
    for out in outs:
        assert (out[idx] == want).all()
    assert len(np.unique(want)) > 8


@pytest.mark.parametrize("batch", [32, 64, 128, 256])
def test_resnet18_at_the_benchmarked_and_sharded_batch_sizes(lite, oracle, batch):
    """Batch 256 is the benchmark's; 128 / 64 / 32 are its shards over 2 / 4 / 8 GPUs. The
    kernel selection changes with the batch (tile width, patch kernel, small-activation
    path), so each size is a different set of launches."""
    from megcc_b200 import zoo
    _sampled_parity(lite, oracle, zoo.resnet18(), batch, f"resnet18_b{batch}")


@pytest.mark.parametrize("batch", [1, 64, 256])
@pytest.mark.parametrize("per_channel", [False, True])
def test_mobilenet_v1_at_the_benchmarked_batch_sizes(lite, oracle, batch, per_channel):
    """MobileNetV1 at batch 1 (latency), 64 and 256, with one filter scale per tensor and with
    one per output channel (the form the configuration names; an extension over the reference,
    checked against the same formula with flt_scale[oc]). From batch 64 up the stride-1
    depthwise layers over 128, 256 and 512 channels run on the tensor cores."""
    from megcc_b200 import zoo
    _sampled_parity(lite, oracle, zoo.mobilenet_v1(per_channel=per_channel), batch,
                    f"mbv1_b{batch}_{per_channel}")


def test_resnet18_per_channel_scales_at_batch_256(lite, oracle):
    from megcc_b200 import zoo
    _sampled_parity(lite, oracle, zoo.resnet18(per_channel=True), 256, "resnet18_pc_b256",
                    samples=3)


# ---- models as MegCC's --enable_nchw44 hands them over ----
@pytest.mark.parametrize("which", ["resnet18", "mobilenet_v1"])
def test_nchw44_models_match_oracle(lite, oracle, which):
    """Filters in the NCHW44 layouts (first-layer form on the NCHW image, dense,
    channel-wise), repacked by the Init step at load; the logits come back as
    [N, C/4, 1, 1, 4], which for one pixel is the channel order."""
    from megcc_b200 import zoo
    spec = getattr(zoo, which)()
    x = cases.rng_for(which + "_nchw44").integers(-128, 128, (4, 3, 224, 224), dtype=np.int8)
    g = spec.to_graph(nchw44=True)
    model = g.compile([4])
    assert all("_NHWC44" in s for s in g.kernel_symbols() if "conv2d" in s)
    want = netwalk.run(spec, x, oracle)
    for out in run_model(lite, model, x, want.shape, forwards=3):
        assert (out == want).all()


@pytest.mark.parametrize("batch", [1, 5])
def test_nchw44_input_and_spatial_output(lite, oracle, batch):
    spec = cases.nchw44_block_spec()
    x = cases.rng_for("nchw44_block").integers(-128, 128, (batch, 16, 30, 34), dtype=np.int8)
    want = oracle.nchw_to_nchw44(netwalk.run(spec, x, oracle))
    model = spec.to_graph(nchw44=True).compile([batch])
    assert want.shape == (batch, 24, 15, 17, 4)
    for out in run_model(lite, model, oracle.nchw_to_nchw44(x), want.shape, forwards=3):
        assert (out == want).all()


def test_nchw44_model_through_generated_kernel_tables(lite, oracle, tmp_path):
    """The same block with every Opr run as kernels[kernel_id](...) from stubs compiled as C:
    the NCHW44 Init stub repacks the filter, the Relayout stubs convert at the boundary."""
    from test_gpu_kernel_tables import build_kernel_library, tables
    spec = cases.nchw44_block_spec(seed=1)
    x = cases.rng_for("nchw44_tables").integers(-128, 128, (3, 16, 30, 34), dtype=np.int8)
    want = oracle.nchw_to_nchw44(netwalk.run(spec, x, oracle))
    g = spec.to_graph(nchw44=True)
    model = g.compile([3])
    handle, n = build_kernel_library(g, str(tmp_path))
    net = lite.Network(model, kernel_tables=tables(handle, n))
    for _ in range(2):
        net.set_input("data", oracle.nchw_to_nchw44(x))
        net.forward()
        net.wait()
        assert (net.output(net.output_names()[0]).reshape(want.shape) == want).all()
    net.close()


def test_model_with_a_bare_metal_device_model_beside_the_cuda_one(lite, oracle):
    """One artefact for both runtimes (tests/test_bare_metal_model.py runs the other half on
    the reference's C runtime): this runtime takes the CUDA DeviceModels of the file."""
    from megcc_b200 import zoo
    spec = zoo.resnet18(seed=5)
    x = cases.rng_for("dual_model").integers(-128, 128, (2, 3, 224, 224), dtype=np.int8)
    g = spec.to_graph()
    g.set_option("bare_metal_model", 1)
    want = netwalk.run(spec, x, oracle)
    out = run_model(lite, g.compile([2]), x, want.shape, forwards=2)[1]
    assert (out == want).all()


def test_cycling_device_input_buffers_replays_captured_graphs(lite, oracle):
    """A caller that alternates between a few device input buffers: each address gets its own
    captured graph, kept (up to four) and replayed, and every forward is still bit-exact."""
    from megcc_b200 import zoo
    spec = zoo.resnet18(hw=64, classes=64, seed=7)
    model = spec.to_graph().compile([8])
    net = lite.Network(model)
    name_in, name_out = net.input_names()[0], net.output_names()[0]
    r = cases.rng_for("cycle_inputs")
    xs = [r.integers(-128, 128, (8, 3, 64, 64), dtype=np.int8) for _ in range(3)]
    wants = [netwalk.run(spec, x, oracle).reshape(-1) for x in xs]
    devs = [torch.from_numpy(x).cuda() for x in xs]
    for turn in range(4):  # eager pass, three captures, then replays only
        for d, want in zip(devs, wants):
            net.set_input_ptr(name_in, d.data_ptr(), d.numel())
            net.forward()
            net.wait()
            assert (net.output(name_out) == want).all(), turn
    net.close()
