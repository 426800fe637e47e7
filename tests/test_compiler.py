"""Compile side on CPU: kernel selection through the KernelFunc interface, the static
memory plan, the tinynn writer (checked with our loader's parser AND with the reference's
own flatcc reader) and the generated host stubs."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def describe(model_bytes):
    from megcc_b200 import _lib
    buf = C.create_string_buffer(4 << 20)
    rc = _lib.lib().mb200_tinynn_describe(model_bytes, len(model_bytes), buf, len(buf))
    return rc, buf.value.decode()


def test_kernel_pack_symbols_follow_reference_naming():
    from megcc_b200.compiler import probe_conv_symbol
    ok, sym = probe_conv_symbol(64, 64, 56, 56, 3, 1, 1, nonline="RELU")
    assert ok
    # the reference's x86 symbol for the same operator is
    # kernel_conv2d_3x3_NCHW_DENSE_p1x1_s1x1_d1x1_qsi8qsi8qsi32qsi8_bias_RELU
    assert sym == "cuda_sm100_conv2d_3x3_NHWC_DENSE_p1x1_s1x1_d1x1_qsi8qsi8qsi32qsi8_bias_RELU"
    ok, sym = probe_conv_symbol(32, 32, 112, 112, 3, 2, 1, groups=32, nonline="H_SWISH", bias=False)
    assert ok and sym == "cuda_sm100_conv2d_3x3_NHWC_GROUP_p1x1_s2x2_d1x1_qsi8qsi8qsi32qsi8_H_SWISH"
    # admission is a subset of BareMetal::ConvGeneral::IsAvailable: what it refuses falls
    # through to the CPU kernels in the registry. NCHW44 is admitted with NCHW44 operands
    # only, not with the NCHW shapes this probe passes.
    assert not probe_conv_symbol(64, 64, 56, 56, 3, 1, 1, fmt="NCHW44")[0]
    assert not probe_conv_symbol(64, 64, 56, 56, 3, 1, 1, nonline="SIGMOID")[0]


def test_symbols_match_the_reference_kernels_one_to_one(reference):
    """Every CUDA symbol of the two models has a reference x86 kernel of the same family and
    attributes (the one the checker runs)."""
    from megcc_b200 import zoo
    for spec, pool in ((zoo.resnet18(), 0), (zoo.resnet18(), 1), (zoo.mobilenet_v1(), 0)):
        g = spec.to_graph()
        g.set_option("fuse_conv_pooling", pool)
        g.compile([1])
        assert any(s.endswith("_pool_MAX3x3s2p1") for s in g.kernel_symbols()) == bool(pool)
        for sym in g.kernel_symbols():
            ref = sym.replace("cuda_sm100_", "kernel_").replace("_NHWC_", "_NCHW_")
            if ref.endswith("_pool_MAX3x3s2p1"):
                # ConvBias + the MAX pooling behind it: two reference kernels as well
                assert reference.ref_has(ref[:-len("_pool_MAX3x3s2p1")]), sym
                assert reference.ref_has("kernel_pooling_MAX_NCHW_p1x1_s2x2_w3x3_qsi8qsi8"), sym
                continue
            m = re.match(r"(.*qsi8qsi8qsi32qsi8)qsi8(_bias)_z_(\w+)$", ref)
            if m:  # a fused instruction stands for two reference kernels run back to back
                assert reference.ref_has(m.group(1) + m.group(2)), sym
                assert reference.ref_has(
                    f"kernel_elementwise_multitype_{m.group(3)}_qsi8qsi8qsi8"), sym
                continue
            assert reference.ref_has(ref), f"{sym}: no reference kernel {ref}"


def _parse_plan(text, model=0):
    tensors, oprs, cur = {}, [], -1
    for line in text.splitlines():
        if line.startswith("device_model"):
            cur += 1
        if cur != model:
            continue
        m = re.match(r"tensor (\S+) offset=(\d+) bytes=(\d+)", line)
        if m:
            tensors[m.group(1)] = (int(m.group(2)), int(m.group(3)))
        m = re.match(r"opr (\S+) in=(\S*) out=(\S*) ws=(\d+)\+(\d+)", line)
        if m:
            k = len(oprs)
            oprs.append((m.group(1), [x for x in m.group(2).split(",") if x],
                         [x for x in m.group(3).split(",") if x]))
            if int(m.group(5)):  # a workspace is a buffer that lives for this instruction only
                tensors[f"ws:{k}"] = (int(m.group(4)), int(m.group(5)))
                oprs[-1][1].append(f"ws:{k}")
    return tensors, oprs


@pytest.mark.parametrize("net", ["resnet18", "mobilenet_v1"])
def test_memory_plan_never_overlaps_live_tensors(net):
    from megcc_b200 import zoo
    spec = getattr(zoo, net)()
    g = spec.to_graph()
    model = g.compile([1, 8])
    rc, text = describe(model)
    assert rc == 0
    for mi, batch in enumerate((1, 8)):
        tensors, oprs = _parse_plan(text, mi)
        first, last = {"data": 0}, {}
        for k, (_, ins, outs) in enumerate(oprs):
            for t in ins:
                if t in tensors:
                    first.setdefault(t, k)
                    last[t] = k
            for t in outs:
                first.setdefault(t, k)
                last[t] = max(last.get(t, k), k)
        last[oprs[-1][2][0]] = len(oprs)
        names = [t for t in tensors if t in first]
        for i, a in enumerate(names):
            for b in names[i + 1:]:
                if last[a] < first[b] or last[b] < first[a]:
                    continue
                (oa, sa), (ob, sb) = tensors[a], tensors[b]
                assert oa + sa <= ob or ob + sb <= oa, f"{a} and {b} overlap while both live"
        arena = g.arena_bytes(mi)
        assert all(o % 256 == 0 and o + s <= arena for o, s in tensors.values())
        # the first layer (stride 2, 3 input channels) gets scratch for its space-to-depth
        # tensor: N x 112 x 112 x 16 bytes
        assert tensors["ws:0"][1] == batch * 112 * 112 * 16
        assert arena < 0.5 * g.unplanned_bytes(mi), "the plan should reuse memory"


def test_reference_reader_accepts_our_model(tmp_path):
    """The reference's flatcc-generated reader sees the model we wrote."""
    tool = os.path.join(ROOT, "oracle", "_ref", "ref_tinynn_dump")
    if not os.path.exists(tool):
        pytest.skip("oracle/_ref not built")
    from megcc_b200 import zoo
    spec = zoo.resnet18()
    model = spec.to_graph().compile([2])
    path = tmp_path / "r18.tiny"
    path.write_bytes(model)
    out = subprocess.run([tool, str(path)], capture_output=True, text=True, check=True).stdout
    assert "model name=resnet18_int8" in out
    assert "device=7" in out  # CUDA_SM100, appended to the Device enum
    theirs = [l for l in out.splitlines() if l.startswith("tensor ")]
    rc, ours = describe(model)
    mine = [l for l in ours.splitlines() if l.startswith("tensor ")]
    assert rc == 0 and len(theirs) == len(mine) == 24  # inner results of fused pairs are gone
    for a, b in zip(theirs, mine):
        assert a.split()[1] == b.split()[1]
        assert re.search(r"offset=(\d+)", a).group(1) == re.search(r"offset=(\d+)", b).group(1)
        assert re.search(r"dims=(\S+)", a).group(1) == re.search(r"dims=(\S+)", b).group(1)
        assert re.search(r"stride=(\S+)", a).group(1) == re.search(r"stride=(\S+)", b).group(1)
    # weights arrive byte for byte
    w = [l for l in out.splitlines() if l.startswith("weight stem:filter")][0]
    assert "bytes=9408" in w and "dims=64x3x7x7" in w
    assert len([l for l in out.splitlines() if l.startswith("opr ")]) == 23
    # the same network with fusion off keeps one instruction per operator
    g2 = zoo.resnet18().to_graph()
    g2.set_option("fuse_conv_elemwise", 0)
    rc, plain = describe(g2.compile([2]))
    assert rc == 0 and len([l for l in plain.splitlines() if l.startswith("opr ")]) == 31


def test_truncated_and_corrupt_models_are_rejected_not_crashed():
    from megcc_b200 import zoo
    model = zoo.single_conv().to_graph().compile([1])
    assert describe(model)[0] == 0
    for cut in (0, 3, 7, 64, len(model) // 2, len(model) - 64):
        rc, _ = describe(model[:cut])
        assert rc in (5, 7), f"cut at {cut}: status {rc}"
    rng = np.random.default_rng(7)
    for _ in range(200):
        bad = bytearray(model)
        for pos in rng.integers(0, min(len(bad), 2000), 8):
            bad[pos] = int(rng.integers(0, 256))
        assert describe(bytes(bad))[0] in (0, 4, 5, 6, 7, 10, 11, 12)


def test_unknown_kernel_symbol_is_reported():
    from megcc_b200 import zoo
    model = zoo.single_conv().to_graph().compile([1])
    bad = model.replace(b"cuda_sm100_conv2d_3x3", b"cuda_sm100_conv9d_3x3")
    assert describe(bad)[0] == 5  # TinyNN_ERROR_NO_FOUND


def test_exported_stubs_compile_against_public_headers(tmp_path):
    """kernels.h / kernels.c / <symbol>.c, laid out like the reference exporter's output,
    compile as C against include/ and link against libmegcc_b200.so."""
    from megcc_b200 import zoo, _lib
    g = zoo.resnet18().to_graph()
    g.compile([1])
    g.export_kernels(str(tmp_path))
    files = sorted(os.listdir(tmp_path))
    assert "kernels.h" in files and "kernels.c" in files
    syms = g.kernel_symbols()
    assert all(s + ".c" in files for s in syms)
    srcs = [str(tmp_path / f) for f in files if f.endswith(".c")]
    so = str(tmp_path / "libkernels.so")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-shared", "-fPIC",
                    "-I" + os.path.join(ROOT, "include"), "-I" + str(tmp_path), "-o", so] + srcs
                   + [_lib.LIB_PATH], check=True)
    L = C.CDLL(so)
    L.load_kernel_init_function()
    tab = (C.c_void_p * len(syms)).in_dll(L, "kernels")
    assert all(tab[i] for i in range(len(syms)))


def test_nchw44_model_keeps_its_visible_layout_and_its_stubs_compile(tmp_path):
    """A model handed over as --enable_nchw44 would: filters stay in their NCHW44 layouts in
    the model file (the Init stub repacks them at load), the visible tensors are
    [N, C/4, H, W, 4], Relayout instructions sit at the boundary, and the stubs are C99."""
    from megcc_b200 import zoo, _lib
    g = zoo.mobilenet_v1(hw=64).to_graph(nchw44=True)
    model = g.compile([2])
    rc, text = describe(model)
    assert rc == 0
    assert "weight stem:filter" in text and "dims=8x3x3x3x4" in text      # [OC/4][KH][KW][IC][4]
    assert "dims=8x1x1x3x3x4" in text                                     # channel-wise
    assert "dims=16x8x1x1x4x4" in text                                    # dense
    syms = g.kernel_symbols()
    assert "cuda_sm100_relayout_NHWC_NCHW44_qsi8qsi8" in syms
    assert any("_NHWC44H_DENSE_" in s for s in syms)
    assert any("_NHWC44C_GROUP_" in s for s in syms)
    assert any("_NHWC44D_DENSE_" in s for s in syms)
    g.export_kernels(str(tmp_path))
    srcs = [str(tmp_path / f) for f in sorted(os.listdir(tmp_path)) if f.endswith(".c")]
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-shared", "-fPIC",
                    "-I" + os.path.join(ROOT, "include"), "-I" + str(tmp_path), "-o",
                    str(tmp_path / "libkernels.so")] + srcs + [_lib.LIB_PATH], check=True)
    init = "".join((tmp_path / f).read_text() for f in os.listdir(tmp_path) if "NHWC44C" in f)
    assert "mb200_conv_pack_filter_nchw44" in init
    # an NCHW44 input is declared with five dims
    rc, text = describe(cases.nchw44_block_spec().to_graph(nchw44=True).compile([1]))
    assert rc == 0 and "cuda_sm100_relayout_NCHW44_NHWC_qsi8qsi8" in text
    assert re.search(r"tensor data .*format=2 .*dims=1x4x30x34x4 stride=16320x4080x136x4x1", text)
    assert re.search(r"tensor add:out .*format=2 .*dims=1x24x15x17x4 ", text)


def _matmul_graph():
    from megcc_b200.compiler import Graph
    rng = np.random.default_rng(11)
    g = Graph("gap_matmul")
    x = g.input("data", 64, 8, 8, 0.05)
    f = rng.integers(-127, 128, (64, 64, 3, 3), dtype=np.int8)
    y = g.conv_bias("conv", x, f, None, 1, 1, 0.01, 0.9, "RELU")
    y = g.pooling("gap", y, "AVERAGE", 8, 8, 0)
    b = rng.integers(-127, 128, (64, 200), dtype=np.int8)
    y = g.matmul("fc", y, b, 0.01, 0.3)
    g.mark_output(y)
    return g, f, b


def test_matmul_kernel_func_symbol_stub_and_model(tmp_path):
    """MatrixMul + TypeCvt as an operator of a compiled model: the symbol follows the
    reference's kernel_matmul_<n|t><n|t>_<dtype> scheme, the exported kernel and init stubs
    compile as C99 against the public headers, and this repository's loader lists the
    instruction with its weight."""
    from megcc_b200 import _lib
    g, _, _ = _matmul_graph()
    model = g.compile([4])
    syms = g.kernel_symbols()
    assert "cuda_sm100_matmul_nn_qsi8qsi8qsi32_typecvt_qsi8" in syms
    g.export_kernels(str(tmp_path))
    srcs = [str(tmp_path / f) for f in sorted(os.listdir(tmp_path)) if f.endswith(".c")]
    so = str(tmp_path / "libkernels.so")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-shared", "-fPIC",
                    "-I" + os.path.join(ROOT, "include"), "-I" + str(tmp_path), "-o", so] + srcs
                   + [_lib.LIB_PATH], check=True)
    out = C.create_string_buffer(1 << 16)
    assert _lib.lib().mb200_tinynn_describe(model, len(model), out, len(out)) == 0
    text = out.value.decode()
    assert "cuda_sm100_matmul_nn_qsi8qsi8qsi32_typecvt_qsi8" in text and "fc:B" in text


def test_compile_side_builds_inside_the_reference_kernelgen(tmp_path):
    """The CUDA kernel pack and graph compiler, compiled against the reference's own
    KernelGen.h / TContext.h and linked with its registry (oracle/Makefile), emit byte for
    byte the model the stand-alone build emits."""
    tool = os.path.join(ROOT, "oracle", "_ref", "intree_compile_check")
    if not os.path.exists(tool):
        pytest.skip("oracle/_ref/intree_compile_check not built (needs the reference tree)")
    out = tmp_path / "intree.tiny"
    r = subprocess.run([tool, str(out)], capture_output=True, text=True, check=True)
    assert "reference_pooling_candidates" in r.stdout
    from megcc_b200.compiler import Graph
    g = Graph("intree")
    x = g.input("data", 3, 64, 64, 0.02)
    f1 = ((np.arange(64 * 3 * 7 * 7) * 37) % 255 - 127).astype(np.int8).reshape(64, 3, 7, 7)
    f2 = ((np.arange(64 * 64 * 9) * 53) % 255 - 127).astype(np.int8).reshape(64, 64, 3, 3)
    b = (np.arange(64) * 17 - 500).astype(np.int32)
    y = g.conv_bias("stem", x, f1, b, 2, 3, 0.01, 0.5, "RELU")
    y = g.pooling("pool", y, "MAX", 3, 2, 1)
    z = g.conv_bias("conv", y, f2, b, 1, 1, 0.01, 2.0, "IDENTITY")
    z = g.qelemwise("add", "QFUSE_ADD_RELU", z, y, 2.0)
    g.mark_output(z)
    mine = g.compile([1, 32])
    assert out.read_bytes() == mine
    syms = g.kernel_symbols()
    assert r.stdout.split()[:len(syms)] == syms and any("_z_QFUSE_ADD_RELU" in x for x in syms)
