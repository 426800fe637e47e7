"""The allocation-free ConvBias entry point, through the C ABI.

It exists for programs that cannot call cudaMalloc when they need a convolution (their own
pool owns the device, or they sit in a loop where cudaMalloc's device-wide synchronisation
is not acceptable); its scratch is a fixed array inside the library. This file is collected
last on purpose: should it fail, a run that stops at the first failure has already run every
other test. It passes alone in a fresh process and after the other tests alike.
"""
import ctypes as C

import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def call_noalloc(ops, p, src, flt, bias, flt_scales=None, dst=None):
    from megcc_b200._lib import check, lib
    if dst is None:
        dst = torch.empty((p.n, p.oc) + ops.out_hw(p), dtype=torch.int8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib().mb200_conv_bias_qs8_nchw_noalloc(
        C.byref(p), C.c_void_p(src.data_ptr()), C.c_void_p(flt.data_ptr()),
        None if bias is None else C.c_void_p(bias.data_ptr()),
        None if flt_scales is None else C.c_void_p(flt_scales.data_ptr()),
        C.c_void_p(dst.data_ptr()), st))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def free_device_bytes():
    """cudaMemGetInfo's free figure: anything the driver hands out moves it."""
    return torch.cuda.mem_get_info()[0]


SECOND = dict(name="noalloc_second", n=3, ic=24, oc=40, h=31, w=29, k=5, stride=2, pad=2,
              groups=1, act="H_SWISH", range=(-128, 127), bias_range=(-1000, 1000),
              scales=(0.05, 0.01, 0.7))
GROUPED = dict(name="noalloc_grouped", n=2, ic=24, oc=36, h=17, w=19, k=3, stride=1, pad=1,
               groups=6, act="RELU", range=(-128, 127), bias_range=(-1000, 1000),
               scales=(0.05, 0.01, 0.3))
NO_BIAS = dict(name="noalloc_depthwise_no_bias", n=2, ic=32, oc=32, h=20, w=20, k=3, stride=2,
               pad=1, groups=32, act="IDENTITY", range=(-128, 127), bias=False,
               scales=(0.05, 0.01, 0.02))


def test_noalloc_entry_matches_existing_entry_twice_in_a_row(oracle):
    assert torch.cuda.is_available()
    import golden_util as G
    from megcc_b200 import ops
    # different problems back to back: each call sees its predecessor's leftovers in the
    # shared scratch and must not be affected by them
    for c in (cases.conv_cfg1(5.0), SECOND, GROUPED, NO_BIAS):
        src, flt, bias = cases.conv_inputs(c)
        s0, s1, s2 = c["scales"]
        p = ops.conv_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                           c["pad"], c["groups"], c["act"], s0, s1, s2)
        d_src, d_flt = dev(src), dev(flt)
        d_bias = None if bias is None else dev(bias)
        want = ops.conv_bias_qs8_nchw(p, d_src, d_flt, d_bias).cpu().numpy()
        first = call_noalloc(ops, p, d_src, d_flt, d_bias)
        # the second call writes into a buffer that exists already, so that the free-memory
        # figure around it shows what the entry point itself took from the driver: nothing
        dst = torch.empty_like(torch.from_numpy(first)).cuda()
        torch.cuda.synchronize()
        before = free_device_bytes()
        second = call_noalloc(ops, p, d_src, d_flt, d_bias, dst=dst)
        assert free_device_bytes() == before, "the call changed the device's free memory"
        # integer outputs: the tolerance of every parity test here is zero
        assert (first == want).all() and (second == want).all()
        # and the CPU checker agrees (the first case is also a committed golden vector)
        cpu = oracle.conv_bias_qs8(src, flt, bias, c["stride"], c["pad"], s0, s1, s2, c["act"],
                                   groups=c["groups"])
        assert (first == cpu).all()
        if c["name"].startswith("cfg1"):
            G.check("conv_bias_qs8", c["name"], first, src, flt, bias)


def test_noalloc_entry_with_one_scale_per_output_channel(oracle):
    from megcc_b200 import ops
    c = SECOND
    src, flt, bias = cases.conv_inputs(c)
    s0, _, s2 = c["scales"]
    scales = cases.rng_for("noalloc_channel_scales").uniform(0.005, 0.02, c["oc"]).astype(np.float32)
    p = ops.conv_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                       c["pad"], 1, c["act"], s0, float(scales.mean()), s2)
    got = call_noalloc(ops, p, dev(src), dev(flt), dev(bias), flt_scales=dev(scales))
    want = ops.conv_bias_qs8_nchw(p, dev(src), dev(flt), dev(bias), dev(scales)).cpu().numpy()
    cpu = oracle.conv_bias_qs8(src, flt, bias, c["stride"], c["pad"], s0, scales, s2, c["act"])
    assert (got == want).all() and (got == cpu).all()


def test_noalloc_entry_refuses_problems_beyond_its_scratch():
    from megcc_b200 import ops
    from megcc_b200._lib import MegccError, check, lib
    assert lib().mb200_conv_bias_qs8_nchw_noalloc_max_scratch() == 8 << 20
    p = ops.conv_param(64, 64, 56, 56, 64, 3, 3, 1, 1, 1, "RELU", 0.05, 0.01, 0.1)  # 25 MB
    z = torch.zeros(16, dtype=torch.int8, device="cuda")
    with pytest.raises(MegccError) as e:
        check(lib().mb200_conv_bias_qs8_nchw_noalloc(
            C.byref(p), C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()), None, None,
            C.c_void_p(z.data_ptr()), None))
    assert e.value.status == 4 and "scratch" in str(e.value)
