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


def call_noalloc(ops, p, src, flt, bias):
    from megcc_b200._lib import check, lib
    dst = torch.empty((p.n, p.oc) + ops.out_hw(p), dtype=torch.int8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib().mb200_conv_bias_qs8_nchw_noalloc(
        C.byref(p), C.c_void_p(src.data_ptr()), C.c_void_p(flt.data_ptr()),
        C.c_void_p(bias.data_ptr()), None, C.c_void_p(dst.data_ptr()), st))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def test_noalloc_entry_matches_existing_entry_twice_in_a_row():
    assert torch.cuda.is_available()
    from megcc_b200 import ops
    # two different problems back to back: the second call sees the first one's leftovers in
    # the shared scratch and must not be affected by them
    for c in (cases.conv_cfg1(5.0),
              dict(name="noalloc_second", n=3, ic=24, oc=40, h=31, w=29, k=5, stride=2, pad=2,
                   groups=1, act="H_SWISH", range=(-128, 127), bias_range=(-1000, 1000),
                   scales=(0.05, 0.01, 0.7))):
        src, flt, bias = cases.conv_inputs(c)
        s0, s1, s2 = c["scales"]
        p = ops.conv_param(c["n"], c["ic"], c["h"], c["w"], c["oc"], c["k"], c["k"], c["stride"],
                           c["pad"], c["groups"], c["act"], s0, s1, s2)
        d_src, d_flt, d_bias = dev(src), dev(flt), dev(bias)
        want = ops.conv_bias_qs8_nchw(p, d_src, d_flt, d_bias).cpu().numpy()
        first = call_noalloc(ops, p, d_src, d_flt, d_bias)
        second = call_noalloc(ops, p, d_src, d_flt, d_bias)
        # integer outputs: the tolerance of every parity test here is zero
        assert (first == want).all() and (second == want).all()


def test_noalloc_entry_refuses_problems_beyond_its_scratch():
    from megcc_b200 import ops
    from megcc_b200._lib import MegccError, lib
    assert lib().mb200_conv_bias_qs8_nchw_noalloc_max_scratch() == 8 << 20
    p = ops.conv_param(64, 64, 56, 56, 64, 3, 3, 1, 1, 1, "RELU", 0.05, 0.01, 0.1)  # 25 MB
    z = torch.zeros(16, dtype=torch.int8, device="cuda")
    with pytest.raises(MegccError) as e:
        lib_call = lib().mb200_conv_bias_qs8_nchw_noalloc
        from megcc_b200._lib import check
        check(lib_call(C.byref(p), C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()), None, None,
                       C.c_void_p(z.data_ptr()), None))
    assert e.value.status == 4 and "scratch" in str(e.value)
