"""The give-up path of the bounded device waits, and arena sharing between two networks.

Nothing here faults, traps or hangs the GPU: the self-test entry point shortens a wait's
limit to about a millisecond and leaves one pipeline stage unfilled, the kernel notices, records
a status code, drains what it started, frees its tensor memory and returns normally."""
import ctypes as C

import numpy as np
import pytest

import cases
from oracle import netwalk

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ERR_MMA_WAIT = 0x102


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _selftest(ops, p, src, packed, dst, stream):
    from megcc_b200._lib import check, lib
    check(lib().mb200_selftest_wait_expiry(
        C.byref(p), C.c_void_p(src.data_ptr()), C.c_void_p(packed.data_ptr()),
        C.c_void_p(dst.data_ptr()), 2_000_000, C.c_void_p(stream)))


def test_bounded_wait_runs_out_and_the_context_stays_usable(oracle):
    from megcc_b200 import ops
    c = dict(name="wait_expiry", n=2, ic=64, oc=64, h=40, w=40, k=3, stride=1, pad=1, groups=1,
             act="RELU", range=(-128, 127), bias_range=(-1000, 1000), scales=(0.05, 0.01, 0.9))
    src, flt, bias = cases.conv_inputs(c)
    p = ops.conv_param(2, 64, 40, 40, 64, 3, 3, 1, 1, 1, "RELU", 0.05, 0.01, 0.9)
    nhwc = ops.nchw_to_nhwc(dev(src))
    packed = ops.pack_filter(p, dev(flt))
    dst = torch.zeros((2, 40, 40, 64), dtype=torch.int8, device="cuda")
    assert ops.device_status() == 0
    _selftest(ops, p, nhwc, packed, dst, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    assert ops.device_status() == ERR_MMA_WAIT
    assert ops.device_status() == 0  # reading cleared it
    # the very next normal launch of the same kernel is bit-exact
    out = ops.conv_bias_qs8_nhwc(p, nhwc, packed, dev(bias), algo="umma")
    torch.cuda.synchronize()
    want = oracle.conv_bias_qs8(src, flt, bias, 1, 1, 0.05, 0.01, 0.9, "RELU")
    assert (out.cpu().numpy().transpose(0, 3, 1, 2) == want).all()
    assert ops.device_status() == 0


def test_lite_wait_reports_a_kernel_that_gave_up_and_only_on_its_own_network(oracle):
    from megcc_b200 import lite, ops, zoo
    from megcc_b200.lite import LiteError
    spec = zoo.single_conv(ic=64, oc=64, hw=40, s_dst=0.9)
    x = cases.rng_for("wait_expiry_net").integers(-128, 128, (2, 64, 40, 40), dtype=np.int8)
    model = spec.to_graph().compile([2])
    want = netwalk.run(spec, x, oracle).reshape(-1)
    a, b = lite.Network(model), lite.Network(model)
    for net in (a, b):
        net.set_input("data", x)
        net.forward()
        net.wait()
    # a kernel gives up on network a's stream
    p = ops.conv_param(2, 64, 40, 40, 64, 3, 3, 1, 1, 1, "RELU", 0.05, 0.01, 0.9)
    nhwc = ops.nchw_to_nhwc(dev(x))
    packed = ops.pack_filter(p, dev(spec.layers[0]["flt"]))
    dst = torch.zeros((2, 40, 40, 64), dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    _selftest(ops, p, nhwc, packed, dst, a.stream())
    # network b neither sees nor clears it
    b.forward()
    b.wait()
    assert (b.output(b.output_names()[0]) == want).all()
    a.forward()
    with pytest.raises(LiteError) as e:
        a.wait()
    assert e.value.status == 3 and "0x102" in str(e.value)  # TinyNN_ERROR_RUNTIME
    # and the network works again afterwards
    a.forward()
    a.wait()
    assert (a.output(a.output_names()[0]) == want).all()
    a.close()
    b.close()


def test_two_networks_share_one_runtime_arena(oracle):
    """LITE_share_runtime_memroy (runtime/src/lite/network.c:285-303 in the reference): both
    networks lay their tensors into one arena sized for the larger; used one after the other
    they give the results they give alone."""
    from megcc_b200 import lite, zoo
    from megcc_b200.lite import LiteError
    small = zoo.single_conv(ic=64, oc=64, hw=40, s_dst=0.9, seed=3)
    big = zoo.resnet18(hw=64, classes=64, seed=4)
    xs = cases.rng_for("share_small").integers(-128, 128, (2, 64, 40, 40), dtype=np.int8)
    xb = cases.rng_for("share_big").integers(-128, 128, (4, 3, 64, 64), dtype=np.int8)
    ws, wb = netwalk.run(small, xs, oracle).reshape(-1), netwalk.run(big, xb, oracle).reshape(-1)
    before = torch.cuda.mem_get_info()[0]
    n_small = lite.Network(small.to_graph().compile([2]))
    n_big = lite.Network(big.to_graph().compile([4]))
    lite.check(lite.lib().LITE_share_runtime_memroy(n_small._net, n_big._net))
    for _ in range(3):  # eager, capture, replay: alternating on the shared arena
        n_small.set_input("data", xs)
        n_small.forward()
        n_small.wait()
        got_small = n_small.output(n_small.output_names()[0])
        n_big.set_input("data", xb)
        n_big.forward()
        n_big.wait()
        got_big = n_big.output(n_big.output_names()[0])
        assert (got_small == ws).all() and (got_big == wb).all()
    # sharing after a run is refused, as in the reference
    with pytest.raises(LiteError):
        lite.check(lite.lib().LITE_share_runtime_memroy(n_small._net, n_big._net))
    n_small.close()
    n_big.close()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= before - (8 << 20)  # the arena went back
