"""Generate tests/golden/*.npz from the reference's OWN x86 kernels.

Run in a container that has the reference tree (oracle/Makefile builds oracle/_ref from
it):

    python tests/golden/make_golden.py

Every output stored here was computed by oracle/_ref/libmegcc_ref_kernels.so, i.e. by the
C code the reference's KernelGen emits for Arch::BAREMETAL, compiled with the strict-IEEE
flags of its x86 unit tests. Inputs are not stored: tests/cases.py rebuilds them from the
case name; a CRC of each input set is stored to catch PRNG drift.
"""
import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle import oracle as O  # noqa: E402


def crc(*arrays):
    c = 0
    for a in arrays:
        if a is not None:
            c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return np.uint32(c)


BIG = 65536


def put(out, name, result, *inputs):
    """Small results are stored whole; large ones as a CRC-32 of their bytes."""
    if result.size > BIG:
        out[name + "/out_crc"] = crc(result)
        out[name + "/shape"] = np.array(result.shape, np.int64)
    else:
        out[name] = result
    out[name + "/crc"] = crc(*inputs)


def put_f32(out, name, result, *inputs):
    """fp32 results: 4096 elements at fixed pseudo-random positions (whole when smaller)."""
    flat = result.reshape(-1)
    if flat.size > 4096:
        idx = np.random.Generator(np.random.PCG64(zlib.crc32(name.encode()))).choice(
            flat.size, 4096, replace=False)
        idx.sort()
        out[name + "/idx"] = idx.astype(np.int64)
        out[name] = flat[idx]
    else:
        out[name] = flat
    out[name + "/shape"] = np.array(result.shape, np.int64)
    out[name + "/crc"] = crc(*inputs)


def main():
    O.build(with_reference=True)
    assert O.ref_lib() is not None, "needs the reference tree to build oracle/_ref"

    out = {}
    conv_cases = (cases.conv_naive_catalogue() + cases.conv_im2col_catalogue()
                  + [cases.conv_cfg1(0.1), cases.conv_cfg1(5.0)] + cases.conv_model_shapes())
    for c in conv_cases:
        src, flt, bias = cases.conv_inputs(c)
        s0, s1, s2 = c["scales"]
        dst = O.ref_conv_bias_qs8(src, flt, bias, c["stride"], c["pad"], s0, s1, s2, c["act"],
                                  c["groups"])
        put(out, c["name"], dst, src, flt, bias)
    np.savez_compressed(os.path.join(HERE, "conv_bias_qs8.npz"), **out)

    # format NCHW44: outputs of the reference's ConvGeneral generated for NCHW44 / NCHW_NCHW44
    out = {}
    for c in cases.conv_nchw44_catalogue():
        src, flt44, bias = cases.conv_nchw44_inputs(c, O)
        s0, s1, s2 = c["scales"]
        dst = O.ref_conv_bias_qs8_nchw44(src, flt44, bias, c["stride"], c["pad"], s0, s1, s2,
                                         c["form"], c["act"])
        put(out, c["name"], dst, src, flt44, bias)
    np.savez_compressed(os.path.join(HERE, "conv_bias_nchw44.npz"), **out)

    out = {}
    for c in cases.pool_catalogue():
        x = cases.pool_input(c)
        put(out, c["name"],
            O.ref_pooling_qs8(x, c["mode"], c["window"], c["stride"], c["pad"], 0.7), x)
    np.savez_compressed(os.path.join(HERE, "pooling_qs8.npz"), **out)

    out = {}
    for c in cases.qelem_catalogue():
        a, b = cases.qelem_inputs(c)
        s0, s1, s2 = c["scales"]
        put(out, c["name"], O.ref_qelemwise(c["mode"], a, b, s0, s1, s2), a, b)
    np.savez_compressed(os.path.join(HERE, "qelemwise.npz"), **out)

    out = {}
    for c in cases.typecvt_catalogue():
        x = cases.typecvt_input(c)
        put(out, c["name"], O.ref_typecvt_qs32_qs8(x, c["s_src"], c["s_dst"]), x)
    np.savez_compressed(os.path.join(HERE, "typecvt_qs32_qs8.npz"), **out)
    # fp32 path: outputs of the reference's GeneralIntrinsic ConvBias (im2col) and MatrixMul
    # (4x12) kernels, stored as a checksum-free float digest: mean, standard deviation and 64
    # sampled elements per case (the GPU is compared within 1e-4 / 1e-5, not bit for bit)
    out = {}
    for c in cases.f32_conv_catalogue():
        src, flt, bias = cases.f32_conv_inputs(c)
        put_f32(out, c["name"], O.ref_conv_bias_f32(src, flt, bias, c["stride"], c["pad"], c["act"]),
                src, flt, bias)
    for c in cases.f32_matmul_catalogue():
        a, b = cases.f32_matmul_inputs(c)
        put_f32(out, c["name"], O.ref_matmul_f32(a, b), a, b)
    np.savez_compressed(os.path.join(HERE, "f32_ops.npz"), **out)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
