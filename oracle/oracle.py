"""TEST INFRASTRUCTURE: numpy-facing bindings of the checker.

Two back ends, same call shapes:

* ``restated``  -> oracle/libmegcc_oracle.so, our C restatement (oracle/megcc_oracle.c)
* ``reference`` -> oracle/_ref/libmegcc_ref_kernels.so, the reference's own generated
  x86 kernels (built by oracle/Makefile from the reference sources; only the kernels
  listed in oracle/ref_specs.txt exist)

Only tests/, the smoke check and the CPU-baseline leg of bench.py import this module.
The product package never does.

All tensors are the reference's model-visible layouts: activations NCHW, dense filter
OIHW, grouped filter [G, OCpg, ICpg, KH, KW], bias [OC] int32.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# the one place that names where the reference tree is expected (override: MEGCC_REFERENCE_DIR)
DEFAULT_REFERENCE_DIR = "/root/reference"
ACT = {"IDENTITY": 0, "RELU": 1, "H_SWISH": 2}
POOL = {"MAX": 0, "AVERAGE": 1, "AVERAGE_COUNT_EXCLUDE_PADDING": 2}
QELEM = {"QADD": 0, "QFUSE_ADD_RELU": 1, "QMUL": 2, "QRELU": 3}

_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def reference_tree():
    """Where the reference's source tree lies: $MEGCC_REFERENCE_DIR, else the default the
    Makefile also uses. None when its KernelGen sources are not there."""
    root = os.environ.get("MEGCC_REFERENCE_DIR", DEFAULT_REFERENCE_DIR)
    return root if os.path.isdir(os.path.join(root, "compiler", "lib", "KernelGen")) else None


def build(with_reference=True):
    """Compile the checker (and, when the reference tree is present, oracle/_ref)."""
    targets = ["oracle"]
    args = []
    if with_reference and reference_tree():
        targets.append("ref")
        args.append("REF=" + reference_tree())
    subprocess.run(["make", "-s", "-j8", "-C", HERE] + args + targets, check=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "libmegcc_oracle.so")
        if not os.path.exists(path):
            build(with_reference=False)
        L = C.CDLL(path)
        L.oracle_conv_bias_qs8.restype = C.c_int
        L.oracle_conv_bias_qs8.argtypes = (
            [_i8p, _i8p, C.c_void_p, _i8p, C.c_void_p] + [C.c_int] * 14
            + [C.c_float, _f32p, C.c_int, C.c_float, C.c_int])
        L.oracle_pooling_qs8.restype = None
        L.oracle_pooling_qs8.argtypes = [_i8p, _i8p] + [C.c_int] * 11
        L.oracle_qelemwise.restype = None
        L.oracle_qelemwise.argtypes = [
            _i8p, C.c_void_p, _i8p, C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_int,
            C.c_float, C.c_float, C.c_float]
        L.oracle_typecvt_qs32_qs8.restype = None
        L.oracle_typecvt_qs32_qs8.argtypes = [_i32p, _i8p, C.c_size_t, C.c_float, C.c_float]
        L.oracle_matmul_s8_s32.restype = None
        L.oracle_matmul_s8_s32.argtypes = [_i8p, _i8p, _i32p, C.c_int, C.c_int, C.c_int]
        L.oracle_typecvt_f32_qs8.restype = None
        L.oracle_typecvt_f32_qs8.argtypes = [_f32p, _i8p, C.c_size_t, C.c_float, C.c_float]
        L.oracle_typecvt_qs8_f32.restype = None
        L.oracle_typecvt_qs8_f32.argtypes = [_i8p, _f32p, C.c_size_t, C.c_float, C.c_float]
        L.oracle_conv_bias_f32.restype = None
        L.oracle_conv_bias_f32.argtypes = [_f32p, _f32p, C.c_void_p, C.c_void_p, _f32p] + [C.c_int] * 13
        L.oracle_matmul_f32.restype = None
        L.oracle_matmul_f32.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.oracle_elemwise_f32.restype = None
        L.oracle_elemwise_f32.argtypes = [C.c_int, _f32p, C.c_void_p, _f32p, C.c_size_t]
        L.oracle_pooling_f32.restype = None
        L.oracle_pooling_f32.argtypes = [_f32p, _f32p] + [C.c_int] * 11
        L.oracle_resize_nearest_f32.restype = None
        L.oracle_resize_nearest_f32.argtypes = [_f32p, _f32p] + [C.c_int] * 6
        _lib = L
    return _lib


def out_extent(i, k, s, p, d=1):
    return (i + 2 * p - d * (k - 1) - 1) // s + 1


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def conv_bias_qs8(src, flt, bias, stride, pad, s_src, s_flt, s_dst, act="IDENTITY",
                  groups=1, dilate=1, return_acc=False):
    """qint8 ConvBias; ``s_flt`` a float (per tensor) or an [OC] array (per channel)."""
    src, flt = _c(src, np.int8), _c(flt, np.int8)
    n, ic, ih, iw = src.shape
    kh, kw = flt.shape[-2:]
    oc = flt.shape[0] if flt.ndim == 4 else flt.shape[0] * flt.shape[1]
    oh, ow = out_extent(ih, kh, stride, pad, dilate), out_extent(iw, kw, stride, pad, dilate)
    dst = np.empty((n, oc, oh, ow), np.int8)
    acc = np.empty((n, oc, oh, ow), np.int32) if return_acc else None
    per_channel = int(np.ndim(s_flt) > 0)
    fs = _c(np.atleast_1d(s_flt), np.float32)
    b = None if bias is None else _c(np.asarray(bias).reshape(-1), np.int32)
    rc = lib().oracle_conv_bias_qs8(
        src, flt, None if b is None else b.ctypes.data, dst,
        None if acc is None else acc.ctypes.data, n, ic, ih, iw, oc, kh, kw, stride, stride,
        pad, pad, dilate, dilate, groups, np.float32(s_src), fs, per_channel,
        np.float32(s_dst), ACT[act])
    assert rc == 0
    return (dst, acc) if return_acc else dst


def pooling_qs8(src, mode, window, stride, pad):
    src = _c(src, np.int8)
    n, c, ih, iw = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = np.empty((n, c, oh, ow), np.int8)
    lib().oracle_pooling_qs8(src, dst, POOL[mode], n, c, ih, iw, window, window, stride,
                             stride, pad, pad)
    return dst


def _bcast(a, b):
    if b is None or a.shape == b.shape:
        return 0, 1, 1
    if b.size == 1:
        return 1, 1, 1
    assert b.size == a.shape[1], "only same-shape, scalar or per-channel operands"
    return 2, a.shape[1], int(np.prod(a.shape[2:]))


def qelemwise(mode, a, b, s0, s1, s_dst):
    a = _c(a, np.int8)
    b = None if b is None else _c(b, np.int8)
    bc, ch, inner = _bcast(a, b)
    dst = np.empty(a.shape, np.int8)
    lib().oracle_qelemwise(a, None if b is None else b.ctypes.data, dst, QELEM[mode], a.size,
                           bc, ch, inner, np.float32(s0), np.float32(s1), np.float32(s_dst))
    return dst


def typecvt_qs32_qs8(src, s_src, s_dst):
    src = _c(src, np.int32)
    dst = np.empty(src.shape, np.int8)
    lib().oracle_typecvt_qs32_qs8(src, dst, src.size, np.float32(s_src), np.float32(s_dst))
    return dst


def typecvt_f32_qs8(src, s_src, s_dst):
    src = _c(src, np.float32)
    dst = np.empty(src.shape, np.int8)
    lib().oracle_typecvt_f32_qs8(src, dst, src.size, np.float32(s_src), np.float32(s_dst))
    return dst


def typecvt_qs8_f32(src, s_src, s_dst):
    src = _c(src, np.int8)
    dst = np.empty(src.shape, np.float32)
    lib().oracle_typecvt_qs8_f32(src, dst, src.size, np.float32(s_src), np.float32(s_dst))
    return dst


def matmul_s8_s32(a, b):
    a, b = _c(a, np.int8), _c(b, np.int8)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.int32)
    lib().oracle_matmul_s8_s32(a, b, c, m, n, k)
    return c


# ----------------------------------------------------------------------------------------
# fp32 path (restated)
# ----------------------------------------------------------------------------------------
F32_ACT = {"IDENTITY": 0, "RELU": 1, "H_SWISH": 2, "SIGMOID": 3, "SILU": 4}
ELEM = {"RELU": 0, "SIGMOID": 1, "SILU": 2, "H_SWISH": 3, "EXP": 4, "ADD": 16, "SUB": 17,
        "MUL": 18, "MAX": 19, "FUSE_ADD_RELU": 20}


def conv_bias_f32(src, flt, bias, stride, pad, act="IDENTITY", groups=1, z=None):
    """fp32 ConvBias (NCHW, OIHW), activation, then optionally + z."""
    src, flt = _c(src, np.float32), _c(flt, np.float32)
    n, ic, ih, iw = src.shape
    kh, kw = flt.shape[-2:]
    oc = flt.shape[0] if flt.ndim == 4 else flt.shape[0] * flt.shape[1]
    oh, ow = out_extent(ih, kh, stride, pad), out_extent(iw, kw, stride, pad)
    dst = np.empty((n, oc, oh, ow), np.float32)
    b = None if bias is None else _c(np.asarray(bias).reshape(-1), np.float32)
    zz = None if z is None else _c(z, np.float32)
    lib().oracle_conv_bias_f32(src, flt, None if b is None else b.ctypes.data,
                               None if zz is None else zz.ctypes.data, dst, n, ic, ih, iw, oc,
                               kh, kw, stride, stride, pad, pad, groups, F32_ACT[act])
    return dst


def matmul_f32(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    lib().oracle_matmul_f32(a, b, c, m, n, k)
    return c


def elemwise_f32(mode, a, b=None):
    a = _c(a, np.float32)
    bb = None if b is None else _c(b, np.float32)
    dst = np.empty(a.shape, np.float32)
    lib().oracle_elemwise_f32(ELEM[mode], a, None if bb is None else bb.ctypes.data, dst, a.size)
    return dst


def pooling_f32(src, mode, window, stride, pad):
    src = _c(src, np.float32)
    n, c, ih, iw = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = np.empty((n, c, oh, ow), np.float32)
    lib().oracle_pooling_f32(src, dst, POOL[mode], n, c, ih, iw, window, window, stride, stride,
                             pad, pad)
    return dst


def resize_nearest_f32(src, oh, ow):
    src = _c(src, np.float32)
    n, c, ih, iw = src.shape
    dst = np.empty((n, c, oh, ow), np.float32)
    lib().oracle_resize_nearest_f32(src, dst, n, c, ih, iw, oh, ow)
    return dst


def concat_f32(tensors):
    """Concat along channels, NCHW (BareMetal/Concat.cpp:23-78 with axis 1)."""
    return np.concatenate([_c(t, np.float32) for t in tensors], axis=1)


def focus_f32(src, c_out=None):
    """The Focus stem's four stride-2 slices concatenated along channels (optionally padded
    with zero channels up to c_out)."""
    x = _c(src, np.float32)
    parts = [x[:, :, 0::2, 0::2], x[:, :, 1::2, 0::2], x[:, :, 0::2, 1::2], x[:, :, 1::2, 1::2]]
    out = np.concatenate(parts, axis=1)
    if c_out is not None and c_out > out.shape[1]:
        pad = np.zeros((out.shape[0], c_out - out.shape[1]) + out.shape[2:], np.float32)
        out = np.concatenate([out, pad], axis=1)
    return np.ascontiguousarray(out)


# ----------------------------------------------------------------------------------------
# the reference's own kernels
# ----------------------------------------------------------------------------------------
class _RefOperand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int), ("scale", C.c_float),
                ("ndim", C.c_int), ("dims", C.c_int * 7)]


_DT = {np.dtype(np.int8): 100, np.dtype(np.int32): 101, np.dtype(np.float32): 0}
_ref = None


def ref_lib():
    """The reference-kernel library, or None when it was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libmegcc_ref_kernels.so")
        if not os.path.exists(path):
            return None
        L = C.CDLL(path)
        L.megcc_ref_call.restype = C.c_int
        L.megcc_ref_call.argtypes = [C.c_char_p, C.POINTER(_RefOperand), C.c_int,
                                     C.POINTER(_RefOperand), C.c_int]
        L.megcc_ref_has.restype = C.c_int
        L.megcc_ref_has.argtypes = [C.c_char_p]
        _ref = L
    return _ref


def ref_has(symbol):
    L = ref_lib()
    return bool(L and L.megcc_ref_has(symbol.encode()))


def _operand(a, scale):
    o = _RefOperand()
    o.ptr = a.ctypes.data
    o.dtype = _DT[a.dtype]
    o.scale = scale
    o.ndim = a.ndim
    for i, d in enumerate(a.shape):
        o.dims[i] = d
    return o


def ref_call(symbol, ins, outs):
    """ins/outs: lists of (contiguous ndarray, scale)."""
    L = ref_lib()
    if L is None:
        raise RuntimeError("oracle/_ref was not built (reference tree absent at build time)")
    ia = (_RefOperand * len(ins))(*[_operand(a, s) for a, s in ins])
    oa = (_RefOperand * len(outs))(*[_operand(a, s) for a, s in outs])
    rc = L.megcc_ref_call(symbol.encode(), ia, len(ins), oa, len(outs))
    if rc != 0:
        raise RuntimeError(f"reference kernel {symbol}: status {rc}")


def conv_symbol(k, stride, pad, groups, act, bias=True):
    """Symbol naming of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:144-176."""
    sparse = "DENSE" if groups == 1 else "GROUP"
    s = (f"kernel_conv2d_{k}x{k}_NCHW_{sparse}_p{pad}x{pad}_s{stride}x{stride}_d1x1_"
         f"qsi8qsi8qsi32qsi8")
    if bias:
        s += "_bias"
    if act != "IDENTITY":
        s += "_" + act
    return s


def ref_conv_bias_qs8(src, flt, bias, stride, pad, s_src, s_flt, s_dst, act="IDENTITY",
                      groups=1):
    src, flt = _c(src, np.int8), _c(flt, np.int8)
    n, ic, ih, iw = src.shape
    kh, kw = flt.shape[-2:]
    if groups > 1 and flt.ndim == 4:
        flt = flt.reshape(groups, flt.shape[0] // groups, flt.shape[1], kh, kw)
    oc = flt.shape[0] if flt.ndim == 4 else flt.shape[0] * flt.shape[1]
    oh, ow = out_extent(ih, kh, stride, pad), out_extent(iw, kw, stride, pad)
    dst = np.empty((n, oc, oh, ow), np.int8)
    if bias is None:
        b = np.zeros((0,), np.int32)
        ins = [(src, s_src), (flt, s_flt), (b, s_src * s_flt)]
    else:
        b = _c(np.asarray(bias).reshape(1, oc, 1, 1), np.int32)
        ins = [(src, s_src), (flt, s_flt), (b, s_src * s_flt)]
    ref_call(conv_symbol(kh, stride, pad, groups, act, bias is not None), ins, [(dst, s_dst)])
    return dst


# ---- NCHW44: the layouts of a model compiled with --enable_nchw44 ----
def nchw_to_nchw44(x):
    """[N, C, H, W] -> [N, C/4, H, W, 4] (compiler/lib/KernelGen/BareMetal/FormatHelper.cpp:23-26:
    offset = n*s0 + (c/4)*s1 + h*s2 + w*s3 + c%4)."""
    n, c, h, w = x.shape
    assert c % 4 == 0
    return np.ascontiguousarray(x.reshape(n, c // 4, 4, h, w).transpose(0, 1, 3, 4, 2))


def nchw44_to_nchw(x):
    n, cb, h, w, four = x.shape
    assert four == 4
    return np.ascontiguousarray(x.transpose(0, 1, 4, 2, 3).reshape(n, cb * 4, h, w))


def filter_to_nchw44(flt, form):
    """OIHW (dense, first_layer) or [G, 1, 1, KH, KW] (channel_wise) -> the NCHW44 filter
    layouts of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:48-62,88-101."""
    flt = np.asarray(flt)
    if form == "dense":  # [OC/4][IC/4][KH][KW][4 ic][4 oc]
        oc, ic, kh, kw = flt.shape
        return np.ascontiguousarray(
            flt.reshape(oc // 4, 4, ic // 4, 4, kh, kw).transpose(0, 2, 4, 5, 3, 1))
    if form == "channel_wise":  # [G/4][1][1][KH][KW][4]
        g = flt.shape[0]
        kh, kw = flt.shape[-2:]
        return np.ascontiguousarray(
            flt.reshape(g // 4, 4, kh, kw).transpose(0, 2, 3, 1).reshape(g // 4, 1, 1, kh, kw, 4))
    if form == "first_layer":  # [OC/4][KH][KW][IC][4 oc]
        oc, ic, kh, kw = flt.shape
        return np.ascontiguousarray(flt.reshape(oc // 4, 4, ic, kh, kw).transpose(0, 3, 4, 2, 1))
    raise ValueError(form)


def filter_from_nchw44(flt44, form):
    """Inverse of filter_to_nchw44: back to OIHW, or [G, 1, 1, KH, KW] for channel_wise."""
    flt44 = np.asarray(flt44)
    if form == "dense":
        ob, ib, kh, kw, _, _ = flt44.shape
        return np.ascontiguousarray(
            flt44.transpose(0, 5, 1, 4, 2, 3).reshape(ob * 4, ib * 4, kh, kw))
    if form == "channel_wise":
        gb, _, _, kh, kw, _ = flt44.shape
        return np.ascontiguousarray(
            flt44.reshape(gb, kh, kw, 4).transpose(0, 3, 1, 2).reshape(gb * 4, 1, 1, kh, kw))
    if form == "first_layer":
        ob, kh, kw, ic, _ = flt44.shape
        return np.ascontiguousarray(flt44.transpose(0, 4, 3, 1, 2).reshape(ob * 4, ic, kh, kw))
    raise ValueError(form)


def conv_bias_qs8_nchw44(src, flt44, bias, stride, pad, s_src, s_flt, s_dst, form,
                         act="IDENTITY"):
    """ConvBias of an NCHW44 model, restated as layout conversions around the NCHW
    restatement: src [N, C/4, H, W, 4] (NCHW for form "first_layer"), result [N, OC/4, OH, OW, 4].
    Pinned to the reference's own NCHW44 kernels by tests/test_oracle_vs_reference.py."""
    x = np.asarray(src) if form == "first_layer" else nchw44_to_nchw(np.asarray(src))
    flt = filter_from_nchw44(flt44, form)
    groups = flt.shape[0] if form == "channel_wise" else 1
    out = conv_bias_qs8(x, flt, bias, stride, pad, s_src, s_flt, s_dst, act, groups=groups)
    return nchw_to_nchw44(out)


def ref_conv_bias_qs8_nchw44(src, flt44, bias, stride, pad, s_src, s_flt, s_dst, form,
                             act="IDENTITY"):
    """The reference's ConvGeneral generated for format NCHW44 (symbol naming of
    compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:144-176 with get_format's NCHW_NCHW44)."""
    src, flt44 = _c(src, np.int8), _c(flt44, np.int8)
    oc = flt44.shape[0] * 4
    if form == "first_layer":
        kh, kw = flt44.shape[1:3]
        fmt, sparse = "NCHW_NCHW44", "DENSE"
    elif form == "channel_wise":
        kh, kw = flt44.shape[3:5]
        fmt, sparse = "NCHW44", "GROUP"
    else:
        kh, kw = flt44.shape[2:4]
        fmt, sparse = "NCHW44", "DENSE"
    ih, iw = src.shape[2], src.shape[3]
    oh, ow = out_extent(ih, kh, stride, pad), out_extent(iw, kw, stride, pad)
    dst = np.empty((src.shape[0], oc // 4, oh, ow, 4), np.int8)
    b = (np.zeros((0,), np.int32) if bias is None
         else _c(np.asarray(bias).reshape(1, oc // 4, 1, 1, 4), np.int32))
    sym = (f"kernel_conv2d_{kh}x{kw}_{fmt}_{sparse}_p{pad}x{pad}_s{stride}x{stride}_d1x1_"
           f"qsi8qsi8qsi32qsi8")
    if bias is not None:
        sym += "_bias"
    if act != "IDENTITY":
        sym += "_" + act
    ref_call(sym, [(src, s_src), (flt44, s_flt), (b, s_src * s_flt)], [(dst, s_dst)])
    return dst


def ref_pooling_qs8(src, mode, window, stride, pad, scale=1.0):
    src = _c(src, np.int8)
    n, c, ih, iw = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = np.empty((n, c, oh, ow), np.int8)
    sym = (f"kernel_pooling_{mode}_NCHW_p{pad}x{pad}_s{stride}x{stride}_w{window}x{window}"
           f"_qsi8qsi8")
    ref_call(sym, [(src, scale)], [(dst, scale)])
    return dst


def ref_qelemwise(mode, a, b, s0, s1, s_dst):
    a = _c(a, np.int8)
    dst = np.empty(a.shape, np.int8)
    if mode == "QRELU":
        ref_call("kernel_elementwise_multitype_QRELU_qsi8qsi8", [(a, s0)], [(dst, s_dst)])
    else:
        b = _c(b, np.int8)
        ref_call(f"kernel_elementwise_multitype_{mode}_qsi8qsi8qsi8", [(a, s0), (b, s1)],
                 [(dst, s_dst)])
    return dst


def ref_typecvt_f32_qs8(src, s_src, s_dst):
    src = _c(src, np.float32)
    dst = np.empty(src.shape, np.int8)
    ref_call("GI_kernel_typecvt_f32qsi8", [(src, s_src)], [(dst, s_dst)])
    return dst


def ref_typecvt_qs8_f32(src, s_src, s_dst):
    src = _c(src, np.int8)
    dst = np.empty(src.shape, np.float32)
    ref_call("GI_kernel_typecvt_qsi8f32", [(src, s_src)], [(dst, s_dst)])
    return dst


def ref_typecvt_qs32_qs8(src, s_src, s_dst):
    src = _c(src, np.int32)
    dst = np.empty(src.shape, np.int8)
    ref_call("kernel_typecvt_qsi32qsi8", [(src, s_src)], [(dst, s_dst)])
    return dst


# ---- the reference's fp32 kernels (GeneralIntrinsic im2col ConvBias and 4x12 MatrixMul,
# GI / BareMetal Elemwise, BareMetal Concat / Resize / Pooling) ----
def ref_conv_bias_f32(src, flt, bias, stride, pad, act="IDENTITY"):
    """ConvBias fp32 with the reference's own nonlinearities (IDENTITY / RELU / SIGMOID)."""
    src, flt = _c(src, np.float32), _c(flt, np.float32)
    n, ic, ih, iw = src.shape
    oc, _, kh, kw = flt.shape
    oh, ow = out_extent(ih, kh, stride, pad), out_extent(iw, kw, stride, pad)
    dst = np.empty((n, oc, oh, ow), np.float32)
    sym = f"GI_kernel_conv2d_im2col_{kh}x{kw}_NCHW_DENSE_p{pad}x{pad}_s{stride}x{stride}_d1x1"
    if bias is not None:
        sym += "_bias"
        b = _c(np.asarray(bias).reshape(1, oc, 1, 1), np.float32)
    else:
        b = np.zeros((0,), np.float32)
    if act != "IDENTITY":
        sym += "_" + act
    ref_call(sym + "f32", [(src, 1.0), (flt, 1.0), (b, 1.0)], [(dst, 1.0)])
    return dst


def ref_matmul_f32(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    c = np.empty((a.shape[0], b.shape[1]), np.float32)
    ref_call("GI_kernel_fp32_matmul_4x12_nn", [(a, 1.0), (b, 1.0)], [(c, 1.0)])
    return c


def ref_elemwise_f32(mode, a, b=None):
    a = _c(a, np.float32)
    dst = np.empty(a.shape, np.float32)
    if mode == "SILU":
        ref_call("kernel_elementwise_SILU_f32f32", [(a, 1.0)], [(dst, 1.0)])
    elif b is None:
        ref_call(f"GI_kernel_elementwise_{mode}_f32_unary_vec_vec_f32f32", [(a, 1.0)], [(dst, 1.0)])
    else:
        ref_call(f"GI_kernel_elementwise_{mode}_f32_binary_VEC_VEC_f32f32f32",
                 [(a, 1.0), (_c(b, np.float32), 1.0)], [(dst, 1.0)])
    return dst


def ref_concat_f32(tensors):
    ts = [_c(t, np.float32) for t in tensors]
    shape = list(ts[0].shape)
    shape[1] = sum(t.shape[1] for t in ts)
    dst = np.empty(shape, np.float32)
    ref_call("kernel_concat_byte_4_axis_1", [(t, 1.0) for t in ts], [(dst, 1.0)])
    return dst


def ref_resize_nearest_f32(src, oh, ow):
    src = _c(src, np.float32)
    dst = np.empty(src.shape[:2] + (oh, ow), np.float32)
    ref_call("kernel_resize_linear_NCHW_NEAREST_f32", [(src, 1.0)], [(dst, 1.0)])
    return dst


def ref_pooling_f32(src, mode, window, stride, pad):
    src = _c(src, np.float32)
    n, c, ih, iw = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = np.empty((n, c, oh, ow), np.float32)
    ref_call(f"kernel_pooling_{mode}_NCHW_p{pad}x{pad}_s{stride}x{stride}_w{window}x{window}_f32f32",
             [(src, 1.0)], [(dst, 1.0)])
    return dst
