"""ctypes face of the compile-side library (include/megcc_b200_compiler.h): build a
quantised network operator by operator, compile it to a tinynn model for the CUDA device."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmegcc_b200_compiler.so")

_P = C.c_void_p
SIGNATURES = {
    "mb200c_graph_create": (_P, [C.c_char_p]),
    "mb200c_graph_destroy": (None, [_P]),
    "mb200c_last_error": (C.c_char_p, []),
    "mb200c_add_input": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_float]),
    "mb200c_add_conv_bias": (C.c_int, [_P, C.c_char_p] + [C.c_int] * 7 + [
        C.c_char_p, _P, C.c_float, _P, _P, C.c_float]),
    "mb200c_add_input_nchw44": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_float]),
    "mb200c_add_conv_bias_nchw44": (C.c_int, [_P, C.c_char_p] + [C.c_int] * 7 + [
        C.c_char_p, _P, C.c_float, _P, _P, C.c_float]),
    "mb200c_add_matmul": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, _P, C.c_float, C.c_float]),
    "mb200c_add_pooling": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_char_p] + [C.c_int] * 3),
    "mb200c_add_qelemwise": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_float]),
    "mb200c_add_input_f32": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, C.c_int]),
    "mb200c_add_conv_f32": (C.c_int, [_P, C.c_char_p] + [C.c_int] * 7 + [C.c_char_p, _P, _P,
                                                                        C.c_int]),
    "mb200c_add_matmul_f32": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, _P]),
    "mb200c_add_elemwise_f32": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.c_int, C.c_int]),
    "mb200c_add_concat": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_int), C.c_int]),
    "mb200c_add_focus": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int]),
    "mb200c_add_resize_nearest": (C.c_int, [_P, C.c_char_p, C.c_int, C.c_int, C.c_int]),
    "mb200c_mark_output": (C.c_int, [_P, C.c_int]),
    "mb200c_set_option": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "mb200c_compile": (C.c_int, [_P, C.POINTER(C.c_int), C.c_int, C.POINTER(_P),
                                 C.POINTER(C.c_size_t)]),
    "mb200c_kernel_symbols": (C.c_char_p, [_P]),
    "mb200c_arena_bytes": (C.c_size_t, [_P, C.c_int]),
    "mb200c_unplanned_bytes": (C.c_size_t, [_P, C.c_int]),
    "mb200c_export_kernels": (C.c_int, [_P, C.c_char_p]),
    "mb200c_probe_conv_symbol": (C.c_int, [C.c_int] * 8 + [C.c_char_p, C.c_int, C.c_char_p,
                                                          C.c_char_p, C.c_size_t]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m megcc_b200.build`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class CompileError(RuntimeError):
    pass


def _check(rc):
    if rc < 0:
        raise CompileError(lib().mb200c_last_error().decode())
    return rc


class Graph:
    """A static-shape qint8 network. Tensor handles are plain ints."""

    def __init__(self, name="model"):
        self._g = lib().mb200c_graph_create(name.encode())
        self._keep = []

    def __del__(self):
        if getattr(self, "_g", None):
            lib().mb200c_graph_destroy(self._g)
            self._g = None

    def input(self, name, c, h, w, scale):
        return _check(lib().mb200c_add_input(self._g, name.encode(), c, h, w, scale))

    def conv_bias(self, name, src, flt, bias, stride, pad, flt_scale, dst_scale,
                  nonline="IDENTITY", groups=1, channel_scales=None):
        flt = np.ascontiguousarray(flt, np.int8)
        kh, kw = flt.shape[-2:]
        oc = flt.shape[0] if flt.ndim == 4 else flt.shape[0] * flt.shape[1]
        b = None if bias is None else np.ascontiguousarray(np.asarray(bias).reshape(-1), np.int32)
        cs = None if channel_scales is None else np.ascontiguousarray(channel_scales, np.float32)
        return _check(lib().mb200c_add_conv_bias(
            self._g, name.encode(), src, oc, kh, kw, stride, pad, groups, nonline.encode(),
            flt.ctypes.data, flt_scale, None if b is None else b.ctypes.data,
            None if cs is None else cs.ctypes.data, dst_scale))

    def input_nchw44(self, name, c, h, w, scale):
        """Input of a model compiled with --enable_nchw44: the buffer is [N, C/4, H, W, 4]."""
        return _check(lib().mb200c_add_input_nchw44(self._g, name.encode(), c, h, w, scale))

    def conv_bias_nchw44(self, name, src, flt44, bias, stride, pad, flt_scale, dst_scale, form,
                         nonline="IDENTITY", channel_scales=None):
        """ConvBias whose filter comes in an NCHW44 layout; form names it: "dense"
        [OC/4, IC/4, KH, KW, 4, 4], "channel_wise" [G/4, 1, 1, KH, KW, 4] or, on an NCHW model
        input, "first_layer" [OC/4, KH, KW, IC, 4]."""
        flt44 = np.ascontiguousarray(flt44, np.int8)
        oc = flt44.shape[0] * 4
        if form == "first_layer":
            assert flt44.ndim == 5 and flt44.shape[4] == 4
            kh, kw, groups = flt44.shape[1], flt44.shape[2], 1
        elif form == "channel_wise":
            assert flt44.ndim == 6 and flt44.shape[1:3] == (1, 1) and flt44.shape[5] == 4
            kh, kw, groups = flt44.shape[3], flt44.shape[4], oc
        elif form == "dense":
            assert flt44.ndim == 6 and flt44.shape[4:] == (4, 4)
            kh, kw, groups = flt44.shape[2], flt44.shape[3], 1
        else:
            raise ValueError(f"unknown NCHW44 filter form {form!r}")
        b = None if bias is None else np.ascontiguousarray(np.asarray(bias).reshape(-1), np.int32)
        cs = None if channel_scales is None else np.ascontiguousarray(channel_scales, np.float32)
        return _check(lib().mb200c_add_conv_bias_nchw44(
            self._g, name.encode(), src, oc, kh, kw, stride, pad, groups, nonline.encode(),
            flt44.ctypes.data, flt_scale, None if b is None else b.ctypes.data,
            None if cs is None else cs.ctypes.data, dst_scale))

    def matmul(self, name, src, b, b_scale, dst_scale):
        """MatrixMul + TypeCvt: src is a [batch][K] tensor (h = w = 1), b a [K, N] int8 array."""
        b = np.ascontiguousarray(b, dtype=np.int8)
        return _check(lib().mb200c_add_matmul(self._g, name.encode(), src, b.shape[1],
                                              b.ctypes.data, b_scale, dst_scale))

    # ---- fp32 operators ----
    def input_f32(self, name, c, h, w):
        return _check(lib().mb200c_add_input_f32(self._g, name.encode(), c, h, w))

    def conv_f32(self, name, src, flt, bias, stride, pad, nonline="IDENTITY", groups=1, z=None):
        flt = np.ascontiguousarray(flt, np.float32)
        kh, kw = flt.shape[-2:]
        oc = flt.shape[0] if flt.ndim == 4 else flt.shape[0] * flt.shape[1]
        b = None if bias is None else np.ascontiguousarray(np.asarray(bias).reshape(-1),
                                                           np.float32)
        return _check(lib().mb200c_add_conv_f32(
            self._g, name.encode(), src, oc, kh, kw, stride, pad, groups, nonline.encode(),
            flt.ctypes.data, None if b is None else b.ctypes.data, -1 if z is None else z))

    def matmul_f32(self, name, src, b):
        b = np.ascontiguousarray(b, np.float32)
        return _check(lib().mb200c_add_matmul_f32(self._g, name.encode(), src, b.shape[1],
                                                  b.ctypes.data))

    def elemwise_f32(self, name, mode, a, b=None):
        return _check(lib().mb200c_add_elemwise_f32(self._g, name.encode(), mode.encode(), a,
                                                    -1 if b is None else b))

    def concat(self, name, srcs):
        arr = (C.c_int * len(srcs))(*srcs)
        return _check(lib().mb200c_add_concat(self._g, name.encode(), arr, len(srcs)))

    def focus(self, name, src, c_out):
        return _check(lib().mb200c_add_focus(self._g, name.encode(), src, c_out))

    def resize_nearest(self, name, src, oh, ow):
        return _check(lib().mb200c_add_resize_nearest(self._g, name.encode(), src, oh, ow))

    def pooling(self, name, src, mode, window, stride, pad):
        return _check(lib().mb200c_add_pooling(self._g, name.encode(), src, mode.encode(), window,
                                               stride, pad))

    def qelemwise(self, name, mode, a, b, dst_scale):
        return _check(lib().mb200c_add_qelemwise(self._g, name.encode(), mode.encode(), a,
                                                 -1 if b is None else b, dst_scale))

    def set_option(self, name, value):
        _check(lib().mb200c_set_option(self._g, name.encode(), int(value)))

    def mark_output(self, t):
        _check(lib().mb200c_mark_output(self._g, t))

    def compile(self, batches):
        """-> bytes of the tinynn model with one DeviceModel per batch size."""
        arr = (C.c_int * len(batches))(*batches)
        ptr, n = _P(), C.c_size_t()
        _check(lib().mb200c_compile(self._g, arr, len(batches), C.byref(ptr), C.byref(n)))
        return C.string_at(ptr.value, n.value)

    def kernel_symbols(self):
        return lib().mb200c_kernel_symbols(self._g).decode().split()

    def arena_bytes(self, i=0):
        return lib().mb200c_arena_bytes(self._g, i)

    def unplanned_bytes(self, i=0):
        return lib().mb200c_unplanned_bytes(self._g, i)

    def export_kernels(self, directory):
        _check(lib().mb200c_export_kernels(self._g, directory.encode()))


def probe_conv_symbol(ic, oc, h, w, k, stride, pad, groups=1, nonline="IDENTITY", bias=True,
                      fmt="NCHW"):
    """(available, symbol) from the CUDA KernelGen pack for a ConvBias description."""
    buf = C.create_string_buffer(256)
    ok = lib().mb200c_probe_conv_symbol(ic, oc, h, w, k, stride, pad, groups, nonline.encode(),
                                        int(bias), fmt.encode(), buf, 256)
    return bool(ok), buf.value.decode()
