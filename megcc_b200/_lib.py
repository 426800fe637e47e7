"""Loads libmegcc_b200.so. There is no fallback: without the built CUDA library every
operator call raises."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmegcc_b200.so")


class ConvParam(C.Structure):
    """Mirror of ``mb200_conv_param`` (include/megcc_b200.h)."""
    _fields_ = [(k, C.c_int) for k in (
        "n", "ic", "ih", "iw", "oc", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w",
        "dilate_h", "dilate_w", "groups", "nonline")] + [
        ("src_scale", C.c_float), ("flt_scale", C.c_float), ("dst_scale", C.c_float)]


class ConvF32Param(C.Structure):
    """Mirror of ``mb200_conv_f32_param``."""
    _fields_ = [(k, C.c_int) for k in (
        "n", "ic", "ih", "iw", "oc", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w",
        "groups", "nonline")]


class ConvFuse(C.Structure):
    """Mirror of ``mb200_conv_fuse``."""
    _fields_ = [("z", C.c_void_p), ("mode", C.c_int), ("z_scale", C.c_float),
                ("out_scale", C.c_float)]


_lib = None

# name -> (restype, argtypes); every symbol declared in include/megcc_b200.h
_P = C.c_void_p
SIGNATURES = {
    "mb200_version": (C.c_char_p, []),
    "mb200_last_error": (C.c_char_p, []),
    "mb200_device_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "mb200_set_option": (C.c_int, [C.c_char_p, C.c_int]),
    "mb200_get_option": (C.c_int, [C.c_char_p, C.POINTER(C.c_int)]),
    "mb200_measure_mma_rate": (C.c_int, [C.c_int, _P, C.POINTER(C.c_double)]),
    "mb200_selftest_wait_expiry": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P, C.c_longlong, _P]),
    "mb200_register_readable_range": (C.c_int, [_P, C.c_size_t]),
    "mb200_unregister_readable_range": (C.c_int, [_P]),
    "mb200_tinynn_describe": (C.c_int, [_P, C.c_size_t, C.c_char_p, C.c_size_t]),
    "mb200_conv_packed_filter_bytes": (C.c_size_t, [C.POINTER(ConvParam)]),
    "mb200_conv_pack_filter": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P]),
    "mb200_conv_pack_filter_nchw44": (C.c_int, [C.POINTER(ConvParam), C.c_int, _P, _P, _P]),
    "mb200_relayout_nchw44_to_nhwc_s8": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
    "mb200_relayout_nhwc_to_nchw44_s8": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
    "mb200_conv_bias_qs8_nhwc": (C.c_int, [C.POINTER(ConvParam), _P, C.c_int, _P, _P, _P, _P,
                                           C.c_int, _P]),
    "mb200_conv_bias_qs8_nhwc_fused": (C.c_int, [C.POINTER(ConvParam), _P, C.c_int, _P, _P, _P, _P,
                                                 _P, C.c_int, _P]),
    "mb200_conv_s2d_supported": (C.c_int, [C.POINTER(ConvParam)]),
    "mb200_conv_s2d_filter_bytes": (C.c_size_t, [C.POINTER(ConvParam)]),
    "mb200_conv_s2d_workspace_bytes": (C.c_size_t, [C.POINTER(ConvParam)]),
    "mb200_conv_s2d_pack_filter": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P]),
    "mb200_conv_bias_qs8_s2d": (C.c_int, [C.POINTER(ConvParam), _P, C.c_int, _P, _P, _P, _P, _P,
                                          C.c_size_t, _P]),
    "mb200_conv_bias_pool_qs8_s2d": (C.c_int, [C.POINTER(ConvParam), _P, C.c_int, _P, _P, _P, _P, _P,
                                          C.c_size_t, _P]),
    "mb200_conv_s2d_pool_supported": (C.c_int, [C.POINTER(ConvParam)]),
    "mb200_conv_bias_qs8_nchw_workspace": (C.c_size_t, [C.POINTER(ConvParam)]),
    "mb200_conv_bias_qs8_nchw": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P, _P, _P, _P,
                                           C.c_size_t, C.c_int, _P]),
    "mb200_conv_bias_qs8_nchw_noalloc_max_scratch": (C.c_size_t, []),
    "mb200_conv_bias_qs8_nchw_noalloc": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P, _P, _P, _P]),
    "mb200_conv_acc_qs8_nhwc": (C.c_int, [C.POINTER(ConvParam), _P, _P, _P, _P, _P]),
    "mb200_requant_fast_constants": (C.c_int, [C.c_float, C.c_float, C.c_float, C.c_int,
                                               C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mb200_matmul_pack_b": (C.c_int, [C.c_int, C.c_int, _P, _P, _P]),
    "mb200_matmul_s8_s32": (C.c_int, [C.c_int, C.c_int, C.c_int, _P, _P, _P, _P]),
    "mb200_matmul_s8_qs8": (C.c_int, [C.c_int, C.c_int, C.c_int, _P, _P, _P, C.c_float, C.c_float,
                                      _P]),
    "mb200_pooling_qs8_nhwc": (C.c_int, [_P, _P] + [C.c_int] * 11 + [_P]),
    "mb200_qelemwise_qs8": (C.c_int, [_P, _P, _P, C.c_int, C.c_size_t, C.c_float, C.c_float,
                                      C.c_float, _P]),
    "mb200_typecvt_qs32_qs8": (C.c_int, [_P, _P, C.c_size_t, C.c_float, C.c_float, _P]),
    "mb200_typecvt_f32_qs8": (C.c_int, [_P, _P, C.c_size_t, C.c_float, C.c_float, _P]),
    "mb200_typecvt_qs8_f32": (C.c_int, [_P, _P, C.c_size_t, C.c_float, C.c_float, _P]),
    "mb200_qelemwise_qs8_bcast": (C.c_int, [_P, _P, _P, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t,
                                            C.c_float, C.c_float, C.c_float, _P]),
    "mb200_relayout_nchw_to_nhwc_s8": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
    "mb200_relayout_nhwc_to_nchw_s8": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
    # fp32 path
    "mb200_conv_f32_packed_filter_bytes": (C.c_size_t, [C.POINTER(ConvF32Param)]),
    "mb200_conv_f32_pack_filter": (C.c_int, [C.POINTER(ConvF32Param), _P, _P, _P]),
    "mb200_conv_f32_workspace_bytes": (C.c_size_t, [C.POINTER(ConvF32Param)]),
    "mb200_conv_bias_f32_nhwc": (C.c_int, [C.POINTER(ConvF32Param), _P, _P, _P, _P, _P,
                                           C.c_longlong, _P, C.c_size_t, C.c_int, _P]),
    "mb200_matmul_f32_packed_b_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "mb200_matmul_f32_pack_b": (C.c_int, [C.c_int, C.c_int, _P, _P, _P]),
    "mb200_matmul_f32_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "mb200_matmul_f32": (C.c_int, [C.c_int, C.c_int, C.c_int, _P, _P, _P, _P, C.c_size_t, _P]),
    "mb200_elemwise_f32": (C.c_int, [C.c_int, _P, _P, _P, C.c_size_t, _P]),
    "mb200_concat_f32_nhwc": (C.c_int, [C.POINTER(_P), C.POINTER(C.c_int), C.c_int, _P,
                                        C.c_size_t, _P]),
    "mb200_resize_nearest_f32_nhwc": (C.c_int, [_P, _P] + [C.c_int] * 6 + [_P]),
    "mb200_pooling_f32_nhwc": (C.c_int, [_P, _P] + [C.c_int] * 11 + [_P]),
    "mb200_focus_f32": (C.c_int, [_P, _P] + [C.c_int] * 5 + [_P]),
    "mb200_relayout_nchw_to_nhwc_f32": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
    "mb200_relayout_nhwc_to_nchw_f32": (C.c_int, [_P, _P] + [C.c_int] * 4 + [_P]),
}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m megcc_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class MegccError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"TinyNNStatus {status}: {msg}")
        self.status = status


def check(status):
    if status != 0:
        raise MegccError(status, lib().mb200_last_error().decode())
