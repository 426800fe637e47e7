"""Operator calls over device buffers (torch tensors are used only as device memory).

Each function mirrors one kernel family of the reference's KernelGen and calls straight
into the C ABI of libmegcc_b200.so on the current torch CUDA stream.
"""
import ctypes as C

import torch

from ._lib import ConvParam, check, lib

ACT = {"IDENTITY": 0, "RELU": 1, "H_SWISH": 2}
POOL = {"MAX": 0, "AVERAGE": 1, "AVERAGE_COUNT_EXCLUDE_PADDING": 2}
QELEM = {"QADD": 0, "QFUSE_ADD_RELU": 1, "QMUL": 2, "QRELU": 3}
ALGO = {"auto": 0, "direct": 1, "umma": 2, "patch": 3}


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def conv_param(n, ic, ih, iw, oc, kh, kw, stride, pad, groups, act, s_src, s_flt, s_dst,
               dilate=1):
    p = ConvParam()
    p.n, p.ic, p.ih, p.iw, p.oc, p.kh, p.kw = n, ic, ih, iw, oc, kh, kw
    p.stride_h = p.stride_w = stride
    p.pad_h = p.pad_w = pad
    p.dilate_h = p.dilate_w = dilate
    p.groups = groups
    p.nonline = ACT[act]
    p.src_scale, p.flt_scale, p.dst_scale = s_src, s_flt, s_dst
    return p


def out_hw(p):
    oh = (p.ih + 2 * p.pad_h - p.dilate_h * (p.kh - 1) - 1) // p.stride_h + 1
    ow = (p.iw + 2 * p.pad_w - p.dilate_w * (p.kw - 1) - 1) // p.stride_w + 1
    return oh, ow


def pack_filter(p, flt_oihw):
    """OIHW / [G,OCpg,ICpg,KH,KW] int8 device tensor -> K-major packed filter."""
    packed = torch.empty(lib().mb200_conv_packed_filter_bytes(C.byref(p)), dtype=torch.int8,
                         device=flt_oihw.device)
    check(lib().mb200_conv_pack_filter(C.byref(p), _ptr(flt_oihw), _ptr(packed), _stream()))
    return packed


def conv_bias_qs8_nhwc(p, src, flt_packed, bias, dst=None, flt_scales=None, algo="auto",
                       src_is_nchw=False):
    oh, ow = out_hw(p)
    if dst is None:
        dst = torch.empty((p.n, oh, ow, p.oc), dtype=torch.int8, device=src.device)
    check(lib().mb200_conv_bias_qs8_nhwc(
        C.byref(p), _ptr(src), int(src_is_nchw), _ptr(flt_packed), _ptr(bias), _ptr(flt_scales),
        _ptr(dst), ALGO[algo], _stream()))
    return dst


def conv_bias_qs8_nhwc_fused(p, src, flt_packed, bias, z, mode, z_scale, out_scale, algo="auto"):
    """ConvBias (p.nonline must be IDENTITY) followed by QADD / QFUSE_ADD_RELU with the int8
    tensor z of the output's NHWC shape, in one kernel."""
    from ._lib import ConvFuse
    oh, ow = out_hw(p)
    dst = torch.empty((p.n, oh, ow, p.oc), dtype=torch.int8, device=src.device)
    fuse = ConvFuse(z.data_ptr(), QELEM[mode], z_scale, out_scale)
    check(lib().mb200_conv_bias_qs8_nhwc_fused(
        C.byref(p), _ptr(src), 0, _ptr(flt_packed), _ptr(bias), None, C.byref(fuse), _ptr(dst),
        ALGO[algo], _stream()))
    return dst


def conv_acc_qs8_nhwc(p, src, flt_packed, bias):
    oh, ow = out_hw(p)
    acc = torch.empty((p.n, oh, ow, p.oc), dtype=torch.int32, device=src.device)
    check(lib().mb200_conv_acc_qs8_nhwc(C.byref(p), _ptr(src), _ptr(flt_packed), _ptr(bias),
                                        _ptr(acc), _stream()))
    return acc


def conv_bias_qs8_nchw(p, src, flt_oihw, bias, flt_scales=None, algo="auto"):
    """ConvBias in the reference's own layouts (NCHW activations, OIHW filter)."""
    oh, ow = out_hw(p)
    dst = torch.empty((p.n, p.oc, oh, ow), dtype=torch.int8, device=src.device)
    nbytes = lib().mb200_conv_bias_qs8_nchw_workspace(C.byref(p))
    ws = torch.empty(nbytes + 256, dtype=torch.int8, device=src.device)
    off = (-ws.data_ptr()) % 256
    check(lib().mb200_conv_bias_qs8_nchw(
        C.byref(p), _ptr(src), _ptr(flt_oihw), _ptr(bias), _ptr(flt_scales), _ptr(dst),
        C.c_void_p(ws.data_ptr() + off), nbytes, ALGO[algo], _stream()))
    return dst


def matmul_pack_b(b):
    """[K, N] int8 device tensor -> K-major [N, K] copy for the matrix product."""
    k, n = b.shape
    out = torch.empty((n, k), dtype=torch.int8, device=b.device)
    check(lib().mb200_matmul_pack_b(k, n, _ptr(b), _ptr(out), _stream()))
    return out


def matmul_s8_s32(a, b_packed):
    m, k = a.shape
    n = b_packed.shape[0]
    c = torch.empty((m, n), dtype=torch.int32, device=a.device)
    check(lib().mb200_matmul_s8_s32(m, n, k, _ptr(a), _ptr(b_packed), _ptr(c), _stream()))
    return c


def matmul_s8_qs8(a, b_packed, acc_scale, dst_scale):
    m, k = a.shape
    n = b_packed.shape[0]
    c = torch.empty((m, n), dtype=torch.int8, device=a.device)
    check(lib().mb200_matmul_s8_qs8(m, n, k, _ptr(a), _ptr(b_packed), _ptr(c), acc_scale,
                                    dst_scale, _stream()))
    return c


def pooling_qs8_nhwc(src, mode, window, stride, pad):
    n, ih, iw, c = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = torch.empty((n, oh, ow, c), dtype=torch.int8, device=src.device)
    check(lib().mb200_pooling_qs8_nhwc(_ptr(src), _ptr(dst), POOL[mode], n, c, ih, iw, window,
                                       window, stride, stride, pad, pad, _stream()))
    return dst


def qelemwise_qs8(mode, a, b, s0, s1, s_dst):
    dst = torch.empty_like(a)
    check(lib().mb200_qelemwise_qs8(_ptr(a), _ptr(b), _ptr(dst), QELEM[mode], a.numel(), s0, s1,
                                    s_dst, _stream()))
    return dst


def typecvt_qs32_qs8(src, s_src, s_dst):
    dst = torch.empty(src.shape, dtype=torch.int8, device=src.device)
    check(lib().mb200_typecvt_qs32_qs8(_ptr(src), _ptr(dst), src.numel(), s_src, s_dst, _stream()))
    return dst


def nchw_to_nhwc(src):
    n, c, h, w = src.shape
    dst = torch.empty((n, h, w, c), dtype=torch.int8, device=src.device)
    check(lib().mb200_relayout_nchw_to_nhwc_s8(_ptr(src), _ptr(dst), n, c, h, w, _stream()))
    return dst


def nhwc_to_nchw(src):
    n, h, w, c = src.shape
    dst = torch.empty((n, c, h, w), dtype=torch.int8, device=src.device)
    check(lib().mb200_relayout_nhwc_to_nchw_s8(_ptr(src), _ptr(dst), n, c, h, w, _stream()))
    return dst


def set_option(name, value):
    """Kernel-selection switch (see mb200_set_option); returns the previous value."""
    old = C.c_int(0)
    check(lib().mb200_get_option(name.encode(), C.byref(old)))
    check(lib().mb200_set_option(name.encode(), int(value)))
    return old.value


def measure_mma_rate(kind="i8"):
    """Sustained tcgen05.mma rate of the current GPU in TOP/s ("i8") or TFLOP/s ("tf32")."""
    v = C.c_double(0)
    check(lib().mb200_measure_mma_rate(0 if kind == "i8" else 1, _stream(), C.byref(v)))
    return v.value


def device_status():
    s = C.c_int(0)
    check(lib().mb200_device_status(_stream(), C.byref(s)))
    return s.value


# ----------------------------------------------------------------------------------------
# fp32 path (NHWC float32 device tensors)
# ----------------------------------------------------------------------------------------
F32_ACT = {"IDENTITY": 0, "RELU": 1, "H_SWISH": 2, "SIGMOID": 3, "SILU": 4}
ELEM = {"RELU": 0, "SIGMOID": 1, "SILU": 2, "H_SWISH": 3, "EXP": 4, "ADD": 16, "SUB": 17,
        "MUL": 18, "MAX": 19, "FUSE_ADD_RELU": 20}


def conv_f32_param(n, ic, ih, iw, oc, kh, kw, stride, pad, groups=1, act="IDENTITY"):
    from ._lib import ConvF32Param
    p = ConvF32Param()
    p.n, p.ic, p.ih, p.iw, p.oc, p.kh, p.kw = n, ic, ih, iw, oc, kh, kw
    p.stride_h = p.stride_w = stride
    p.pad_h = p.pad_w = pad
    p.groups = groups
    p.nonline = F32_ACT[act]
    return p


def _scratch(nbytes, device):
    """256-byte aligned device scratch of at least nbytes (None when nbytes == 0)."""
    if nbytes == 0:
        return None, None
    buf = torch.empty(nbytes + 256, dtype=torch.int8, device=device)
    return buf, buf.data_ptr() + (-buf.data_ptr()) % 256


def pack_filter_f32(p, flt_oihw):
    nbytes = lib().mb200_conv_f32_packed_filter_bytes(C.byref(p))
    packed = torch.empty(nbytes // 4, dtype=torch.float32, device=flt_oihw.device)
    check(lib().mb200_conv_f32_pack_filter(C.byref(p), _ptr(flt_oihw), _ptr(packed), _stream()))
    return packed


def conv_bias_f32_nhwc(p, src, flt_packed, bias=None, z=None, dst=None, dst_pitch=0,
                       algo="auto"):
    oh = (p.ih + 2 * p.pad_h - p.kh) // p.stride_h + 1
    ow = (p.iw + 2 * p.pad_w - p.kw) // p.stride_w + 1
    if dst is None:
        dst = torch.empty((p.n, oh, ow, p.oc), dtype=torch.float32, device=src.device)
    nbytes = lib().mb200_conv_f32_workspace_bytes(C.byref(p))
    keep, ws = _scratch(nbytes, src.device)
    check(lib().mb200_conv_bias_f32_nhwc(
        C.byref(p), _ptr(src), _ptr(flt_packed), _ptr(bias), _ptr(z), _ptr(dst), dst_pitch,
        None if ws is None else C.c_void_p(ws), nbytes, ALGO[algo], _stream()))
    torch.cuda.current_stream().synchronize()  # the scratch must outlive the kernels
    return dst


def matmul_f32(a, b):
    """C = A[M, K] @ B[K, N] (fp32 device tensors) through pack + product."""
    m, k = a.shape
    n = b.shape[1]
    packed = torch.empty(lib().mb200_matmul_f32_packed_b_bytes(k, n) // 4, dtype=torch.float32,
                         device=a.device)
    check(lib().mb200_matmul_f32_pack_b(k, n, _ptr(b), _ptr(packed), _stream()))
    c = torch.empty((m, n), dtype=torch.float32, device=a.device)
    nbytes = lib().mb200_matmul_f32_workspace_bytes(m, k)
    keep, ws = _scratch(nbytes, a.device)
    check(lib().mb200_matmul_f32(m, n, k, _ptr(a), _ptr(packed), _ptr(c),
                                 None if ws is None else C.c_void_p(ws), nbytes, _stream()))
    torch.cuda.current_stream().synchronize()
    return c


def elemwise_f32(mode, a, b=None):
    dst = torch.empty_like(a)
    check(lib().mb200_elemwise_f32(ELEM[mode], _ptr(a), _ptr(b), _ptr(dst), a.numel(), _stream()))
    return dst


def concat_f32_nhwc(tensors):
    n, h, w = tensors[0].shape[:3]
    chans = [t.shape[3] for t in tensors]
    dst = torch.empty((n, h, w, sum(chans)), dtype=torch.float32, device=tensors[0].device)
    ptrs = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    cs = (C.c_int * len(tensors))(*chans)
    check(lib().mb200_concat_f32_nhwc(ptrs, cs, len(tensors), _ptr(dst), n * h * w, _stream()))
    return dst


def resize_nearest_f32_nhwc(src, oh, ow):
    n, ih, iw, c = src.shape
    dst = torch.empty((n, oh, ow, c), dtype=torch.float32, device=src.device)
    check(lib().mb200_resize_nearest_f32_nhwc(_ptr(src), _ptr(dst), n, c, ih, iw, oh, ow,
                                              _stream()))
    return dst


def pooling_f32_nhwc(src, mode, window, stride, pad):
    n, ih, iw, c = src.shape
    oh, ow = (ih + 2 * pad - window) // stride + 1, (iw + 2 * pad - window) // stride + 1
    dst = torch.empty((n, oh, ow, c), dtype=torch.float32, device=src.device)
    check(lib().mb200_pooling_f32_nhwc(_ptr(src), _ptr(dst), POOL[mode], n, c, ih, iw, window,
                                       window, stride, stride, pad, pad, _stream()))
    return dst


def focus_f32(src_nchw, c_out):
    n, c, h, w = src_nchw.shape
    dst = torch.empty((n, h // 2, w // 2, c_out), dtype=torch.float32, device=src_nchw.device)
    check(lib().mb200_focus_f32(_ptr(src_nchw), _ptr(dst), n, c, h, w, c_out, _stream()))
    return dst


def nchw_to_nhwc_f32(x):
    n, c, h, w = x.shape
    y = torch.empty((n, h, w, c), dtype=torch.float32, device=x.device)
    check(lib().mb200_relayout_nchw_to_nhwc_f32(_ptr(x), _ptr(y), n, c, h, w, _stream()))
    return y


def nhwc_to_nchw_f32(x):
    n, h, w, c = x.shape
    y = torch.empty((n, c, h, w), dtype=torch.float32, device=x.device)
    check(lib().mb200_relayout_nhwc_to_nchw_f32(_ptr(x), _ptr(y), n, c, h, w, _stream()))
    return y


def qelemwise_qs8_bcast(mode, a, b, s0, s1, s_dst, channels, inner):
    """ElemwiseMultiType with b broadcast over a: b[(i / inner) % channels], or b[0]."""
    dst = torch.empty_like(a)
    check(lib().mb200_qelemwise_qs8_bcast(_ptr(a), _ptr(b), _ptr(dst), QELEM[mode], a.numel(),
                                          channels, inner, s0, s1, s_dst, _stream()))
    return dst


def typecvt_f32_qs8(src, s_src, s_dst):
    dst = torch.empty(src.shape, dtype=torch.int8, device=src.device)
    check(lib().mb200_typecvt_f32_qs8(_ptr(src), _ptr(dst), src.numel(), s_src, s_dst, _stream()))
    return dst


def typecvt_qs8_f32(src, s_src, s_dst):
    dst = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    check(lib().mb200_typecvt_qs8_f32(_ptr(src), _ptr(dst), src.numel(), s_src, s_dst, _stream()))
    return dst


def conv_s2d_supported(p):
    return bool(lib().mb200_conv_s2d_supported(C.byref(p)))


def conv_bias_qs8_s2d(p, src, flt_packed, bias, flt_scales=None, src_is_nchw=True):
    """First-layer ConvBias (few input channels) through the space-to-depth form; flt_packed
    from mb200_conv_s2d_pack_filter or pack_filter_nchw44."""
    oh, ow = out_hw(p)
    dst = torch.empty((p.n, oh, ow, p.oc), dtype=torch.int8, device=src.device)
    nbytes = lib().mb200_conv_s2d_workspace_bytes(C.byref(p))
    keep, ws = _scratch(nbytes, src.device)
    check(lib().mb200_conv_bias_qs8_s2d(
        C.byref(p), _ptr(src), int(src_is_nchw), _ptr(flt_packed), _ptr(bias), _ptr(flt_scales),
        _ptr(dst), ws, nbytes, _stream()))
    return dst


def pack_filter_s2d(p, flt_oihw):
    """OIHW int8 device tensor -> the space-to-depth packing of the first-layer form."""
    packed = torch.empty(lib().mb200_conv_s2d_filter_bytes(C.byref(p)), dtype=torch.int8,
                         device=flt_oihw.device)
    check(lib().mb200_conv_s2d_pack_filter(C.byref(p), _ptr(flt_oihw), _ptr(packed), _stream()))
    return packed


def conv_s2d_pool_supported(p):
    return bool(lib().mb200_conv_s2d_pool_supported(C.byref(p)))


def conv_bias_pool_qs8_s2d(p, src, flt_packed, bias, flt_scales=None, src_is_nchw=True):
    """First-layer ConvBias + MAX pooling 3x3 / 2 / pad 1 as one kernel; NHWC pooled result."""
    oh, ow = out_hw(p)
    dst = torch.empty((p.n, (oh - 1) // 2 + 1, (ow - 1) // 2 + 1, p.oc), dtype=torch.int8,
                      device=src.device)
    nbytes = lib().mb200_conv_s2d_workspace_bytes(C.byref(p))
    keep, ws = _scratch(nbytes, src.device)
    check(lib().mb200_conv_bias_pool_qs8_s2d(
        C.byref(p), _ptr(src), int(src_is_nchw), _ptr(flt_packed), _ptr(bias), _ptr(flt_scales),
        _ptr(dst), ws, nbytes, _stream()))
    return dst


# ---- NCHW44 (models compiled with --enable_nchw44) ----
NCHW44_FORMS = {"dense": 0, "channel_wise": 1, "first_layer": 2}


def pack_filter_nchw44(p, flt44, form):
    """Filter in an NCHW44 layout (dense [OC/4,IC/4,KH,KW,4,4], channel_wise [G/4,1,1,KH,KW,4],
    first_layer [OC/4,KH,KW,IC,4]) -> the packing the ConvBias entry points read: the
    space-to-depth packing where conv_s2d_supported(p), the K-major one otherwise."""
    s2d = bool(lib().mb200_conv_s2d_supported(C.byref(p)))
    nbytes = (lib().mb200_conv_s2d_filter_bytes if s2d else lib().mb200_conv_packed_filter_bytes)(
        C.byref(p))
    packed = torch.empty(nbytes, dtype=torch.int8, device=flt44.device)
    check(lib().mb200_conv_pack_filter_nchw44(C.byref(p), NCHW44_FORMS[form], _ptr(flt44),
                                              _ptr(packed), _stream()))
    return packed


def nchw44_to_nhwc(src):
    """[N, C/4, H, W, 4] int8 -> [N, H, W, C]"""
    n, cb, h, w, four = src.shape
    assert four == 4
    dst = torch.empty((n, h, w, cb * 4), dtype=torch.int8, device=src.device)
    check(lib().mb200_relayout_nchw44_to_nhwc_s8(_ptr(src), _ptr(dst), n, cb * 4, h, w, _stream()))
    return dst


def nhwc_to_nchw44(src):
    """[N, H, W, C] int8 -> [N, C/4, H, W, 4]"""
    n, h, w, c = src.shape
    dst = torch.empty((n, c // 4, h, w, 4), dtype=torch.int8, device=src.device)
    check(lib().mb200_relayout_nhwc_to_nchw44_s8(_ptr(src), _ptr(dst), n, c, h, w, _stream()))
    return dst
