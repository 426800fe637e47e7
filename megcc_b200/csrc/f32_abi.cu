// extern "C" entry points of the fp32 path declared in include/megcc_b200.h.
#include "f32_internal.h"

using namespace mb200;

namespace {

size_t up256(size_t v) {
    return (v + 255) / 256 * 256;
}

int make_f32_args(const mb200_conv_f32_param* p, long long dst_pitch, ConvF32Args* a) {
    if (!p)
        return set_error(ST_NULL_PTR, "conv param is NULL");
    if (p->n <= 0 || p->ic <= 0 || p->oc <= 0 || p->ih <= 0 || p->iw <= 0 || p->kh <= 0 ||
        p->kw <= 0 || p->stride_h <= 0 || p->stride_w <= 0 || p->pad_h < 0 || p->pad_w < 0 ||
        p->groups <= 0)
        return set_error(ST_INVALID_LAYOUT, "conv param has a non-positive extent");
    if (p->ic % p->groups || p->oc % p->groups)
        return set_error(ST_INVALID_LAYOUT, "channels %d/%d not divisible by groups %d", p->ic,
                         p->oc, p->groups);
    if (p->nonline < 0 || p->nonline > MB200_F32_SILU)
        return set_error(ST_NO_IMPLEMENT, "nonlineMode %d not supported", p->nonline);
    a->n = p->n;
    a->ic = p->ic;
    a->ih = p->ih;
    a->iw = p->iw;
    a->oc = p->oc;
    a->kh = p->kh;
    a->kw = p->kw;
    a->sh = p->stride_h;
    a->sw = p->stride_w;
    a->ph = p->pad_h;
    a->pw = p->pad_w;
    a->groups = p->groups;
    a->oh = out_extent(p->ih, p->kh, p->stride_h, p->pad_h, 1);
    a->ow = out_extent(p->iw, p->kw, p->stride_w, p->pad_w, 1);
    if (a->oh <= 0 || a->ow <= 0)
        return set_error(ST_INVALID_LAYOUT, "filter larger than the padded input");
    const long long m = (long long)p->n * a->oh * a->ow;
    if (m > 0x3fffffffLL)
        return set_error(ST_OUT_OF_RANGE, "too many output pixels");
    a->m = (int)m;
    a->act = p->nonline;
    a->src_pitch = p->ic;
    a->dst_pitch = dst_pitch > 0 ? dst_pitch : p->oc;
    a->z_pitch = p->oc;
    if (a->dst_pitch < p->oc)
        return set_error(ST_INVALID_LAYOUT, "dst_pitch %lld is below the channel count %d",
                         a->dst_pitch, p->oc);
    return ST_SUCCESS;
}

// does the packed filter of this shape carry the tf32 planes?
bool split_eligible(const ConvF32Args& a) {
    return a.groups == 1 && (a.ic == 16 || a.ic % 32 == 0);
}

size_t plain_filter_bytes(const ConvF32Args& a) {
    return up256((size_t)a.oc * (a.ic / a.groups) * a.kh * a.kw * sizeof(float));
}

}  // namespace

extern "C" {

size_t mb200_conv_f32_packed_filter_bytes(const mb200_conv_f32_param* p) {
    ConvF32Args a{};
    if (make_f32_args(p, 0, &a))
        return 0;
    size_t bytes = plain_filter_bytes(a);
    if (split_eligible(a))
        bytes += up256(conv_f32_split_filter_floats(a) * sizeof(float));
    return bytes;
}

int mb200_conv_f32_pack_filter(
        const mb200_conv_f32_param* p, const float* flt_oihw, float* flt_packed, void* stream) {
    ConvF32Args a{};
    int rc = make_f32_args(p, 0, &a);
    if (rc)
        return rc;
    if (!flt_oihw || !flt_packed)
        return set_error(ST_NULL_PTR, "filter pointer is NULL");
    if (((uintptr_t)flt_oihw & 3) || ((uintptr_t)flt_packed & 15))
        return set_error(ST_INVALID_LAYOUT, "filter must be 4-byte, packed filter 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if ((rc = launch_conv_f32_pack_filter_plain(a, flt_oihw, flt_packed, st)))
        return rc;
    if (split_eligible(a))
        rc = launch_conv_f32_pack_filter_split(
                a, flt_oihw, (float*)((uint8_t*)flt_packed + plain_filter_bytes(a)), st);
    return rc;
}

size_t mb200_conv_f32_workspace_bytes(const mb200_conv_f32_param* p) {
    ConvF32Args a{};
    if (make_f32_args(p, 0, &a))
        return 0;
    return split_eligible(a) ? up256(conv_f32_workspace_bytes(a)) : 0;
}

int mb200_conv_bias_f32_nhwc(
        const mb200_conv_f32_param* p, const float* src, const float* flt_packed,
        const float* bias, const float* z, float* dst, long long dst_pitch, void* workspace,
        size_t workspace_bytes, int algo, void* stream) {
    ConvF32Args a{};
    int rc = make_f32_args(p, dst_pitch, &a);
    if (rc)
        return rc;
    if (!src || !flt_packed || !dst)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (((uintptr_t)src | (uintptr_t)flt_packed | (uintptr_t)dst | (uintptr_t)bias |
         (uintptr_t)z) & 3)
        return set_error(ST_INVALID_LAYOUT, "fp32 operands must be 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const bool umma_ok = split_eligible(a) && conv_f32_umma_supported(a, src, dst) &&
                         workspace_bytes >= conv_f32_workspace_bytes(a) &&
                         (((uintptr_t)workspace | (uintptr_t)flt_packed | (uintptr_t)bias |
                           (uintptr_t)z) & 15) == 0;
    if (algo == MB200_ALGO_UMMA && !umma_ok)
        return set_error(ST_NO_IMPLEMENT,
                         "tensor-core fp32 ConvBias needs a dense filter, ic == 16 or ic %% 32 == 0, "
                         "16-byte aligned operands and >= 128 KiB of input");
    if (algo == MB200_ALGO_UMMA || (algo == MB200_ALGO_AUTO && umma_ok))
        return launch_conv_f32_umma(
                a, src, (const float*)((const uint8_t*)flt_packed + plain_filter_bytes(a)), bias, z,
                dst, workspace, st);
    if (algo != MB200_ALGO_AUTO && algo != MB200_ALGO_DIRECT)
        return set_error(ST_OUT_OF_RANGE, "unknown algo %d", algo);
    return launch_conv_f32_direct(a, src, flt_packed, bias, z, dst, st);
}

// ---- fp32 matrix product: a 1x1 ConvBias over M "pixels" with K channels ----
static int matmul_f32_param(int m, int n, int k, mb200_conv_f32_param* p) {
    if (m <= 0 || n <= 0 || k <= 0)
        return set_error(ST_INVALID_LAYOUT, "matmul extents must be positive");
    memset(p, 0, sizeof(*p));
    p->n = m;
    p->ic = k;
    p->ih = p->iw = 1;
    p->oc = n;
    p->kh = p->kw = 1;
    p->stride_h = p->stride_w = 1;
    p->groups = 1;
    p->nonline = MB200_F32_IDENTITY;
    return ST_SUCCESS;
}

size_t mb200_matmul_f32_packed_b_bytes(int k, int n) {
    mb200_conv_f32_param p;
    if (matmul_f32_param(1, n, k, &p))
        return 0;
    // [N][K] transposed copy first (the conv's OIHW filter), then what the conv packs from it
    return up256((size_t)k * n * sizeof(float)) + mb200_conv_f32_packed_filter_bytes(&p);
}

int mb200_matmul_f32_pack_b(int k, int n, const float* b, float* b_packed, void* stream) {
    mb200_conv_f32_param p;
    int rc = matmul_f32_param(1, n, k, &p);
    if (rc)
        return rc;
    if (!b || !b_packed)
        return set_error(ST_NULL_PTR, "matmul operand pointer is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    // [K][N] row-major -> [N][K] = the OIHW filter of a 1x1 conv
    if ((rc = launch_transpose_f32(b, b_packed, 1, k, n, st)))
        return rc;
    return mb200_conv_f32_pack_filter(
            &p, b_packed, (float*)((uint8_t*)b_packed + up256((size_t)k * n * sizeof(float))), st);
}

size_t mb200_matmul_f32_workspace_bytes(int m, int k) {
    mb200_conv_f32_param p;
    if (matmul_f32_param(m, 1, k, &p))
        return 0;
    return mb200_conv_f32_workspace_bytes(&p);
}

int mb200_matmul_f32(
        int m, int n, int k, const float* a, const float* b_packed, float* c, void* workspace,
        size_t workspace_bytes, void* stream) {
    mb200_conv_f32_param p;
    int rc = matmul_f32_param(m, n, k, &p);
    if (rc)
        return rc;
    if (!a || !b_packed || !c)
        return set_error(ST_NULL_PTR, "matmul operand pointer is NULL");
    const float* packed =
            (const float*)((const uint8_t*)b_packed + up256((size_t)k * n * sizeof(float)));
    return mb200_conv_bias_f32_nhwc(&p, a, packed, nullptr, nullptr, c, 0, workspace,
                                    workspace_bytes, MB200_ALGO_AUTO, stream);
}

int mb200_elemwise_f32(
        int mode, const float* a, const float* b, float* dst, size_t nr_elem, void* stream) {
    const bool unary = mode >= MB200_ELEM_RELU && mode <= MB200_ELEM_EXP;
    const bool binary = mode >= MB200_ELEM_ADD && mode <= MB200_ELEM_FUSE_ADD_RELU;
    if (!unary && !binary)
        return set_error(ST_NO_IMPLEMENT, "elemwise mode %d not supported", mode);
    if (!a || !dst || (binary && !b))
        return set_error(ST_NULL_PTR, "elemwise tensor pointer is NULL");
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)dst) & 3)
        return set_error(ST_INVALID_LAYOUT, "fp32 operands must be 4-byte aligned");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_elemwise_f32(mode, a, binary ? b : a, dst, nr_elem, (cudaStream_t)stream);
}

int mb200_concat_f32_nhwc(
        const float* const* srcs, const int* channels, int nr_inputs, float* dst, size_t pixels,
        void* stream) {
    if (!srcs || !channels || !dst)
        return set_error(ST_NULL_PTR, "concat pointer is NULL");
    if (pixels == 0)
        return ST_SUCCESS;
    return launch_concat_f32(srcs, channels, nr_inputs, dst, pixels, (cudaStream_t)stream);
}

int mb200_resize_nearest_f32_nhwc(
        const float* src, float* dst, int n, int c, int ih, int iw, int oh, int ow, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "resize tensor pointer is NULL");
    if (n <= 0 || c <= 0 || ih <= 0 || iw <= 0 || oh <= 0 || ow <= 0)
        return set_error(ST_INVALID_LAYOUT, "resize extents must be positive");
    return launch_resize_nearest_f32(src, dst, n, c, ih, iw, oh, ow, (cudaStream_t)stream);
}

int mb200_pooling_f32_nhwc(
        const float* src, float* dst, int mode, int n, int c, int ih, int iw, int window_h,
        int window_w, int stride_h, int stride_w, int pad_h, int pad_w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "pooling tensor pointer is NULL");
    if (mode < 0 || mode > 2)
        return set_error(ST_NO_IMPLEMENT, "pooling mode %d not supported", mode);
    if (n <= 0 || c <= 0 || ih <= 0 || iw <= 0 || window_h <= 0 || window_w <= 0 ||
        stride_h <= 0 || stride_w <= 0 || pad_h < 0 || pad_w < 0 ||
        ih + 2 * pad_h < window_h || iw + 2 * pad_w < window_w || pad_h >= window_h ||
        pad_w >= window_w)
        return set_error(ST_INVALID_LAYOUT, "pooling extents are invalid");
    return launch_pooling_f32(src, dst, mode, n, c, ih, iw, window_h, window_w, stride_h,
                              stride_w, pad_h, pad_w, (cudaStream_t)stream);
}

int mb200_focus_f32(
        const float* src_nchw, float* dst_nhwc, int n, int c, int h, int w, int c_out,
        void* stream) {
    if (!src_nchw || !dst_nhwc)
        return set_error(ST_NULL_PTR, "focus tensor pointer is NULL");
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || (h & 1) || (w & 1) || c_out < 4 * c)
        return set_error(ST_INVALID_LAYOUT, "focus needs even extents and c_out >= 4 * c");
    return launch_focus_f32(src_nchw, dst_nhwc, n, c, h, w, c_out, (cudaStream_t)stream);
}

int mb200_relayout_nchw_to_nhwc_f32(
        const float* src, float* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    return launch_transpose_f32(src, dst, n, c, h * w, (cudaStream_t)stream);
}

int mb200_relayout_nhwc_to_nchw_f32(
        const float* src, float* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    return launch_transpose_f32(src, dst, n, h * w, c, (cudaStream_t)stream);
}

}  // extern "C"
