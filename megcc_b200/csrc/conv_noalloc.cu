// ConvBias in the reference's layouts for callers that must not allocate device memory.
//
// Some users of this library cannot call cudaMalloc at the point where they need a
// convolution: an inference service that has handed the whole device to its own memory pool
// at start-up and has nothing left for the driver to give, or a latency-critical loop in
// which the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.
// mb200_conv_bias_qs8_nchw needs scratch memory from its caller for the NHWC copies and the
// packed filter; this variant takes that scratch from a fixed array that is part of the
// library image instead. Every GPU that loads the library carries the array (8 MiB) until
// the process exits, which is why it is kept modest and why larger problems are refused.
#include <stdint.h>

#include "../../include/megcc_b200.h"
#include "internal.h"

namespace {

constexpr size_t kScratchBytes = MB200_NOALLOC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime, not a device address: the address
// a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) uint8_t g_scratch[kScratchBytes];

// device address of g_scratch per CUDA ordinal, resolved on the first call on that device
uint8_t* g_scratch_addr[64] = {nullptr};

size_t align_up(size_t v, size_t a) {
    return (v + a - 1) / a * a;
}

int out_extent(int in, int k, int s, int p, int d) {
    return (in + 2 * p - d * (k - 1) - 1) / s + 1;
}

}  // namespace

using namespace mb200;

extern "C" {

size_t mb200_conv_bias_qs8_nchw_noalloc_max_scratch(void) {
    return kScratchBytes;
}

int mb200_conv_bias_qs8_nchw_noalloc(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_oihw,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* stream) {
    if (!p)
        return set_error(ST_NULL_PTR, "conv param is NULL");
    if (!src || !flt_oihw || !dst)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (p->n <= 0 || p->ic <= 0 || p->oc <= 0 || p->ih <= 0 || p->iw <= 0 || p->kh <= 0 ||
        p->kw <= 0 || p->stride_h <= 0 || p->stride_w <= 0 || p->pad_h < 0 || p->pad_w < 0 ||
        p->dilate_h <= 0 || p->dilate_w <= 0 || p->groups <= 0 || p->ic % p->groups ||
        p->oc % p->groups)
        return set_error(ST_INVALID_LAYOUT, "conv param has an invalid extent");
    if (p->nonline < 0 || p->nonline > 2)
        return set_error(ST_NO_IMPLEMENT, "nonlineMode %d not supported", p->nonline);

    ConvArgs a{};
    a.n = p->n;
    a.ic = p->ic;
    a.ih = p->ih;
    a.iw = p->iw;
    a.oc = p->oc;
    a.kh = p->kh;
    a.kw = p->kw;
    a.sh = p->stride_h;
    a.sw = p->stride_w;
    a.ph = p->pad_h;
    a.pw = p->pad_w;
    a.dh = p->dilate_h;
    a.dw = p->dilate_w;
    a.groups = p->groups;
    a.oh = out_extent(p->ih, p->kh, p->stride_h, p->pad_h, p->dilate_h);
    a.ow = out_extent(p->iw, p->kw, p->stride_w, p->pad_w, p->dilate_w);
    if (a.oh <= 0 || a.ow <= 0)
        return set_error(ST_INVALID_LAYOUT, "filter larger than the padded input");
    const long long m = (long long)p->n * a.oh * a.ow;
    if (m > 0x7fffffffLL)
        return set_error(ST_OUT_OF_RANGE, "too many output pixels");
    a.m = (int)m;
    a.act = p->nonline;
    a.src_is_nchw = 0;
    a.s_src = p->src_scale;
    a.s_flt = p->flt_scale;
    a.s_dst = p->dst_scale;

    // scratch layout: [src as NHWC][dst as NHWC][filter packed K-major], 256-byte aligned
    const size_t src_bytes = align_up((size_t)a.n * a.ih * a.iw * a.ic, 256);
    const size_t dst_bytes = align_up((size_t)a.m * a.oc, 256);
    const size_t flt_bytes = align_up((size_t)a.oc * (a.ic / a.groups) * a.kh * a.kw, 256);
    const size_t need = src_bytes + dst_bytes + flt_bytes;
    if (need > kScratchBytes)
        return set_error(ST_OUT_OF_RANGE,
                         "this convolution needs %zu bytes of scratch, the built-in scratch "
                         "holds %zu: use mb200_conv_bias_qs8_nchw with caller memory instead",
                         need, kScratchBytes);

    // one-time set-up per device, with that device current: resolve the array's device address
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64)
        return set_error(ST_RUNTIME, "no usable current CUDA device");
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_scratch);
        if (e != cudaSuccess || !ptr)
            return set_error(ST_RUNTIME, "cudaGetSymbolAddress(scratch): %s",
                             cudaGetErrorString(e));
        g_scratch_addr[dev] = (uint8_t*)ptr;
    }
    uint8_t* scratch = g_scratch_addr[dev];

    cudaStream_t st = (cudaStream_t)stream;
    int8_t* ws_src = (int8_t*)scratch;
    int8_t* ws_dst = ws_src + src_bytes;
    int8_t* ws_flt = ws_dst + dst_bytes;
    // Nothing in the scratch has to start at zero: every byte a kernel reads below is written
    // earlier in this same call, so whatever the previous call left behind is never seen.
    int rc = launch_transpose_s8(src, ws_src, a.n, a.ic, a.ih * a.iw, st);
    if (rc)
        return rc;
    if ((rc = launch_pack_filter(a, flt_oihw, ws_flt, st)))
        return rc;
    if ((rc = launch_conv_direct(a, ws_src, ws_flt, bias, flt_scales, ws_dst, nullptr, st)))
        return rc;
    return launch_transpose_s8(ws_dst, dst, a.n, a.oh * a.ow, a.oc, st);
}

}  // extern "C"
