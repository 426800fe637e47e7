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

#include <atomic>

#include "../../include/megcc_b200.h"
#include "internal.h"

namespace {

constexpr size_t kScratchBytes = MB200_NOALLOC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime, not a device address: the address
// a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) uint8_t g_scratch[kScratchBytes];

// device address of g_scratch per CUDA ordinal, resolved on the first call on that device.
// Atomic: several host threads may make their first call at once; each would store the same
// address.
std::atomic<uint8_t*> g_scratch_addr[64];

}  // namespace

using namespace mb200;

extern "C" {

size_t mb200_conv_bias_qs8_nchw_noalloc_max_scratch(void) {
    return kScratchBytes;
}

int mb200_conv_bias_qs8_nchw_noalloc(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_oihw,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* stream) {
    // the same validation and argument block as every other ConvBias entry point
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!src || !flt_oihw || !dst)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (((uintptr_t)bias | (uintptr_t)flt_scales) & 3)
        return set_error(ST_INVALID_LAYOUT, "bias and channel scales must be 4-byte aligned");

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
    uint8_t* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_scratch);
        if (e != cudaSuccess || !ptr)
            return set_error(ST_RUNTIME, "cudaGetSymbolAddress(scratch): %s",
                             cudaGetErrorString(e));
        scratch = (uint8_t*)ptr;
        g_scratch_addr[dev].store(scratch, std::memory_order_release);
    }

    cudaStream_t st = (cudaStream_t)stream;
    int8_t* ws_src = (int8_t*)scratch;
    int8_t* ws_dst = ws_src + src_bytes;
    int8_t* ws_flt = ws_dst + dst_bytes;
    // Nothing in the scratch has to start at zero: every byte a kernel reads below is written
    // earlier in this same call, so whatever the previous call left behind is never seen.
    rc = launch_transpose_s8(src, ws_src, a.n, a.ic, a.ih * a.iw, st);
    if (rc)
        return rc;
    if ((rc = launch_pack_filter(a, flt_oihw, ws_flt, st)))
        return rc;
    if ((rc = launch_conv_direct(a, ws_src, ws_flt, bias, flt_scales, ws_dst, nullptr, st)))
        return rc;
    return launch_transpose_s8(ws_dst, dst, a.n, a.oh * a.ow, a.oc, st);
}

}  // extern "C"
