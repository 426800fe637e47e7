// extern "C" operator-level entry points declared in include/megcc_b200.h.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/megcc_b200.h"
#include <map>
#include <mutex>

#include "internal.h"
#include "tuning.h"

namespace mb200 {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return set_error(ST_RUNTIME, "%s: %s", what, cudaGetErrorString(e));
    return ST_SUCCESS;
}

// One status word per (device, stream): a kernel whose bounded wait runs out records its
// code in the word of the stream it was launched on, so that a network waiting on its own
// stream never consumes another network's error. The words of a device come from one small
// allocation made at first use; a stream first seen while it is capturing (no set-up may
// happen then) and streams beyond the pool's capacity share word 0.
int* device_status_word(cudaStream_t st) {
    constexpr int kWords = 4096;
    struct Pool {
        int* base = nullptr;
        std::map<cudaStream_t, int> index;
        int next = 1;
    };
    static Pool pools[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_error(ST_RUNTIME, "no current CUDA device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    Pool& pool = pools[dev];
    if (!pool.base) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (st && cudaStreamIsCapturing(st, &cap) == cudaSuccess &&
            cap != cudaStreamCaptureStatusNone) {
            set_error(ST_RUNTIME, "first use of the library on this device during stream capture");
            return nullptr;
        }
        int* p = nullptr;
        if (cudaMalloc(&p, kWords * sizeof(int)) != cudaSuccess ||
            cudaMemset(p, 0, kWords * sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            set_error(ST_MALLOC, "cannot allocate the device status words");
            return nullptr;
        }
        pool.base = p;
    }
    auto it = pool.index.find(st);
    if (it != pool.index.end())
        return pool.base + it->second;
    if (pool.next >= kWords)
        return pool.base;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (st && cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return pool.base;
    cudaGetLastError();
    const int idx = pool.next++;
    pool.index[st] = idx;
    return pool.base + idx;
}

namespace {
struct TuningField {
    const char* name;
    const char* env;
    int Tuning::*field;
    bool env_negates;  // the variable switches the feature OFF
};
const TuningField kTuningFields[] = {
        {"conv_bn", "MB200_CONV_BN", &Tuning::conv_bn, false},
        {"conv_pair", "MB200_CONV_PAIR", &Tuning::conv_pair, false},
        {"conv_splitk", "MB200_CONV_SPLITK", &Tuning::conv_splitk, false},
        {"wide128", "MB200_NO_WIDE128", &Tuning::wide128, true},
        {"patch_ctas", "MB200_PATCH_CTAS", &Tuning::patch_ctas, false},
        {"patch_alone", "MB200_PATCH_ALONE", &Tuning::patch_alone, false},
        {"patch_plain", "MB200_PATCH_PLAIN", &Tuning::patch_plain, false},
        {"overlap_loads", "MB200_OVERLAP_LOADS", &Tuning::overlap_loads, false},
        {"dw_tensor", "MB200_DW_TENSOR", &Tuning::dw_tensor, false},
        {"dw_out", "MB200_DW_OUT", &Tuning::dw_out, false},
        {"dw_one_output", "MB200_DW_ONE_OUTPUT", &Tuning::dw_one_output, false},
        {"fast_requant", "MB200_NO_FAST_REQUANT", &Tuning::fast_requant, true},
        {"debug", "MB200_DEBUG", &Tuning::debug, false},
        {"pdl", "MB200_NO_PDL", &Tuning::pdl, true},
};
}  // namespace

Tuning& tuning() {
    static Tuning t = [] {
        Tuning v;
        for (const TuningField& f : kTuningFields) {
            const char* e = getenv(f.env);
            if (!e || !*e)
                continue;
            const int n = atoi(e);
            v.*(f.field) = f.env_negates ? (n != 0 ? 0 : 1) : n;
        }
        return v;
    }();
    return t;
}

int out_extent(int in, int k, int s, int p, int d) {
    return (in + 2 * p - d * (k - 1) - 1) / s + 1;
}

int make_args(const mb200_conv_param* p, int src_is_nchw, ConvArgs* a) {
    if (!p)
        return set_error(ST_NULL_PTR, "conv param is NULL");
    if (p->n <= 0 || p->ic <= 0 || p->oc <= 0 || p->ih <= 0 || p->iw <= 0 || p->kh <= 0 ||
        p->kw <= 0 || p->stride_h <= 0 || p->stride_w <= 0 || p->pad_h < 0 || p->pad_w < 0 ||
        p->dilate_h <= 0 || p->dilate_w <= 0 || p->groups <= 0)
        return set_error(ST_INVALID_LAYOUT, "conv param has a non-positive extent");
    if (p->ic % p->groups || p->oc % p->groups)
        return set_error(ST_INVALID_LAYOUT, "channels %d/%d not divisible by groups %d", p->ic,
                         p->oc, p->groups);
    if (p->nonline < 0 || p->nonline > 2)
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
    a->dh = p->dilate_h;
    a->dw = p->dilate_w;
    a->groups = p->groups;
    a->oh = out_extent(p->ih, p->kh, p->stride_h, p->pad_h, p->dilate_h);
    a->ow = out_extent(p->iw, p->kw, p->stride_w, p->pad_w, p->dilate_w);
    if (a->oh <= 0 || a->ow <= 0)
        return set_error(ST_INVALID_LAYOUT, "filter larger than the padded input");
    const long long m = (long long)p->n * a->oh * a->ow;
    if (m > 0x7fffffffLL)
        return set_error(ST_OUT_OF_RANGE, "too many output pixels");
    a->m = (int)m;
    a->act = p->nonline;
    a->src_is_nchw = src_is_nchw;
    a->s_src = p->src_scale;
    a->s_flt = p->flt_scale;
    a->s_dst = p->dst_scale;
    a->z = nullptr;
    a->z_mode = 0;
    a->z_scale = 1.f;
    a->z_out_scale = 1.f;
    a->acc_out = nullptr;
    a->pool = 0;
    a->true_division = division_range_ok(p->src_scale, p->flt_scale, p->dst_scale) ? 0 : 1;
    return ST_SUCCESS;
}

size_t align_up(size_t v, size_t a) {
    return (v + a - 1) / a * a;
}

}  // namespace mb200

using namespace mb200;

namespace mb200 {

namespace {
std::mutex g_ranges_mu;
std::map<uintptr_t, size_t> g_ranges;  // base -> bytes
}  // namespace

bool readable_through(const void* p, size_t bytes) {
    std::lock_guard<std::mutex> lock(g_ranges_mu);
    auto it = g_ranges.upper_bound((uintptr_t)p);
    if (it == g_ranges.begin())
        return false;
    --it;
    return (uintptr_t)p + bytes <= it->first + it->second;
}

int descriptor_images(const ConvArgs& a, const int8_t* src) {
    constexpr size_t kMinMapBytes = 131072;
    const size_t image = (size_t)a.ih * a.iw * (a.dw64 ? a.oc : a.ic);  // (dw64: a.ic is a slice)
    if ((size_t)a.n * image >= kMinMapBytes)
        return a.n;
    const size_t images = (kMinMapBytes + image - 1) / image;
    return readable_through(src, images * image) ? (int)images : 0;
}

}  // namespace mb200

extern "C" {

int mb200_register_readable_range(const void* base, size_t bytes) {
    if (!base || !bytes)
        return mb200::set_error(mb200::ST_NULL_PTR, "register_readable_range: empty range");
    std::lock_guard<std::mutex> lock(mb200::g_ranges_mu);
    mb200::g_ranges[(uintptr_t)base] = bytes;
    return 0;
}

int mb200_unregister_readable_range(const void* base) {
    std::lock_guard<std::mutex> lock(mb200::g_ranges_mu);
    mb200::g_ranges.erase((uintptr_t)base);
    return 0;
}


int mb200_set_option(const char* name, int value) {
    if (!name)
        return set_error(ST_NULL_PTR, "option name is NULL");
    for (const TuningField& f : kTuningFields)
        if (strcmp(name, f.name) == 0) {
            tuning().*(f.field) = value;
            return ST_SUCCESS;
        }
    return set_error(ST_OUT_OF_RANGE, "unknown option '%s'", name);
}

int mb200_get_option(const char* name, int* value) {
    if (!name || !value)
        return set_error(ST_NULL_PTR, "option name or value pointer is NULL");
    for (const TuningField& f : kTuningFields)
        if (strcmp(name, f.name) == 0) {
            *value = tuning().*(f.field);
            return ST_SUCCESS;
        }
    return set_error(ST_OUT_OF_RANGE, "unknown option '%s'", name);
}

const char* mb200_version(void) {
    return "megcc_b200 0.1 (sm_100a)";
}

const char* mb200_last_error(void) {
    return g_err;
}

int mb200_device_status(void* stream, int* status_host) {
    if (!status_host)
        return set_error(ST_NULL_PTR, "status_host is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    int* w = device_status_word(st);
    if (!w)
        return ST_MALLOC;
    int v = 0;
    if (cudaMemcpyAsync(&v, w, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
        return set_error(ST_RUNTIME, "reading the device status word failed: %s",
                         cudaGetErrorString(cudaGetLastError()));
    if (v != 0)
        cudaMemsetAsync(w, 0, sizeof(int), st);
    *status_host = v;
    return ST_SUCCESS;
}

size_t mb200_conv_packed_filter_bytes(const mb200_conv_param* p) {
    if (!p || p->groups <= 0)
        return 0;
    return (size_t)p->oc * (p->ic / p->groups) * p->kh * p->kw;
}

int mb200_conv_pack_filter(
        const mb200_conv_param* p, const int8_t* flt_oihw, int8_t* flt_packed, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!flt_oihw || !flt_packed)
        return set_error(ST_NULL_PTR, "filter pointer is NULL");
    return launch_pack_filter(a, flt_oihw, flt_packed, (cudaStream_t)stream);
}

int mb200_conv_pack_filter_nchw44(
        const mb200_conv_param* p, int form, const int8_t* flt_nchw44, int8_t* flt_packed,
        void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!flt_nchw44 || !flt_packed)
        return set_error(ST_NULL_PTR, "filter pointer is NULL");
    const int icpg = a.ic / a.groups;
    if (form < 0 || form > 2 || a.oc % 4 || (form == 0 && (a.groups != 1 || icpg % 4)) ||
        (form == 1 && (a.groups != a.ic || a.oc != a.ic)) || (form == 2 && a.groups != 1))
        return set_error(ST_INVALID_LAYOUT, "filter form %d does not fit %d -> %d channels in %d "
                         "groups", form, a.ic, a.oc, a.groups);
    cudaStream_t st = (cudaStream_t)stream;
    // through OIHW in a scratch buffer of the filter's size: load-time work, so the
    // allocation (and the synchronisation freeing it implies) is acceptable here
    const size_t bytes = (size_t)a.oc * icpg * a.kh * a.kw;
    int8_t* oihw = nullptr;
    if (cudaMalloc(&oihw, bytes) != cudaSuccess) {
        cudaGetLastError();
        return set_error(ST_MALLOC, "cannot allocate %zu bytes of filter scratch", bytes);
    }
    rc = launch_filter_nchw44_to_oihw(a, form, flt_nchw44, oihw, st);
    if (!rc)
        rc = conv_s2d_supported(a) ? launch_conv_s2d_pack_filter(a, oihw, flt_packed, st)
                                   : launch_pack_filter(a, oihw, flt_packed, st);
    cudaStreamSynchronize(st);
    cudaFree(oihw);
    return rc;
}

int mb200_relayout_nchw44_to_nhwc_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    if (c % 4 || (((uintptr_t)src | (uintptr_t)dst) & 3))
        return set_error(ST_INVALID_LAYOUT, "NCHW44 needs channels %% 4 == 0 and 4-byte aligned "
                                            "tensors");
    // [N][C/4][HW] four-byte groups -> [N][HW][C/4]
    return launch_transpose_f32((const float*)src, (float*)dst, n, c / 4, h * w,
                                (cudaStream_t)stream);
}

int mb200_relayout_nhwc_to_nchw44_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    if (c % 4 || (((uintptr_t)src | (uintptr_t)dst) & 3))
        return set_error(ST_INVALID_LAYOUT, "NCHW44 needs channels %% 4 == 0 and 4-byte aligned "
                                            "tensors");
    return launch_transpose_f32((const float*)src, (float*)dst, n, h * w, c / 4,
                                (cudaStream_t)stream);
}

int mb200_conv_bias_qs8_nhwc(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_packed,
        const int32_t* bias, const float* flt_scales, int8_t* dst, int algo, void* stream) {
    return mb200_conv_bias_qs8_nhwc_fused(
            p, src, src_is_nchw, flt_packed, bias, flt_scales, nullptr, dst, algo, stream);
}

int mb200_conv_bias_qs8_nhwc_fused(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_packed,
        const int32_t* bias, const float* flt_scales, const mb200_conv_fuse* fuse, int8_t* dst,
        int algo, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, src_is_nchw, &a);
    if (rc)
        return rc;
    if (fuse) {
        if (!fuse->z)
            return set_error(ST_NULL_PTR, "fused operand z is NULL");
        if (fuse->mode != MB200_QADD && fuse->mode != MB200_QFUSE_ADD_RELU)
            return set_error(ST_NO_IMPLEMENT, "fused elemwise mode %d not supported", fuse->mode);
        if (p->nonline != MB200_IDENTITY)
            return set_error(ST_NO_IMPLEMENT, "a fused elemwise step needs a ConvBias without "
                                              "activation");
        if ((uintptr_t)fuse->z & 15)
            return set_error(ST_INVALID_LAYOUT, "fused operand z must be 16-byte aligned");
        a.z = fuse->z;
        a.z_mode = fuse->mode == MB200_QADD ? 1 : 2;
        a.z_scale = fuse->z_scale;
        a.z_out_scale = fuse->out_scale;
    }
    if (!src || !flt_packed || !dst)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (((uintptr_t)bias | (uintptr_t)flt_scales) & 3)
        return set_error(ST_INVALID_LAYOUT, "bias and channel scales must be 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    // the vector kernels load bias and channel scales 16 bytes at a time
    // ... and divide by a constant in three instructions, which is exact inside a scale range
    const bool side_ok =
            ((((uintptr_t)bias | (uintptr_t)flt_scales) & 15) == 0) && !a.true_division;
    if (algo == MB200_ALGO_PATCH && a.groups > 1) {
        // a depthwise ConvBias asked onto the halo-patch kernel: its block-diagonal form
        if (!side_ok || !conv_patch_dw_supported(a, src, flt_packed, dst, true))
            return set_error(ST_NO_IMPLEMENT,
                             "halo-patch depthwise ConvBias needs 3x3, stride 1, channels %% 64 "
                             "== 0 (or 32 channels, even width, padding 1), NHWC, 16-byte aligned "
                             "tensors and >= 128 KiB of input");
        return launch_conv_patch_dw(a, src, flt_packed, bias, flt_scales, dst, st);
    }
    const bool patch_ok = side_ok && conv_patch_supported(a, src, flt_packed, dst);
    if (algo == MB200_ALGO_PATCH && !patch_ok)
        return set_error(ST_NO_IMPLEMENT,
                         "halo-patch ConvBias needs dense, stride 1, NHWC, ic in {16, 32k <= 128}, "
                         "16-byte aligned tensors and >= 128 KiB of input");
    // the patch kernel pays for partial 16x8 patches; below 3/4 useful rows im2col wins
    const bool umma_ok = side_ok && conv_umma_supported(a, src, flt_packed, dst);
    // a pointwise convolution has no halo to share: the plain-matrix loads of the im2col
    // kernel measured equal or up to 18 % faster (128 -> 256 channels at 28 x 28, batch 256)
    const bool pointwise = a.kh == 1 && a.kw == 1 && umma_ok;
    if (algo == MB200_ALGO_PATCH ||
        (algo == MB200_ALGO_AUTO && patch_ok && !pointwise && conv_patch_efficiency(a) >= 0.75f))
        return launch_conv_patch(a, src, flt_packed, bias, flt_scales, dst, st);
    if (algo == MB200_ALGO_UMMA && !umma_ok)
        return set_error(ST_NO_IMPLEMENT,
                         "tensor-core ConvBias needs dense, NHWC, ic %% 64 == 0, oc %% 8 == 0, "
                         "16-byte aligned tensors and >= 128 KiB of input");
    if (algo == MB200_ALGO_UMMA || (algo == MB200_ALGO_AUTO && umma_ok))
        return launch_conv_umma(a, src, flt_packed, bias, flt_scales, dst, st);
    if (algo != MB200_ALGO_AUTO && algo != MB200_ALGO_DIRECT)
        return set_error(ST_OUT_OF_RANGE, "unknown algo %d", algo);
    // depthwise 3x3 / stride 1 over whole 64-channel slices: the halo-patch tensor-core kernel
    // with a block-diagonal filter (63 of 64 MACs multiply zeros, and it is still the faster
    // form: the CUDA-core kernel below is bound by instruction issue)
    if (algo == MB200_ALGO_AUTO && side_ok && tuning().dw_tensor &&
        conv_patch_dw_supported(a, src, flt_packed, dst))
        return launch_conv_patch_dw(a, src, flt_packed, bias, flt_scales, dst, st);
    // depthwise 3x3: vector loads and dp4a over taps
    if (algo == MB200_ALGO_AUTO && side_ok && conv_dw_supported(a, src, flt_packed, dst))
        return launch_conv_dw(a, src, flt_packed, bias, flt_scales, dst, st);
    return launch_conv_direct(a, src, flt_packed, bias, flt_scales, dst, nullptr, st);
}

int mb200_selftest_wait_expiry(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_packed, int8_t* dst,
        long long limit_cycles, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!src || !flt_packed || !dst)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (limit_cycles < 1000 || limit_cycles > (1LL << 31))
        return set_error(ST_OUT_OF_RANGE, "limit of %lld cycles is outside [1000, 2^31]",
                         limit_cycles);
    if (!conv_umma_supported(a, src, flt_packed, dst) || a.kh * a.kw * (a.ic / 64) < 3)
        return set_error(ST_NO_IMPLEMENT, "the self-test needs a shape of the tensor-core "
                                          "ConvBias with at least three pipeline steps");
    a.test_wait_cycles = limit_cycles;
    a.test_skip_step = 1;
    return launch_conv_umma(a, src, flt_packed, nullptr, nullptr, dst, (cudaStream_t)stream);
}

int mb200_conv_acc_qs8_nhwc(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_packed,
        const int32_t* bias, int32_t* acc, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!src || !flt_packed || !acc)
        return set_error(ST_NULL_PTR, "conv tensor pointer is NULL");
    if (((uintptr_t)bias | (uintptr_t)acc) & 3)
        return set_error(ST_INVALID_LAYOUT, "bias and acc must be 4-byte aligned");
    return launch_conv_direct(
            a, src, flt_packed, bias, nullptr, nullptr, acc, (cudaStream_t)stream);
}

int mb200_conv_s2d_supported(const mb200_conv_param* p) {
    ConvArgs a{};
    if (make_args(p, 0, &a))
        return 0;
    return conv_s2d_supported(a) ? 1 : 0;
}

size_t mb200_conv_s2d_filter_bytes(const mb200_conv_param* p) {
    ConvArgs a{};
    if (make_args(p, 0, &a))
        return 0;
    return conv_s2d_filter_bytes(a);
}

size_t mb200_conv_s2d_workspace_bytes(const mb200_conv_param* p) {
    ConvArgs a{};
    if (make_args(p, 0, &a))
        return 0;
    return conv_s2d_workspace_bytes(a);
}

int mb200_conv_s2d_pack_filter(
        const mb200_conv_param* p, const int8_t* flt_oihw, int8_t* flt_s2d, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!flt_oihw || !flt_s2d)
        return set_error(ST_NULL_PTR, "filter pointer is NULL");
    if (!conv_s2d_supported(a))
        return set_error(ST_NO_IMPLEMENT, "the space-to-depth path does not apply to this conv");
    return launch_conv_s2d_pack_filter(a, flt_oihw, flt_s2d, (cudaStream_t)stream);
}

int mb200_conv_bias_qs8_s2d(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_s2d,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, src_is_nchw, &a);
    if (rc)
        return rc;
    if (!src || !flt_s2d || !dst || !workspace)
        return set_error(ST_NULL_PTR, "conv tensor or workspace pointer is NULL");
    if (!conv_s2d_supported(a))
        return set_error(ST_NO_IMPLEMENT, "the space-to-depth path does not apply to this conv");
    if (a.true_division)
        return set_error(ST_OUT_OF_RANGE, "scales %g * %g / %g are outside the range of the "
                         "tensor-core epilogue: use mb200_conv_bias_qs8_nhwc", p->src_scale,
                         p->flt_scale, p->dst_scale);
    if (workspace_bytes < conv_s2d_workspace_bytes(a))
        return set_error(ST_OUT_OF_RANGE, "workspace of %zu bytes is too small", workspace_bytes);
    if (((uintptr_t)workspace | (uintptr_t)flt_s2d | (uintptr_t)dst) & 15)
        return set_error(ST_INVALID_LAYOUT, "workspace, filter and dst must be 16-byte aligned");
    return launch_conv_s2d(a, src, flt_s2d, bias, flt_scales, dst, workspace, (cudaStream_t)stream);
}

int mb200_conv_s2d_pool_supported(const mb200_conv_param* p) {
    ConvArgs a{};
    if (make_args(p, 0, &a))
        return 0;
    return conv_s2d_pool_supported(a) && !a.true_division ? 1 : 0;
}

int mb200_conv_bias_pool_qs8_s2d(
        const mb200_conv_param* p, const int8_t* src, int src_is_nchw, const int8_t* flt_s2d,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, src_is_nchw, &a);
    if (rc)
        return rc;
    if (!src || !flt_s2d || !dst || !workspace)
        return set_error(ST_NULL_PTR, "conv tensor or workspace pointer is NULL");
    if (!conv_s2d_pool_supported(a) || a.true_division)
        return set_error(ST_NO_IMPLEMENT, "ConvBias + MAX pooling 3x3/2 does not apply to this "
                                          "conv: see mb200_conv_s2d_pool_supported");
    if (workspace_bytes < conv_s2d_workspace_bytes(a))
        return set_error(ST_OUT_OF_RANGE, "workspace of %zu bytes is too small", workspace_bytes);
    if (((uintptr_t)workspace | (uintptr_t)flt_s2d | (uintptr_t)dst) & 15)
        return set_error(ST_INVALID_LAYOUT, "workspace, filter and dst must be 16-byte aligned");
    a.pool = 1;
    return launch_conv_s2d(a, src, flt_s2d, bias, flt_scales, dst, workspace, (cudaStream_t)stream);
}

size_t mb200_conv_bias_qs8_nchw_workspace(const mb200_conv_param* p) {
    ConvArgs a{};
    if (make_args(p, 0, &a))
        return 0;
    const size_t dst = align_up((size_t)a.m * a.oc, 256);
    if (conv_s2d_supported(a))
        return dst + align_up(conv_s2d_filter_bytes(a), 256) + conv_s2d_workspace_bytes(a);
    const size_t src = align_up((size_t)a.n * a.ih * a.iw * a.ic, 256);
    const size_t flt = align_up(mb200_conv_packed_filter_bytes(p), 256);
    return src + dst + flt;
}

int mb200_conv_bias_qs8_nchw(
        const mb200_conv_param* p, const int8_t* src, const int8_t* flt_oihw,
        const int32_t* bias, const float* flt_scales, int8_t* dst, void* workspace,
        size_t workspace_bytes, int algo, void* stream) {
    ConvArgs a{};
    int rc = make_args(p, 0, &a);
    if (rc)
        return rc;
    if (!src || !flt_oihw || !dst || !workspace)
        return set_error(ST_NULL_PTR, "conv tensor or workspace pointer is NULL");
    if (workspace_bytes < mb200_conv_bias_qs8_nchw_workspace(p))
        return set_error(ST_OUT_OF_RANGE, "workspace of %zu bytes is too small", workspace_bytes);
    if ((uintptr_t)workspace & 255)
        return set_error(ST_INVALID_LAYOUT, "workspace must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (conv_s2d_supported(a) && algo != MB200_ALGO_DIRECT && !a.true_division) {
        // first-layer form: the input is read in place, only the output needs a transpose
        int8_t* ws_dst = (int8_t*)workspace;
        int8_t* ws_flt = ws_dst + align_up((size_t)a.m * a.oc, 256);
        int8_t* ws_s2d = ws_flt + align_up(conv_s2d_filter_bytes(a), 256);
        a.src_is_nchw = 1;
        if ((rc = launch_conv_s2d_pack_filter(a, flt_oihw, ws_flt, st)))
            return rc;
        if ((rc = launch_conv_s2d(a, src, ws_flt, bias, flt_scales, ws_dst, ws_s2d, st)))
            return rc;
        return launch_transpose_s8(ws_dst, dst, a.n, a.oh * a.ow, a.oc, st);
    }
    if (conv_s2d_supported(a)) {
        // the general kernel on this shape: same scratch budget, standard packing
        const size_t need = align_up((size_t)a.n * a.ih * a.iw * a.ic, 256) +
                            align_up((size_t)a.m * a.oc, 256) +
                            align_up(mb200_conv_packed_filter_bytes(p), 256);
        if (workspace_bytes < need)
            return set_error(ST_OUT_OF_RANGE, "workspace of %zu bytes is too small",
                             workspace_bytes);
    }
    int8_t* ws_src = (int8_t*)workspace;
    int8_t* ws_dst = ws_src + align_up((size_t)a.n * a.ih * a.iw * a.ic, 256);
    int8_t* ws_flt = ws_dst + align_up((size_t)a.m * a.oc, 256);
    // NCHW -> NHWC is a [C][HW] -> [HW][C] transpose per image
    if ((rc = launch_transpose_s8(src, ws_src, a.n, a.ic, a.ih * a.iw, st)))
        return rc;
    if ((rc = launch_pack_filter(a, flt_oihw, ws_flt, st)))
        return rc;
    if ((rc = mb200_conv_bias_qs8_nhwc(p, ws_src, 0, ws_flt, bias, flt_scales, ws_dst, algo, st)))
        return rc;
    return launch_transpose_s8(ws_dst, dst, a.n, a.oh * a.ow, a.oc, st);
}

int mb200_requant_fast_constants(
        float src_scale, float flt_scale, float dst_scale, int nonline, float* mul, float* add) {
    float c = 0.f, d = 0.f;
    const int ops = requant_fast_constants(src_scale, flt_scale, dst_scale, nonline, &c, &d);
    if (mul)
        *mul = c;
    if (add)
        *add = d;
    return ops;
}

// ---- int8 matrix product: a 1x1 ConvBias over M "pixels" with K channels ----
static int matmul_args(int m, int n, int k, ConvArgs* a) {
    if (m <= 0 || n <= 0 || k <= 0)
        return set_error(ST_INVALID_LAYOUT, "matmul extents must be positive");
    mb200_conv_param p;
    memset(&p, 0, sizeof(p));
    p.n = m;
    p.ic = k;
    p.ih = p.iw = 1;
    p.oc = n;
    p.kh = p.kw = 1;
    p.stride_h = p.stride_w = p.dilate_h = p.dilate_w = 1;
    p.groups = 1;
    p.nonline = MB200_IDENTITY;
    p.src_scale = p.flt_scale = p.dst_scale = 1.f;
    return make_args(&p, 0, a);
}

int mb200_matmul_pack_b(int k, int n, const int8_t* b, int8_t* b_packed, void* stream) {
    if (!b || !b_packed)
        return set_error(ST_NULL_PTR, "matmul operand pointer is NULL");
    if (k <= 0 || n <= 0)
        return set_error(ST_INVALID_LAYOUT, "matmul extents must be positive");
    // [K][N] row-major -> [N][K]: K-major rows, the layout the filter of a 1x1 conv has
    return launch_transpose_s8(b, b_packed, 1, k, n, (cudaStream_t)stream);
}

int mb200_matmul_s8_s32(
        int m, int n, int k, const int8_t* a, const int8_t* b_packed, int32_t* c, void* stream) {
    ConvArgs args{};
    int rc = matmul_args(m, n, k, &args);
    if (rc)
        return rc;
    if (!a || !b_packed || !c)
        return set_error(ST_NULL_PTR, "matmul operand pointer is NULL");
    if ((uintptr_t)c & 3)
        return set_error(ST_INVALID_LAYOUT, "the int32 product must be 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (conv_umma_supported(args, a, b_packed, (const int8_t*)c)) {
        args.acc_out = c;
        return launch_conv_umma(args, a, b_packed, nullptr, nullptr, (int8_t*)c, st);
    }
    return launch_conv_direct(args, a, b_packed, nullptr, nullptr, nullptr, c, st);
}

int mb200_matmul_s8_qs8(
        int m, int n, int k, const int8_t* a, const int8_t* b_packed, int8_t* c, float acc_scale,
        float dst_scale, void* stream) {
    ConvArgs args{};
    int rc = matmul_args(m, n, k, &args);
    if (rc)
        return rc;
    if (!a || !b_packed || !c)
        return set_error(ST_NULL_PTR, "matmul operand pointer is NULL");
    // requantisation of the int32 product by the TypeCvt rule val * src_scale / dst_scale:
    // the ConvBias form acc * s_src * s_flt / s_dst with s_flt = 1 (a multiplication by 1.0f
    // is exact), so both are the same float operations in the same order
    args.s_src = acc_scale;
    args.s_flt = 1.f;
    args.s_dst = dst_scale;
    args.true_division = division_range_ok(acc_scale, 1.f, dst_scale) ? 0 : 1;
    cudaStream_t st = (cudaStream_t)stream;
    if (!args.true_division && conv_umma_supported(args, a, b_packed, c))
        return launch_conv_umma(args, a, b_packed, nullptr, nullptr, c, st);
    return launch_conv_direct(args, a, b_packed, nullptr, nullptr, c, nullptr, st);
}

int mb200_pooling_qs8_nhwc(
        const int8_t* src, int8_t* dst, int mode, int n, int c, int ih, int iw, int window_h,
        int window_w, int stride_h, int stride_w, int pad_h, int pad_w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "pooling tensor pointer is NULL");
    if (mode < 0 || mode > 2)
        return set_error(ST_NO_IMPLEMENT, "pooling mode %d not supported", mode);
    if (n <= 0 || c <= 0 || ih <= 0 || iw <= 0 || window_h <= 0 || window_w <= 0 ||
        stride_h <= 0 || stride_w <= 0 || pad_h < 0 || pad_w < 0 ||
        ih + 2 * pad_h < window_h || iw + 2 * pad_w < window_w)
        return set_error(ST_INVALID_LAYOUT, "pooling extents are invalid");
    return launch_pooling(
            src, dst, mode, n, c, ih, iw, window_h, window_w, stride_h, stride_w, pad_h, pad_w,
            (cudaStream_t)stream);
}

int mb200_qelemwise_qs8(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, float scale_a,
        float scale_b, float scale_dst, void* stream) {
    if (mode < 0 || mode > 3)
        return set_error(ST_NO_IMPLEMENT, "elemwise mode %d not supported", mode);
    if (!a || !dst || (mode != MB200_QRELU && !b))
        return set_error(ST_NULL_PTR, "elemwise tensor pointer is NULL");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_qelemwise(
            a, mode == MB200_QRELU ? a : b, dst, mode, nr_elem, scale_a, scale_b, scale_dst,
            (cudaStream_t)stream);
}

int mb200_qelemwise_qs8_bcast(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem,
        size_t b_channels, size_t inner, float scale_a, float scale_b, float scale_dst,
        void* stream) {
    if (mode < 0 || mode > 2)
        return set_error(ST_NO_IMPLEMENT, "elemwise mode %d takes no second operand to broadcast",
                         mode);
    if (!a || !b || !dst)
        return set_error(ST_NULL_PTR, "elemwise tensor pointer is NULL");
    if (b_channels > 0xffffffffull || inner > 0xffffffffull || (b_channels && !inner))
        return set_error(ST_INVALID_LAYOUT, "broadcast extents are invalid");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_qelemwise_bcast(a, b, dst, mode, nr_elem, (unsigned)b_channels, (unsigned)inner,
                                  scale_a, scale_b, scale_dst, (cudaStream_t)stream);
}

int mb200_typecvt_f32_qs8(
        const float* src, int8_t* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "typecvt tensor pointer is NULL");
    if ((uintptr_t)src & 3)
        return set_error(ST_INVALID_LAYOUT, "typecvt source must be 4-byte aligned");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_typecvt_f32_qs8(src, dst, nr_elem, src_scale, dst_scale, (cudaStream_t)stream);
}

int mb200_typecvt_qs8_f32(
        const int8_t* src, float* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "typecvt tensor pointer is NULL");
    if ((uintptr_t)dst & 3)
        return set_error(ST_INVALID_LAYOUT, "typecvt destination must be 4-byte aligned");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_typecvt_qs8_f32(src, dst, nr_elem, src_scale, dst_scale, (cudaStream_t)stream);
}

int mb200_typecvt_qs32_qs8(
        const int32_t* src, int8_t* dst, size_t nr_elem, float src_scale, float dst_scale,
        void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "typecvt tensor pointer is NULL");
    if ((uintptr_t)src & 3)
        return set_error(ST_INVALID_LAYOUT, "typecvt source must be 4-byte aligned");
    if (nr_elem == 0)
        return ST_SUCCESS;
    return launch_typecvt_qs32_qs8(
            src, dst, nr_elem, src_scale, dst_scale, (cudaStream_t)stream);
}

int mb200_relayout_nchw_to_nhwc_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    return launch_transpose_s8(src, dst, n, c, h * w, (cudaStream_t)stream);
}

int mb200_relayout_nhwc_to_nchw_s8(
        const int8_t* src, int8_t* dst, int n, int c, int h, int w, void* stream) {
    if (!src || !dst)
        return set_error(ST_NULL_PTR, "relayout tensor pointer is NULL");
    return launch_transpose_s8(src, dst, n, h * w, c, (cudaStream_t)stream);
}

}  // extern "C"
