// Internal declarations shared by the kernel translation units and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace mb200 {

// TinyNNStatus values used by this library (runtime/src/tinynn.h:9-24 in the reference)
enum Status : int {
    ST_SUCCESS = 0,
    ST_NULL_PTR = 1,
    ST_RUNTIME = 3,
    ST_OUT_OF_RANGE = 4,
    ST_NO_IMPLEMENT = 6,
    ST_MODEL_PARSE = 7,
    ST_OPEN_FILE = 8,
    ST_MALLOC = 9,
    ST_UNSUPPORTED_INST = 10,
    ST_UNSUPPORTED_DTYPE = 11,
    ST_INVALID_LAYOUT = 12,
    ST_ERROR = 13,
};

// Everything a conv kernel needs, by value.
struct ConvArgs {
    int n, ic, ih, iw, oc, oh, ow;
    int kh, kw, sh, sw, ph, pw, dh, dw, groups;
    int m;  // n * oh * ow
    int act;
    int src_is_nchw;
    float s_src, s_flt, s_dst;
    // optional fused ElemwiseMultiType step after the ConvBias (see conv_epilogue.cuh):
    // s_dst is then the scale of the ConvBias result, z_out_scale that of the final output
    const int8_t* z;
    int z_mode;  // 0 none, 1 QADD, 2 QFUSE_ADD_RELU
    float z_scale, z_out_scale;
    // tensor-core kernels only: store the int32 accumulators here instead of int8 results
    int32_t* acc_out;
    // halo-patch kernel only (reached through the space-to-depth path): 1 = the MAX pooling
    // 3x3 / stride 2 / pad 1 that follows the ConvBias is taken in its epilogue and dst is the
    // pooled tensor [n][(oh-1)/2+1][(ow-1)/2+1][oc]
    int pool;
    // halo-patch kernel only: `a` is the dense view of a depthwise 3x3 convolution over
    // a.oc channels taken 64 at a time (a.ic == 64, a.groups == 1): every CTA reads its own
    // 64 input channels and builds the block-diagonal filter tile from the raw [C][3][3] filter.
    // 2: 32 channels, a.iw / a.ow count pixel PAIRS (64-byte rows), a.oc == 64.
    int dw64;
    // general kernel only: divide by s_dst with the true division (scales outside the range
    // in which the three-instruction division by a constant is exact, see common.cuh)
    int true_division;
    // self-test of the bounded device waits (conv_umma only): when test_wait_cycles > 0 the
    // waits give up after that many clock cycles and the producer leaves out pipeline step
    // test_skip_step of every tile
    long long test_wait_cycles;
    int test_skip_step;
};

}  // namespace mb200
struct mb200_conv_param;
namespace mb200 {
// validates the public parameter block and fills the kernels' argument block (abi.cu)
int make_args(const mb200_conv_param* p, int src_is_nchw, ConvArgs* a);
int out_extent(int in, int k, int s, int p, int d);
size_t align_up(size_t v, size_t a);

// records a message for mb200_last_error() and returns `code`
int set_error(int code, const char* fmt, ...);
// cudaGetLastError() after a launch -> status
int check_launch(const char* what);
// the int that kernels launched on `st` set when a bounded wait runs out (one per device
// and stream, see abi.cu)
int* device_status_word(cudaStream_t st);

int launch_pack_filter(const ConvArgs& a, const int8_t* src, int8_t* dst, cudaStream_t st);
int launch_filter_nchw44_to_oihw(
        const ConvArgs& a, int form, const int8_t* src, int8_t* dst, cudaStream_t st);
int launch_transpose_f32(
        const float* src, float* dst, int batch, int rows, int cols, cudaStream_t st);
int launch_conv_direct(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, int32_t* acc, cudaStream_t st);
// depthwise 3x3 over NHWC with channels % 16 == 0 (conv_dw.cu)
bool conv_dw_supported(const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst);
int launch_conv_dw(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);
// requant_verify.cu: the shortest form clamp_s8(trunc(fma(f, mul, +-add))), f = (float)acc
// [* s_src [* s_flt]], that equals the reference's three-step requantisation for EVERY int32
// acc (checked on both sides of every step of the reference's staircase). Returns the number
// of float operations (1..3), or 0 and zeros when none passed
int requant_fast_constants(
        float s_src, float s_flt, float s_dst, int act, float* mul_out, float* add_out);
// the same idea for the fused residual step (mode 1 QADD, 2 QFUSE_ADD_RELU): a and b with
// trunc(fma(z, b, conv * a) +- 0.49999997) equal to the reference's five float operations on
// all 65536 (conv, z) pairs; false (and zeros) when no candidate passes
bool residual_fast_constants(
        float s_conv, float s_z, float out_scale, int mode, float* a_out, float* b_out);

// Images the activation's tensor map describes. TMA maps are only built over at least
// 128 KiB (smaller tensors need a descriptor fix-up on current drivers that this library does
// not apply). A smaller activation is described with more images than it has, as many as
// reach 128 KiB, when the bytes behind it are known to be readable (a registered range,
// mb200_register_readable_range): the kernels never use what they load from there. 0 = the
// tensor is too small and nothing is known about the memory behind it.
int descriptor_images(const ConvArgs& a, const int8_t* src);
bool readable_through(const void* p, size_t bytes);

// tensor-core implicit GEMM; conv_umma_supported() says whether the shape qualifies
bool conv_umma_supported(const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst);
// the same implicit GEMM on a pair of SMs (cta_group::2), 256 x 256 tiles: wide layers
bool conv_pair_supported(const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst);
int launch_conv_pair(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);
int launch_conv_umma(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);
// stride-1 tensor-core ConvBias with halo-patch tiles and a resident filter (conv_patch.cu)
bool conv_patch_supported(const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst);
// Depthwise 3x3 / stride 1 over a multiple of 64 channels (or 32 channels as pixel pairs) on
// the tensor cores: the halo-patch kernel with a block-diagonal filter built on chip. `a` is the depthwise convolution itself
// (groups == ic == oc), `flt` its packed filter [C][3][3]. `whatever_the_size`: leave out the
// two checks that only say whether it pays (enough patches per CTA, few partial patches).
bool conv_patch_dw_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst,
        bool whatever_the_size = false);
int launch_conv_patch_dw(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);
float conv_patch_efficiency(const ConvArgs& a);
int launch_conv_patch(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);
// stride-2 ConvBias with <= 4 input channels via 2x2 space-to-depth (conv_s2d.cu)
bool conv_s2d_supported(const ConvArgs& a);
size_t conv_s2d_filter_bytes(const ConvArgs& a);
size_t conv_s2d_workspace_bytes(const ConvArgs& a);
int launch_conv_s2d_pack_filter(
        const ConvArgs& a, const int8_t* flt_oihw, int8_t* out, cudaStream_t st);
int launch_conv_s2d(
        const ConvArgs& a, const int8_t* src, const int8_t* flt_s2d, const int32_t* bias,
        const float* flt_scales, int8_t* dst, void* workspace, cudaStream_t st);
// may a.pool be set for this ConvBias (first-layer form on the halo-patch kernel)?
bool conv_s2d_pool_supported(const ConvArgs& a);
int launch_pooling(
        const int8_t* src, int8_t* dst, int mode, int n, int c, int ih, int iw, int wh, int ww,
        int sh, int sw, int ph, int pw, cudaStream_t st);
int launch_qelemwise(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, float s0,
        float s1, float s_dst, cudaStream_t st);
int launch_qelemwise_bcast(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, unsigned channels,
        unsigned inner, float s0, float s1, float s_dst, cudaStream_t st);
int launch_typecvt_f32_qs8(
        const float* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst, cudaStream_t st);
int launch_typecvt_qs8_f32(
        const int8_t* src, float* dst, size_t nr_elem, float s_src, float s_dst, cudaStream_t st);
int launch_typecvt_qs32_qs8(
        const int32_t* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst,
        cudaStream_t st);
int launch_transpose_s8(
        const int8_t* src, int8_t* dst, int batch, int rows, int cols, cudaStream_t st);

}  // namespace mb200
