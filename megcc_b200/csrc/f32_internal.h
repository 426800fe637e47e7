// Internal declarations of the fp32 path (conv_f32.cu, f32_ops.cu, f32_abi.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include "../../include/megcc_b200.h"
#include "internal.h"

namespace mb200 {

// Everything an fp32 conv kernel needs, by value. Pitches are in floats.
struct ConvF32Args {
    int n, ic, ih, iw, oc, oh, ow;
    int kh, kw, sh, sw, ph, pw, groups;
    int m;    // n * oh * ow
    int act;  // MB200_F32_*
    long long src_pitch;  // floats between consecutive pixels of src (>= ic)
    long long dst_pitch;  // ... of dst (>= oc): lets a conv write its slice of a concat buffer
    long long z_pitch;    // ... of the optional residual operand
};

int conv_f32_padded_ic(int ic);
size_t conv_f32_split_filter_floats(const ConvF32Args& a);
bool conv_f32_umma_supported(const ConvF32Args& a, const float* src, const float* dst);
size_t conv_f32_workspace_bytes(const ConvF32Args& a);
int launch_conv_f32_pack_filter_split(
        const ConvF32Args& a, const float* flt_oihw, float* out, cudaStream_t st);
int launch_conv_f32_pack_filter_plain(
        const ConvF32Args& a, const float* flt_oihw, float* out, cudaStream_t st);
int launch_conv_f32_direct(
        const ConvF32Args& a, const float* src, const float* flt_plain, const float* bias,
        const float* z, float* dst, cudaStream_t st);
int launch_conv_f32_umma(
        const ConvF32Args& a, const float* src, const float* flt_split, const float* bias,
        const float* z, float* dst, void* workspace, cudaStream_t st);

int launch_elemwise_f32(
        int mode, const float* a, const float* b, float* dst, size_t nr_elem, cudaStream_t st);
int launch_concat_f32(
        const float* const* srcs, const int* channels, int nr, float* dst, size_t pixels,
        cudaStream_t st);
int launch_resize_nearest_f32(
        const float* src, float* dst, int n, int c, int ih, int iw, int oh, int ow,
        cudaStream_t st);
int launch_pooling_f32(
        const float* src, float* dst, int mode, int n, int c, int ih, int iw, int wh, int ww,
        int sh, int sw, int ph, int pw, cudaStream_t st);
int launch_focus_f32(
        const float* src_nchw, float* dst_nhwc, int n, int c, int h, int w, int c_out,
        cudaStream_t st);
int launch_transpose_f32(
        const float* src, float* dst, int batch, int rows, int cols, cudaStream_t st);

}  // namespace mb200
