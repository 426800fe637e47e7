// Shared device helpers: the bit-exact requantisation epilogue and small utilities.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

enum Act : int { ACT_IDENTITY = 0, ACT_RELU = 1, ACT_H_SWISH = 2 };

// float -> int8 exactly as the reference's generated C does it on x86:
// `int res = roundf(src); clamp to [-128,127]`
// (compiler/lib/KernelGen/BareMetal/Activation.cpp:50-56). roundf is round-half-away.
// A float beyond the int range converts to INT_MIN on x86 (cvttss2si), which the clamp
// then turns into -128; __float2int_rz would saturate instead, so that case is spelled out.
__device__ __forceinline__ int f32_to_i32_x86(float r) {
    return (fabsf(r) < 2147483648.f) ? __float2int_rz(r) : (int)0x80000000;
}

__device__ __forceinline__ int fp32_to_int8(float x) {
    int res = f32_to_i32_x86(roundf(x));
    res = res > 127 ? 127 : res;
    res = res < -128 ? -128 : res;
    return res;
}

// Activation bodies of compiler/lib/KernelGen/BareMetal/Activation.cpp:9-30, each
// float operation individually rounded (no FMA contraction).
__device__ __forceinline__ float apply_act(int act, float x) {
    if (act == ACT_RELU) {
        return x > 0.f ? x : 0.f;
    }
    if (act == ACT_H_SWISH) {
        float t = __fadd_rn(x, 3.f);
        t = t > 0.f ? t : 0.f;
        t = t > 6.f ? 6.f : t;
        return __fmul_rn(__fmul_rn(x, t), 1.f / 6.f);
    }
    return x;
}

// ConvBias requantisation: the reference composes "dval*scale*flt_scale/dst_scale",
// evaluated left to right in float with a true division, then the activation, then the
// int8 conversion (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113).
__device__ __forceinline__ int requant_conv(
        int acc, float s_src, float s_flt, float s_dst, int act) {
    float x = __fdiv_rn(__fmul_rn(__fmul_rn(__int2float_rn(acc), s_src), s_flt), s_dst);
    return fp32_to_int8(apply_act(act, x));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

}  // namespace mb200
