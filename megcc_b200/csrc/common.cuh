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

// ---- the same arithmetic in fewer instructions, still bit-exact ----
//
// Division: with r = RN(1/d) (computed on the host), q0 = RN(t*r), rem = t - q0*d (exact in
// one FMA) and q = RN(q0 + rem*r) equals RN(t/d) as long as no intermediate leaves the normal
// range. tests/requant_math_check.c checks it on the host for every mantissa of t, a list of
// divisors that includes the range ends below, and around every int8 step of the accumulator
// chain. Three instructions instead of the general division routine.
//
// Precondition (division_range_ok): no intermediate may leave the normal range. With t the
// product acc * s_src * s_flt of a non-zero int32 accumulator: 2^-100 <= |s_src * s_flt| <=
// 2^69 keeps t and rem = t * 2^-24 normal, 2^-100 <= |s_dst| <= 2^100 keeps d and 1 / d normal,
// and 2^-60 <= |s_src * s_flt / s_dst| <= 2^60 keeps the quotient normal. (Activation scales
// of a deep network with large accumulators legitimately reach 1e20 and beyond.) The launchers
// check it for per-tensor scales and send anything else to the general kernel with the true
// division; one scale per output channel must satisfy it by contract.
__host__ __device__ inline bool division_range_ok(float s_src, float s_flt, float s_dst) {
    const float prod = fabsf(s_src * s_flt), d = fabsf(s_dst);
    if (!(prod >= 0x1p-100f && prod <= 0x1p69f && d >= 0x1p-100f && d <= 0x1p100f))
        return false;
    const float ratio = prod / d;
    return ratio >= 0x1p-60f && ratio <= 0x1p60f;
}
__device__ __forceinline__ float div_rn_by_const(float t, float d, float r) {
    const float q0 = __fmul_rn(t, r);
    const float rem = __fmaf_rn(-q0, d, t);
    return __fmaf_rn(rem, r, q0);
}

// roundf (half away from zero) followed by the x86 float->int conversion and the int8
// clamp. trunc(x + copysign(0.49999997f, x)) == roundf(x) for every float below 2^31 in
// magnitude (0.49999997f is the largest float below one half); larger magnitudes convert
// to INT_MIN on x86 and therefore clamp to -128.
__device__ __forceinline__ int round_clamp_s8(float x) {
    const float y = __fadd_rn(x, copysignf(0.49999997f, x));
    int q = __float2int_rz(y);
    q = min(max(q, -128), 127);
    return (fabsf(x) < 2147483648.f) ? q : -128;
}

__device__ __forceinline__ int requant_conv_fast(
        int acc, float s_src, float s_flt, float s_dst, float inv_dst, int act) {
    const float t = __fmul_rn(__fmul_rn(__int2float_rn(acc), s_src), s_flt);
    return round_clamp_s8(apply_act(act, div_rn_by_const(t, s_dst, inv_dst)));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

}  // namespace mb200
