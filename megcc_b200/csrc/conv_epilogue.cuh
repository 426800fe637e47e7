// The ConvBias epilogue shared by the tensor-core kernels: 32 int32 accumulators of one
// output pixel -> + bias -> requantisation in the reference's operation order
// (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113) -> activation -> int8 -> store.
#pragma once
#include "common.cuh"
#include "umma_ptx.cuh"

namespace mb200 {

struct EpilogueParams {
    int oc;
    int act;
    // 1 when the host has shown that |x| stays far below 2^31 for every possible int32
    // accumulator, so that the x86 "out of range converts to INT_MIN" case cannot occur and
    // one saturating conversion does round-to-int and clamp together
    int bounded;
    float s_src, s_flt, s_dst, inv_dst;
    const int32_t* bias;
    const float* flt_scales;
};

// host: is |(float)acc * s_src * s_flt / s_dst| < 2^30 for every int32 acc?
inline bool requant_is_bounded(float s_src, float s_flt, float s_dst) {
    const double m = 2147483648.0 * (double)fabsf(s_src) * (double)fabsf(s_flt) / (double)fabsf(s_dst);
    return m == m && m < 1073741824.0;
}

template <int ACT, bool BOUNDED>
__device__ __forceinline__ int requant_one(
        int acc, float s_src, float s_flt, float s_dst, float inv_dst) {
    const float t = __fmul_rn(__fmul_rn(__int2float_rn(acc), s_src), s_flt);
    float x = div_rn_by_const(t, s_dst, inv_dst);
    if (!BOUNDED)
        return round_clamp_s8(apply_act(ACT, x));
    int q;
    if (ACT == ACT_RELU) {
        // x >= 0 after the max: no sign to carry into the rounding offset
        const float y = __fadd_rn(fmaxf(x, 0.f), 0.49999997f);
        asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    } else {
        x = apply_act(ACT, x);
        const float y = __fadd_rn(x, copysignf(0.49999997f, x));
        asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    }
    return q;
}

template <int ACT, bool PER_CHANNEL, bool BOUNDED>
__device__ __forceinline__ void epilogue_store32_t(
        const uint32_t (&v)[32], const EpilogueParams& e, int8_t* out, int ch0) {
    if (ch0 + 32 <= e.oc && (e.oc % 16) == 0) {
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int4 b = make_int4(0, 0, 0, 0);
            if (e.bias)
                b = __ldg(reinterpret_cast<const int4*>(e.bias + ch0) + j);
            float4 s = make_float4(e.s_flt, e.s_flt, e.s_flt, e.s_flt);
            if (PER_CHANNEL)
                s = __ldg(reinterpret_cast<const float4*>(e.flt_scales + ch0) + j);
            const int r0 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 0] + b.x, e.s_src, s.x, e.s_dst,
                                                     e.inv_dst);
            const int r1 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 1] + b.y, e.s_src, s.y, e.s_dst,
                                                     e.inv_dst);
            const int r2 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 2] + b.z, e.s_src, s.z, e.s_dst,
                                                     e.inv_dst);
            const int r3 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 3] + b.w, e.s_src, s.w, e.s_dst,
                                                     e.inv_dst);
            packed[j] = umma::pack4_prmt(r0, r1, r2, r3);
        }
        reinterpret_cast<uint4*>(out)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        reinterpret_cast<uint4*>(out)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
        // ragged channel tail, or a channel count that rules out vector stores (fully
        // unrolled with a predicate so the accumulators stay in registers)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (ch0 + i < e.oc) {
                const int acc = (int)v[i] + (e.bias ? e.bias[ch0 + i] : 0);
                const float s = PER_CHANNEL ? e.flt_scales[ch0 + i] : e.s_flt;
                out[i] = (int8_t)requant_one<ACT, false>(acc, e.s_src, s, e.s_dst, e.inv_dst);
            }
        }
    }
}

// run-time dispatch on (activation, per-channel scales, bounded); uniform across the CTA
__device__ __forceinline__ void epilogue_store32(
        const uint32_t (&v)[32], const EpilogueParams& e, int8_t* out, int ch0) {
    const bool pc = e.flt_scales != nullptr;
    if (e.bounded && !pc) {
        switch (e.act) {
            case ACT_IDENTITY: epilogue_store32_t<ACT_IDENTITY, false, true>(v, e, out, ch0); break;
            case ACT_RELU: epilogue_store32_t<ACT_RELU, false, true>(v, e, out, ch0); break;
            default: epilogue_store32_t<ACT_H_SWISH, false, true>(v, e, out, ch0); break;
        }
        return;
    }
    switch (e.act * 2 + (pc ? 1 : 0)) {
        case 0: epilogue_store32_t<ACT_IDENTITY, false, false>(v, e, out, ch0); break;
        case 1: epilogue_store32_t<ACT_IDENTITY, true, false>(v, e, out, ch0); break;
        case 2: epilogue_store32_t<ACT_RELU, false, false>(v, e, out, ch0); break;
        case 3: epilogue_store32_t<ACT_RELU, true, false>(v, e, out, ch0); break;
        case 4: epilogue_store32_t<ACT_H_SWISH, false, false>(v, e, out, ch0); break;
        default: epilogue_store32_t<ACT_H_SWISH, true, false>(v, e, out, ch0); break;
    }
}

}  // namespace mb200
