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
    // Optional fused quantised elementwise step (the residual add of a ResNet block): the
    // ConvBias result, requantised to int8 at scale s_dst exactly as the stand-alone kernel
    // would store it, is combined with the int8 tensor z (same NHWC shape as the output) by
    // the ElemwiseMultiType formula (compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp
    // :38-46,158): fp32_to_int8((s_dst*conv + z_scale*z [max 0]) * z_div), z_div = 1.f/out_scale.
    const int8_t* z;
    int z_mode;  // 0 none, 1 QADD, 2 QFUSE_ADD_RELU
    float z_scale, z_div;
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

// conv (already int8, as int) combined with one z value
template <int ZMODE>
__device__ __forceinline__ int fuse_z(int conv_q, int zv, const EpilogueParams& e) {
    if (ZMODE == 0)
        return conv_q;
    float t = __fadd_rn(__fmul_rn(e.s_dst, __int2float_rn(conv_q)),
                        __fmul_rn(e.z_scale, __int2float_rn(zv)));
    if (ZMODE == 2)
        t = t > 0.f ? t : 0.f;
    // |t * z_div| is bounded by the two int8 operands: far from the int range
    const float x = __fmul_rn(t, e.z_div);
    const float y = __fadd_rn(x, copysignf(0.49999997f, x));
    int q;
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    return q;
}

template <int ACT, bool PER_CHANNEL, bool BOUNDED, int ZMODE>
__device__ __forceinline__ void epilogue_store32_t(
        const uint32_t (&v)[32], const EpilogueParams& e, int8_t* out, const int8_t* zin,
        int ch0) {
    if (ch0 + 32 <= e.oc && (e.oc % 16) == 0) {
        uint32_t packed[8];
        uint32_t zw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (ZMODE != 0) {
            const uint4 z0 = __ldg(reinterpret_cast<const uint4*>(zin));
            const uint4 z1 = __ldg(reinterpret_cast<const uint4*>(zin) + 1);
            zw[0] = z0.x; zw[1] = z0.y; zw[2] = z0.z; zw[3] = z0.w;
            zw[4] = z1.x; zw[5] = z1.y; zw[6] = z1.z; zw[7] = z1.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int4 b = make_int4(0, 0, 0, 0);
            if (e.bias)
                b = __ldg(reinterpret_cast<const int4*>(e.bias + ch0) + j);
            float4 s = make_float4(e.s_flt, e.s_flt, e.s_flt, e.s_flt);
            if (PER_CHANNEL)
                s = __ldg(reinterpret_cast<const float4*>(e.flt_scales + ch0) + j);
            int r0 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 0] + b.x, e.s_src, s.x, e.s_dst,
                                               e.inv_dst);
            int r1 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 1] + b.y, e.s_src, s.y, e.s_dst,
                                               e.inv_dst);
            int r2 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 2] + b.z, e.s_src, s.z, e.s_dst,
                                               e.inv_dst);
            int r3 = requant_one<ACT, BOUNDED>((int)v[j * 4 + 3] + b.w, e.s_src, s.w, e.s_dst,
                                               e.inv_dst);
            if (ZMODE != 0) {
                r0 = fuse_z<ZMODE>(r0, (int)(int8_t)(zw[j]), e);
                r1 = fuse_z<ZMODE>(r1, (int)(int8_t)(zw[j] >> 8), e);
                r2 = fuse_z<ZMODE>(r2, (int)(int8_t)(zw[j] >> 16), e);
                r3 = fuse_z<ZMODE>(r3, (int)(int8_t)(zw[j] >> 24), e);
            }
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
                int r = requant_one<ACT, false>(acc, e.s_src, s, e.s_dst, e.inv_dst);
                if (ZMODE != 0)
                    r = fuse_z<ZMODE>(r, (int)zin[i], e);
                out[i] = (int8_t)r;
            }
        }
    }
}

// run-time dispatch on (activation, per-channel scales, bounded, fused step); uniform across
// the CTA. `off` is the element offset of the pixel's first channel of this chunk in the
// output tensor (and in z, which has the same shape).
__device__ __forceinline__ void epilogue_store32(
        const uint32_t (&v)[32], const EpilogueParams& e, int8_t* dst, size_t off, int ch0) {
    int8_t* out = dst + off;
    const bool pc = e.flt_scales != nullptr;
    if (e.z_mode != 0) {
        // the fused form follows a ConvBias without activation
        const int8_t* zin = e.z + off;
        if (e.z_mode == 1) {
            if (pc)
                epilogue_store32_t<ACT_IDENTITY, true, false, 1>(v, e, out, zin, ch0);
            else if (e.bounded)
                epilogue_store32_t<ACT_IDENTITY, false, true, 1>(v, e, out, zin, ch0);
            else
                epilogue_store32_t<ACT_IDENTITY, false, false, 1>(v, e, out, zin, ch0);
        } else {
            if (pc)
                epilogue_store32_t<ACT_IDENTITY, true, false, 2>(v, e, out, zin, ch0);
            else if (e.bounded)
                epilogue_store32_t<ACT_IDENTITY, false, true, 2>(v, e, out, zin, ch0);
            else
                epilogue_store32_t<ACT_IDENTITY, false, false, 2>(v, e, out, zin, ch0);
        }
        return;
    }
    if (e.bounded && !pc) {
        switch (e.act) {
            case ACT_IDENTITY:
                epilogue_store32_t<ACT_IDENTITY, false, true, 0>(v, e, out, nullptr, ch0);
                break;
            case ACT_RELU:
                epilogue_store32_t<ACT_RELU, false, true, 0>(v, e, out, nullptr, ch0);
                break;
            default:
                epilogue_store32_t<ACT_H_SWISH, false, true, 0>(v, e, out, nullptr, ch0);
                break;
        }
        return;
    }
    switch (e.act * 2 + (pc ? 1 : 0)) {
        case 0: epilogue_store32_t<ACT_IDENTITY, false, false, 0>(v, e, out, nullptr, ch0); break;
        case 1: epilogue_store32_t<ACT_IDENTITY, true, false, 0>(v, e, out, nullptr, ch0); break;
        case 2: epilogue_store32_t<ACT_RELU, false, false, 0>(v, e, out, nullptr, ch0); break;
        case 3: epilogue_store32_t<ACT_RELU, true, false, 0>(v, e, out, nullptr, ch0); break;
        case 4: epilogue_store32_t<ACT_H_SWISH, false, false, 0>(v, e, out, nullptr, ch0); break;
        default: epilogue_store32_t<ACT_H_SWISH, true, false, 0>(v, e, out, nullptr, ch0); break;
    }
}

}  // namespace mb200
