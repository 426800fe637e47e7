// The ConvBias epilogue shared by the tensor-core kernels: 32 int32 accumulators of one
// output pixel -> + bias -> requantisation in the reference's operation order
// (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113) -> activation -> int8 -> store.
#pragma once
#include "common.cuh"
#include "umma_ptx.cuh"

namespace mb200 {

// what an absent bias reads: the vector path then loads unconditionally instead of testing the
// pointer and clearing four registers for each group of four channels
__device__ __align__(32) const int32_t kZeroBias[32] = {};

struct EpilogueParams {
    int oc;
    int act;
    // 1 when the host has shown that |x| stays far below 2^31 for every possible int32
    // accumulator, so that the x86 "out of range converts to INT_MIN" case cannot occur and
    // one saturating conversion does round-to-int and clamp together
    int bounded;
    float s_src, s_flt, s_dst, inv_dst;
    // non-zero: multiplier and rounding offset of the one-FMA form that the host has checked
    // against the three-step chain on every step of its staircase (requant_verify.cu);
    // per-tensor scales, IDENTITY / RELU only
    float fast_mul, fast_add;
    int fast_ops;  // 0: none; 1..3: float operations of the verified form (see requant_pair_fast)
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
    // non-zero: the fused step in its verified short form (requant_verify.cu): a and b with
    // fma(z, b, conv * a) rounded as below equal to the reference's five float operations
    // on all 65536 (conv, z) pairs
    float z_fast_a, z_fast_b;
    // when set, the int32 accumulators (+ bias) are stored here instead of the int8 result
    // (same [pixel][channel] indexing); used by the int8 -> int32 matrix product
    int32_t* acc_out;
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

// ---- two floats per instruction (sm_100 f32x2 forms; each half is the IEEE RN operation) ----
// CAUTION: unlike the scalar intrinsics, a packed multiply whose result feeds a packed add IS
// contracted into a fused multiply-add by the assembler (explicit .rn and -fmad=false
// notwithstanding). Sequences here are multiply -> multiply, multiply -> fma, fma -> add,
// none of which can be contracted; where a product must be rounded before it is added, the
// scalar intrinsics are used.
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// the constants of one requantisation, each duplicated into both halves
struct RequantPair {
    uint64_t s_src, s_flt, neg_dst, inv_dst, half;
    __device__ __forceinline__ explicit RequantPair(const EpilogueParams& e)
            : s_src(f2_pack(e.s_src, e.s_src)),
              s_flt(f2_pack(e.s_flt, e.s_flt)),
              neg_dst(f2_pack(-e.s_dst, -e.s_dst)),
              inv_dst(f2_pack(e.inv_dst, e.inv_dst)),
              half(f2_pack(0.49999997f, 0.49999997f)) {}
};

// Bounded, per-tensor requantisation of two accumulators: the float operations of
// requant_one<ACT, true> on both halves at once. With RELU the max is NOT applied here: the
// caller clears negative bytes after packing (a value below zero rounds to something <= 0
// either way, and max(., 0) commutes with the monotonic round-and-saturate).
template <int ACT>
__device__ __forceinline__ void requant_pair(
        int acc0, int acc1, const RequantPair& c, int& q0, int& q1) {
    const uint64_t f = f2_pack(__int2float_rn(acc0), __int2float_rn(acc1));
    const uint64_t t = f2_mul(f2_mul(f, c.s_src), c.s_flt);
    // t / s_dst correctly rounded (div_rn_by_const); fma(-q, d, t) == fma(q, -d, t)
    const uint64_t qa = f2_mul(t, c.inv_dst);
    const uint64_t rem = f2_fma(qa, c.neg_dst, t);
    const uint64_t x = f2_fma(rem, c.inv_dst, qa);
    uint64_t y;
    if (ACT == ACT_RELU) {
        y = f2_add(x, c.half);
    } else {
        float x0, x1;
        f2_unpack(x, x0, x1);
        y = f2_add(x, f2_pack(copysignf(0.49999997f, x0), copysignf(0.49999997f, x1)));
    }
    float y0, y1;
    f2_unpack(y, y0, y1);
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(y0));
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(y1));
}

// The verified form (EpilogueParams::fast_mul / fast_add) on two accumulators: ONE fused
// multiply-add, trunc(fma((float)acc, c, +-d)), saturated. It is written as an explicit fma because
// the assembler contracts a packed multiply followed by a packed add into one anyway (seen on
// a tie: 15000 * 1e-4f + 0.49999997f is 2.0 in two steps and 1.9999999 fused), and the host's
// value-by-value check (requant_verify.cu) evaluates exactly this fused form.
template <int ACT, int OPS>
__device__ __forceinline__ void requant_pair_fast(
        int acc0, int acc1, const EpilogueParams& e, int& q0, int& q1) {
    // scalar operations: the packed form would need the two converted values moved into a
    // register pair and the results moved out again, which costs what it saves. OPS - 1
    // leading multiplications of the reference chain are kept, the rest is one fma.
    float f0 = __int2float_rn(acc0), f1 = __int2float_rn(acc1);
    if (OPS >= 2) {
        f0 = __fmul_rn(f0, e.s_src);
        f1 = __fmul_rn(f1, e.s_src);
    }
    if (OPS >= 3) {
        f0 = __fmul_rn(f0, e.s_flt);
        f1 = __fmul_rn(f1, e.s_flt);
    }
    const float y0 = __fmaf_rn(f0, e.fast_mul, ACT == ACT_RELU ? e.fast_add : copysignf(e.fast_add, f0));
    const float y1 = __fmaf_rn(f1, e.fast_mul, ACT == ACT_RELU ? e.fast_add : copysignf(e.fast_add, f1));
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(y0));
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(y1));
}

// four packed int8: bytes below zero become zero (byte-wise sign masks from PRMT)
__device__ __forceinline__ uint32_t relu_s8x4(uint32_t p) {
    // selector nibbles 8..B: bytes 0..3 with bit 3 set, which replicates the byte's sign bit
    // (the __byte_perm intrinsic masks that bit off, hence the instruction itself)
    uint32_t neg;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(neg) : "r"(p), "r"(0u), "r"(0xBA98u));
    return p & ~neg;
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

// NV = 16 or 32 accumulators (consecutive channels from ch0) of one output pixel
// The verified short form of fuse_z (EpilogueParams::z_fast_a / z_fast_b). QFUSE_ADD_RELU:
// trunc(fma(z, b, fma(conv, a, 0.49999997))) with negatives cleared afterwards; QADD: the
// rounding offset takes the sign of the sum, so it is added last. Scalar intrinsics: none
// of these may be contracted or reordered.
template <int ZMODE>
__device__ __forceinline__ int fuse_z_fast(int conv_q, int zv, float a, float b) {
    const float qf = __int2float_rn(conv_q), zf = __int2float_rn(zv);
    float y;
    if (ZMODE == 2) {
        y = __fmaf_rn(zf, b, __fmaf_rn(qf, a, 0.49999997f));
    } else {
        const float v = __fmaf_rn(zf, b, __fmul_rn(qf, a));
        y = __fadd_rn(v, copysignf(0.49999997f, v));
    }
    int q;
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    return q;
}

template <int NV, int ACT, bool PER_CHANNEL, bool BOUNDED, int ZMODE, int FAST = 0,
          bool ZFAST = false>
__device__ __forceinline__ void epilogue_store_t(
        const uint32_t (&v)[NV], const EpilogueParams& e, int8_t* out, const int8_t* zin,
        int ch0) {
    static_assert(NV == 16 || NV == 32, "16 or 32 channels per call");
    // a pixel's channels start at a multiple of oc bytes: 16-byte vectors when oc allows,
    // 8-byte ones for oc % 8 == 0 (a 1000-class classifier), bytes otherwise
    if (ch0 + NV <= e.oc && (e.oc % 8) == 0) {
        const bool wide = (e.oc % 16) == 0;
        uint32_t packed[NV / 4];
        uint32_t zw[NV / 4];
#pragma unroll
        for (int j = 0; j < NV / 4; ++j)
            zw[j] = 0;
        if (ZMODE != 0) {
            if (NV == 32 && (e.oc % 32) == 0 && ((uintptr_t)zin & 31) == 0) {
                // one 256-bit load of the sector that the store below will mirror
                asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(zw[0]), "=r"(zw[1]), "=r"(zw[2]), "=r"(zw[3]),
                               "=r"(zw[NV / 4 - 4]), "=r"(zw[NV / 4 - 3]), "=r"(zw[NV / 4 - 2]),
                               "=r"(zw[NV / 4 - 1])
                             : "l"(zin));
            } else if (wide) {
#pragma unroll
                for (int h = 0; h < NV / 16; ++h) {
                    const uint4 z0 = __ldg(reinterpret_cast<const uint4*>(zin) + h);
                    zw[h * 4 + 0] = z0.x; zw[h * 4 + 1] = z0.y;
                    zw[h * 4 + 2] = z0.z; zw[h * 4 + 3] = z0.w;
                }
            } else {
#pragma unroll
                for (int h = 0; h < NV / 8; ++h) {
                    const uint2 z0 = __ldg(reinterpret_cast<const uint2*>(zin) + h);
                    zw[h * 2 + 0] = z0.x; zw[h * 2 + 1] = z0.y;
                }
            }
        }
        constexpr bool kPaired = BOUNDED && !PER_CHANNEL && ACT != ACT_H_SWISH;
        static_assert(FAST == 0 || kPaired, "the verified form exists for the paired path only");
        static_assert(ZMODE == 0 || ACT == ACT_IDENTITY, "the fused step follows a plain ConvBias");
        const RequantPair rp(e);
        const int4* bias4 = reinterpret_cast<const int4*>(e.bias ? e.bias + ch0 : kZeroBias);
#pragma unroll
        for (int j = 0; j < NV / 4; ++j) {
            const int4 b = __ldg(bias4 + j);
            if (kPaired) {
                int r0, r1, r2, r3;
                if (FAST != 0) {
                    requant_pair_fast<ACT, FAST>((int)v[j * 4 + 0] + b.x, (int)v[j * 4 + 1] + b.y, e,
                                                 r0, r1);
                    requant_pair_fast<ACT, FAST>((int)v[j * 4 + 2] + b.z, (int)v[j * 4 + 3] + b.w, e,
                                                 r2, r3);
                } else {
                    requant_pair<ACT>((int)v[j * 4 + 0] + b.x, (int)v[j * 4 + 1] + b.y, rp, r0, r1);
                    requant_pair<ACT>((int)v[j * 4 + 2] + b.z, (int)v[j * 4 + 3] + b.w, rp, r2, r3);
                }
                if (ZMODE != 0 && ZFAST) {
                    r0 = fuse_z_fast<ZMODE>(r0, (int)(int8_t)(zw[j]), e.z_fast_a, e.z_fast_b);
                    r1 = fuse_z_fast<ZMODE>(r1, (int)(int8_t)(zw[j] >> 8), e.z_fast_a, e.z_fast_b);
                    r2 = fuse_z_fast<ZMODE>(r2, (int)(int8_t)(zw[j] >> 16), e.z_fast_a, e.z_fast_b);
                    r3 = fuse_z_fast<ZMODE>(r3, (int)(int8_t)(zw[j] >> 24), e.z_fast_a, e.z_fast_b);
                } else if (ZMODE != 0) {
                    // scalar operations with explicit rounding: a packed multiply feeding a
                    // packed add would be contracted, and this sum must not be
                    r0 = fuse_z<ZMODE>(r0, (int)(int8_t)(zw[j]), e);
                    r1 = fuse_z<ZMODE>(r1, (int)(int8_t)(zw[j] >> 8), e);
                    r2 = fuse_z<ZMODE>(r2, (int)(int8_t)(zw[j] >> 16), e);
                    r3 = fuse_z<ZMODE>(r3, (int)(int8_t)(zw[j] >> 24), e);
                }
                const uint32_t pk = umma::pack4_prmt(r0, r1, r2, r3);
                // RELU of the conv, or of the fused sum in its short form, on packed bytes
                packed[j] = ((ACT == ACT_RELU && ZMODE == 0) || (ZMODE == 2 && ZFAST))
                                    ? relu_s8x4(pk)
                                    : pk;
                continue;
            }
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
        if (NV == 32 && (e.oc % 32) == 0 && ((uintptr_t)out & 31) == 0) {
            // the chunk's 32 bytes are one whole, aligned sector: one 256-bit store (two
            // 16-byte stores would each touch half a sector of 32 different lines per warp)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out),
                         "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]),
                         "r"(packed[NV / 4 - 4]), "r"(packed[NV / 4 - 3]), "r"(packed[NV / 4 - 2]),
                         "r"(packed[NV / 4 - 1])
                         : "memory");
        } else if (wide) {
#pragma unroll
            for (int h = 0; h < NV / 16; ++h)
                reinterpret_cast<uint4*>(out)[h] = make_uint4(
                        packed[h * 4 + 0], packed[h * 4 + 1], packed[h * 4 + 2], packed[h * 4 + 3]);
        } else {
#pragma unroll
            for (int h = 0; h < NV / 8; ++h)
                reinterpret_cast<uint2*>(out)[h] = make_uint2(packed[h * 2 + 0], packed[h * 2 + 1]);
        }
    } else {
        // ragged channel tail, or a channel count that rules out vector stores (fully
        // unrolled with a predicate so the accumulators stay in registers)
#pragma unroll
        for (int i = 0; i < NV; ++i) {
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

// Four consecutive channels (from ch0, a multiple of 4) of one output of a ConvBias without a
// fused elementwise step: accumulators + bias `b` -> four packed int8, by the same
// arithmetic and the same choice of form as epilogue_store() makes for whole chunks. `s` are
// the channels' filter scales when e.flt_scales is set (else ignored). IDENTITY / RELU only.
__device__ __forceinline__ uint32_t epilogue_word(
        const uint32_t (&v)[4], const int4 b, const float4 s, const EpilogueParams& e) {
    const int a0 = (int)v[0] + b.x, a1 = (int)v[1] + b.y, a2 = (int)v[2] + b.z,
              a3 = (int)v[3] + b.w;
    const bool relu = e.act == ACT_RELU;
    int r0, r1, r2, r3;
    if (e.fast_ops != 0) {
#define MB200_WORD_FAST(OPS)                                             \
    if (relu) {                                                          \
        requant_pair_fast<ACT_RELU, OPS>(a0, a1, e, r0, r1);             \
        requant_pair_fast<ACT_RELU, OPS>(a2, a3, e, r2, r3);             \
    } else {                                                             \
        requant_pair_fast<ACT_IDENTITY, OPS>(a0, a1, e, r0, r1);         \
        requant_pair_fast<ACT_IDENTITY, OPS>(a2, a3, e, r2, r3);         \
    }
        if (e.fast_ops == 1) {
            MB200_WORD_FAST(1)
        } else if (e.fast_ops == 2) {
            MB200_WORD_FAST(2)
        } else {
            MB200_WORD_FAST(3)
        }
#undef MB200_WORD_FAST
        const uint32_t pk = umma::pack4_prmt(r0, r1, r2, r3);
        return relu ? relu_s8x4(pk) : pk;
    }
    if (e.bounded && !e.flt_scales) {
        const RequantPair rp(e);
        if (relu) {
            requant_pair<ACT_RELU>(a0, a1, rp, r0, r1);
            requant_pair<ACT_RELU>(a2, a3, rp, r2, r3);
        } else {
            requant_pair<ACT_IDENTITY>(a0, a1, rp, r0, r1);
            requant_pair<ACT_IDENTITY>(a2, a3, rp, r2, r3);
        }
        const uint32_t pk = umma::pack4_prmt(r0, r1, r2, r3);
        return relu ? relu_s8x4(pk) : pk;
    }
    const float4 sc = e.flt_scales ? s : make_float4(e.s_flt, e.s_flt, e.s_flt, e.s_flt);
    if (relu) {
        r0 = requant_one<ACT_RELU, false>(a0, e.s_src, sc.x, e.s_dst, e.inv_dst);
        r1 = requant_one<ACT_RELU, false>(a1, e.s_src, sc.y, e.s_dst, e.inv_dst);
        r2 = requant_one<ACT_RELU, false>(a2, e.s_src, sc.z, e.s_dst, e.inv_dst);
        r3 = requant_one<ACT_RELU, false>(a3, e.s_src, sc.w, e.s_dst, e.inv_dst);
    } else {
        r0 = requant_one<ACT_IDENTITY, false>(a0, e.s_src, sc.x, e.s_dst, e.inv_dst);
        r1 = requant_one<ACT_IDENTITY, false>(a1, e.s_src, sc.y, e.s_dst, e.inv_dst);
        r2 = requant_one<ACT_IDENTITY, false>(a2, e.s_src, sc.z, e.s_dst, e.inv_dst);
        r3 = requant_one<ACT_IDENTITY, false>(a3, e.s_src, sc.w, e.s_dst, e.inv_dst);
    }
    return umma::pack4_prmt(r0, r1, r2, r3);
}

// run-time dispatch on (activation, per-channel scales, bounded, fused step); uniform across
// the CTA. `off` is the element offset of the pixel's first channel of this chunk in the
// output tensor (and in z, which has the same shape).
// ---- one 32-column chunk with its TMEM load split in two ----
// The epilogue warps are bound by the latency of their own chain (wait, tcgen05.ld,
// requantisation, store), so the chunk's accumulators are fetched as two 16-column loads and
// the second is in flight while the first half is requantised (halo-patch kernel, batch 256,
// same box: first layer 134 -> 117 us with its space-to-depth pass, 64 -> 64 layers 44 -> 40 us).
// Written for the two commonest epilogues only, each with everything fixed at compile time:
// RELU and QFUSE_ADD_RELU in the verified one-FMA form; everything else takes
// epilogue_store(). How this is compiled decides whether it pays: twelve instantiations (every
// verified form and activation) made the compiler spill the accumulators in the tile loop
// (first layer 142 us), one instantiation per fused-step mode with the operation count and
// the activation as run-time values was slower than no overlap at all (149 against 141 us),
// and as functions of their own (__noinline__) the variants crash ptxas 12.9.
//
// Can the chunk at channel ch0 take this path? (Uniform over the warp.)
__device__ __forceinline__ bool epilogue_chunk_overlappable(
        const EpilogueParams& e, const int8_t* dst, int ch0) {
    if (e.fast_ops != 1 || e.acc_out || e.flt_scales || (e.oc % 32) != 0 || ch0 + 32 > e.oc)
        return false;
    if (((uintptr_t)dst & 31) != 0)
        return false;
    // the two commonest epilogues only: RELU without a fused step, QFUSE_ADD_RELU
    if (!(e.z_mode == 0 && e.act == ACT_RELU) && e.z_mode != 2)
        return false;
    if (e.z_mode != 0 && (e.z_fast_a == 0.f || ((uintptr_t)e.z & 31) != 0))
        return false;
    return true;
}

// ZMODE 0: ConvBias with RELU; 2: QFUSE_ADD_RELU behind an IDENTITY ConvBias. `release_bar`
// (or null): the accumulator buffer's "drained" barrier, on which the thread arrives once all
// its accumulators are in registers. Every lane of the warp must call (the loads are
// warp-wide); `valid` guards the reads of z and the store.
template <int ZMODE>
__device__ __forceinline__ void epilogue_chunk_overlapped_t(
        uint32_t taddr, const EpilogueParams& e, int8_t* out, const int8_t* zin, int ch0,
        bool valid, uint64_t* release_bar) {
    uint32_t lo[16], hi[16], packed[8], zw[8];
    umma::tmem_ld16_nowait(taddr, lo);
    if (ZMODE != 0 && valid)
        asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(zw[0]), "=r"(zw[1]), "=r"(zw[2]), "=r"(zw[3]), "=r"(zw[4]),
                       "=r"(zw[5]), "=r"(zw[6]), "=r"(zw[7])
                     : "l"(zin));
    const int4* bias4 = reinterpret_cast<const int4*>(e.bias ? e.bias + ch0 : kZeroBias);
    constexpr bool relu = ZMODE == 0;
    umma::tmem_ld_wait16(lo);
    umma::tmem_ld16_nowait(taddr + 16u, hi);
    auto half = [&](const uint32_t (&v)[16], int base) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int4 b = __ldg(bias4 + base + j);
            int r0, r1, r2, r3;
            constexpr int kAct = ZMODE == 0 ? ACT_RELU : ACT_IDENTITY;
            requant_pair_fast<kAct, 1>((int)v[4 * j] + b.x, (int)v[4 * j + 1] + b.y, e, r0, r1);
            requant_pair_fast<kAct, 1>((int)v[4 * j + 2] + b.z, (int)v[4 * j + 3] + b.w, e, r2, r3);
            if (ZMODE != 0) {
                const uint32_t z = zw[base + j];
                r0 = fuse_z_fast<ZMODE>(r0, (int)(int8_t)(z), e.z_fast_a, e.z_fast_b);
                r1 = fuse_z_fast<ZMODE>(r1, (int)(int8_t)(z >> 8), e.z_fast_a, e.z_fast_b);
                r2 = fuse_z_fast<ZMODE>(r2, (int)(int8_t)(z >> 16), e.z_fast_a, e.z_fast_b);
                r3 = fuse_z_fast<ZMODE>(r3, (int)(int8_t)(z >> 24), e.z_fast_a, e.z_fast_b);
            }
            const uint32_t pk = umma::pack4_prmt(r0, r1, r2, r3);
            // RELU of the ConvBias, or of the fused sum, on packed bytes
            packed[base + j] = (relu || ZMODE == 2) ? relu_s8x4(pk) : pk;
        }
    };
    half(lo, 0);
    umma::tmem_ld_wait16(hi);
    if (release_bar) {
        // all of this thread's accumulators are in registers: hand the buffer back
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        umma::mbar_arrive(release_bar);
    }
    half(hi, 4);
    if (valid)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out),
                     "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]),
                     "r"(packed[4]), "r"(packed[5]), "r"(packed[6]), "r"(packed[7])
                     : "memory");
}

// `taddr`: the chunk's first TMEM column for this thread's lane; `off`: element offset of the
// pixel's channel ch0 in dst (and z). The caller has checked epilogue_chunk_overlappable().
__device__ __forceinline__ void epilogue_chunk_overlapped(
        uint32_t taddr, const EpilogueParams& e, int8_t* dst, size_t off, int ch0, bool valid,
        uint64_t* release_bar) {
    int8_t* out = dst + off;
    if (e.z_mode == 0)
        epilogue_chunk_overlapped_t<0>(taddr, e, out, nullptr, ch0, valid, release_bar);
    else
        epilogue_chunk_overlapped_t<2>(taddr, e, out, e.z + off, ch0, valid, release_bar);
}

template <int NV>
__device__ __forceinline__ void epilogue_store(
        const uint32_t (&v)[NV], const EpilogueParams& e, int8_t* dst, size_t off, int ch0) {
    if (e.acc_out) {
        int32_t* o = e.acc_out + off;
        if (ch0 + NV <= e.oc && (e.oc % 4) == 0) {
#pragma unroll
            for (int j = 0; j < NV / 4; ++j) {
                int4 b = make_int4(0, 0, 0, 0);
                if (e.bias)
                    b = __ldg(reinterpret_cast<const int4*>(e.bias + ch0) + j);
                reinterpret_cast<int4*>(o)[j] =
                        make_int4((int)v[j * 4 + 0] + b.x, (int)v[j * 4 + 1] + b.y,
                                  (int)v[j * 4 + 2] + b.z, (int)v[j * 4 + 3] + b.w);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (ch0 + i < e.oc)
                    o[i] = (int)v[i] + (e.bias ? e.bias[ch0 + i] : 0);
        }
        return;
    }
    int8_t* out = dst + off;
    const bool pc = e.flt_scales != nullptr;
    if (e.fast_ops != 0) {
        // set by the host only together with `bounded`, per-tensor scales, IDENTITY / RELU
        const int8_t* zin = e.z_mode != 0 ? e.z + off : nullptr;
        const bool zfast = e.z_mode != 0 && e.z_fast_a != 0.f;
#define MB200_FAST_CASE(OPS)                                                                      \
    if (zfast && e.z_mode == 1)                                                                   \
        epilogue_store_t<NV, ACT_IDENTITY, false, true, 1, OPS, true>(v, e, out, zin, ch0);       \
    else if (zfast)                                                                               \
        epilogue_store_t<NV, ACT_IDENTITY, false, true, 2, OPS, true>(v, e, out, zin, ch0);       \
    else if (e.z_mode == 1)                                                                       \
        epilogue_store_t<NV, ACT_IDENTITY, false, true, 1, OPS>(v, e, out, zin, ch0);             \
    else if (e.z_mode == 2)                                                                       \
        epilogue_store_t<NV, ACT_IDENTITY, false, true, 2, OPS>(v, e, out, zin, ch0);             \
    else if (e.act == ACT_RELU)                                                                   \
        epilogue_store_t<NV, ACT_RELU, false, true, 0, OPS>(v, e, out, nullptr, ch0);             \
    else                                                                                          \
        epilogue_store_t<NV, ACT_IDENTITY, false, true, 0, OPS>(v, e, out, nullptr, ch0);
        if (e.fast_ops == 1) {
            MB200_FAST_CASE(1)
        } else if (e.fast_ops == 2) {
            MB200_FAST_CASE(2)
        } else {
            MB200_FAST_CASE(3)
        }
#undef MB200_FAST_CASE
        return;
    }
    if (e.z_mode != 0) {
        // the fused form follows a ConvBias without activation
        const int8_t* zin = e.z + off;
        if (e.z_mode == 1) {
            if (pc)
                epilogue_store_t<NV, ACT_IDENTITY, true, false, 1>(v, e, out, zin, ch0);
            else if (e.bounded)
                epilogue_store_t<NV, ACT_IDENTITY, false, true, 1>(v, e, out, zin, ch0);
            else
                epilogue_store_t<NV, ACT_IDENTITY, false, false, 1>(v, e, out, zin, ch0);
        } else {
            if (pc)
                epilogue_store_t<NV, ACT_IDENTITY, true, false, 2>(v, e, out, zin, ch0);
            else if (e.bounded)
                epilogue_store_t<NV, ACT_IDENTITY, false, true, 2>(v, e, out, zin, ch0);
            else
                epilogue_store_t<NV, ACT_IDENTITY, false, false, 2>(v, e, out, zin, ch0);
        }
        return;
    }
    if (e.bounded && !pc) {
        switch (e.act) {
            case ACT_IDENTITY:
                epilogue_store_t<NV, ACT_IDENTITY, false, true, 0>(v, e, out, nullptr, ch0);
                break;
            case ACT_RELU:
                epilogue_store_t<NV, ACT_RELU, false, true, 0>(v, e, out, nullptr, ch0);
                break;
            default:
                epilogue_store_t<NV, ACT_H_SWISH, false, true, 0>(v, e, out, nullptr, ch0);
                break;
        }
        return;
    }
    switch (e.act * 2 + (pc ? 1 : 0)) {
        case 0: epilogue_store_t<NV, ACT_IDENTITY, false, false, 0>(v, e, out, nullptr, ch0); break;
        case 1: epilogue_store_t<NV, ACT_IDENTITY, true, false, 0>(v, e, out, nullptr, ch0); break;
        case 2: epilogue_store_t<NV, ACT_RELU, false, false, 0>(v, e, out, nullptr, ch0); break;
        case 3: epilogue_store_t<NV, ACT_RELU, true, false, 0>(v, e, out, nullptr, ch0); break;
        case 4: epilogue_store_t<NV, ACT_H_SWISH, false, false, 0>(v, e, out, nullptr, ch0); break;
        default: epilogue_store_t<NV, ACT_H_SWISH, true, false, 0>(v, e, out, nullptr, ch0); break;
    }
}

}  // namespace mb200
