// qint8 depthwise ConvBias (groups == channels, one filter per channel), NHWC, 3x3 filter,
// any stride and padding: no reduction over channels, so no tensor cores.
//
// Two kernels. conv_dw_kernel: one thread = one output pixel x 16 channels. Its taps are
// 16-byte vector loads (the 16 channels of one input pixel); a tap outside the image
// contributes zeros. dp4a is used the other way round: the bytes of four taps are transposed
// (8 PRMTs per 4 taps x 4 channels) into one word per channel holding that channel's four
// taps, and one dp4a per channel multiplies them with the channel's four weights: 0.75
// instructions per multiply-add instead of 3 for extract-extract-multiply. The filter, packed
// [C][KH*KW] like every group filter, is re-laid once per CTA into shared memory as words of
// four taps each (zero beyond the ninth tap), ordered [tap group][channel quad within 16]
// [16-channel group][4 channels] so that a warp's 16-byte reads are consecutive. It serves
// stride 2 and the fused residual step. conv_dw3x3_row_kernel (further down): two or four
// adjacent outputs per thread, the default at stride 1.
//
// Arithmetic: the reference's order (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:305-344,
// Activation.cpp:105-113) or its verified one-FMA form for per-tensor scales, per-tensor or
// per-channel filter scales, optional fused residual step as in the other ConvBias kernels.
#include <stdlib.h>

#include "internal.h"
#include "tuning.h"

namespace mb200 {

namespace {

constexpr int kTapWords = 3;  // 12 taps at most

struct DwParams {
    ConvArgs a;
    int c16;    // channels / 16
    float inv_dst, z_div;
    // the verified one-FMA requantisation (requant_verify.cu), per-tensor scales only:
    // fast_ops == 1 -> trunc(fma((float)acc, fast_mul, +-fast_add)) saturated
    int fast_ops;
    float fast_mul, fast_add;
};

// four words, byte i = channel i of taps a..d  ->  four words, byte j = tap j of one channel
__device__ __forceinline__ void transpose4x4(
        uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&ch)[4]) {
    const uint32_t ab_lo = __byte_perm(a, b, 0x5140), cd_lo = __byte_perm(c, d, 0x5140);
    const uint32_t ab_hi = __byte_perm(a, b, 0x7362), cd_hi = __byte_perm(c, d, 0x7362);
    ch[0] = __byte_perm(ab_lo, cd_lo, 0x5410);
    ch[1] = __byte_perm(ab_lo, cd_lo, 0x7632);
    ch[2] = __byte_perm(ab_hi, cd_hi, 0x5410);
    ch[3] = __byte_perm(ab_hi, cd_hi, 0x7632);
}

template <int KH, int KW>
__global__ void __launch_bounds__(256) conv_dw_kernel(
        const DwParams p, const uint4* __restrict__ src, const int8_t* __restrict__ flt,
        const int32_t* __restrict__ bias, const float* __restrict__ flt_scales,
        uint4* __restrict__ dst) {
    extern __shared__ uint4 w_smem[];  // [kTapWords][4 quads][c16] vectors of 4 channels
    const ConvArgs& a = p.a;
    constexpr int kTaps = KH * KW;
    for (int c = threadIdx.x; c < a.ic; c += blockDim.x) {
        uint32_t w[kTapWords] = {0, 0, 0};
        for (int t = 0; t < kTaps; ++t)
            w[t >> 2] |= (uint32_t)(uint8_t)flt[(size_t)c * kTaps + t] << (8 * (t & 3));
        const int cvv = c >> 4, q = (c >> 2) & 3, i = c & 3;
#pragma unroll
        for (int g = 0; g < kTapWords; ++g)
            reinterpret_cast<uint32_t*>(w_smem)[((g * 4 + q) * p.c16 + cvv) * 4 + i] = w[g];
    }
    __syncthreads();

    const unsigned total = (unsigned)a.m * p.c16;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % p.c16;
        unsigned m = idx / p.c16;
        const int ox = (int)(m % a.ow);
        m /= a.ow;
        const int oy = (int)(m % a.oh);
        const int n = (int)(m / a.oh);
        // the taps, 12 slots, zeros where the filter or the image ends
        uint4 v[4 * kTapWords];
#pragma unroll
        for (int t = 0; t < 4 * kTapWords; ++t) {
            v[t] = make_uint4(0, 0, 0, 0);
            if (t < kTaps) {
                const int fy = t / KW, fx = t - fy * KW;
                const int iy = oy * a.sh + fy - a.ph, ix = ox * a.sw + fx - a.pw;
                if ((unsigned)iy < (unsigned)a.ih && (unsigned)ix < (unsigned)a.iw)
                    v[t] = __ldg(src + ((size_t)((unsigned)n * a.ih + iy) * a.iw + ix) * p.c16 + cv);
            }
        }
        int acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
            acc[i] = 0;
#pragma unroll
        for (int g = 0; g < kTapWords; ++g) {
            if (4 * g >= kTaps)
                break;
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // channel quad = word q of every tap vector
                const uint32_t ta = q == 0 ? v[4 * g].x : q == 1 ? v[4 * g].y : q == 2 ? v[4 * g].z : v[4 * g].w;
                const uint32_t tb = q == 0 ? v[4 * g + 1].x : q == 1 ? v[4 * g + 1].y : q == 2 ? v[4 * g + 1].z : v[4 * g + 1].w;
                const uint32_t tc = q == 0 ? v[4 * g + 2].x : q == 1 ? v[4 * g + 2].y : q == 2 ? v[4 * g + 2].z : v[4 * g + 2].w;
                const uint32_t td = q == 0 ? v[4 * g + 3].x : q == 1 ? v[4 * g + 3].y : q == 2 ? v[4 * g + 3].z : v[4 * g + 3].w;
                uint32_t ch[4];
                transpose4x4(ta, tb, tc, td, ch);
                const uint4 w = w_smem[(g * 4 + q) * p.c16 + cv];
                acc[q * 4 + 0] = __dp4a((int)ch[0], (int)w.x, acc[q * 4 + 0]);
                acc[q * 4 + 1] = __dp4a((int)ch[1], (int)w.y, acc[q * 4 + 1]);
                acc[q * 4 + 2] = __dp4a((int)ch[2], (int)w.z, acc[q * 4 + 2]);
                acc[q * 4 + 3] = __dp4a((int)ch[3], (int)w.w, acc[q * 4 + 3]);
            }
        }
        const int c0 = (int)cv * 16;
        uint32_t zw[4] = {0, 0, 0, 0};
        if (a.z_mode != 0 && a.z) {
            const uint4 zv = __ldg(reinterpret_cast<const uint4*>(a.z) + idx);
            zw[0] = zv.x; zw[1] = zv.y; zw[2] = zv.z; zw[3] = zv.w;
        }
        uint32_t out[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int4 b = make_int4(0, 0, 0, 0);
            if (bias)
                b = __ldg(reinterpret_cast<const int4*>(bias + c0) + q);
            float4 s = make_float4(a.s_flt, a.s_flt, a.s_flt, a.s_flt);
            if (flt_scales)
                s = __ldg(reinterpret_cast<const float4*>(flt_scales + c0) + q);
            const int bb[4] = {b.x, b.y, b.z, b.w};
            const float ss[4] = {s.x, s.y, s.z, s.w};
            int r[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (p.fast_ops == 1) {
                    const float f = __int2float_rn(acc[q * 4 + i] + bb[i]);
                    const float y = __fmaf_rn(
                            f, p.fast_mul,
                            a.act == ACT_RELU ? p.fast_add : copysignf(p.fast_add, f));
                    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r[i]) : "f"(y));
                    if (a.act == ACT_RELU)
                        r[i] = max(r[i], 0);
                } else {
                    r[i] = requant_conv_fast(acc[q * 4 + i] + bb[i], a.s_src, ss[i], a.s_dst,
                                             p.inv_dst, a.act);
                }
                if (a.z_mode != 0 && a.z) {
                    // fused ElemwiseMultiType step (ElemwiseMultiType.cpp:38-46,158)
                    const int zi = (int)(int8_t)(zw[q] >> (8 * i));
                    float t = __fadd_rn(__fmul_rn(a.s_dst, __int2float_rn(r[i])),
                                        __fmul_rn(a.z_scale, __int2float_rn(zi)));
                    if (a.z_mode == 2)
                        t = t > 0.f ? t : 0.f;
                    r[i] = fp32_to_int8(__fmul_rn(t, p.z_div));
                }
            }
            out[q] = pack4(r[0], r[1], r[2], r[3]);
        }
        dst[idx] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// ------------------------------------------------------------------------------------------
// OUT (2 or 4) horizontally adjacent outputs per thread (3x3, stride 1 or 2, no fused residual step)
// ------------------------------------------------------------------------------------------
// The kernel above spends 41 instructions per output and is bound by instruction issue.
// Here a thread walks the (OUT - 1) S + 3 input columns its outputs touch. A column is loaded
// once (three vectors: the three filter rows), transposed once into one word per channel
// holding (top, middle, bottom, 0), and every output that uses the column adds one dp4a per
// channel with the word of its filter column (w(0,dx), w(1,dx), w(2,dx), 0). Against one
// output per thread: half the vector loads, two thirds of the permutes at stride 1, a quarter
// of the index arithmetic. Filter columns live in shared memory as [dx][channel quad of the
// vector][16-channel vector][4 channels] words.
__device__ __forceinline__ uint32_t quad_word(const uint4& v, int q) {
    return q == 0 ? v.x : q == 1 ? v.y : q == 2 ? v.z : v.w;
}

template <int S, int OUT>
__global__ void __launch_bounds__(128, OUT == 4 ? 4 : 6) conv_dw3x3_row_kernel(
        const DwParams p, const uint4* __restrict__ src, const int8_t* __restrict__ flt,
        const int32_t* __restrict__ bias, const float* __restrict__ flt_scales,
        uint4* __restrict__ dst) {
    extern __shared__ uint4 w_smem[];  // [3 dx][4 quads][c16] vectors of 4 channel words
    const ConvArgs& a = p.a;
    constexpr int kOut = OUT, kCols = (kOut - 1) * S + 3;
    for (int c = threadIdx.x; c < a.ic; c += blockDim.x) {
        const int cvv = c >> 4, q = (c >> 2) & 3, i = c & 3;
#pragma unroll
        for (int dx = 0; dx < 3; ++dx) {
            uint32_t w = 0;
#pragma unroll
            for (int fy = 0; fy < 3; ++fy)
                w |= (uint32_t)(uint8_t)flt[(size_t)c * 9 + fy * 3 + dx] << (8 * fy);
            reinterpret_cast<uint32_t*>(w_smem)[((dx * 4 + q) * p.c16 + cvv) * 4 + i] = w;
        }
    }
    __syncthreads();

    const unsigned groups = (unsigned)(a.ow + kOut - 1) / kOut;
    const unsigned total = (unsigned)a.n * a.oh * groups * p.c16;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % p.c16;
        unsigned t = idx / p.c16;
        const int ox0 = (int)(t % groups) * kOut;
        t /= groups;
        const int oy = (int)(t % a.oh);
        const int n = (int)(t / a.oh);
        const int iy0 = oy * S - a.ph, ix0 = ox0 * S - a.pw;
        int acc[kOut][16];
#pragma unroll
        for (int o = 0; o < kOut; ++o)
#pragma unroll
            for (int i = 0; i < 16; ++i)
                acc[o][i] = 0;
        const uint4* base = src + (size_t)((unsigned)n * a.ih) * a.iw * p.c16 + cv;
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
            const int ix = ix0 + j;
            uint4 r[3];
#pragma unroll
            for (int fy = 0; fy < 3; ++fy) {
                const int iy = iy0 + fy;
                r[fy] = make_uint4(0, 0, 0, 0);
                if ((unsigned)iy < (unsigned)a.ih && (unsigned)ix < (unsigned)a.iw)
                    r[fy] = __ldg(base + ((size_t)iy * a.iw + ix) * p.c16);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t ch[4];  // channel 4q + i: bytes (top, middle, bottom, 0)
                transpose4x4(quad_word(r[0], q), quad_word(r[1], q), quad_word(r[2], q), 0u, ch);
#pragma unroll
                for (int o = 0; o < kOut; ++o) {
                    const int dx = j - o * S;  // this column's place in output o's window
                    if (dx < 0 || dx > 2)
                        continue;
                    const uint4 w = w_smem[(dx * 4 + q) * p.c16 + cv];
                    acc[o][q * 4 + 0] = __dp4a((int)ch[0], (int)w.x, acc[o][q * 4 + 0]);
                    acc[o][q * 4 + 1] = __dp4a((int)ch[1], (int)w.y, acc[o][q * 4 + 1]);
                    acc[o][q * 4 + 2] = __dp4a((int)ch[2], (int)w.z, acc[o][q * 4 + 2]);
                    acc[o][q * 4 + 3] = __dp4a((int)ch[3], (int)w.w, acc[o][q * 4 + 3]);
                }
            }
        }
        const int c0 = (int)cv * 16;
        uint4* out = dst + ((size_t)((unsigned)n * a.oh + oy) * a.ow + ox0) * p.c16 + cv;
#pragma unroll
        for (int o = 0; o < kOut; ++o) {
            if (ox0 + o >= a.ow)
                break;
            uint32_t packed[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                int4 b = make_int4(0, 0, 0, 0);
                if (bias)
                    b = __ldg(reinterpret_cast<const int4*>(bias + c0) + q);
                float4 s = make_float4(a.s_flt, a.s_flt, a.s_flt, a.s_flt);
                if (flt_scales)
                    s = __ldg(reinterpret_cast<const float4*>(flt_scales + c0) + q);
                const int bb[4] = {b.x, b.y, b.z, b.w};
                const float ss[4] = {s.x, s.y, s.z, s.w};
                int r4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int x = acc[o][q * 4 + i] + bb[i];
                    if (p.fast_ops == 1) {
                        const float f = __int2float_rn(x);
                        const float y = __fmaf_rn(
                                f, p.fast_mul,
                                a.act == ACT_RELU ? p.fast_add : copysignf(p.fast_add, f));
                        asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r4[i]) : "f"(y));
                        if (a.act == ACT_RELU)
                            r4[i] = max(r4[i], 0);
                    } else {
                        r4[i] = requant_conv_fast(x, a.s_src, ss[i], a.s_dst, p.inv_dst, a.act);
                    }
                }
                packed[q] = pack4(r4[0], r4[1], r4[2], r4[3]);
            }
            out[(size_t)o * p.c16] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
    }
}

}  // namespace

bool conv_dw_supported(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int8_t* dst) {
    if (a.groups != a.ic || a.oc != a.ic || a.src_is_nchw)
        return false;
    if (a.ic % 16 != 0 || a.kh != 3 || a.kw != 3 || a.dh != 1 || a.dw != 1)
        return false;
    if ((size_t)a.m * (a.ic / 16) >= (1ull << 31) ||
        (size_t)a.n * a.ih * a.iw * (a.ic / 16) >= (1ull << 31))
        return false;
    if ((size_t)a.ic * kTapWords * 4 > 96 * 1024)
        return false;
    if (((uintptr_t)src | (uintptr_t)dst) & 15)
        return false;
    return flt != nullptr;
}

// `flt`: the packed group filter [C][KH][KW] (one input channel per group)
int launch_conv_dw(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st) {
    if (((uintptr_t)bias & 15) || ((uintptr_t)flt_scales & 15) || ((uintptr_t)a.z & 15))
        return set_error(ST_INVALID_LAYOUT, "bias, channel scales and z must be 16-byte aligned");
    DwParams p;
    p.a = a;
    p.c16 = a.ic / 16;
    p.inv_dst = 1.0f / a.s_dst;         // RN(1/d), as the division by a constant needs
    p.z_div = 1.0f / a.z_out_scale;     // the reference's scale_div = 1.f / scale_dst
    p.fast_ops = 0;
    p.fast_mul = p.fast_add = 0.f;
    if (!flt_scales) {
        // (the search itself refuses scales whose results could leave the int range)
        p.fast_ops = requant_fast_constants(a.s_src, a.s_flt, a.s_dst, a.act, &p.fast_mul,
                                            &p.fast_add);
        if (p.fast_ops != 1)
            p.fast_ops = 0;
    }
    const size_t work = (size_t)a.m * p.c16;
    size_t grid = (work + 255) / 256;
    const size_t cap = (size_t)148 * 8;
    if (grid > cap)
        grid = cap;
    if (grid < 1)
        grid = 1;
    const int smem = a.ic * kTapWords * 4;
    // Several outputs per thread. Measured on the MobileNetV1 layers at batch 64: two outputs
    // per thread are 10-20 % faster than one at stride 1 (40 against 49 us for 32 channels
    // at 112x112) and four are no better than two (130 registers, 18 % of the warp slots,
    // latency-bound); at stride 2 adjacent outputs share one input column only and the
    // one-output kernel stays ahead. MB200_DW_OUT=2|4 forces a form at either stride,
    // MB200_DW_ONE_OUTPUT=1 the one-output kernel (tests and experiments).
    const int forced = tuning().dw_out;
    if (a.sh == a.sw && (a.sh == 1 || (a.sh == 2 && forced != 0)) && !(a.z_mode != 0 && a.z) &&
        !tuning().dw_one_output) {
        const int outs = forced == 4 ? 4 : 2;
        const size_t items = (size_t)a.n * a.oh * ((a.ow + outs - 1) / outs) * p.c16;
        size_t blocks = (items + 127) / 128;
        const size_t most = (size_t)148 * 16;
        if (blocks > most)
            blocks = most;
        if (blocks < 1)
            blocks = 1;
        auto kernel = outs == 4 ? (a.sh == 1 ? conv_dw3x3_row_kernel<1, 4> : conv_dw3x3_row_kernel<2, 4>)
                                : (a.sh == 1 ? conv_dw3x3_row_kernel<1, 2> : conv_dw3x3_row_kernel<2, 2>);
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
                    cudaSuccess)
            return check_launch("conv_dw smem attribute");
        kernel<<<(int)blocks, 128, smem, st>>>(p, (const uint4*)src, flt, bias, flt_scales,
                                               (uint4*)dst);
        return check_launch("conv_dw_row");
    }
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(conv_dw_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem) != cudaSuccess)
        return check_launch("conv_dw smem attribute");
    conv_dw_kernel<3, 3><<<(int)grid, 256, smem, st>>>(
            p, (const uint4*)src, flt, bias, flt_scales, (uint4*)dst);
    return check_launch("conv_dw");
}

}  // namespace mb200
