// CUDA-core kernels of the hot path: the general (any shape) ConvBias, filter packing,
// pooling, quantised elementwise, type conversion and layout transforms. The tensor-core
// ConvBias lives in conv_umma.cu; everything here is bandwidth- or latency-bound work.
#include "internal.h"
#include "pdl.h"

namespace mb200 {

// ------------------------------------------------------------------------------------------
// filter packing: OIHW (dense) or [G][OCpg][ICpg][KH][KW] (group) -> [OC][KH][KW][ICpg]
// ------------------------------------------------------------------------------------------
__global__ void pack_filter_kernel(
        const int8_t* __restrict__ src, int8_t* __restrict__ dst, int oc, int icpg, int kh,
        int kw) {
    const size_t total = (size_t)oc * icpg * kh * kw;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        // i indexes dst: [o][fy][fx][c]
        int c = (int)(i % icpg);
        size_t t = i / icpg;
        int fx = (int)(t % kw);
        t /= kw;
        int fy = (int)(t % kh);
        int o = (int)(t / kh);
        dst[i] = src[(((size_t)o * icpg + c) * kh + fy) * kw + fx];
    }
}

// ------------------------------------------------------------------------------------------
// NCHW44 filters (what a model compiled with --enable_nchw44 carries) -> OIHW, after which
// the usual packing applies. Index formulas of compiler/lib/KernelGen/BareMetal/ConvKernel.cpp
// :48-62,88-101:
//   form 0 dense        [OC/4][IC/4][KH][KW][4 ic][4 oc]
//   form 1 channel-wise [G/4][1][1][KH][KW][4]            (one input channel per group)
//   form 2 first layer  [OC/4][KH][KW][IC][4 oc]          (NCHW input, NCHW44 output)
// dst: OIHW, or [G][1][1][KH][KW] for form 1
// ------------------------------------------------------------------------------------------
__global__ void filter_nchw44_to_oihw_kernel(
        const int8_t* __restrict__ src, int8_t* __restrict__ dst, int form, int oc, int icpg,
        int kh, int kw) {
    const size_t total = (size_t)oc * icpg * kh * kw;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        // i indexes dst: [o][c][fy][fx]
        const int fx = (int)(i % kw);
        size_t t = i / kw;
        const int fy = (int)(t % kh);
        t /= kh;
        const int c = (int)(t % icpg);
        const int o = (int)(t / icpg);
        size_t off;
        if (form == 0)
            off = (size_t)(o / 4) * ((size_t)icpg * kh * kw * 4) + (size_t)(c / 4) * (kh * kw * 16) +
                  (size_t)fy * (kw * 16) + (size_t)fx * 16 + (c % 4) * 4 + (o % 4);
        else if (form == 1)
            off = (size_t)(o / 4) * (kh * kw * 4) + (size_t)fy * (kw * 4) + (size_t)fx * 4 + (o % 4);
        else
            off = (size_t)(o / 4) * ((size_t)4 * kh * kw * icpg) + (size_t)fy * (kw * icpg * 4) +
                  (size_t)fx * (icpg * 4) + (size_t)c * 4 + (o % 4);
        dst[i] = src[off];
    }
}

// ------------------------------------------------------------------------------------------
// general direct ConvBias. One thread per (output pixel, output channel), channel fastest,
// so a warp shares one input window (broadcast loads) and writes 32 contiguous bytes.
// ------------------------------------------------------------------------------------------
template <bool kRequant>
__global__ void __launch_bounds__(256) conv_direct_kernel(
        ConvArgs a, const int8_t* __restrict__ src, const int8_t* __restrict__ flt,
        const int32_t* __restrict__ bias, const float* __restrict__ flt_scales,
        int8_t* __restrict__ dst, int32_t* __restrict__ acc_out) {
    const size_t total = (size_t)a.m * a.oc;
    const int icpg = a.ic / a.groups, ocpg = a.oc / a.groups;
    // 4-byte loads only where every (pixel, group) run and every filter tap starts on a
    // 4-byte boundary: icpg % 4 == 0 keeps the strides aligned, the base pointers are the
    // caller's (a tensor sliced at an odd byte takes the byte loop)
    const bool vec4 = !a.src_is_nchw && (icpg % 4 == 0) &&
                      ((((uintptr_t)src) | ((uintptr_t)flt)) & 3) == 0;
    const float inv_dst = __fdiv_rn(1.f, a.s_dst);  // RN(1/d), as the fast division needs
    const float z_div = __fdiv_rn(1.f, a.z_out_scale);
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(idx % a.oc);
        const int m = (int)(idx / a.oc);
        const int ow_ = m % a.ow;
        const int t = m / a.ow;
        const int oh_ = t % a.oh;
        const int n = t / a.oh;
        const int g = o / ocpg;
        const int8_t* w = flt + (size_t)o * a.kh * a.kw * icpg;
        int acc = 0;
        for (int fy = 0; fy < a.kh; ++fy) {
            const int iy = oh_ * a.sh + fy * a.dh - a.ph;
            if ((unsigned)iy >= (unsigned)a.ih)
                continue;
            for (int fx = 0; fx < a.kw; ++fx) {
                const int ix = ow_ * a.sw + fx * a.dw - a.pw;
                if ((unsigned)ix >= (unsigned)a.iw)
                    continue;
                const int8_t* wk = w + (size_t)(fy * a.kw + fx) * icpg;
                if (vec4) {
                    const int8_t* s =
                            src + (((size_t)n * a.ih + iy) * a.iw + ix) * a.ic + g * icpg;
                    const int* s4 = reinterpret_cast<const int*>(s);
                    const int* w4 = reinterpret_cast<const int*>(wk);
                    for (int c = 0; c < icpg / 4; ++c)
                        acc = __dp4a(__ldg(s4 + c), __ldg(w4 + c), acc);
                } else if (!a.src_is_nchw) {
                    const int8_t* s =
                            src + (((size_t)n * a.ih + iy) * a.iw + ix) * a.ic + g * icpg;
                    for (int c = 0; c < icpg; ++c)
                        acc += (int)s[c] * (int)wk[c];
                } else {
                    const size_t plane = (size_t)a.ih * a.iw;
                    const int8_t* s = src + ((size_t)n * a.ic + g * icpg) * plane +
                                      (size_t)iy * a.iw + ix;
                    for (int c = 0; c < icpg; ++c)
                        acc += (int)s[c * plane] * (int)wk[c];
                }
            }
        }
        if (bias)
            acc += bias[o];
        if (kRequant) {
            const float sf = flt_scales ? flt_scales[o] : a.s_flt;
            int q = a.true_division
                            ? requant_conv(acc, a.s_src, sf, a.s_dst, a.act)
                            : requant_conv_fast(acc, a.s_src, sf, a.s_dst, inv_dst, a.act);
            if (a.z_mode != 0 && a.z) {
                // fused ElemwiseMultiType step (ElemwiseMultiType.cpp:38-46,158)
                float t = __fadd_rn(__fmul_rn(a.s_dst, __int2float_rn(q)),
                                    __fmul_rn(a.z_scale, __int2float_rn((int)a.z[idx])));
                if (a.z_mode == 2)
                    t = t > 0.f ? t : 0.f;
                q = fp32_to_int8(__fmul_rn(t, z_div));
            }
            dst[idx] = (int8_t)q;
        } else {
            acc_out[idx] = acc;
        }
    }
}

// ------------------------------------------------------------------------------------------
// pooling, NHWC, one thread per output element (channel fastest -> coalesced)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pooling_kernel(
        const int8_t* __restrict__ src, int8_t* __restrict__ dst, int mode, int n, int c, int ih,
        int iw, int oh, int ow, int wh, int ww, int sh, int sw, int ph, int pw) {
    pdl_start();
    const size_t total = (size_t)n * oh * ow * c;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ch = (int)(idx % c);
        size_t t = idx / c;
        const int x = (int)(t % ow);
        t /= ow;
        const int y = (int)(t % oh);
        const int b = (int)(t / oh);
        int mx = -128, sum = 0, count = 0;
        for (int fy = 0; fy < wh; ++fy) {
            const int iy = y * sh + fy - ph;
            if ((unsigned)iy >= (unsigned)ih)
                continue;
            for (int fx = 0; fx < ww; ++fx) {
                const int ix = x * sw + fx - pw;
                if ((unsigned)ix >= (unsigned)iw)
                    continue;
                const int v = src[(((size_t)b * ih + iy) * iw + ix) * c + ch];
                mx = v > mx ? v : mx;
                sum += v;
                ++count;
            }
        }
        int r;
        if (mode == 0) {
            r = mx;
        } else {
            // roundf((float)sum / count), stored through an int (Pooling.cpp:131-146)
            const float d = (mode == 1) ? (float)(wh * ww) : (float)count;
            r = f32_to_i32_x86(roundf(__fdiv_rn(__int2float_rn(sum), d)));
        }
        dst[idx] = (int8_t)r;
    }
}

// MAX pooling, 16 channels (one 16-byte vector) per thread; per-byte signed max in SIMD
__global__ void __launch_bounds__(256) pooling_max_vec16_kernel(
        const uint4* __restrict__ src, uint4* __restrict__ dst, int n, int c16, int ih, int iw,
        int oh, int ow, int wh, int ww, int sh, int sw, int ph, int pw) {
    pdl_start();
    const size_t total = (size_t)n * oh * ow * c16;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int cv = (int)(idx % c16);
        size_t t = idx / c16;
        const int x = (int)(t % ow);
        t /= ow;
        const int y = (int)(t % oh);
        const int b = (int)(t / oh);
        uint4 m = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // -128
        for (int fy = 0; fy < wh; ++fy) {
            const int iy = y * sh + fy - ph;
            if ((unsigned)iy >= (unsigned)ih)
                continue;
            for (int fx = 0; fx < ww; ++fx) {
                const int ix = x * sw + fx - pw;
                if ((unsigned)ix >= (unsigned)iw)
                    continue;
                const uint4 v = __ldg(src + (((size_t)b * ih + iy) * iw + ix) * c16 + cv);
                m.x = __vmaxs4(m.x, v.x);
                m.y = __vmaxs4(m.y, v.y);
                m.z = __vmaxs4(m.z, v.z);
                m.w = __vmaxs4(m.w, v.w);
            }
        }
        dst[idx] = m;
    }
}

// MAX pooling with a 3x3 window and stride 2 (the ResNet stem's pool), 16 channels per
// thread and TWO horizontally adjacent outputs per thread: their windows share a column, so
// 15 loads serve both (instead of 18), all issued before the first use. 32-bit index
// arithmetic (the launcher checks the sizes). The kernel is bound by HBM: every input byte
// is read once from DRAM, the re-reads between neighbouring threads hit L1 / L2.
__device__ __forceinline__ uint4 vmax16(uint4 a, uint4 b) {
    return make_uint4(__vmaxs4(a.x, b.x), __vmaxs4(a.y, b.y), __vmaxs4(a.z, b.z),
                      __vmaxs4(a.w, b.w));
}

__global__ void __launch_bounds__(256, 4) pooling_max_3x3s2_vec16_kernel(
        const uint4* __restrict__ src, uint4* __restrict__ dst, int n, int c16, int ih, int iw,
        int oh, int ow, int ph, int pw) {
    pdl_start();
    const int owp = (ow + 1) / 2;  // output pairs per row
    const unsigned total = (unsigned)n * oh * owp * c16;
    const uint4 lowest = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // -128
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % c16;
        unsigned t = idx / c16;
        const int xp = (int)(t % owp);
        t /= owp;
        const int y = (int)(t % oh);
        const int b = (int)(t / oh);
        const int x0 = 2 * xp;
        const int ix0 = 2 * x0 - pw, iy0 = 2 * y - ph;
        uint4 v[3][5];
#pragma unroll
        for (int fy = 0; fy < 3; ++fy) {
            const int iy = iy0 + fy;
            const bool row_ok = (unsigned)iy < (unsigned)ih;
            const uint4* row = src + ((size_t)((unsigned)b * ih + (row_ok ? iy : 0)) * iw) * c16 + cv;
#pragma unroll
            for (int fx = 0; fx < 5; ++fx) {
                const int ix = ix0 + fx;
                v[fy][fx] = (row_ok && (unsigned)ix < (unsigned)iw) ? __ldg(row + (size_t)ix * c16)
                                                                     : lowest;
            }
        }
        // Column maxima, then the two windows. Signed bytes are compared as the HIGH bytes of
        // signed 16-bit lanes (one three-input s16x2 maximum per lane pair; the byte-wise
        // intrinsic is emulated with a dozen instructions and made this kernel ALU-bound at
        // 53 % of the DRAM bandwidth): odd bytes already are high bytes, even bytes after a
        // shift by 8; what sits in a lane's low byte only breaks ties between equal high
        // bytes and is dropped when the two halves are merged.
        uint32_t odd[5][4], even[5][4];
#pragma unroll
        for (int fx = 0; fx < 5; ++fx) {
            const uint32_t r0[4] = {v[0][fx].x, v[0][fx].y, v[0][fx].z, v[0][fx].w};
            const uint32_t r1[4] = {v[1][fx].x, v[1][fx].y, v[1][fx].z, v[1][fx].w};
            const uint32_t r2[4] = {v[2][fx].x, v[2][fx].y, v[2][fx].z, v[2][fx].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                odd[fx][k] = __vimax3_s16x2(r0[k], r1[k], r2[k]);
                even[fx][k] = __vimax3_s16x2(r0[k] << 8, r1[k] << 8, r2[k] << 8);
            }
        }
        uint32_t o0[4], o1[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // bytes 1 and 3 of both halves -> bytes (even, odd, even, odd)
            o0[k] = __byte_perm(__vimax3_s16x2(even[0][k], even[1][k], even[2][k]),
                                __vimax3_s16x2(odd[0][k], odd[1][k], odd[2][k]), 0x7351);
            o1[k] = __byte_perm(__vimax3_s16x2(even[2][k], even[3][k], even[4][k]),
                                __vimax3_s16x2(odd[2][k], odd[3][k], odd[4][k]), 0x7351);
        }
        uint4* out = dst + ((size_t)((unsigned)b * oh + y) * ow + x0) * c16 + cv;
        out[0] = make_uint4(o0[0], o0[1], o0[2], o0[3]);
        if (x0 + 1 < ow)
            out[c16] = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    }
}

// AVERAGE pooling over the whole image (the classifier's global pool), 16 channels per thread:
// wh * ww vector loads, sixteen int sums, then roundf((float)sum / count) as pooling_kernel.
__global__ void __launch_bounds__(64) pooling_global_avg_vec16_kernel(
        const uint4* __restrict__ src, uint4* __restrict__ dst, int n, int c16, int pixels) {
    pdl_start();
    const unsigned total = (unsigned)n * c16;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % c16, b = idx / c16;
        const uint4* p = src + (size_t)b * pixels * c16 + cv;
        int sum[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
            sum[i] = 0;
        // seven loads in flight at a time (the accumulation would otherwise serialise them)
        for (int px0 = 0; px0 < pixels; px0 += 7) {
            uint4 v[7];
#pragma unroll
            for (int k = 0; k < 7; ++k)
                v[k] = px0 + k < pixels ? __ldg(p + (size_t)(px0 + k) * c16) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int k = 0; k < 7; ++k) {
                const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    sum[i] += (int)(int8_t)(w[i >> 2] >> (8 * (i & 3)));
            }
        }
        const float d = (float)pixels;
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int r[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                r[i] = f32_to_i32_x86(roundf(__fdiv_rn(__int2float_rn(sum[k * 4 + i]), d)));
            o[k] = pack4(r[0], r[1], r[2], r[3]);
        }
        dst[idx] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// The same with the pixels of one image split over the four warps of a CTA: a classifier's
// global pool has few outputs (batch x C/16 vectors) but 49 loads and 800 additions behind
// each, and one thread per output leaves most SMs with a single busy warp (21 us for
// 256 x 7 x 7 x 512). A CTA takes 32 consecutive 16-channel vectors of one image; warp g sums
// pixels g, g+4, ...; the partial sums meet in shared memory and every thread finishes four
// channels. The integer sum is exact in any order, the division is the one of
// pooling_kernel.
__global__ void __launch_bounds__(128) pooling_global_avg_split_kernel(
        const uint4* __restrict__ src, uint32_t* __restrict__ dst, int c16, int pixels,
        int blocks_per_image) {
    pdl_start();
    __shared__ int part[4][16][32];
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int b = blockIdx.x / blocks_per_image;
    const int cv = (blockIdx.x - b * blocks_per_image) * 32 + lane;
    const bool live = cv < c16;
    int sum[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        sum[i] = 0;
    if (live) {
        const uint4* p = src + (size_t)b * pixels * c16 + cv;
        for (int px0 = g; px0 < pixels; px0 += 4 * 7) {
            uint4 v[7];
#pragma unroll
            for (int k = 0; k < 7; ++k)
                v[k] = px0 + 4 * k < pixels ? __ldg(p + (size_t)(px0 + 4 * k) * c16)
                                            : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int k = 0; k < 7; ++k) {
                const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    sum[i] += (int)(int8_t)(w[i >> 2] >> (8 * (i & 3)));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
        part[g][i][lane] = sum[i];
    __syncthreads();
    if (!live)
        return;
    // thread (g, lane): channels 4g .. 4g+3 of vector `cv`
    const float d = (float)pixels;
    int r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s = part[0][4 * g + i][lane] + part[1][4 * g + i][lane] +
                      part[2][4 * g + i][lane] + part[3][4 * g + i][lane];
        r[i] = f32_to_i32_x86(roundf(__fdiv_rn(__int2float_rn(s), d)));
    }
    dst[((size_t)b * c16 + cv) * 4 + g] = pack4(r[0], r[1], r[2], r[3]);
}

// ------------------------------------------------------------------------------------------
// quantised elementwise, same-shape operands, 16 bytes per thread
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int qelem_one(
        int mode, int v0, int v1, float s0, float s1, float scale_div, float scale_mul) {
    if (mode == 0) {  // QADD: (s0*v0 + s1*v1) * scale_div
        float x = __fmul_rn(
                __fadd_rn(__fmul_rn(s0, __int2float_rn(v0)), __fmul_rn(s1, __int2float_rn(v1))),
                scale_div);
        return fp32_to_int8(x);
    } else if (mode == 1) {  // QFUSE_ADD_RELU
        float t = __fadd_rn(__fmul_rn(s0, __int2float_rn(v0)), __fmul_rn(s1, __int2float_rn(v1)));
        t = t > 0.f ? t : 0.f;
        return fp32_to_int8(__fmul_rn(t, scale_div));
    } else if (mode == 2) {  // QMUL: v0*v1*scale_mul, the product formed in int first
        return fp32_to_int8(__fmul_rn(__int2float_rn(v0 * v1), scale_mul));
    } else {  // QRELU
        float t = __fmul_rn(s0, __int2float_rn(v0));
        t = t > 0.f ? t : 0.f;
        return fp32_to_int8(__fmul_rn(t, scale_div));
    }
}

__global__ void __launch_bounds__(256) qelemwise_kernel(
        const int8_t* __restrict__ a, const int8_t* __restrict__ b, int8_t* __restrict__ dst,
        int mode, size_t nr_elem, float s0, float s1, float scale_div, float scale_mul,
        int vec_ok) {
    pdl_start();
    const size_t nvec = vec_ok ? nr_elem / 16 : 0;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t nthr = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < nvec; i += nthr) {
        const int4 va = __ldg(reinterpret_cast<const int4*>(a) + i);
        int4 vb = make_int4(0, 0, 0, 0);
        if (mode != 3)
            vb = __ldg(reinterpret_cast<const int4*>(b) + i);
        const int wa[4] = {va.x, va.y, va.z, va.w};
        const int wb[4] = {vb.x, vb.y, vb.z, vb.w};
        int wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int q[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int v0 = (int)(int8_t)(wa[j] >> (8 * k));
                const int v1 = (int)(int8_t)(wb[j] >> (8 * k));
                q[k] = qelem_one(mode, v0, v1, s0, s1, scale_div, scale_mul);
            }
            wo[j] = (int)pack4(q[0], q[1], q[2], q[3]);
        }
        reinterpret_cast<int4*>(dst)[i] = make_int4(wo[0], wo[1], wo[2], wo[3]);
    }
    for (size_t i = nvec * 16 + tid; i < nr_elem; i += nthr) {
        const int v1 = (mode != 3) ? (int)b[i] : 0;
        dst[i] = (int8_t)qelem_one(mode, (int)a[i], v1, s0, s1, scale_div, scale_mul);
    }
}

// Broadcast forms of ElemwiseMultiType (compiler/test/kernel/opr/naive/elemwise_multitype.cpp
// :33-62: a {2,3,4,5} operand combined with {1,3,1,1} or a scalar): element i of a meets
// b[(i / inner) % channels], or b[0] when channels == 0.
__global__ void __launch_bounds__(256) qelemwise_bcast_kernel(
        const int8_t* __restrict__ a, const int8_t* __restrict__ b, int8_t* __restrict__ dst,
        int mode, size_t nr_elem, unsigned channels, unsigned inner, float s0, float s1,
        float scale_div, float scale_mul) {
    pdl_start();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nr_elem;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t bi = channels ? (i / inner) % channels : 0;
        dst[i] = (int8_t)qelem_one(mode, (int)a[i], (int)b[bi], s0, s1, scale_div, scale_mul);
    }
}

// ------------------------------------------------------------------------------------------
// TypeCvt between fp32 and qsi8 as the reference's x86 build performs it: these dtype pairs
// resolve to the GeneralIntrinsic kernel, whose rule is NOT the BareMetal one
// (compiler/lib/KernelGen/GeneralIntrinsic/Typecvt.cpp:258-267 and :176-190): scale =
// src_scale / dst_scale is computed once in float, with the scale of the float side taken as
// 1 whatever the tensor says (:56-69), then every element is clamp(round(v * scale)), half
// away from zero. With the flags of the reference's x86 builds (no -msse4.2,
// compiler/script/compile_target_cmake.cmake:33) only GI_SSE2_INTRINSICS is defined and the
// SIMD groups of 16 take the same round() as the trailing elements
// (immigration/include/gi_int.h:1332-1340, gi_common.h:71-76); an SSE4.2 build would convert
// the SIMD groups as trunc(v * scale +- 0.5) instead, which differs next to ties.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) typecvt_f32_qs8_kernel(
        const float* __restrict__ src, int8_t* __restrict__ dst, size_t nr_elem, float scale) {
    pdl_start();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nr_elem;
         i += (size_t)gridDim.x * blockDim.x) {
        float r = roundf(__fmul_rn(src[i], scale));
        r = r >= 127.f ? 127.f : r;
        r = r <= -128.f ? -128.f : r;
        dst[i] = (int8_t)__float2int_rn(r);
    }
}

__global__ void __launch_bounds__(256) typecvt_qs8_f32_kernel(
        const int8_t* __restrict__ src, float* __restrict__ dst, size_t nr_elem, float scale) {
    pdl_start();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nr_elem;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __fmul_rn(__int2float_rn((int)src[i]), scale);
}

// ------------------------------------------------------------------------------------------
// typecvt qsi32 -> qsi8: saturate(roundf(val * src_scale / dst_scale))
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) typecvt_qs32_qs8_kernel(
        const int32_t* __restrict__ src, int8_t* __restrict__ dst, size_t nr_elem, float s_src,
        float s_dst) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nr_elem;
         i += (size_t)gridDim.x * blockDim.x) {
        const float x = __fdiv_rn(__fmul_rn(__int2float_rn(src[i]), s_src), s_dst);
        dst[i] = (int8_t)fp32_to_int8(x);
    }
}

// ------------------------------------------------------------------------------------------
// [R][C] -> [C][R] byte transpose per batch item, 32x32 tiles through shared memory
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_s8_kernel(
        const int8_t* __restrict__ src, int8_t* __restrict__ dst, int rows, int cols) {
    pdl_start();
    __shared__ int8_t tile[32][33];
    const size_t base = (size_t)blockIdx.z * rows * cols;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols)
            tile[j][threadIdx.x] = src[base + (size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols)
            dst[base + (size_t)c * rows + r] = tile[threadIdx.x][j];
    }
}

// ------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------
static int grid_for(size_t work, int block) {
    size_t g = (work + block - 1) / block;
    const size_t cap = (size_t)148 * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

int launch_pack_filter(
        const ConvArgs& a, const int8_t* src, int8_t* dst, cudaStream_t st) {
    const int icpg = a.ic / a.groups;
    const size_t total = (size_t)a.oc * icpg * a.kh * a.kw;
    pack_filter_kernel<<<grid_for(total, 256), 256, 0, st>>>(src, dst, a.oc, icpg, a.kh, a.kw);
    return check_launch("pack_filter");
}

int launch_filter_nchw44_to_oihw(
        const ConvArgs& a, int form, const int8_t* src, int8_t* dst, cudaStream_t st) {
    const int icpg = a.ic / a.groups;
    const size_t total = (size_t)a.oc * icpg * a.kh * a.kw;
    filter_nchw44_to_oihw_kernel<<<grid_for(total, 256), 256, 0, st>>>(src, dst, form, a.oc, icpg,
                                                                       a.kh, a.kw);
    return check_launch("filter_nchw44_to_oihw");
}

int launch_conv_direct(
        const ConvArgs& a, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, int32_t* acc, cudaStream_t st) {
    const size_t total = (size_t)a.m * a.oc;
    const int grid = grid_for(total, 256);
    if (acc)
        conv_direct_kernel<false><<<grid, 256, 0, st>>>(a, src, flt, bias, flt_scales, dst, acc);
    else
        conv_direct_kernel<true><<<grid, 256, 0, st>>>(a, src, flt, bias, flt_scales, dst, acc);
    return check_launch("conv_direct");
}

int launch_pooling(
        const int8_t* src, int8_t* dst, int mode, int n, int c, int ih, int iw, int wh, int ww,
        int sh, int sw, int ph, int pw, cudaStream_t st) {
    const int oh = (ih + 2 * ph - wh) / sh + 1, ow = (iw + 2 * pw - ww) / sw + 1;
    const size_t total = (size_t)n * oh * ow * c;
    const bool vec16 = mode == 0 && c % 16 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0);
    if (vec16 && wh == 3 && ww == 3 && sh == 2 && sw == 2 && ph <= 2 && pw <= 2 &&
        (size_t)n * ih * iw * (c / 16) < (1u << 30) && oh > 0 && ow > 0) {
        // a window with no valid element cannot occur: padding is below the window size
        const size_t pairs = (size_t)n * oh * ((ow + 1) / 2) * (c / 16);
        launch_pdl(pooling_max_3x3s2_vec16_kernel, dim3(grid_for(pairs, 256)), dim3(256), 0, st,
                   (const uint4*)src, (uint4*)dst, n, c / 16, ih, iw, oh, ow, ph, pw);
        return check_launch("pooling_max_3x3s2_vec16");
    }
    if (mode != 0 && c % 16 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) && wh == ih &&
        ww == iw && ph == 0 && pw == 0 && (size_t)n * (c / 16) < (1u << 31)) {
        // one window per image and no padding: both AVERAGE modes divide by wh * ww
        const size_t work = (size_t)n * (c / 16);
        const int per_image = (c / 16 + 31) / 32;
        if (ih * iw >= 8 && (size_t)n * per_image < (1u << 30)) {
            launch_pdl(pooling_global_avg_split_kernel, dim3(n * per_image), dim3(128), 0, st,
                       (const uint4*)src, (uint32_t*)dst, c / 16, ih * iw, per_image);
            return check_launch("pooling_global_avg_split");
        }
        launch_pdl(pooling_global_avg_vec16_kernel, dim3(grid_for(work, 64)), dim3(64), 0, st,
                   (const uint4*)src, (uint4*)dst, n, c / 16, ih * iw);
        return check_launch("pooling_global_avg_vec16");
    }
    if (vec16) {
        launch_pdl(pooling_max_vec16_kernel, dim3(grid_for(total / 16, 256)), dim3(256), 0, st,
                   (const uint4*)src, (uint4*)dst, n, c / 16, ih, iw, oh, ow, wh, ww, sh, sw, ph, pw);
        return check_launch("pooling_max_vec16");
    }
    launch_pdl(pooling_kernel, dim3(grid_for(total, 256)), dim3(256), 0, st, src, dst, mode, n, c, ih,
               iw, oh, ow, wh, ww, sh, sw, ph, pw);
    return check_launch("pooling");
}

int launch_qelemwise(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, float s0,
        float s1, float s_dst, cudaStream_t st) {
    // scale_div = 1.f / scale_dst; scale_mul = s0 * s1 * scale_div, computed on the host in
    // float exactly like the reference's generated C (ElemwiseMultiType.cpp:158-159)
    volatile float scale_div = 1.f / s_dst;
    volatile float t = s0 * s1;
    volatile float scale_mul = t * scale_div;
    const int vec_ok = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)dst) & 15) == 0;
    const size_t work = nr_elem / 16 + 1;
    launch_pdl(qelemwise_kernel, dim3(grid_for(work, 256)), dim3(256), 0, st,
               a, b, dst, mode, nr_elem, s0, s1, scale_div, scale_mul, vec_ok);
    return check_launch("qelemwise");
}

int launch_qelemwise_bcast(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, unsigned channels,
        unsigned inner, float s0, float s1, float s_dst, cudaStream_t st) {
    volatile float scale_div = 1.f / s_dst;
    volatile float t = s0 * s1;
    volatile float scale_mul = t * scale_div;
    launch_pdl(qelemwise_bcast_kernel, dim3(grid_for(nr_elem, 256)), dim3(256), 0, st, a, b, dst,
               mode, nr_elem, channels, inner ? inner : 1u, s0, s1, (float)scale_div,
               (float)scale_mul);
    return check_launch("qelemwise_bcast");
}

int launch_typecvt_f32_qs8(
        const float* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst, cudaStream_t st) {
    (void)s_src;  // a float tensor's scale counts as 1 (GeneralIntrinsic/Typecvt.cpp:56-69)
    volatile float scale = 1.f / s_dst;
    launch_pdl(typecvt_f32_qs8_kernel, dim3(grid_for(nr_elem, 256)), dim3(256), 0, st, src, dst,
               nr_elem, (float)scale);
    return check_launch("typecvt_f32_qs8");
}

int launch_typecvt_qs8_f32(
        const int8_t* src, float* dst, size_t nr_elem, float s_src, float s_dst, cudaStream_t st) {
    (void)s_dst;  // a float tensor's scale counts as 1
    volatile float scale = s_src / 1.f;
    launch_pdl(typecvt_qs8_f32_kernel, dim3(grid_for(nr_elem, 256)), dim3(256), 0, st, src, dst,
               nr_elem, (float)scale);
    return check_launch("typecvt_qs8_f32");
}

int launch_typecvt_qs32_qs8(
        const int32_t* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst,
        cudaStream_t st) {
    typecvt_qs32_qs8_kernel<<<grid_for(nr_elem, 256), 256, 0, st>>>(
            src, dst, nr_elem, s_src, s_dst);
    return check_launch("typecvt_qs32_qs8");
}

int launch_transpose_s8(
        const int8_t* src, int8_t* dst, int batch, int rows, int cols, cudaStream_t st) {
    if (batch <= 0 || rows <= 0 || cols <= 0)
        return 0;
    if (batch > 65535)
        return set_error(4, "transpose: batch %d exceeds the grid z limit", batch);
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
    launch_pdl(transpose_s8_kernel, grid, block, 0, st, src, dst, rows, cols);
    return check_launch("transpose_s8");
}

}  // namespace mb200
