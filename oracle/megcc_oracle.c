/* TEST INFRASTRUCTURE - CPU restatement of the reference's hot-path arithmetic.
 *
 * This file is the checker that the GPU results are compared with. It is used by
 * tests/, by the smoke check and by the CPU-baseline leg of bench.py only; the
 * product (megcc_b200/) never links, imports or calls it.
 *
 * Parity status: PINNED. Every function below is checked bit-for-bit against the
 * reference's own generated x86 kernels (oracle/_ref, built from the reference
 * sources by oracle/Makefile) in tests/test_oracle_vs_reference.py, and against
 * the committed golden vectors under tests/golden/ that were produced by those
 * same reference kernels.
 *
 * Layouts are the reference's model-visible ones: activations NCHW, dense filter
 * OIHW, grouped filter [G][OCpg][ICpg][KH][KW]
 * (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:50-52,89-91,217-220).
 * Integer accumulation is exact (wrap-around int32), so the loop order used here
 * for speed does not change any result; the float requantisation keeps the
 * reference's operation order literally. Build with -ffp-contract=off and without
 * fast-math (oracle/Makefile does).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ACT_IDENTITY = 0, ACT_RELU = 1, ACT_H_SWISH = 2 };

/* compiler/lib/KernelGen/BareMetal/Activation.cpp:50-56 */
static inline int8_t fp32_to_int8(float src) {
    int res = (int)roundf(src);
    res = res > 127 ? 127 : res;
    res = res < -128 ? -128 : res;
    return (int8_t)res;
}

/* compiler/lib/KernelGen/BareMetal/Activation.cpp:9-30 */
static inline float apply_act(int act, float x) {
    if (act == ACT_RELU)
        return x > 0 ? x : 0;
    if (act == ACT_H_SWISH) {
        float t = x + 3;
        t = t > 0.f ? t : 0.f;
        t = t > 6.f ? 6.f : t;
        return x * t * (1.f / 6.f);
    }
    return x;
}

/* compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113: the generator composes
 * "dval*scale*flt_scale/dst_scale", evaluated left to right in float, the
 * activation applied to that quotient. */
static inline int8_t requant(int acc, float s_src, float s_flt, float s_dst, int act) {
    float x = (float)acc * s_src * s_flt / s_dst;
    return fp32_to_int8(apply_act(act, x));
}

static int out_extent(int in, int k, int s, int p, int d) {
    return (in + 2 * p - d * (k - 1) - 1) / s + 1;
}

/* int32 accumulators (bias already added) of the quantised convolution.
 * Follows the loop nest of BareMetal/ConvKernel.cpp:305-344 and the bias add of
 * :374-382; out-of-range taps are skipped (:314-319). acc is [N][OC][OH][OW]. */
void oracle_conv_qs8_acc(
        const int8_t* src, const int8_t* flt, const int32_t* bias, int32_t* acc, int n,
        int ic, int ih, int iw, int oc, int kh, int kw, int sh, int sw, int ph, int pw,
        int dh, int dw, int groups) {
    const int oh = out_extent(ih, kh, sh, ph, dh), ow = out_extent(iw, kw, sw, pw, dw);
    const int icpg = ic / groups, ocpg = oc / groups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b) {
        for (int o = 0; o < oc; ++o) {
            const int g = o / ocpg;
            int32_t* a = acc + ((size_t)b * oc + o) * oh * ow;
            const int32_t b0 = bias ? bias[o] : 0;
            for (int i = 0; i < oh * ow; ++i)
                a[i] = 0;
            for (int c = 0; c < icpg; ++c) {
                const int8_t* s = src + ((size_t)b * ic + g * icpg + c) * ih * iw;
                const int8_t* f = flt + ((size_t)o * icpg + c) * kh * kw;
                for (int fy = 0; fy < kh; ++fy) {
                    for (int fx = 0; fx < kw; ++fx) {
                        const int w = f[fy * kw + fx];
                        for (int y = 0; y < oh; ++y) {
                            const int iy = y * sh + fy * dh - ph;
                            if (iy < 0 || iy >= ih)
                                continue;
                            /* valid x range: 0 <= x*sw + fx*dw - pw < iw */
                            int x0 = 0, off = fx * dw - pw;
                            if (off < 0)
                                x0 = (-off + sw - 1) / sw;
                            int x1 = ow;
                            if (iw - 1 - off < 0)
                                x1 = 0;
                            else if (off + (ow - 1) * sw >= iw)
                                x1 = (iw - 1 - off) / sw + 1;
                            const int8_t* srow = s + (size_t)iy * iw + off;
                            int32_t* arow = a + (size_t)y * ow;
                            if (sw == 1) {
                                for (int x = x0; x < x1; ++x)
                                    arow[x] += (int)srow[x] * w;
                            } else {
                                for (int x = x0; x < x1; ++x)
                                    arow[x] += (int)srow[x * sw] * w;
                            }
                        }
                    }
                }
            }
            for (int i = 0; i < oh * ow; ++i)
                a[i] += b0;
        }
    }
}

/* Full ConvBias: accumulate, add bias, requantise, activate, store int8 NCHW.
 * flt_scales: per-tensor scale when per_channel==0 (the only form the reference
 * can express, runtime/src/data_struct.h:12-20), else one scale per output
 * channel (an extension; same formula with flt_scale[oc]). acc_out may be NULL. */
int oracle_conv_bias_qs8(
        const int8_t* src, const int8_t* flt, const int32_t* bias, int8_t* dst,
        int32_t* acc_out, int n, int ic, int ih, int iw, int oc, int kh, int kw, int sh,
        int sw, int ph, int pw, int dh, int dw, int groups, float s_src,
        const float* flt_scales, int per_channel, float s_dst, int act) {
    const int oh = out_extent(ih, kh, sh, ph, dh), ow = out_extent(iw, kw, sw, pw, dw);
    const size_t total = (size_t)n * oc * oh * ow;
    int32_t* acc = acc_out ? acc_out : (int32_t*)malloc(total * sizeof(int32_t));
    if (!acc)
        return 1;
    oracle_conv_qs8_acc(
            src, flt, bias, acc, n, ic, ih, iw, oc, kh, kw, sh, sw, ph, pw, dh, dw,
            groups);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)total; ++i) {
        const int o = (int)((i / ((long)oh * ow)) % oc);
        const float sf = per_channel ? flt_scales[o] : flt_scales[0];
        dst[i] = requant(acc[i], s_src, sf, s_dst, act);
    }
    if (!acc_out)
        free(acc);
    return 0;
}

/* Pooling on qint8 NCHW. mode 0 MAX, 1 AVERAGE, 2 AVERAGE_COUNT_EXCLUDE_PADDING.
 * compiler/lib/KernelGen/BareMetal/Pooling.cpp:89-95 (init -128), :118-146
 * (average = roundf((float)sum / count), assigned to an int then to int8),
 * :222-243 (padding taps skipped). */
void oracle_pooling_qs8(
        const int8_t* src, int8_t* dst, int mode, int n, int c, int ih, int iw, int wh,
        int ww, int sh, int sw, int ph, int pw) {
    const int oh = (ih + 2 * ph - wh) / sh + 1, ow = (iw + 2 * pw - ww) / sw + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b) {
        for (int ch = 0; ch < c; ++ch) {
            const int8_t* s = src + ((size_t)b * c + ch) * ih * iw;
            int8_t* d = dst + ((size_t)b * c + ch) * oh * ow;
            for (int y = 0; y < oh; ++y) {
                for (int x = 0; x < ow; ++x) {
                    int8_t mx = -128;
                    int sum = 0, count = 0;
                    for (int fy = 0; fy < wh; ++fy) {
                        for (int fx = 0; fx < ww; ++fx) {
                            const int iy = y * sh + fy - ph, ix = x * sw + fx - pw;
                            if (iy < 0 || iy >= ih || ix < 0 || ix >= iw)
                                continue;
                            const int8_t v = s[(size_t)iy * iw + ix];
                            mx = v > mx ? v : mx;
                            sum += v;
                            ++count;
                        }
                    }
                    if (mode == 0) {
                        d[(size_t)y * ow + x] = mx;
                    } else {
                        int r;
                        if (mode == 1)
                            r = (int)roundf((float)sum / (float)(wh * ww));
                        else
                            r = (int)roundf((float)sum / (float)count);
                        d[(size_t)y * ow + x] = (int8_t)r;
                    }
                }
            }
        }
    }
}

/* Quantised elementwise. mode 0 QADD, 1 QFUSE_ADD_RELU, 2 QMUL, 3 QRELU (b unused).
 * compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp:26-56 (formulas),
 * :158-159 (scale_div = 1.f/scale_dst; scale_mul = s0*s1*scale_div).
 * bcast 0: same shape; 1: b is a single element; 2: b is per-channel [C] over a
 * [N][C][inner] tensor (:183-197). */
void oracle_qelemwise(
        const int8_t* a, const int8_t* b, int8_t* dst, int mode, size_t nr_elem, int bcast,
        int channels, int inner, float s0, float s1, float s_dst) {
    const float scale_div = 1.f / s_dst;
    const float scale_mul = s0 * s1 * scale_div;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)nr_elem; ++i) {
        const int v0 = a[i];
        int v1 = 0;
        if (mode != 3) {
            if (bcast == 0)
                v1 = b[i];
            else if (bcast == 1)
                v1 = b[0];
            else
                v1 = b[(i / inner) % channels];
        }
        int8_t out;
        if (mode == 0) {
            out = fp32_to_int8((s0 * v0 + s1 * v1) * scale_div);
        } else if (mode == 1) {
            float val0 = s0 * v0;
            float val1 = s1 * v1;
            out = fp32_to_int8(((val0 + val1) > 0 ? (val0 + val1) : 0) * scale_div);
        } else if (mode == 2) {
            out = fp32_to_int8(v0 * v1 * scale_mul);
        } else {
            out = fp32_to_int8(((s0 * v0) > 0 ? (s0 * v0) : 0) * scale_div);
        }
        dst[i] = out;
    }
}

/* qsi32 -> qsi8: compiler/lib/KernelGen/BareMetal/Typecvt.cpp:46-53 (saturate with
 * roundf), :91-96 (val * src_scale / dst_scale). */
void oracle_typecvt_qs32_qs8(
        const int32_t* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)nr_elem; ++i) {
        int v = (int)roundf((float)src[i] * s_src / s_dst);
        v = v >= 127 ? 127 : v;
        v = v <= -128 ? -128 : v;
        dst[i] = (int8_t)v;
    }
}

/* int8 x int8 -> int32 GEMM, C[m][n] = sum_k A[m][k] * B[k][n]. The reference has
 * no x86 kernel for it (BareMetal/MatrixMul.cpp:13-23 admits f32/f16 only), so this
 * is the exact integer definition; requantisation reuses the typecvt rule above. */
void oracle_matmul_s8_s32(
        const int8_t* a, const int8_t* b, int32_t* c, int m, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        int32_t* row = c + (size_t)i * n;
        for (int j = 0; j < n; ++j)
            row[j] = 0;
        for (int p = 0; p < k; ++p) {
            const int av = a[(size_t)i * k + p];
            const int8_t* brow = b + (size_t)p * n;
            for (int j = 0; j < n; ++j)
                row[j] += av * (int)brow[j];
        }
    }
}

/* ==========================================================================================
 * fp32 path. Parity status: pinned within tolerance, not bit for bit: the functions below
 * are compared with the reference's own fp32 kernels (GI im2col ConvBias, GI 4x12 MatrixMul,
 * GI / BareMetal Elemwise, BareMetal Pooling / Resize / Concat) in
 * tests/test_oracle_vs_reference.py at 1e-5 relative; fp32 sums in a different order cannot
 * agree to the last bit. The GPU is then held to 1e-4 relative / 1e-5 absolute against these.
 * ========================================================================================== */
enum { F32_IDENTITY = 0, F32_RELU = 1, F32_H_SWISH = 2, F32_SIGMOID = 3, F32_SILU = 4 };

/* BareMetal/Activation.cpp:9-42 (RELU, H_SWISH, SIGMOID) and
 * BareMetal/ElemwiseKernel.cpp:52-53 (SILU: val / (1 + expf(-val))) */
static inline float act_f32(int act, float x) {
    switch (act) {
        case F32_RELU:
            return x > 0 ? x : 0;
        case F32_H_SWISH: {
            float t = x + 3;
            t = t > 0.f ? t : 0.f;
            t = t > 6.f ? 6.f : t;
            return x * t * (1.f / 6.f);
        }
        case F32_SIGMOID:
            return 1.f / (1.f + expf(-x));
        case F32_SILU:
            return x / (1.f + expf(-x));
        default:
            return x;
    }
}

/* fp32 ConvBias, NCHW / OIHW ([G][OCpg][ICpg][KH][KW] when grouped), then the activation,
 * then an optional tensor z of the output's shape added (the bottleneck shortcut). The sum
 * runs in double and is rounded once: the tightest statement of "the fp32 result" that both
 * the reference's SIMD GEMM order and the GPU's tensor-core order are compared with. */
void oracle_conv_bias_f32(
        const float* src, const float* flt, const float* bias, const float* z, float* dst,
        int n, int ic, int ih, int iw, int oc, int kh, int kw, int sh, int sw, int ph, int pw,
        int groups, int act) {
    const int oh = out_extent(ih, kh, sh, ph, 1), ow = out_extent(iw, kw, sw, pw, 1);
    const int icpg = ic / groups, ocpg = oc / groups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; ++b) {
        for (int o = 0; o < oc; ++o) {
            const int g = o / ocpg;
            double* a = (double*)calloc((size_t)oh * ow, sizeof(double));
            for (int c = 0; c < icpg; ++c) {
                const float* s = src + ((size_t)b * ic + g * icpg + c) * ih * iw;
                const float* f = flt + ((size_t)o * icpg + c) * kh * kw;
                for (int fy = 0; fy < kh; ++fy)
                    for (int fx = 0; fx < kw; ++fx) {
                        const double w = f[fy * kw + fx];
                        for (int y = 0; y < oh; ++y) {
                            const int iy = y * sh + fy - ph;
                            if (iy < 0 || iy >= ih)
                                continue;
                            for (int x = 0; x < ow; ++x) {
                                const int ix = x * sw + fx - pw;
                                if (ix < 0 || ix >= iw)
                                    continue;
                                a[(size_t)y * ow + x] += (double)s[(size_t)iy * iw + ix] * w;
                            }
                        }
                    }
            }
            float* d = dst + ((size_t)b * oc + o) * oh * ow;
            const float* zz = z ? z + ((size_t)b * oc + o) * oh * ow : NULL;
            for (int i = 0; i < oh * ow; ++i) {
                float r = act_f32(act, (float)(a[i] + (bias ? (double)bias[o] : 0.0)));
                if (zz)
                    r += zz[i];
                d[i] = r;
            }
            free(a);
        }
    }
}

/* C[M][N] = A[M][K] * B[K][N], row-major; double sum, one rounding */
void oracle_matmul_f32(const float* a, const float* b, float* c, int m, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        double* row = (double*)calloc((size_t)n, sizeof(double));
        for (int kk = 0; kk < k; ++kk) {
            const double av = a[(size_t)i * k + kk];
            const float* br = b + (size_t)kk * n;
            for (int j = 0; j < n; ++j)
                row[j] += av * (double)br[j];
        }
        for (int j = 0; j < n; ++j)
            c[(size_t)i * n + j] = (float)row[j];
        free(row);
    }
}

/* Elemwise modes of BareMetal/ElemwiseKernel.cpp:20-120 (codes as in include/megcc_b200.h) */
void oracle_elemwise_f32(int mode, const float* a, const float* b, float* dst, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float x = a[i];
        float r;
        switch (mode) {
            case 0: r = x > 0 ? x : 0; break;
            case 1: r = 1.f / (1.f + expf(-x)); break;
            case 2: r = x / (1.f + expf(-x)); break;
            case 3: r = act_f32(F32_H_SWISH, x); break;
            case 4: r = expf(x); break;
            case 16: r = x + b[i]; break;
            case 17: r = x - b[i]; break;
            case 18: r = x * b[i]; break;
            case 19: r = x > b[i] ? x : b[i]; break;
            case 20: r = x + b[i]; r = r > 0 ? r : 0; break;
            default: r = x; break;
        }
        dst[i] = r;
    }
}

/* fp32 pooling, NCHW (BareMetal/Pooling.cpp:66-150,166-273): MAX starts from -FLT_MAX and
 * skips padding; AVERAGE divides by the window, AVERAGE_COUNT_EXCLUDE_PADDING by the taps */
void oracle_pooling_f32(
        const float* src, float* dst, int mode, int n, int c, int ih, int iw, int wh, int ww,
        int sh, int sw, int ph, int pw) {
    const int oh = (ih + 2 * ph - wh) / sh + 1, ow = (iw + 2 * pw - ww) / sw + 1;
#pragma omp parallel for schedule(static)
    for (int bc = 0; bc < n * c; ++bc) {
        const float* s = src + (size_t)bc * ih * iw;
        float* d = dst + (size_t)bc * oh * ow;
        for (int y = 0; y < oh; ++y)
            for (int x = 0; x < ow; ++x) {
                float mx = -3.402823466e38f, sum = 0.f;
                int count = 0;
                for (int fy = 0; fy < wh; ++fy) {
                    const int iy = y * sh + fy - ph;
                    if (iy < 0 || iy >= ih)
                        continue;
                    for (int fx = 0; fx < ww; ++fx) {
                        const int ix = x * sw + fx - pw;
                        if (ix < 0 || ix >= iw)
                            continue;
                        const float v = s[(size_t)iy * iw + ix];
                        mx = v > mx ? v : mx;
                        sum += v;
                        ++count;
                    }
                }
                d[(size_t)y * ow + x] =
                        mode == 0 ? mx : sum / (mode == 1 ? (float)(wh * ww) : (float)count);
            }
    }
}

/* Resize NEAREST, NCHW (compiler/lib/KernelGen/Common/Resize.h:155-156 with
 * scale = (float)out / in as BareMetal/Resize.cpp computes it) */
void oracle_resize_nearest_f32(
        const float* src, float* dst, int n, int c, int ih, int iw, int oh, int ow) {
    const float scale_h = (float)oh / ih, scale_w = (float)ow / iw;
    for (int bc = 0; bc < n * c; ++bc)
        for (int y = 0; y < oh; ++y) {
            int sy = (int)(y / scale_h);
            sy = sy < ih - 1 ? sy : ih - 1;
            for (int x = 0; x < ow; ++x) {
                int sx = (int)(x / scale_w);
                sx = sx < iw - 1 ? sx : iw - 1;
                dst[((size_t)bc * oh + y) * ow + x] = src[((size_t)bc * ih + sy) * iw + sx];
            }
        }
}

/* fp32 <-> qsi8 TypeCvt as the reference's x86 build performs it: the GeneralIntrinsic kernel
 * (compiler/lib/KernelGen/GeneralIntrinsic/Typecvt.cpp:258-267: scale = src_scale / dst_scale
 * with the float side's scale forced to 1, :56-69). Built with the reference's x86 flags (no
 * -msse4.2) its SIMD groups go through the plain round() of immigration/include/gi_int.h
 * :1332-1340, the same rule as the trailing elements (Typecvt.cpp:176-183). */
void oracle_typecvt_f32_qs8(
        const float* src, int8_t* dst, size_t nr_elem, float s_src, float s_dst) {
    (void)s_src;
    const float scale = 1.f / s_dst;
    for (size_t i = 0; i < nr_elem; ++i) {
        float r = roundf(src[i] * scale);
        r = r >= 127.f ? 127.f : r;
        r = r <= -128.f ? -128.f : r;
        dst[i] = (int8_t)(int)r;
    }
}

void oracle_typecvt_qs8_f32(
        const int8_t* src, float* dst, size_t nr_elem, float s_src, float s_dst) {
    (void)s_dst;
    const float scale = s_src / 1.f;
    for (size_t i = 0; i < nr_elem; ++i)
        dst[i] = (float)src[i] * scale;
}
