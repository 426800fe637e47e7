// Bandwidth-bound fp32 operators of the detector configuration, all over NHWC tensors
// (channels innermost), 16 bytes per thread where the shapes allow:
//   elementwise   SILU / SIGMOID / RELU / H_SWISH / EXP, ADD / SUB / MUL / MAX / FUSE_ADD_RELU
//                 (compiler/lib/KernelGen/BareMetal/ElemwiseKernel.cpp:20-120)
//   concat        along channels (BareMetal/Concat.cpp:23-78: a strided copy per input)
//   resize        NEAREST (compiler/lib/KernelGen/Common/Resize.h:155-156)
//   pooling       MAX / AVERAGE with any window (BareMetal/Pooling.cpp:66-150,166-273)
//   focus         the stem's four stride-2 slices concatenated along channels: the reference
//                 expresses it as four Subtensor views (zero-copy MemForward,
//                 runtime/src/vm/memforward.c:41-51) feeding a Concat
//   transpose     model-boundary NCHW <-> NHWC
#include "f32_internal.h"
#include "pdl.h"
#include "umma_ptx.cuh"

namespace mb200 {

namespace {

int grid_for_f32(size_t work, int block) {
    size_t g = (work + block - 1) / block;
    const size_t most = (size_t)umma::sm_count() * 16;
    if (g > most)
        g = most;
    return g < 1 ? 1 : (int)g;
}

__device__ __forceinline__ float unary_f32(int mode, float x) {
    switch (mode) {
        case MB200_ELEM_RELU:
            return x > 0.f ? x : 0.f;
        case MB200_ELEM_SIGMOID:
            return 1.f / (1.f + expf(-x));
        case MB200_ELEM_SILU:
            return x / (1.f + expf(-x));
        case MB200_ELEM_EXP:
            return expf(x);
        case MB200_ELEM_H_SWISH: {
            float t = x + 3.f;
            t = t > 0.f ? t : 0.f;
            t = t > 6.f ? 6.f : t;
            return x * t / 6.f;
        }
        default:
            return x;
    }
}

__device__ __forceinline__ float binary_f32(int mode, float x, float y) {
    switch (mode) {
        case MB200_ELEM_ADD:
            return x + y;
        case MB200_ELEM_SUB:
            return x - y;
        case MB200_ELEM_MUL:
            return x * y;
        case MB200_ELEM_MAX:
            return x > y ? x : y;
        case MB200_ELEM_FUSE_ADD_RELU: {
            const float s = x + y;
            return s > 0.f ? s : 0.f;
        }
        default:
            return x;
    }
}

__global__ void __launch_bounds__(256) elemwise_f32_kernel(
        int mode, const float* __restrict__ a, const float* __restrict__ b,
        float* __restrict__ dst, size_t nr_elem, int vec_ok) {
    pdl_start();
    const bool binary = mode >= MB200_ELEM_ADD;
    const size_t vecs = vec_ok ? nr_elem / 4 : 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < vecs;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(a) + i);
        float4 r;
        if (binary) {
            const float4 y = __ldg(reinterpret_cast<const float4*>(b) + i);
            r.x = binary_f32(mode, x.x, y.x);
            r.y = binary_f32(mode, x.y, y.y);
            r.z = binary_f32(mode, x.z, y.z);
            r.w = binary_f32(mode, x.w, y.w);
        } else {
            r.x = unary_f32(mode, x.x);
            r.y = unary_f32(mode, x.y);
            r.z = unary_f32(mode, x.z);
            r.w = unary_f32(mode, x.w);
        }
        reinterpret_cast<float4*>(dst)[i] = r;
    }
    // tail (or everything, when a pointer is not 16-byte aligned)
    for (size_t i = vecs * 4 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nr_elem;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = binary ? binary_f32(mode, a[i], b[i]) : unary_f32(mode, a[i]);
}

constexpr int kMaxConcat = 8;
struct ConcatArgs {
    const float* src[kMaxConcat];
    int channels[kMaxConcat];
    int offset[kMaxConcat];  // first output channel of input i
    int nr, c_out, vec;
};

// one thread per (pixel, 4 output channels) when every channel count is a multiple of 4
__global__ void __launch_bounds__(256) concat_f32_kernel(ConcatArgs a, float* __restrict__ dst,
                                                         size_t pixels) {
    pdl_start();
    const int step = a.vec ? 4 : 1;
    const int per_pixel = a.c_out / step;
    const size_t total = pixels * (size_t)per_pixel;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t px = idx / per_pixel;
        const int ch = (int)(idx - px * per_pixel) * step;
        int k = 0;
#pragma unroll
        for (int i = 1; i < kMaxConcat; ++i)
            if (i < a.nr && ch >= a.offset[i])
                k = i;
        const float* s = a.src[k] + px * (size_t)a.channels[k] + (ch - a.offset[k]);
        float* d = dst + px * (size_t)a.c_out + ch;
        if (a.vec)
            *reinterpret_cast<float4*>(d) = __ldg(reinterpret_cast<const float4*>(s));
        else
            *d = *s;
    }
}

__global__ void __launch_bounds__(256) resize_nearest_f32_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int n, int c, int ih, int iw,
        int oh, int ow, float scale_h, float scale_w, int vec) {
    pdl_start();
    const int step = vec ? 4 : 1;
    const int cv = c / step;
    const size_t total = (size_t)n * oh * ow * cv;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ch = (int)(idx % cv) * step;
        size_t t = idx / cv;
        const int x = (int)(t % ow);
        t /= ow;
        const int y = (int)(t % oh);
        const int b = (int)(t / oh);
        // ih = min((int)(oh / scale_h), IH - 1) with scale = out / in, computed in float
        // as the reference's generated C does
        int sy = (int)((float)y / scale_h);
        int sx = (int)((float)x / scale_w);
        sy = sy < ih - 1 ? sy : ih - 1;
        sx = sx < iw - 1 ? sx : iw - 1;
        const float* s = src + (((size_t)b * ih + sy) * iw + sx) * c + ch;
        float* d = dst + (((size_t)b * oh + y) * ow + x) * c + ch;
        if (vec)
            *reinterpret_cast<float4*>(d) = __ldg(reinterpret_cast<const float4*>(s));
        else
            *d = *s;
    }
}

// mode 0 MAX, 1 AVERAGE (divide by the window), 2 AVERAGE_COUNT_EXCLUDE_PADDING
__global__ void __launch_bounds__(256) pooling_f32_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int mode, int n, int c, int ih,
        int iw, int oh, int ow, int wh, int ww, int sh, int sw, int ph, int pw, int vec) {
    pdl_start();
    const int step = vec ? 4 : 1;
    const int cv = c / step;
    const size_t total = (size_t)n * oh * ow * cv;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ch = (int)(idx % cv) * step;
        size_t t = idx / cv;
        const int x = (int)(t % ow);
        t /= ow;
        const int y = (int)(t % oh);
        const int b = (int)(t / oh);
        float4 acc = mode == 0 ? make_float4(-3.402823466e38f, -3.402823466e38f, -3.402823466e38f,
                                             -3.402823466e38f)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
        int count = 0;
        for (int fy = 0; fy < wh; ++fy) {
            const int iy = y * sh + fy - ph;
            if ((unsigned)iy >= (unsigned)ih)
                continue;
            for (int fx = 0; fx < ww; ++fx) {
                const int ix = x * sw + fx - pw;
                if ((unsigned)ix >= (unsigned)iw)
                    continue;
                const float* s = src + (((size_t)b * ih + iy) * iw + ix) * c + ch;
                float4 v;
                if (vec)
                    v = __ldg(reinterpret_cast<const float4*>(s));
                else
                    v = make_float4(*s, 0.f, 0.f, 0.f);
                if (mode == 0) {
                    acc.x = fmaxf(acc.x, v.x); acc.y = fmaxf(acc.y, v.y);
                    acc.z = fmaxf(acc.z, v.z); acc.w = fmaxf(acc.w, v.w);
                } else {
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                ++count;
            }
        }
        if (mode != 0) {
            const float d = mode == 1 ? (float)(wh * ww) : (float)count;
            acc.x /= d; acc.y /= d; acc.z /= d; acc.w /= d;
        }
        float* o = dst + (((size_t)b * oh + y) * ow + x) * c + ch;
        if (vec)
            *reinterpret_cast<float4*>(o) = acc;
        else
            *o = acc.x;
    }
}

// Focus: out[b][y][x][k * C + ch] = in[b][ch][2y + dy_k][2x + dx_k] with the slice order
// (dy, dx) = (0,0), (1,0), (0,1), (1,1); output channels beyond 4 * C are written as zeros so
// that the 16-channel rows the first ConvBias loads hold no stale data. One thread per
// output pixel.
__global__ void __launch_bounds__(256) focus_f32_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int n, int c, int h, int w,
        int c_out) {
    pdl_start();
    const int h2 = h / 2, w2 = w / 2;
    const size_t total = (size_t)n * h2 * w2;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int x = (int)(idx % w2);
        size_t t = idx / w2;
        const int y = (int)(t % h2);
        const int b = (int)(t / h2);
        float* o = dst + idx * c_out;
        for (int k = 0; k < 4; ++k) {
            const int dy = k & 1, dx = k >> 1;
            for (int ch = 0; ch < c; ++ch)
                o[k * c + ch] =
                        __ldg(src + (((size_t)b * c + ch) * h + 2 * y + dy) * w + 2 * x + dx);
        }
        for (int ch = 4 * c; ch < c_out; ++ch)
            o[ch] = 0.f;
    }
}

__global__ void __launch_bounds__(256) transpose_f32_kernel(
        const float* __restrict__ src, float* __restrict__ dst, int rows, int cols) {
    pdl_start();
    __shared__ float tile[32][33];
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

}  // namespace

int launch_elemwise_f32(
        int mode, const float* a, const float* b, float* dst, size_t nr_elem, cudaStream_t st) {
    const int vec_ok = ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)dst) & 15) == 0) ? 1 : 0;
    launch_pdl(elemwise_f32_kernel, dim3(grid_for_f32(nr_elem / 4 + 1, 256)), dim3(256), 0, st, mode,
               a, b, dst, nr_elem, vec_ok);
    return check_launch("elemwise_f32");
}

int launch_concat_f32(
        const float* const* srcs, const int* channels, int nr, float* dst, size_t pixels,
        cudaStream_t st) {
    if (nr < 1 || nr > kMaxConcat)
        return set_error(ST_OUT_OF_RANGE, "concat takes 1..%d inputs, not %d", kMaxConcat, nr);
    ConcatArgs a;
    a.nr = nr;
    a.c_out = 0;
    a.vec = (((uintptr_t)dst & 15) == 0) ? 1 : 0;
    for (int i = 0; i < kMaxConcat; ++i) {
        a.src[i] = i < nr ? srcs[i] : nullptr;
        a.channels[i] = i < nr ? channels[i] : 0;
        a.offset[i] = a.c_out;
        if (i < nr) {
            if (channels[i] <= 0 || !srcs[i])
                return set_error(ST_INVALID_LAYOUT, "concat input %d is empty", i);
            a.c_out += channels[i];
            if ((channels[i] & 3) || ((uintptr_t)srcs[i] & 15))
                a.vec = 0;
        }
    }
    const size_t work = pixels * (size_t)(a.c_out / (a.vec ? 4 : 1));
    launch_pdl(concat_f32_kernel, dim3(grid_for_f32(work, 256)), dim3(256), 0, st, a, dst, pixels);
    return check_launch("concat_f32");
}

int launch_resize_nearest_f32(
        const float* src, float* dst, int n, int c, int ih, int iw, int oh, int ow,
        cudaStream_t st) {
    const int vec = (c % 4 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0)) ? 1 : 0;
    // scale = (float)out / in, the reference's own float expression
    const float scale_h = (float)oh / ih, scale_w = (float)ow / iw;
    const size_t work = (size_t)n * oh * ow * (c / (vec ? 4 : 1));
    launch_pdl(resize_nearest_f32_kernel, dim3(grid_for_f32(work, 256)), dim3(256), 0, st, src, dst,
               n, c, ih, iw, oh, ow, scale_h, scale_w, vec);
    return check_launch("resize_nearest_f32");
}

int launch_pooling_f32(
        const float* src, float* dst, int mode, int n, int c, int ih, int iw, int wh, int ww,
        int sh, int sw, int ph, int pw, cudaStream_t st) {
    const int oh = (ih + 2 * ph - wh) / sh + 1, ow = (iw + 2 * pw - ww) / sw + 1;
    const int vec = (c % 4 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0)) ? 1 : 0;
    const size_t work = (size_t)n * oh * ow * (c / (vec ? 4 : 1));
    launch_pdl(pooling_f32_kernel, dim3(grid_for_f32(work, 256)), dim3(256), 0, st, src, dst, mode, n,
               c, ih, iw, oh, ow, wh, ww, sh, sw, ph, pw, vec);
    return check_launch("pooling_f32");
}

int launch_focus_f32(
        const float* src_nchw, float* dst_nhwc, int n, int c, int h, int w, int c_out,
        cudaStream_t st) {
    const size_t work = (size_t)n * (h / 2) * (w / 2);
    launch_pdl(focus_f32_kernel, dim3(grid_for_f32(work, 256)), dim3(256), 0, st, src_nchw, dst_nhwc,
               n, c, h, w, c_out);
    return check_launch("focus_f32");
}

int launch_transpose_f32(
        const float* src, float* dst, int batch, int rows, int cols, cudaStream_t st) {
    if (batch <= 0 || rows <= 0 || cols <= 0)
        return 0;
    if (batch > 65535)
        return set_error(ST_OUT_OF_RANGE, "transpose: batch %d exceeds the grid z limit", batch);
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
    launch_pdl(transpose_f32_kernel, grid, block, 0, st, src, dst, rows, cols);
    return check_launch("transpose_f32");
}

}  // namespace mb200
