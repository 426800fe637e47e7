// Stride-2 ConvBias with at most 4 input channels (the first layer of an image network) on
// the tensor cores.
//
// Three input channels cannot feed a TMA row (16 bytes minimum) or a K=32 MMA step, so the
// input goes through a 2x2 space-to-depth step first: pixel (y, x) channel c of the
// [N, C, H, W] input becomes channel (dy*2+dx)*C + c of pixel (y/2, x/2) in an
// [N, H/2, W/2, 16] int8 tensor (unused channels zero). A k x k stride-2 filter becomes a
// ceil-sized stride-1 filter over those 16-channel pixels (7x7 -> 4x4, 3x3 -> 2x2), its
// weights placed accordingly and zero elsewhere; integer sums are unchanged by the added
// zero products, so the accumulators are exactly those of the direct convolution
// (compiler/lib/KernelGen/BareMetal/ConvKernel.cpp:305-344). The transformed convolution
// runs on the TAP16 geometry of conv_umma.cu. The space-to-depth tensor is scratch memory
// the caller provides (the Opr workspace).
#include "conv_s2d_geom.h"
#include "internal.h"
#include "pdl.h"

namespace mb200 {

namespace {

S2dGeom s2d_geom(const ConvArgs& a) {
    return s2d_geometry(a.n, a.ic, a.ih, a.iw, a.oc, a.kh, a.kw, a.sh, a.sw, a.ph, a.pw, a.dh,
                        a.dw, a.groups);
}

// one thread per half-resolution pixel: gathers 2x2xC bytes, writes one 16-byte vector
__global__ void __launch_bounds__(256) space_to_depth_kernel(
        const int8_t* __restrict__ src, uint4* __restrict__ dst, int n, int c, int h, int w,
        int h2, int w2, long long sn, long long sc, long long sy, long long sx) {
    pdl_start();
    const size_t total = (size_t)n * h2 * w2;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int x2 = (int)(idx % w2);
        size_t t = idx / w2;
        const int y2 = (int)(t % h2);
        const int b = (int)(t / h2);
        uint32_t words[4] = {0, 0, 0, 0};
        for (int dy = 0; dy < 2; ++dy) {
            const int y = 2 * y2 + dy;
            if (y >= h)
                continue;
            for (int dx = 0; dx < 2; ++dx) {
                const int x = 2 * x2 + dx;
                if (x >= w)
                    continue;
                for (int ch = 0; ch < c; ++ch) {
                    const int slot = (dy * 2 + dx) * c + ch;
                    const uint32_t v = (uint8_t)src[b * sn + ch * sc + y * sy + x * sx];
                    words[slot >> 2] |= v << (8 * (slot & 3));
                }
            }
        }
        dst[idx] = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

// The same for an NCHW source with an even width and an even base address: one thread per
// half-resolution pixel again, but the two horizontally adjacent bytes of a channel row come
// in one 16-bit load, so a warp's loads are contiguous 64-byte runs and its stores one
// contiguous 512 bytes. 32-bit index arithmetic.
__global__ void __launch_bounds__(256) space_to_depth_nchw2_kernel(
        const int8_t* __restrict__ src, uint4* __restrict__ dst, int n, int c, int h, int w,
        int h2, int w2) {
    pdl_start();
    const unsigned total = (unsigned)n * h2 * w2;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const int x2 = (int)(idx % w2);
        unsigned t = idx / w2;
        const int y2 = (int)(t % h2);
        const int b = (int)(t / h2);
        uint32_t pair[2][4];  // [dy][ch]: bytes (x, x+1) of one channel row
#pragma unroll
        for (int dy = 0; dy < 2; ++dy) {
            const int y = 2 * y2 + dy;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                pair[dy][ch] = 0;
                if (ch < c && y < h)
                    pair[dy][ch] = __ldg(reinterpret_cast<const unsigned short*>(
                            src + (((size_t)b * c + ch) * h + y) * w + 2 * x2));
            }
        }
        uint32_t words[4] = {0, 0, 0, 0};
#pragma unroll
        for (int dy = 0; dy < 2; ++dy) {
#pragma unroll
            for (int dx = 0; dx < 2; ++dx) {
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    if (ch < c) {
                        const uint32_t v = (pair[dy][ch] >> (8 * dx)) & 0xffu;
                        const int slot = (dy * 2 + dx) * c + ch;
                        words[slot >> 2] |= v << (8 * (slot & 3));
                    }
                }
            }
        }
        dst[idx] = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

// Three channels, NCHW, width a multiple of 8, 8-byte aligned base: one thread makes FOUR
// adjacent half-resolution pixels from six 8-byte loads (two source rows of three channel
// planes) and writes 64 contiguous bytes. The twelve bytes of a pixel are put in place by
// seven byte permutes instead of a shift, a mask and an OR each: the general kernels above
// execute some 380 instructions per pixel and are bound by instruction issue (measured: 46 us
// for a 256 x 3 x 224 x 224 input, 80 % issue-active, 12 % of the DRAM bandwidth).
// Slot order: (dy*2 + dx)*3 + ch, so word 0 = [c0 c1 c2 | c0'] of the upper row's left and
// right byte, word 1 = [c1' c2' | lower row c0 c1], word 2 = [c2 | c0' c1' c2'], word 3 = 0.
__global__ void __launch_bounds__(256) space_to_depth_nchw3_x4_kernel(
        const int8_t* __restrict__ src, uint4* __restrict__ dst, int n, int h, int w, int h2) {
    pdl_start();
    const unsigned w8 = (unsigned)w / 8;  // groups of four half-resolution pixels per row
    const unsigned total = (unsigned)n * h2 * w8;
    const size_t plane = (size_t)h * w;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const unsigned xg = idx % w8;
        const unsigned t = idx / w8;
        const unsigned y2 = t % h2, b = t / h2;
        const int8_t* row = src + ((size_t)b * 3 * h + 2 * y2) * w + 8 * xg;
        uint2 r[2][3];
#pragma unroll
        for (int dy = 0; dy < 2; ++dy) {
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                r[dy][ch] = make_uint2(0, 0);
                if ((int)(2 * y2) + dy < h)
                    r[dy][ch] = __ldg(reinterpret_cast<const uint2*>(row + ch * plane + (size_t)dy * w));
            }
        }
        uint4* out = dst + (size_t)idx * 4;  // half-resolution pixels are w/2 = 4*w8 per row
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            // source bytes 2p (left) and 2p + 1 (right) of every row: byte o / o + 1 of a word
            constexpr unsigned kFromY = 4;
            const unsigned o = (unsigned)(p & 1) * 2;
            const uint32_t a0 = p < 2 ? r[0][0].x : r[0][0].y, a1 = p < 2 ? r[0][1].x : r[0][1].y,
                           a2 = p < 2 ? r[0][2].x : r[0][2].y;
            const uint32_t b0 = p < 2 ? r[1][0].x : r[1][0].y, b1 = p < 2 ? r[1][1].x : r[1][1].y,
                           b2 = p < 2 ? r[1][2].x : r[1][2].y;
            const uint32_t t0 = __byte_perm(a0, a1, o | (kFromY + o) << 4 | (o + 1) << 12);
            const uint32_t w0 = __byte_perm(t0, a2, 0x3010u | (kFromY + o) << 8);
            const uint32_t t1 = __byte_perm(a1, a2, (o + 1) | (kFromY + o + 1) << 4);
            const uint32_t t2 = __byte_perm(b0, b1, o | (kFromY + o) << 4);
            const uint32_t w1 = __byte_perm(t1, t2, 0x5410u);
            const uint32_t t3 = __byte_perm(b2, b0, o | (kFromY + o + 1) << 4 | (o + 1) << 12);
            const uint32_t w2 = __byte_perm(t3, b1, 0x3010u | (kFromY + o + 1) << 8);
            out[p] = make_uint4(w0, w1, w2, 0u);
        }
    }
}

// OIHW -> [OC][kh2][kw2][16]
__global__ void __launch_bounds__(256) s2d_pack_filter_kernel(
        const int8_t* __restrict__ src, int8_t* __restrict__ dst, int oc, int ic, int kh, int kw,
        int ph, int pw, int a_min_h, int a_min_w, int kh2, int kw2) {
    const size_t total = (size_t)oc * kh2 * kw2 * 16;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int slot = (int)(idx % 16);
        size_t t = idx / 16;
        const int tb = (int)(t % kw2);
        t /= kw2;
        const int ta = (int)(t % kh2);
        const int o = (int)(t / kh2);
        int8_t v = 0;
        if (slot < 4 * ic) {
            const int ch = slot % ic, d = slot / ic;
            const int dy = d >> 1, dx = d & 1;
            const int fy = 2 * (ta + a_min_h) + dy + ph, fx = 2 * (tb + a_min_w) + dx + pw;
            if (fy >= 0 && fy < kh && fx >= 0 && fx < kw)
                v = src[(((size_t)o * ic + ch) * kh + fy) * kw + fx];
        }
        dst[idx] = v;
    }
}

int grid_for(size_t work) {
    size_t g = (work + 255) / 256;
    const size_t cap = (size_t)148 * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

int launch_conv_umma_geom(
        const ConvArgs& a, int geom, const int8_t* src, const int8_t* flt, const int32_t* bias,
        const float* flt_scales, int8_t* dst, cudaStream_t st);

bool conv_s2d_supported(const ConvArgs& a) {
    return s2d_geom(a).ok;
}

bool conv_s2d_pool_supported(const ConvArgs& a) {
    return s2d_pool_fusable(s2d_geom(a), a.oc) && a.act != ACT_H_SWISH && !a.z && !a.acc_out &&
           a.s_src > 0.f && a.s_flt > 0.f && a.s_dst > 0.f;
}

size_t conv_s2d_filter_bytes(const ConvArgs& a) {
    return s2d_geom(a).filter_bytes;
}

size_t conv_s2d_workspace_bytes(const ConvArgs& a) {
    return s2d_geom(a).workspace_bytes;
}

int launch_conv_s2d_pack_filter(
        const ConvArgs& a, const int8_t* flt_oihw, int8_t* out, cudaStream_t st) {
    const S2dGeom g = s2d_geom(a);
    s2d_pack_filter_kernel<<<grid_for(conv_s2d_filter_bytes(a)), 256, 0, st>>>(
            flt_oihw, out, a.oc, a.ic, a.kh, a.kw, a.ph, a.pw, g.a_min_h, g.a_min_w, g.kh2, g.kw2);
    return check_launch("s2d_pack_filter");
}

int launch_conv_s2d(
        const ConvArgs& a, const int8_t* src, const int8_t* flt_s2d, const int32_t* bias,
        const float* flt_scales, int8_t* dst, void* workspace, cudaStream_t st) {
    const S2dGeom g = s2d_geom(a);
    long long sn, sc, sy, sx;
    if (a.src_is_nchw) {
        sx = 1;
        sy = a.iw;
        sc = (long long)a.ih * a.iw;
        sn = sc * a.ic;
    } else {
        sc = 1;
        sx = a.ic;
        sy = (long long)a.iw * a.ic;
        sn = sy * a.ih;
    }
    if (a.src_is_nchw && a.ic == 3 && a.iw % 8 == 0 && ((uintptr_t)src & 7) == 0 &&
        g.w2 == a.iw / 2 && (size_t)a.n * g.h2 * g.w2 < (1u << 31)) {
        launch_pdl(space_to_depth_nchw3_x4_kernel, dim3(grid_for((size_t)a.n * g.h2 * (a.iw / 8))),
                   dim3(256), 0, st, src, (uint4*)workspace, a.n, a.ih, a.iw, g.h2);
    } else if (a.src_is_nchw && a.iw % 2 == 0 && ((uintptr_t)src & 1) == 0 && g.w2 == a.iw / 2 &&
               (size_t)a.n * g.h2 * g.w2 < (1u << 31)) {
        launch_pdl(space_to_depth_nchw2_kernel, dim3(grid_for((size_t)a.n * g.h2 * g.w2)), dim3(256),
                   0, st, src, (uint4*)workspace, a.n, a.ic, a.ih, a.iw, g.h2, g.w2);
    } else {
        launch_pdl(space_to_depth_kernel, dim3(grid_for((size_t)a.n * g.h2 * g.w2)), dim3(256), 0, st,
                   src, (uint4*)workspace, a.n, a.ic, a.ih, a.iw, g.h2, g.w2, sn, sc, sy, sx);
    }
    int rc = check_launch("space_to_depth");
    if (rc)
        return rc;
    ConvArgs t = a;  // the stride-1 convolution over the half-resolution 16-channel tensor
    t.ic = 16;
    t.ih = g.h2;
    t.iw = g.w2;
    t.kh = g.kh2;
    t.kw = g.kw2;
    t.sh = t.sw = 1;
    t.ph = -g.a_min_h;
    t.pw = -g.a_min_w;
    t.src_is_nchw = 0;
    // oh / ow / m stay those of the original convolution
    if (conv_patch_supported(t, (const int8_t*)workspace, flt_s2d, dst))
        return launch_conv_patch(t, (const int8_t*)workspace, flt_s2d, bias, flt_scales, dst, st);
    if (a.pool)  // only the halo-patch kernel has the pooled epilogue
        return set_error(ST_NO_IMPLEMENT, "ConvBias + pooling does not apply to this shape");
    return launch_conv_umma_geom(t, 1, (const int8_t*)workspace, flt_s2d, bias, flt_scales, dst, st);
}

}  // namespace mb200
