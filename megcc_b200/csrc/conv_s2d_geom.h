// Geometry of the space-to-depth form of a stride-2, <= 4 input channel convolution.
// Plain C++ shared by the CUDA side (conv_s2d.cu) and the compile side (workspace sizing in
// the CUDA KernelGen pack), so both always agree on when the path applies and how much
// scratch it needs.
#pragma once
#include <stddef.h>

namespace mb200 {

struct S2dGeom {
    bool ok;               // the path applies
    int a_min_h, a_min_w;  // first tap of the transformed filter, in half-resolution pixels
    int kh2, kw2;          // transformed filter extent (padded so that kh2*kw2 % 4 == 0)
    int h2, w2;            // half-resolution input extent
    size_t filter_bytes;   // [OC][kh2][kw2][16]
    size_t workspace_bytes;  // [N][h2][w2][16], rounded up to 256
};

inline int s2d_floor_div(int a, int b) {
    int q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0)))
        --q;
    return q;
}

inline S2dGeom s2d_geometry(
        int n, int ic, int ih, int iw, int oc, int kh, int kw, int sh, int sw, int ph, int pw,
        int dh, int dw, int groups) {
    S2dGeom g{};
    g.a_min_h = s2d_floor_div(-ph, 2);
    g.a_min_w = s2d_floor_div(-pw, 2);
    g.kh2 = s2d_floor_div(kh - 1 - ph, 2) - g.a_min_h + 1;
    g.kw2 = s2d_floor_div(kw - 1 - pw, 2) - g.a_min_w + 1;
    if (g.kw2 % 2)
        ++g.kw2;
    if ((g.kh2 * g.kw2) % 4)
        ++g.kh2;
    g.h2 = (ih + 1) / 2;
    g.w2 = (iw + 1) / 2;
    g.filter_bytes = (size_t)oc * g.kh2 * g.kw2 * 16;
    const size_t raw = (size_t)n * g.h2 * g.w2 * 16;
    g.workspace_bytes = (raw + 255) / 256 * 256;
    g.ok = groups == 1 && sh == 2 && sw == 2 && dh == 1 && dw == 1 && ic * 4 <= 16 &&
           kh <= 15 && kw <= 15 && ph <= 15 && pw <= 15 &&
           // TMA im2col maps of very small tensors are mis-encoded by the driver
           raw >= 131072;
    return g;
}

// May the MAX pooling 3x3 / stride 2 / pad 1 that follows such a ConvBias be folded into it?
// (64 output channels at most, in whole 16-channel groups: the pooled epilogue of the
// halo-patch kernel works on one 64-column accumulator tile.) The activation must be
// IDENTITY or RELU and the scales positive; the callers check those.
inline bool s2d_pool_fusable(const S2dGeom& g, int oc) {
    return g.ok && oc <= 64 && oc % 16 == 0 && g.kh2 <= 8 && g.kw2 <= 8;
}

}  // namespace mb200
