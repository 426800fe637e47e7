// Host-side search for a one-FMA requantisation that is PROVEN equal to the reference's
// three-step float chain on every int32 accumulator.
//
// The reference computes  q = clamp_s8(roundf(act(((float)acc * s_src) * s_flt / s_dst)))
// (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113): three rounded float operations
// before the activation. The epilogue of the tensor-core kernels is bound by instruction
// issue, and  q' = clamp_s8(trunc(fma((float)acc, c, +-d)))  (RELU applied afterwards) needs
// one. With positive scales and IDENTITY / RELU both are monotonic staircases over the
// integers, so they are the same function if and only if they agree on both sides of every
// step of the reference (and at INT_MIN / INT_MAX). The steps, at most 255, are found by
// bisection on the reference chain; for a candidate multiplier c the offsets d that put
// every step in the right place form an interval that is computed directly, and a float
// from inside it is then CHECKED through the exact device arithmetic (fmaf is correctly
// rounded) on every step edge. Candidates for c are the correctly rounded ratio and its
// neighbours. If nothing passes, the kernel keeps the three-step chain. Verdicts are cached
// per scale triple; the whole search costs well under a millisecond.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "internal.h"
#include "tuning.h"

namespace mb200 {

namespace {

// every operation below is one correctly rounded IEEE single operation, as on the device;
// volatile keeps the compiler from contracting or reassociating them
inline float fmul(float a, float b) {
    volatile float r = a * b;
    return r;
}
inline float fdiv(float a, float b) {
    volatile float r = a / b;
    return r;
}

inline int clamp_s8(float r) {
    // |r| stays far below 2^31 here (the caller has checked the bound)
    int q = (int)r;
    return q < -128 ? -128 : (q > 127 ? 127 : q);
}

inline int reference_chain(int acc, float s_src, float s_flt, float s_dst, bool relu) {
    float x = fdiv(fmul(fmul((float)acc, s_src), s_flt), s_dst);
    if (relu)
        x = x > 0.f ? x : 0.f;
    return clamp_s8(roundf(x));
}

// what the device's fast path computes: ONE fused multiply-add, trunc(fma((float)acc, c, +-d))
// saturated to int8, the offset taking the accumulator's sign (always +d under RELU, which
// is applied afterwards)
// `ops` = 1: f is the converted accumulator; 2: f = RN(acc * s_src) first; 3: also * s_flt
// (the leading operations of the reference chain kept as they are, the rest merged)
inline float fast_operand(long long acc, int ops, float s_src, float s_flt) {
    float f = (float)acc;
    if (ops >= 2)
        f = fmul(f, s_src);
    if (ops >= 3)
        f = fmul(f, s_flt);
    return f;
}

inline int fast_chain(
        long long acc, int ops, float s_src, float s_flt, float c, float d, bool relu) {
    const float f = fast_operand(acc, ops, s_src, s_flt);
    volatile float y = fmaf(f, c, relu ? d : copysignf(d, f));
    float t = truncf(y);
    int q = t < -128.f ? -128 : (t > 127.f ? 127 : (int)t);
    if (relu && q < 0)
        q = 0;
    return q;
}

struct Staircase {
    // up[k-1]: the smallest accumulator whose reference output is >= k (k = 1..n_up);
    // down[k-1]: the largest accumulator whose reference output is <= -k (k = 1..n_down)
    long long up[127], down[128];
    int n_up, n_down;
};

bool search(
        float s_src, float s_flt, float s_dst, bool relu, int ops, float* c_out, float* d_out) {
    if (!(s_src > 0.f) || !(s_flt > 0.f) || !(s_dst > 0.f))
        return false;
    const double ratio = (double)s_src * (double)s_flt / (double)s_dst;
    if (!(ratio > 0.0) || !isfinite(ratio))
        return false;
    if (2147483648.0 * ratio >= 1073741824.0)  // results must stay far inside the int range
        return false;
    const long long lo_acc = -2147483648LL, hi_acc = 2147483647LL;
    auto ref = [&](long long acc) { return reference_chain((int)acc, s_src, s_flt, s_dst, relu); };
    Staircase st;
    st.n_up = st.n_down = 0;
    const int top = ref(hi_acc), bottom = ref(lo_acc);
    for (int k = 1; k <= top && k <= 127; ++k) {
        long long lo = lo_acc, hi = hi_acc;  // ref(hi) >= k holds
        while (lo < hi) {
            const long long mid = lo + (hi - lo) / 2;
            if (ref(mid) >= k)
                hi = mid;
            else
                lo = mid + 1;
        }
        st.up[st.n_up++] = lo;
    }
    for (int k = 1; -k >= bottom && k <= 128; ++k) {
        long long lo = lo_acc, hi = hi_acc;  // ref(lo) <= -k holds
        while (lo < hi) {
            const long long mid = lo + (hi - lo + 1) / 2;
            if (ref(mid) <= -k)
                lo = mid;
            else
                hi = mid - 1;
        }
        st.down[st.n_down++] = lo;
    }
    auto agrees = [&](float c, float d) {
        if (fast_chain(lo_acc, ops, s_src, s_flt, c, d, relu) != bottom || fast_chain(hi_acc, ops, s_src, s_flt, c, d, relu) != top ||
            fast_chain(0, ops, s_src, s_flt, c, d, relu) != ref(0))
            return false;
        for (int i = 0; i < st.n_up; ++i) {
            const long long a = st.up[i];
            if (fast_chain(a, ops, s_src, s_flt, c, d, relu) != ref(a) ||
                (a > lo_acc && fast_chain(a - 1, ops, s_src, s_flt, c, d, relu) != ref(a - 1)))
                return false;
        }
        for (int i = 0; i < st.n_down; ++i) {
            const long long a = st.down[i];
            if (fast_chain(a, ops, s_src, s_flt, c, d, relu) != ref(a) ||
                (a < hi_acc && fast_chain(a + 1, ops, s_src, s_flt, c, d, relu) != ref(a + 1)))
                return false;
        }
        return true;
    };
    // what is left to merge into the multiplier
    const double rest = ops == 1 ? ratio
                        : ops == 2 ? (double)s_flt / (double)s_dst
                                   : 1.0 / (double)s_dst;
    auto operand = [&](long long acc) { return (double)fast_operand(acc, ops, s_src, s_flt); };
    float cands[17];
    cands[0] = (float)rest;
    for (int i = 0; i < 8; ++i) {
        cands[1 + 2 * i] = nextafterf(i ? cands[2 * i - 1] : cands[0], INFINITY);
        cands[2 + 2 * i] = nextafterf(i ? cands[2 * i] : cands[0], 0.f);
    }
    for (float c : cands) {
        if (!(c > 0.f))
            continue;
        // offsets that place every step correctly, in real arithmetic
        double lo_d = 0.0, hi_d = 1.0;
        for (int i = 0; i < st.n_up; ++i) {
            const double k = i + 1;
            lo_d = fmax(lo_d, k - (double)c * operand(st.up[i]));
            hi_d = fmin(hi_d, k - (double)c * operand(st.up[i] - 1));
        }
        for (int i = 0; i < st.n_down; ++i) {
            const double k = i + 1;
            lo_d = fmax(lo_d, k + (double)c * operand(st.down[i]));
            hi_d = fmin(hi_d, k + (double)c * operand(st.down[i] + 1));
        }
        if (!(lo_d < hi_d))
            continue;
        // a few floats from inside the interval, each put through the exact check
        const float mids[5] = {(float)(0.5 * (lo_d + hi_d)), (float)(0.75 * lo_d + 0.25 * hi_d),
                               (float)(0.25 * lo_d + 0.75 * hi_d), 0.49999997f, 0.5f};
        for (float d : mids) {
            if (!(d > 0.f) || !(d < 1.f) || (double)d < lo_d || (double)d > hi_d)
                continue;
            if (agrees(c, d)) {
                *c_out = c;
                *d_out = d;
                return true;
            }
        }
    }
    return false;
}

// the reference's fused ElemwiseMultiType step on one (conv, z) pair
// (compiler/lib/KernelGen/BareMetal/ElemwiseMultiType.cpp:38-46,158)
inline int reference_residual(int q, int z, float s_conv, float s_z, float z_div, bool relu) {
    volatile float t = fmul(s_conv, (float)q) + fmul(s_z, (float)z);
    float tt = t;
    if (relu)
        tt = tt > 0.f ? tt : 0.f;
    return clamp_s8(roundf(fmul(tt, z_div)));
}

inline int fast_residual(int q, int z, float a, float b, bool relu) {
    volatile float y;
    if (relu) {
        volatile float u = fmaf((float)q, a, 0.49999997f);
        y = fmaf((float)z, b, u);
    } else {
        volatile float v = fmaf((float)z, b, fmul((float)q, a));
        y = v + copysignf(0.49999997f, v);
    }
    const float t = truncf(y);
    int r = t < -128.f ? -128 : (t > 127.f ? 127 : (int)t);
    if (relu && r < 0)
        r = 0;
    return r;
}

}  // namespace

// a, b for the short form of the fused residual step (conv_epilogue.cuh fuse_z_fast), equal to
// the reference on all 65536 pairs of int8 values, or false. mode: 1 QADD, 2 QFUSE_ADD_RELU.
bool residual_fast_constants(
        float s_conv, float s_z, float out_scale, int mode, float* a_out, float* b_out) {
    *a_out = *b_out = 0.f;
    if (!tuning().fast_requant || (mode != 1 && mode != 2))
        return false;
    if (!(s_conv > 0.f) || !(s_z > 0.f) || !(out_scale > 0.f))
        return false;
    static std::mutex mu;
    static std::map<std::tuple<uint32_t, uint32_t, uint32_t, int>, std::pair<float, float>> cache;
    auto bits = [](float f) {
        uint32_t u;
        memcpy(&u, &f, 4);
        return u;
    };
    const auto key = std::make_tuple(bits(s_conv), bits(s_z), bits(out_scale), mode);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *a_out = it->second.first;
            *b_out = it->second.second;
            return *a_out != 0.f;
        }
    }
    const float z_div = 1.0f / out_scale;  // the reference's scale_div
    const bool relu = mode == 2;
    auto around = [](double v, float* c) {
        c[0] = (float)v;
        c[1] = nextafterf(c[0], INFINITY);
        c[2] = nextafterf(c[0], 0.f);
        c[3] = nextafterf(c[1], INFINITY);
        c[4] = nextafterf(c[2], 0.f);
    };
    float ca[5], cb[5];
    around((double)s_conv * (double)z_div, ca);
    around((double)s_z * (double)z_div, cb);
    float fa = 0.f, fb = 0.f;
    for (int i = 0; i < 5 && fa == 0.f; ++i) {
        for (int j = 0; j < 5 && fa == 0.f; ++j) {
            bool same = true;
            for (int q = -128; q <= 127 && same; ++q)
                for (int z = -128; z <= 127 && same; ++z)
                    same = reference_residual(q, z, s_conv, s_z, z_div, relu) ==
                           fast_residual(q, z, ca[i], cb[j], relu);
            if (same) {
                fa = ca[i];
                fb = cb[j];
            }
        }
    }
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = std::make_pair(fa, fb);
    *a_out = fa;
    *b_out = fb;
    return fa != 0.f;
}

// The shortest verified form: returns its number of float operations (1: fma(acc, mul, +-add);
// 2: fma(acc * s_src, mul, +-add); 3: fma(acc * s_src * s_flt, mul, +-add)) with mul and add,
// each equal to the reference chain for every int32 accumulator; 0 when none passed, the
// activation is not IDENTITY / RELU, a scale is not positive, or MB200_NO_FAST_REQUANT is set.
int requant_fast_constants(
        float s_src, float s_flt, float s_dst, int act, float* mul_out, float* add_out) {
    *mul_out = *add_out = 0.f;
    if (act != ACT_IDENTITY && act != ACT_RELU)
        return 0;
    if (!tuning().fast_requant)
        return 0;
    struct Verdict {
        int ops;
        float c, d;
    };
    static std::mutex mu;
    static std::map<std::tuple<uint32_t, uint32_t, uint32_t, int>, Verdict> cache;
    auto bits = [](float f) {
        uint32_t u;
        memcpy(&u, &f, 4);
        return u;
    };
    const auto key = std::make_tuple(bits(s_src), bits(s_flt), bits(s_dst), act);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *mul_out = it->second.c;
            *add_out = it->second.d;
            return it->second.ops;
        }
    }
    Verdict v{0, 0.f, 0.f};
    for (int ops = 1; ops <= 3 && v.ops == 0; ++ops) {
        float c = 0.f, d = 0.f;
        if (search(s_src, s_flt, s_dst, act == ACT_RELU, ops, &c, &d))
            v = Verdict{ops, c, d};
    }
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = v;
    *mul_out = v.c;
    *add_out = v.d;
    return v.ops;
}

}  // namespace mb200
