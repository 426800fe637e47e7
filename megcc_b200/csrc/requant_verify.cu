// Host-side search for a one-multiplication requantisation that is PROVEN equal to the
// reference's three-step float chain on every accumulator value that can matter.
//
// The reference computes  q = clamp_s8(roundf(act(((float)acc * s_src) * s_flt / s_dst)))
// (compiler/lib/KernelGen/BareMetal/Activation.cpp:105-113): three rounded float operations
// before the activation. The epilogue of the tensor-core kernels is bound by instruction
// issue, and  q' = clamp_s8(trunc(fma((float)acc, c, +-0.49999997)))  needs one. For given scales the two
// agree unless some acc lands a half-integer boundary between the two products, and whether
// that happens can simply be checked: both chains are monotonic in acc (positive scales,
// IDENTITY or RELU), so beyond the first acc on either side where BOTH saturate they agree
// for ever, and in between there are about 260 * s_dst / (s_src * s_flt) integers, usually a
// few hundred thousand. Every one of them is evaluated through both chains, for the
// correctly rounded ratio and its neighbouring floats as candidates for c; the first
// candidate without a single difference is used, and if none passes (or the range is too
// long to walk) the kernel keeps the three-step chain. Verdicts are cached per scale triple.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "internal.h"

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

// what the device's fast path computes: ONE fused multiply-add, trunc(fma((float)acc, c,
// +-0.49999997f)) saturated to int8, RELU applied afterwards (fmaf is correctly rounded)
inline int fast_chain(int acc, float c, bool relu) {
    const float f = (float)acc;
    volatile float y = fmaf(f, c, relu ? 0.49999997f : copysignf(0.49999997f, f));
    float t = truncf(y);
    int q = t < -128.f ? -128 : (t > 127.f ? 127 : (int)t);
    if (relu && q < 0)
        q = 0;
    return q;
}

float search(float s_src, float s_flt, float s_dst, bool relu) {
    if (!(s_src > 0.f) || !(s_flt > 0.f) || !(s_dst > 0.f))
        return 0.f;
    const double ratio = (double)s_src * (double)s_flt / (double)s_dst;
    if (!(ratio > 0.0) || !isfinite(ratio))
        return 0.f;
    const double span = 130.0 / ratio;
    if (span > 8.0e6)  // too many values to walk at load time
        return 0.f;
    const int r = (int)span + 4;
    // the ends must be saturated in the reference chain (then every acc beyond them is too)
    if (reference_chain(r, s_src, s_flt, s_dst, relu) != 127 ||
        reference_chain(-r, s_src, s_flt, s_dst, relu) != (relu ? 0 : -128))
        return 0.f;
    float cands[5];
    cands[0] = (float)ratio;
    cands[1] = nextafterf(cands[0], INFINITY);
    cands[2] = nextafterf(cands[0], 0.f);
    cands[3] = nextafterf(cands[1], INFINITY);
    cands[4] = nextafterf(cands[2], 0.f);
    for (float c : cands) {
        if (!(c > 0.f))
            continue;
        bool same = true;
        for (int acc = -r; acc <= r && same; ++acc)
            same = reference_chain(acc, s_src, s_flt, s_dst, relu) == fast_chain(acc, c, relu);
        if (same)
            return c;
    }
    return 0.f;
}

}  // namespace

// The multiplier c with clamp_s8(roundf(act((float)acc * c))) equal to the reference chain for
// every int32 acc, or 0 when there is none (or the activation is not IDENTITY / RELU, or the
// scales are not positive, or MB200_NO_FAST_REQUANT is set).
float requant_fast_constant(float s_src, float s_flt, float s_dst, int act) {
    if (act != ACT_IDENTITY && act != ACT_RELU)
        return 0.f;
    if (getenv("MB200_NO_FAST_REQUANT"))
        return 0.f;
    static std::mutex mu;
    static std::map<std::tuple<uint32_t, uint32_t, uint32_t, int>, float> cache;
    auto bits = [](float f) {
        uint32_t u;
        memcpy(&u, &f, 4);
        return u;
    };
    const auto key = std::make_tuple(bits(s_src), bits(s_flt), bits(s_dst), act);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end())
            return it->second;
    }
    const float c = search(s_src, s_flt, s_dst, act == ACT_RELU);
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = c;
    return c;
}

}  // namespace mb200
