/* Exhaustive CPU checks of the two float identities the GPU requantisation epilogue rests on
 * (megcc_b200/csrc/common.cuh). Compiled by tests/test_requant_math.py with strict IEEE
 * flags (-O2 -ffp-contract=off, no fast-math) and run on the host; no GPU involved.
 *
 *   roundf    trunc(x + copysign(0.49999997f, x)) == roundf(x) for EVERY float with
 *             |x| < 2^31 (all 2^32 bit patterns are visited).
 *   division  q0 = RN(t * r), rem = fma(-q0, d, t), q = fma(rem, r, q0) with r = RN(1 / d)
 *             equals RN(t / d): for every divisor of the list (the scales of the golden
 *             vectors and benchmark configurations, powers of two, all-ones and near-one
 *             mantissas, pseudo-random floats), for all 2^23 mantissas of t at several
 *             exponents and both signs, and for t = (float)acc * s over every int32 acc at
 *             the edges of the int8 staircase. The identity is a property of the mantissas
 *             as long as no intermediate leaves the normal range, so the exponent sample
 *             includes the ends of the range the library admits (see `division_range_ok`
 *             in megcc_b200/csrc/common.cuh): 2^-100 <= |t| <= 2^100, 2^-100 <= d <= 2^100,
 *             2^-60 <= |t / d| <= 2^91.
 *
 * Usage: requant_math_check roundf | division <first> <count>
 * Prints "ok <checked>" or "FAIL ..." and exits non-zero.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float from_bits(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static uint32_t to_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static int check_roundf(uint32_t first, uint64_t count) {
    uint64_t checked = 0;
    for (uint64_t i = 0; i < count; ++i) {
        const uint32_t u = first + (uint32_t)i;
        const float x = from_bits(u);
        if (!(fabsf(x) < 2147483648.f))
            continue; /* beyond the int range (and NaN): handled separately by the kernels */
        volatile float y = x + copysignf(0.49999997f, x);
        const float got = truncf(y);
        const float want = roundf(x);
        if (to_bits(got) != to_bits(want) && !(got == 0.f && want == 0.f)) {
            printf("FAIL roundf x=%a got %a want %a\n", x, got, want);
            return 1;
        }
        ++checked;
    }
    printf("ok %llu\n", (unsigned long long)checked);
    return 0;
}

static float div3(float t, float d, float r) {
    volatile float q0 = t * r;
    const float rem = fmaf(-q0, d, t);
    return fmaf(rem, r, q0);
}

static const float kDivisors[] = {
        /* dst scales of the golden vectors, the benchmark configurations and the tests */
        0.1f, 5.0f, 4.0f, 40.25f, 0.7f, 0.5f, 0.3f, 2.0f, 3.0f, 0.9f, 0.37f, 0.8f, 0.4f, 1.0f,
        0.002f, 0.052f, 6.0f / 127.0f, 0.0472440943f,
        /* mantissa extremes */
        1.9999999f, 1.0000001f, 1.5f, 1.25f, 0.99999994f, 3.9999998f,
        /* range ends the library admits */
        0x1p-100f, 0x1.fffffep-100f, 0x1p100f, 0x1.fffffep99f, 0x1p-60f, 0x1p60f,
        0x1.555556p-40f, 0x1.aaaaaap37f, 0x1.8p66f, 0x1.2p-77f,
};

static int check_division(int first, int count) {
    const int n_fixed = (int)(sizeof(kDivisors) / sizeof(kDivisors[0]));
    uint64_t checked = 0;
    uint32_t lcg = 0x1234567u + (uint32_t)first * 977u;
    for (int di = first; di < first + count; ++di) {
        float d;
        if (di < n_fixed) {
            d = kDivisors[di];
        } else {
            /* pseudo-random mantissa, exponent in [-20, 20] */
            lcg = lcg * 1664525u + 1013904223u + (uint32_t)di;
            const uint32_t mant = lcg >> 9;
            lcg = lcg * 1664525u + 1013904223u;
            const int e = (int)(lcg >> 24) % 41 - 20;
            d = from_bits(((uint32_t)(127 + e) << 23) | mant);
        }
        volatile float rv = 1.0f / d;
        const float r = rv;
        static const int exps[] = {-100, -77, -37, -1, 0, 24, 54, 66, 99};
        for (unsigned ei = 0; ei < sizeof(exps) / sizeof(exps[0]); ++ei) {
            /* the quotient's range the library admits: |t / d| from 2^-60 (one accumulator
             * count at the smallest scale ratio) to 2^91 (2^31 counts at the largest) */
            const float lim = fabsf(ldexpf(1.f, exps[ei]) / d);
            if (!(lim >= 0x1p-61f && lim <= 0x1p92f))
                continue;
            for (uint32_t m = 0; m < (1u << 23); ++m) {
                const float t = from_bits(((uint32_t)(127 + exps[ei]) << 23) | m);
                volatile float want = t / d;
                const float got = div3(t, d, r);
                if (to_bits(got) != to_bits(want)) {
                    printf("FAIL division t=%a d=%a got %a want %a\n", t, d, got, (float)want);
                    return 1;
                }
                volatile float wantn = -t / d;
                const float gotn = div3(-t, d, r);
                if ((m & 1023u) == 0 && to_bits(gotn) != to_bits(wantn)) {
                    printf("FAIL division t=%a d=%a got %a want %a\n", -t, d, gotn, (float)wantn);
                    return 1;
                }
                ++checked;
            }
        }
        /* the accumulator chain itself: t = (float)acc * s_src * s_flt for every int32 acc is
         * far too many values per divisor; walk the accumulators around every int8 step of
         * acc * s / d instead (the values that decide an output), for a few s */
        static const float ss[] = {0.05f * 0.01f, 1.0f * 2.0f, 2.5f * 2.5f, 0.0005f, 1.0f};
        for (unsigned si = 0; si < sizeof(ss) / sizeof(ss[0]); ++si) {
            const float s = ss[si];
            for (int q = -129; q <= 128; ++q) {
                const double centre = ((double)q + 0.5) * (double)d / (double)s;
                if (!(fabs(centre) < 2147480000.0))
                    continue;
                for (long long acc = (long long)centre - 64; acc <= (long long)centre + 64; ++acc) {
                    if (acc < -2147483647LL - 1 || acc > 2147483647LL)
                        continue;
                    volatile float t = (float)(int)acc * s;
                    volatile float want = t / d;
                    const float got = div3(t, d, r);
                    if (to_bits(got) != to_bits(want)) {
                        printf("FAIL division acc=%lld s=%a d=%a\n", acc, s, d);
                        return 1;
                    }
                    ++checked;
                }
            }
        }
    }
    printf("ok %llu\n", (unsigned long long)checked);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 4 && strcmp(argv[1], "roundf") == 0)
        return check_roundf((uint32_t)strtoull(argv[2], 0, 0), strtoull(argv[3], 0, 0));
    if (argc >= 4 && strcmp(argv[1], "division") == 0)
        return check_division(atoi(argv[2]), atoi(argv[3]));
    fprintf(stderr, "usage: %s roundf <first bits> <count> | division <first> <count>\n", argv[0]);
    return 2;
}
