/* Test program for the quantizers' quotient: with r = RN(1 / s), the sequence
 *     q = RN(x r);  q = RN(q + RN(x - q s) r);  q = RN(q + RN(x - q s) r);  q = copysign(q, x)
 * (each RN(a + b c) one fused multiply-add) must give the bits of the IEEE division RN(x / s) whenever
 * 2^-60 <= s <= 2^60 and |x| <= 449 s.  Part 1 walks every bf16 significand of x against a stride of the fp32
 * significands of s; part 2 draws 24-bit x and s at random over the exponent range, x down to 2^-30 s; part 3 is zeros
 * and denormals, where the residuals underflow: there both quotients must have the same sign and stay below 2^-10, half
 * the smallest e4m3 subnormal, so that both convert to the same zero code.  Prints the number of mismatches and exits non-zero if there is one.
 * usage: quotient_identity STRIDE RANDOM_CASES */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float quotient(float x, float s, float r) {
    float q = x * r;
    q = fmaf(fmaf(-q, s, x), r, q);
    q = fmaf(fmaf(-q, s, x), r, q);
    return copysignf(q, x);
}

static long bad = 0;
static void check(float x, float s) {
    const float want = x / s, got = quotient(x, s, 1.0f / s);
    if (bits(want) != bits(got) && bad++ < 10) printf("mismatch x=%a s=%a division=%a sequence=%a\n", x, s, want, got);
}

static uint64_t state = 88172645463325252ull;
static uint64_t next(void) { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return state; }

int main(int argc, char** argv) {
    const uint32_t stride = argc > 1 ? (uint32_t)atoi(argv[1]) : 1;
    const long n_random = argc > 2 ? atol(argv[2]) : 100000000L;
    long cases = 0;
    for (uint32_t ms = 0; ms < (1u << 23); ms += stride) {
        const float s = from_bits(0x3F800000u | ms);
        for (uint32_t mx = 0; mx < 128; ++mx, cases += 2) {
            const float x = from_bits(0x40000000u | (mx << 16));
            check(x, s);
            check(-0.5f * x, s);
        }
    }
    for (long i = 0; i < n_random; ++i, ++cases) {
        const uint64_t a = next(), b = next();
        const int es = (int)(a % 121) - 60, ex = (int)(b % 40) - 30;
        const float s = ldexpf(from_bits(0x3F800000u | (uint32_t)((a >> 8) & 0x7FFFFF)), es);
        float x = ldexpf(from_bits(0x3F800000u | (uint32_t)((b >> 8) & 0x7FFFFF)), es + ex);
        if (es < 60) check((b >> 63) ? -x : x, s);
    }
    const float special[] = {0.0f, -0.0f, 1e-45f, -1e-45f, 1e-38f, -3e-39f};
    for (int i = 0; i < 6; ++i, ++cases) {
        const float want = special[i] / 0.37f, got = quotient(special[i], 0.37f, 1.0f / 0.37f);
        if (signbit(want) != signbit(got) || !(fabsf(want) < 0x1p-10f) || !(fabsf(got) < 0x1p-10f)) {
            printf("mismatch (tiny) x=%a division=%a sequence=%a\n", special[i], want, got);
            ++bad;
        }
    }
    printf("cases %ld mismatches %ld\n", cases, bad);
    return bad != 0;
}
