/* CPU check of the quotient shortcut used by the int8 compress kernel.
 *
 * The kernel needs RN(x / s) in binary32 for every element x of a block whose
 * scale is s.  Instead of a division per element it computes, with
 * r = RN(1/s):  q0 = RN(x*r);  e = fma(-q0, s, x);  q = fma(e, r, q0)
 * and falls back to the division when s has an all-ones significand or an
 * exponent outside [2^-63, 2^63].  This program replays both on the host
 * (fmaf is a correctly rounded fused multiply-add) and counts disagreements,
 * over every finite BF16 x with |x| <= 127.5*s for many scales.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float b2f(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t f2b(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

static int fast_ok(float s) {
    uint32_t b = f2b(s), ex = (b >> 23) & 0xFF;
    return ex >= 64 && ex <= 190 && (b & 0x7FFFFF) != 0x7FFFFF;
}

static float kernel_quotient(float x, float s) {
    if (!fast_ok(s)) return x / s;
    float r = 1.0f / s;
    float q0 = x * r;
    float e = fmaf(-q0, s, x);
    return fmaf(e, r, q0);
}

/* amax/127 and amax/448 by the same sequence with a compile-time reciprocal,
 * as the kernels compute the block scale; every positive finite BF16 amax. */
static uint64_t check_div_const(float D) {
    uint64_t bad = 0;
    const float r = 1.0f / D;
    for (uint32_t h = 0; h < 0x7F80; ++h) {
        float a = b2f(h << 16);
        uint32_t ex = (f2b(a) >> 23) & 0xFF;
        float got;
        if (ex >= 64 && ex <= 190) {
            float q0 = a * r, e = fmaf(-q0, D, a);
            got = fmaf(e, r, q0);
        } else {
            got = a / D;
        }
        if (f2b(got) != f2b(a / D)) ++bad;
    }
    return bad;
}

int main(int argc, char** argv) {
    if (check_div_const(127.0f) || check_div_const(448.0f)) { printf("0 1\n"); return 1; }
    uint64_t nscales = argc > 1 ? strtoull(argv[1], 0, 10) : 2000;
    uint64_t bad = 0, checked = 0, seed = 88172645463325252ull;
    for (uint64_t k = 0; k < nscales; ++k) {
        seed ^= seed << 13; seed ^= seed >> 7; seed ^= seed << 17;
        float s;
        if (k % 4 == 0) {          /* scale of a BF16 absmax: amax/127 */
            uint16_t a = (uint16_t)(seed >> 20) & 0x7FFF;
            if (((a >> 7) & 0xFF) == 0xFF) continue;
            s = b2f((uint32_t)a << 16) / 127.0f;
        } else if (k % 4 == 1) {   /* arbitrary binary32 scale */
            s = b2f((uint32_t)(seed >> 16) & 0x7FFFFFFF);
            if (!(s == s) || isinf(s)) continue;
        } else if (k % 4 == 2) {   /* near all-ones significands */
            s = b2f(((uint32_t)(seed >> 40) % 254 + 1) << 23 | (0x7FFFFF - (uint32_t)(seed & 3)));
        } else {                   /* typical activation range */
            s = b2f(0x3A000000u + ((uint32_t)(seed >> 24) & 0x03FFFFFF));
        }
        if (s == 0.0f) continue;
        for (uint32_t h = 0; h < 65536; ++h) {
            if (((h >> 7) & 0xFF) == 0xFF) continue;
            float x = b2f(h << 16);
            if (fabsf(x) > 127.5f * s) continue;
            float q = kernel_quotient(x, s), d = x / s;
            ++checked;
            /* the kernel only uses the rounded integer, but the quotients themselves must agree
               wherever the integer could differ; require full equality outside the flush zone */
            if (f2b(q) != f2b(d)) {
                if (nearbyintf(q) != nearbyintf(d) || fabsf(d) >= 0.25f) {
                    if (bad < 5) fprintf(stderr, "mismatch x=%a s=%a fast=%a div=%a\n", x, s, q, d);
                    ++bad;
                }
            }
        }
    }
    printf("%llu %llu\n", (unsigned long long)checked, (unsigned long long)bad);
    return bad ? 1 : 0;
}
