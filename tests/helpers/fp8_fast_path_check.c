/* Host replay of the FP8 compress kernel's hardware path, checked against the CPU oracle (test infrastructure).
 *
 * The kernel truncates |y| to FP16, sets the lowest mantissa bit, turns magnitudes from 248 up into NaN and converts
 * with round-to-nearest-even to E4M3 (NaN -> 0x7F).  It then looks again only at elements whose code is 0x00 or 0x08.
 * This program models those steps in integer arithmetic for every binary32 magnitude it is given and counts
 *   - magnitudes whose modelled code differs from the oracle's although the code is neither 0x00 nor 0x08 (must be 0),
 *   - magnitudes of code 0x08 / 0x00 that do differ (the two cases the second look exists for).
 * usage: fp8_fast_path_check <stride of the sparse sweep over all magnitudes>
 * output: checked unexpected differ_at_08 differ_at_00 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

unsigned char oracle_fp8_e4m3_encode_bits(float y);

static float b2f(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }

/* binary32 magnitude bits (finite or infinite, not NaN) -> FP16 bits, rounded toward zero */
static uint32_t f32_to_f16_rz(uint32_t a) {
    if (a >= 0x7F800000u) return 0x7C00u;          /* infinity */
    if (a >= 0x477FE000u) return 0x7BFFu;          /* >= 65504: the largest finite FP16 */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    if (e >= -14) return (uint32_t)((e + 15) << 10) | ((m >> 13) & 0x3FFu);
    int sh = 13 + (-14 - e);
    return sh >= 32 ? 0u : (m >> sh);
}

/* positive finite FP16 bits -> E4M3 code, round-to-nearest-even, saturating at 448 */
static uint32_t f16_to_e4m3_rne(uint32_t h) {
    int e = (int)(h >> 10);
    uint32_t m = h & 0x3FFu;
    /* value = (e ? 1024 + m : m) * 2^(max(e,1) - 25) */
    uint64_t sig = e ? (1024u + m) : m;
    int ex = (e ? e : 1) - 25;                     /* value = sig * 2^ex */
    if (sig == 0) return 0;
    /* below 2^-6: multiples of 2^-9 */
    /* compare value with 2^-6: value >= 2^-6  <=>  sig * 2^(ex+6) >= 1 */
    int top = 63 - __builtin_clzll(sig);           /* value in [2^(top+ex), 2^(top+ex+1)) */
    int ve = top + ex;                             /* floor(log2(value)) */
    if (ve < -6) {
        /* q = value * 512 = sig * 2^(ex+9), rounded to nearest even */
        int s = -(ex + 9);
        if (s <= 0) return (uint32_t)(sig << -s);  /* cannot happen below 2^-6 with s <= 0 except tiny sig; exact */
        if (s > 40) return 0;
        uint64_t q = sig >> s, rem = sig & ((1ull << s) - 1), half = 1ull << (s - 1);
        if (rem > half || (rem == half && (q & 1))) ++q;
        return (uint32_t)q;                        /* 8 is code 0x08 = 2^-6 */
    }
    /* normal: 3 mantissa bits */
    int s = top - 3;                               /* keep 4 significant bits */
    uint64_t q = s > 0 ? sig >> s : sig << -s, rem = s > 0 ? sig & ((1ull << s) - 1) : 0, half = s > 0 ? 1ull << (s - 1) : 0;
    if (s > 0 && (rem > half || (rem == half && (q & 1)))) ++q;
    if (q == 16) { q = 8; ++ve; }
    if (ve > 8 || (ve == 8 && q > 14)) return 0x7E; /* above 448: saturate */
    return (uint32_t)(((ve + 7) << 3) | (q - 8));
}

static uint32_t model(uint32_t a) {
    uint32_t h = f32_to_f16_rz(a);
    if (h >= 0x5BC0u) return 0x7F;                 /* 248 and above are made NaN, which converts to 0x7F */
    return f16_to_e4m3_rne(h | 1u);
}

int main(int argc, char** argv) {
    uint64_t stride = argc > 1 ? strtoull(argv[1], 0, 10) : 257;
    uint64_t checked = 0, unexpected = 0, d08 = 0, d00 = 0;
    /* every magnitude in [2^-20, 2^-5), then a sparse sweep over all of them up to infinity */
    for (int pass = 0; pass < 2; ++pass) {
        uint64_t lo = pass ? 0 : 0x35800000u, hi = pass ? 0x7F800001u : 0x3D000000u, st = pass ? stride : 1;
        for (uint64_t a = lo; a < hi; a += st) {
            uint32_t fast = model((uint32_t)a), ref = oracle_fp8_e4m3_encode_bits(b2f((uint32_t)a));
            ++checked;
            if (fast == ref) continue;
            if (fast == 0x08) ++d08;
            else if (fast == 0x00) ++d00;
            else {
                if (!unexpected) fprintf(stderr, "first unexpected: bits %08x fast %02x ref %02x\n", (unsigned)a, fast, ref);
                ++unexpected;
            }
        }
    }
    printf("%llu %llu %llu %llu\n", (unsigned long long)checked, (unsigned long long)unexpected, (unsigned long long)d08, (unsigned long long)d00);
    return unexpected ? 1 : 0;
}
