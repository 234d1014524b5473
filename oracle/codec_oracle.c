/*
 * CPU oracle for the activation offload codec.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the shipped library links, loads or calls this file.  It is used
 * by the test-suite, by the smoke check and by the CPU-baseline leg of the
 * benchmark, always as the checker or the reported baseline, never as the
 * thing that is shipped or measured as the product.
 *
 * It restates, in plain scalar C with IEEE-754 binary32 arithmetic (no FTZ,
 * no fast-math, no FMA contraction: build with -ffp-contract=off), the
 * arithmetic of the reference project's activation offload path:
 *
 *   - BF16 <-> F32 conversion (bit shift up; round-to-nearest-even down, as
 *     __float2bfloat16 does in src/cuda/fp8_dequant.cu:38).
 *   - the software FP8 E4M3 encoder of src/cuda/fp8_quant.cu:19-57 (round
 *     half UP on the 3-bit mantissa, every magnitude >= 248 collapses to
 *     0x7F, sub-normal mantissa clamps to 7) in two independent forms: one
 *     that follows the reference's frexpf control flow and one that uses only
 *     integer bit arithmetic (the form the GPU kernel uses).
 *   - the FP8 E4M3 decoder of src/cuda/fp8_dequant.cu:20-36 (0x7F reads back
 *     as 480, 0x80 as -0.0).
 *   - the fixed-scale element-wise entry points flame_bf16_to_fp8 /
 *     flame_fp8_to_bf16 (src/cuda/fp8_quant.cu:59-93,
 *     src/cuda/fp8_dequant.cu:10-59) as called from
 *     src/activation_offload.rs:543-561 (inv_scale = 1/scale, multiply).
 *   - the symmetric int8 formula of src/sage_attention.rs:510-543
 *     (scale = absmax/127, code = round-to-nearest-even(val / scale)), applied
 *     per block of 128 consecutive elements with a +-127 clamp.
 *   - the per-128-block FP8 variant: scale = absmax/448, inv = 1/scale,
 *     code = enc(x * inv), value = bf16(dec(code) * scale).
 *   - the FP8 weight decoder with transpose of
 *     src/cuda/fused_dequant_transpose.cu:37-72 (a different reading of E4M3
 *     from the activation decoder: exponent 15 with a non-zero mantissa is
 *     NaN there), [M,N] codes -> [N,M] BF16.
 *
 * Parity status.  The FP8 encoder/decoder restatement is checked against the
 * reference's own encoder body compiled from its source (oracle/_ref, built by
 * oracle/Makefile) over every BF16 bit pattern and a dense sweep of binary32
 * values, and against the bytes the reference's two FP8 kernels wrote on a
 * B200 for every BF16 pattern and every code (tests/golden/
 * fp8_reference_kernel_sm100.npz).  The per-128-block int8 results are checked
 * against what the reference's own int8 quantiser (sage_quantize_tensor,
 * src/sage_attention.rs:510-543) wrote on a B200 with row_size = 128
 * (tests/golden/int8_reference_sage_sm100.npz).  The reference has no
 * per-128-block FP8 mode: that variant is the pinned encoder applied to
 * x * (1/scale) with scale = absmax/448, and it is held to what the reference's
 * own kernel wrote on a B200 when it was launched once per 128-element block
 * with that block's 1/scale (tests/golden/fp8_b128_reference_kernel_sm100.npz).
 * The FP8 weight decoder with transpose is held to what the reference's
 * flame_fused_dequant_transpose_bf16 wrote on a B200
 * (tests/golden/fp8_weight_reference_kernel_sm100.npz).
 * The uncompressed BF16 round trip is pinned by the reference test at
 * src/activation_offload.rs:843-889.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_BLOCK 128
#define ORACLE_FLAG_INT8_MUL_INV 1u /* code = rne(x * (1/scale)) instead of rne(x / scale) */
#define ORACLE_FLAG_FP8_OCP 1u      /* OCP RNE / saturate-to-448 encoder instead of the reference's */

static inline float bits_to_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

float oracle_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* Round-to-nearest-even narrowing; NaN becomes the canonical 0x7FFF. */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t b = f32_to_bits(f);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu;
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

/* ---- FP8 E4M3, reference semantics (src/cuda/fp8_quant.cu:19-57) -------- */

/* Form A: follows the reference's control flow (frexpf, float mantissa maths). */
uint8_t oracle_fp8_e4m3_encode_ref(float y) {
    uint8_t s = 0;
    /* NaN: every comparison below is false, frexpf leaves the exponent 0 (biased
     * 6) and the integer conversion of a NaN mantissa yields zero bits, so the
     * reference's arithmetic ends at 0x30 with no sign.  Stated outright here
     * because (int)NaN is undefined in C; 0x30 is what the reference's kernel
     * compiled for sm_100a returns on a B200 and what its encoder compiled for
     * x86-64 returns. */
    if (y != y) return 0x30;
    if (y < 0.0f) { s = 0x80; y = -y; }
    if (y > 448.0f) y = 448.0f;
    if (y == 0.0f) return s;
    int e2;
    float fr = frexpf(y, &e2); /* y = fr * 2^e2, fr in [0.5,1) */
    int be = (e2 - 1) + 7;
    if (be <= 0) {
        float sub = y * 64.0f;
        int m = (int)(sub * 8.0f + 0.5f);
        if (m > 7) m = 7;
        if (m < 0) m = 0;
        return (uint8_t)(s | m);
    }
    if (be >= 15) return (uint8_t)(s | 0x7F);
    float mf = (2.0f * fr - 1.0f) * 8.0f;
    int m = (int)(mf + 0.5f);
    if (m > 7) { m = 0; be += 1; }
    if (be >= 15) return (uint8_t)(s | 0x7F);
    return (uint8_t)(s | (be << 3) | m);
}

/* Form B: integer-only restatement, identical results to form A.
 * Adding 1<<19 to the binary32 pattern rounds the 23-bit mantissa half-up to
 * 3 bits and carries into the exponent; (pattern>>20) is then exponent*8+mant
 * and subtracting (127-7)*8 re-biases it.  Magnitudes below 2^-6 take the
 * reference's float sub-normal arm. */
uint8_t oracle_fp8_e4m3_encode_bits(float y) {
    uint32_t b = f32_to_bits(y);
    uint32_t a = b & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x30; /* NaN, as form A */
    uint8_t s = (y < 0.0f) ? 0x80 : 0x00; /* -0.0 keeps sign 0, as `val < 0` does */
    if (a == 0) return 0;
    if (a < 0x3C800000u) { /* |y| < 2^-6 */
        float v = bits_to_f32(a);
        int m = (int)(v * 512.0f + 0.5f);
        if (m > 7) m = 7;
        return (uint8_t)(s | m);
    }
    uint32_t t = (a + 0x80000u) >> 20;
    uint32_t c = t - 960u;
    if (a >= 0x43800000u || c >= 120u) c = 0x7F; /* >= 256, or rounded up into exponent 15 */
    return (uint8_t)(s | c);
}

/* Decoder (src/cuda/fp8_dequant.cu:20-36). */
float oracle_fp8_e4m3_decode(uint8_t c) {
    int sg = (c >> 7) & 1, e = (c >> 3) & 0xF, m = c & 7;
    float v;
    if (e == 0 && m == 0) v = 0.0f;
    else if (e == 0) v = ldexpf((float)m / 8.0f, -6);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return sg ? -v : v;
}

/* OCP E4M3 (fn) encoder: round-to-nearest-even, saturate to +-448 (0x7E),
 * NaN -> 0x7F.  Not the reference's arithmetic; offered as a labelled extra. */
uint8_t oracle_fp8_e4m3_encode_ocp(float y) {
    uint32_t b = f32_to_bits(y);
    uint32_t a = b & 0x7FFFFFFFu;
    uint8_t s = (uint8_t)((b >> 24) & 0x80u);
    if (a > 0x7F800000u) return (uint8_t)(s | 0x7F);
    float v = bits_to_f32(a);
    if (v >= 448.0f) return (uint8_t)(s | 0x7E);
    if (a < 0x3C800000u) { /* sub-normal target: spacing 2^-9 */
        float r = nearbyintf(v * 512.0f); /* exact scaling, RNE */
        return (uint8_t)(s | (uint8_t)r);  /* r == 8 gives 0x08 = 2^-6, correct */
    }
    uint32_t lsb = (a >> 20) & 1u;
    uint32_t t = (a + 0x7FFFFu + lsb) >> 20;
    uint32_t c = t - 960u;
    if (c > 0x7E) c = 0x7E;
    return (uint8_t)(s | c);
}

/* Sweeps binary32 patterns lo, lo+stride, ... < hi through form B and through
 * `other` (form A, or the reference's own compiled encoder) and counts the
 * patterns on which they disagree, NaN patterns included.  first_bad receives
 * the first disagreeing pattern. */
typedef unsigned char (*oracle_enc_fn)(float);
uint64_t oracle_fp8_encode_sweep(oracle_enc_fn other, uint64_t lo, uint64_t hi, uint64_t stride, uint32_t* first_bad) {
    uint64_t bad = 0;
    if (stride == 0) stride = 1;
    for (uint64_t b = lo; b < hi; b += stride) {
        uint32_t bits = (uint32_t)b;
        float y = bits_to_f32(bits);
        if (oracle_fp8_e4m3_encode_bits(y) != other(y)) {
            if (!bad && first_bad) *first_bad = bits;
            ++bad;
        }
    }
    return bad;
}

void oracle_fp8_encode_many(const float* y, uint8_t* out, size_t n, int form) {
    for (size_t i = 0; i < n; ++i)
        out[i] = form == 0 ? oracle_fp8_e4m3_encode_ref(y[i]) : form == 1 ? oracle_fp8_e4m3_encode_bits(y[i]) : oracle_fp8_e4m3_encode_ocp(y[i]);
}

/* ---- element-wise fixed-scale entry points (legacy mode) ---------------- */

/* Block codecs only: code of x scaled by the block's inv.  Two cases are this
 * library's own definition (the reference has no block codec): a zero element
 * stays zero even when inv is infinite (0*inf would be NaN), and a NaN result
 * saturates with the sign bit of the source element x. */
static inline uint8_t fp8_code_of(float x, float inv, int ocp) {
    float y = (x == 0.0f) ? x : x * inv;
    if (y != y) return (uint8_t)(((f32_to_bits(x) >> 24) & 0x80u) | 0x7Fu);
    return ocp ? oracle_fp8_e4m3_encode_ocp(y) : oracle_fp8_e4m3_encode_bits(y);
}

void oracle_bf16_to_fp8(const uint16_t* in, uint8_t* out, float inv_scale, size_t n) {
    /* src/cuda/fp8_quant.cu:69-70: the plain product, whatever it is (0*inf and NaN included) */
    for (size_t i = 0; i < n; ++i) out[i] = oracle_fp8_e4m3_encode_bits(oracle_bf16_to_f32(in[i]) * inv_scale);
}

void oracle_fp8_to_bf16(const uint8_t* in, uint16_t* out, float scale, size_t n) {
    for (size_t i = 0; i < n; ++i)
        out[i] = oracle_f32_to_bf16(oracle_fp8_e4m3_decode(in[i]) * scale);
}

/* ---- per-128-block codecs ------------------------------------------------ */

static inline float block_absmax(const uint16_t* in, size_t len) {
    float amax = 0.0f;
    for (size_t i = 0; i < len; ++i) {
        float a = fabsf(oracle_bf16_to_f32(in[i]));
        if (a > amax) amax = a; /* NaN never wins the comparison */
    }
    return amax;
}

static inline int8_t int8_code(float q) {
    if (q != q) return 0;
    float r = nearbyintf(q); /* FE_TONEAREST: ties to even */
    if (r > 127.0f) r = 127.0f;
    if (r < -127.0f) r = -127.0f;
    return (int8_t)r;
}

void oracle_quant_int8_b128(const uint16_t* in, int8_t* codes, float* scales, size_t n, unsigned flags) {
    for (size_t b0 = 0, blk = 0; b0 < n; b0 += ORACLE_BLOCK, ++blk) {
        size_t len = n - b0 < ORACLE_BLOCK ? n - b0 : ORACLE_BLOCK;
        float amax = block_absmax(in + b0, len);
        float scale = amax / 127.0f;
        scales[blk] = scale;
        if (amax == 0.0f) { memset(codes + b0, 0, len); continue; }
        if (flags & ORACLE_FLAG_INT8_MUL_INV) {
            float inv = 1.0f / scale;
            for (size_t i = 0; i < len; ++i) codes[b0 + i] = int8_code(oracle_bf16_to_f32(in[b0 + i]) * inv);
        } else {
            for (size_t i = 0; i < len; ++i) codes[b0 + i] = int8_code(oracle_bf16_to_f32(in[b0 + i]) / scale);
        }
    }
}

void oracle_dequant_int8_b128(const int8_t* codes, const float* scales, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i)
        out[i] = oracle_f32_to_bf16((float)codes[i] * scales[i / ORACLE_BLOCK]);
}

void oracle_quant_fp8_b128(const uint16_t* in, uint8_t* codes, float* scales, size_t n, unsigned flags) {
    for (size_t b0 = 0, blk = 0; b0 < n; b0 += ORACLE_BLOCK, ++blk) {
        size_t len = n - b0 < ORACLE_BLOCK ? n - b0 : ORACLE_BLOCK;
        float amax = block_absmax(in + b0, len);
        float scale = amax / 448.0f;
        scales[blk] = scale;
        if (amax == 0.0f) { memset(codes + b0, 0, len); continue; }
        float inv = 1.0f / scale;
        for (size_t i = 0; i < len; ++i)
            codes[b0 + i] = fp8_code_of(oracle_bf16_to_f32(in[b0 + i]), inv, (flags & ORACLE_FLAG_FP8_OCP) != 0);
    }
}

void oracle_dequant_fp8_b128(const uint8_t* codes, const float* scales, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i)
        out[i] = oracle_f32_to_bf16(oracle_fp8_e4m3_decode(codes[i]) * scales[i / ORACLE_BLOCK]);
}

/* ---- packed host layout ---------------------------------------------------
 * codes[n] | zero padding to a 256-byte boundary | scales[ceil(n/128)] fp32 LE */

/* src/cuda/fused_dequant_transpose.cu:37-72: sign, 4-bit exponent, 3-bit mantissa; zero; sub-normal
 * (mant/8) * 2^-6; exponent 15 with mantissa != 0 -> quiet NaN; exponent 15 with mantissa 0 -> 2^8;
 * otherwise (1 + mant/8) * 2^(exp-7); the sign applied after; then val *= scale and
 * __float2bfloat16 (round to nearest even, NaN -> 0x7FFF). */
float oracle_fp8_weight_decode(uint8_t bits) {
  const int sign = (bits >> 7) & 1, ex = (bits >> 3) & 0xF, mant = bits & 0x7;
  float val;
  if (ex == 0 && mant == 0) val = 0.0f;
  else if (ex == 0) val = ldexpf((float)mant / 8.0f, -6);
  else if (ex == 15 && mant != 0) val = bits_to_f32(0x7FC00000u);
  else if (ex == 15) val = ldexpf(1.0f, 15 - 7);
  else val = ldexpf(1.0f + (float)mant / 8.0f, ex - 7);
  return sign ? -val : val;
}

void oracle_fp8_dequant_transpose(const uint8_t* in, uint16_t* out, float scale, int M, int N) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float v = oracle_fp8_weight_decode(in[(size_t)m * N + n]) * scale;
      out[(size_t)n * M + m] = (v != v) ? (uint16_t)0x7FFF : oracle_f32_to_bf16(v);
    }
}

size_t oracle_packed_scales_offset(size_t n) { return (n + 255u) & ~(size_t)255u; }
size_t oracle_packed_bytes(size_t n) {
    return oracle_packed_scales_offset(n) + 4u * ((n + ORACLE_BLOCK - 1) / ORACLE_BLOCK);
}

/* codec: 2 = int8 per-128-block, 3 = fp8 per-128-block (numbering of the C ABI) */
void oracle_pack(const uint16_t* in, uint8_t* packed, size_t n, int codec, unsigned flags) {
    size_t so = oracle_packed_scales_offset(n);
    memset(packed + n, 0, so - n);
    if (codec == 2) oracle_quant_int8_b128(in, (int8_t*)packed, (float*)(packed + so), n, flags);
    else oracle_quant_fp8_b128(in, packed, (float*)(packed + so), n, flags);
}

void oracle_unpack(const uint8_t* packed, uint16_t* out, size_t n, int codec) {
    size_t so = oracle_packed_scales_offset(n);
    if (codec == 2) oracle_dequant_int8_b128((const int8_t*)packed, (const float*)(packed + so), out, n);
    else oracle_dequant_fp8_b128(packed, (const float*)(packed + so), out, n);
}

/* ---- threaded pack+unpack, for the reported CPU baseline ------------------
 * Static partition on 128-element boundaries; each worker quantises its range
 * into the packed buffer and dequantises it back out. */

typedef struct {
    const uint16_t* in; uint8_t* packed; uint16_t* out;
    size_t n, lo, hi; int codec; unsigned flags; int do_unpack;
} oracle_job;

static void* oracle_worker(void* p) {
    oracle_job* j = (oracle_job*)p;
    size_t so = oracle_packed_scales_offset(j->n);
    size_t len = j->hi - j->lo;
    float* sc = (float*)(j->packed + so) + j->lo / ORACLE_BLOCK;
    if (j->codec == 2) {
        oracle_quant_int8_b128(j->in + j->lo, (int8_t*)j->packed + j->lo, sc, len, j->flags);
        if (j->do_unpack) oracle_dequant_int8_b128((int8_t*)j->packed + j->lo, sc, j->out + j->lo, len);
    } else if (j->codec == 3) {
        oracle_quant_fp8_b128(j->in + j->lo, j->packed + j->lo, sc, len, j->flags);
        if (j->do_unpack) oracle_dequant_fp8_b128(j->packed + j->lo, sc, j->out + j->lo, len);
    } else { /* uncompressed: byte copy out and back */
        memcpy(j->packed + 2 * j->lo, j->in + j->lo, 2 * len);
        if (j->do_unpack) memcpy(j->out + j->lo, j->packed + 2 * j->lo, 2 * len);
    }
    return NULL;
}

/* packed must hold oracle_packed_bytes(n) (codec 2/3) or 2*n (codec 0). Returns 0 on success. */
int oracle_roundtrip_mt(const uint16_t* in, uint8_t* packed, uint16_t* out, size_t n,
                        int codec, unsigned flags, int threads, int do_unpack) {
    if (threads < 1) threads = 1;
    if (threads > 1024) threads = 1024;
    size_t nblk = (n + ORACLE_BLOCK - 1) / ORACLE_BLOCK;
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    oracle_job* jobs = (oracle_job*)malloc(sizeof(oracle_job) * (size_t)threads);
    char* live = (char*)calloc((size_t)threads, 1);
    if (!th || !jobs || !live) { free(th); free(jobs); free(live); return -1; }
    if (codec == 2 || codec == 3) {
        size_t so = oracle_packed_scales_offset(n);
        memset(packed + n, 0, so - n);
    }
    for (int t = 0; t < threads; ++t) {
        size_t b_lo = nblk * (size_t)t / (size_t)threads, b_hi = nblk * (size_t)(t + 1) / (size_t)threads;
        size_t lo = b_lo * ORACLE_BLOCK, hi = b_hi * ORACLE_BLOCK;
        if (hi > n) hi = n;
        jobs[t] = (oracle_job){in, packed, out, n, lo, hi, codec, flags, do_unpack};
        if (lo >= hi) continue;
        /* the calling thread takes the last range itself */
        if (t == threads - 1 || pthread_create(&th[t], NULL, oracle_worker, &jobs[t]) != 0) oracle_worker(&jobs[t]);
        else live[t] = 1;
    }
    for (int t = 0; t < threads; ++t) if (live[t]) pthread_join(th[t], NULL);
    free(live);
    free(th); free(jobs);
    return 0;
}
