// Codec kernels of the activation offload path, written for sm_100a.
//
//   compress   : BF16 -> int8 or FP8-E4M3 codes + one fp32 scale per 128 elements
//   dequantise : codes + scales -> BF16, written at its final address
//   element-wise FP8 with a caller-supplied scale (the reference's two kernels,
//   src/cuda/fp8_quant.cu:59-93 and src/cuda/fp8_dequant.cu:10-59)
//
// All of this is HBM-bound byte work: 2 B read + 1 B + 4/128 B written per
// element one way, the mirror image the other way.  There is no contraction,
// so no tensor cores.  What matters is coalescing, bytes in flight per SM and
// an instruction count per element that stays under the issue budget
// (~18 lane-instructions per element at full HBM rate; in practice ~10).
//
// Compress tile: 256 threads x 64 bytes = 8192 elements = 64 blocks of 128.  A
// lane holds 32 consecutive elements (two 32-byte loads), four consecutive
// lanes hold one block: the block's absmax is a tree of packed BF16 maxima in
// the lane and two shuffles across the four lanes, and the per-block work (one
// exactly rounded scale, one exactly rounded reciprocal) is paid once per 32
// elements of a lane.  By default every lane writes its 32 codes with two
// 16-byte stores and one lane in four writes the scale: no shared memory, no
// barrier.  FLAME_ACT_STAGED_STORES selects the variant that stages each warp's
// 1024 codes and 8 scales in a shared-memory slice of its own and lets one lane
// send them out as two bulk asynchronous copies
// (cp.async.bulk.global.shared::cta; warp-level synchronisation only, cluster
// size 1, every copy CTA-local).  Both write the same bytes.
//
// Output addressing is "packed chunks": chunk c of `chunk_elems` elements lives
// at out + c*chunk_stride, codes first, its scales at a byte offset inside the
// chunk.  One launch can therefore fill a staging tile made of several
// self-contained chunks, each of which then crosses the host link as a single
// copy.  The plain (codes*, scales*) entry points are the one-chunk case.
//
// Arithmetic is IEEE binary32 throughout: this file must be compiled WITHOUT
// --use_fast_math and without -ftz; the operations whose rounding matters use
// the explicit _rn intrinsics so that no FMA contraction can change a result.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>
#include <type_traits>
#include <vector>

#include "codec_kernels.cuh"

namespace flame_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kLaneElems = 16;                               // BF16 per 32-byte access
constexpr int kLaneLoads = 2;                                // 32-byte loads per lane per tile: 32 consecutive elements
constexpr int kCompLaneElems = kLaneElems * kLaneLoads;      // 32
constexpr int kTileElems = kThreads * kCompLaneElems;        // 8192
constexpr int kLanesPerBlock = 128 / kLaneElems;             // 8: lanes per block where a lane holds 16 elements (dequantise, producers)
constexpr int kCompLanesPerBlock = 128 / kCompLaneElems;     // 4: lanes per block in the compress kernels
constexpr int kWarpCodes = 32 * kCompLaneElems;              // 1024 codes per warp per tile
constexpr int kWarpScales = kWarpCodes / 128;                // 8 scales per warp per tile
constexpr int kWarpSliceBytes = kWarpCodes + kWarpScales * 4;  // staged variant: one warp's codes then scales (1056, a multiple of 16)
constexpr int kStagedSmemBytes = (kThreads / 32) * 2 * kWarpSliceBytes;  // two slices per warp
constexpr int kDequantUnroll = 4;                            // 16-byte code loads in flight per thread
constexpr int kDequantTileElems = kThreads * kLaneElems * kDequantUnroll;  // 16384

struct U32x8 { uint32_t v[8]; };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared -> global bulk copy, tracked by the per-thread bulk async-group.
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :: "l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" :: "n"(N) : "memory"); }
// Orders this thread's shared-memory writes before later async-proxy reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 32-byte streaming load / store (256-bit accesses exist from sm_100 on).
__device__ __forceinline__ U32x8 ld_stream32(const void* p) {
  U32x8 r;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]),
                 "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7]) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream32(void* p, const U32x8& r) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :: "l"(p), "r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]),
                  "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7]) : "memory");
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ void unpack16(const U32x8& r, float (&x)[16]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { x[2 * i] = bf16lo(r.v[i]); x[2 * i + 1] = bf16hi(r.v[i]); }
}

// max(|a|, |b|) of two packed BF16 pairs in one instruction.  The sign of each result half is the xor of the
// operands' signs and is masked away by the caller.  A NaN operand is ignored (the other one is returned), so a
// NaN element never becomes the absmax; only an all-NaN set gives NaN.
__device__ __forceinline__ uint32_t max_abs_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// absmax of NW words of two BF16 each, as a float (exact: a maximum only selects).
template <int NW>
__device__ __forceinline__ float absmax_words(const uint32_t* w) {
  static_assert(NW >= 2 && (NW & (NW - 1)) == 0, "a power of two of words");
  uint32_t t[NW / 2];
#pragma unroll
  for (int i = 0; i < NW / 2; ++i) t[i] = max_abs_bf16x2(w[2 * i], w[2 * i + 1]);
#pragma unroll
  for (int n = NW / 4; n >= 1; n >>= 1) {
#pragma unroll
    for (int i = 0; i < n; ++i) t[i] = max_abs_bf16x2(t[2 * i], t[2 * i + 1]);
  }
  const float lo = __uint_as_float((t[0] << 16) & 0x7FFF0000u), hi = __uint_as_float(t[0] & 0x7FFF0000u);
  return fmaxf(lo, hi);  // fmaxf ignores a NaN operand
}

// Max over the 8 lanes that hold one 128-element block (16 elements per lane).
__device__ __forceinline__ float absmax_8lanes(float m) {
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  return m;
}
// Max over the 4 lanes that hold one block (32 elements per lane).
__device__ __forceinline__ float absmax_4lanes(float m) {
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  return m;
}

// ---- correctly rounded quotients without a division per element ----------------
// Markstein's sequence: with r = RN(1/s), q0 = RN(x*r), e = x - q0*s (exact, one
// FMA), q = RN(q0 + e*r) equals RN(x/s) provided s's significand is not all ones
// and nothing underflows.  `safe_range` keeps every intermediate normal; the
// rare scale outside it takes the IEEE division.  (Replayed against x/s on the
// host for every BF16 x and thousands of scales by the test-suite.)
__device__ __forceinline__ bool markstein_ok(float s) {
  const uint32_t b = __float_as_uint(s);
  const uint32_t ex = (b >> 23) & 0xFFu;
  return (ex >= 64u) && (ex <= 190u) && ((b & 0x7FFFFFu) != 0x7FFFFFu);
}

// amax / D for the two constants 127 and 448 (neither has an all-ones significand).
template <int D>
__device__ __forceinline__ float div_const(float amax) {
  const uint32_t ex = (__float_as_uint(amax) >> 23) & 0xFFu;
  if (ex >= 64u && ex <= 190u) {
    const float r = 1.0f / (float)D;  // folded at compile time, correctly rounded
    const float q0 = __fmul_rn(amax, r);
    const float e = __fmaf_rn(-q0, (float)D, amax);
    return __fmaf_rn(e, r, q0);
  }
  return __fdiv_rn(amax, (float)D);
}

// ---- int8 -----------------------------------------------------------------

__device__ __forceinline__ int f32_to_s32_rne(float q) {  // NaN -> 0
  int r;
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(r) : "f"(q));
  return r;
}

// Saturate four ints to signed bytes and pack them, e0 in the lowest byte.
__device__ __forceinline__ uint32_t pack_s8x4(int e0, int e1, int e2, int e3) {
  uint32_t hi, d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e3), "r"(e2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(e1), "r"(e0), "r"(hi));
  return d;
}

// The rare scales that Markstein's sequence does not cover (all-ones significand, extreme exponents) take the IEEE
// division; out of line, so that the common path carries neither its code nor its registers.
__device__ __noinline__ int int8_code_by_division(float x, float scale) { return f32_to_s32_rne(__fdiv_rn(x, scale)); }

// NW words (two BF16 each) of one lane -> NW/2 words of four codes.
template <int NW, bool kMulInv>
__device__ __forceinline__ void encode_int8(const uint32_t* raw, float amax, float& scale, uint32_t* out) {
  scale = div_const<127>(amax);
  if (kMulInv) {
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      const uint32_t w0 = raw[2 * i], w1 = raw[2 * i + 1];
      out[i] = pack_s8x4(max(f32_to_s32_rne(__fmul_rn(bf16lo(w0), inv)), -127), max(f32_to_s32_rne(__fmul_rn(bf16hi(w0), inv)), -127),
                         max(f32_to_s32_rne(__fmul_rn(bf16lo(w1), inv)), -127), max(f32_to_s32_rne(__fmul_rn(bf16hi(w1), inv)), -127));  // -inf would pack as -128
    }
  } else if (markstein_ok(scale)) {
    const float inv = __frcp_rn(scale);
    auto q = [&](float x) {
      const float q0 = __fmul_rn(x, inv);
      const float e = __fmaf_rn(-q0, scale, x);
      return f32_to_s32_rne(__fmaf_rn(e, inv, q0));
    };
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      const uint32_t w0 = raw[2 * i], w1 = raw[2 * i + 1];
      out[i] = pack_s8x4(q(bf16lo(w0)), q(bf16hi(w0)), q(bf16lo(w1)), q(bf16hi(w1)));
    }
  } else if (amax == 0.0f) {
    // every element is zero or NaN: x / 0 is NaN either way, which converts to 0
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) out[i] = 0u;
  } else {
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      const uint32_t w0 = raw[2 * i], w1 = raw[2 * i + 1];
      out[i] = pack_s8x4(int8_code_by_division(bf16lo(w0), scale), int8_code_by_division(bf16hi(w0), scale),
                         int8_code_by_division(bf16lo(w1), scale), int8_code_by_division(bf16hi(w1), scale));
    }
  }
}

// ---- FP8 E4M3, the reference's encoder (src/cuda/fp8_quant.cu:19-57) --------
// Exact scalar restatement in integer arithmetic: adding 1<<19 to the magnitude
// bits rounds the mantissa half-up to 3 bits with carry into the exponent; >>20
// leaves exponent*8+mant; -960 re-biases (127-7)*8.  Anything that lands in
// exponent 15 (>= 248) becomes 0x7F.  Magnitudes under 2^-6 use the reference's
// float formula (int)(v*512 + 0.5f) clamped to 7.  The sign comes from `y < 0`,
// so -0.0 encodes as 0x00 while a negative value that rounds to zero is 0x80.
// `x` is the element before scaling: a NaN result takes x's sign bit (the
// reference leaves NaN undefined; this is this library's definition).
__device__ __forceinline__ uint32_t fp8_encode_ref(float y, float x) {
  const uint32_t b = __float_as_uint(y);
  const uint32_t a = b & 0x7FFFFFFFu;
  uint32_t c = ((a + 0x80000u) >> 20) - 960u;
  c = (c >= 120u) ? 0x7Fu : c;
  if (a < 0x3C800000u) {
    const float w = __fadd_rn(__fmul_rn(__uint_as_float(a), 512.0f), 0.5f);
    // floor(w) for 0 <= w < 16: add 2^23 rounding down, read the low bits.
    c = min(__float_as_uint(__fadd_rd(w, 8388608.0f)) & 0xFu, 7u);
  }
  uint32_t s = (y < 0.0f) ? 0x80u : 0u;
  if (a > 0x7F800000u) { s = (__float_as_uint(x) >> 24) & 0x80u; c = 0x7Fu; }
  return s | c;
}

// y = x * inv, except that a zero element stays zero even when inv is infinite.
__device__ __forceinline__ float scaled(float x, float inv) { return x == 0.0f ? x : __fmul_rn(x, inv); }
__device__ __forceinline__ uint32_t fp8_encode_ref_scaled(float x, float inv) { return fp8_encode_ref(scaled(x, inv), x); }
// The element-wise entry point keeps the reference's result for the plain product x * inv in every case
// (src/cuda/fp8_quant.cu:69-70): when the product is NaN (a NaN element, 0 * inf, inf * 0, a NaN inv) none of
// the reference's comparisons holds, its frexpf leaves the exponent 0 and the mantissa converts to 0: 0x30.
__device__ __forceinline__ uint32_t fp8_encode_legacy(float x, float inv) {
  const float y = __fmul_rn(x, inv);
  return (y != y) ? 0x30u : fp8_encode_ref(y, x);
}
// Out of line: called for the few elements the fast path cannot decide, so that the common path carries neither
// the exact encoder's code nor its registers.
template <bool kLegacy>
__device__ __noinline__ uint32_t fp8_encode_exact(float x, float inv) {
  return kLegacy ? fp8_encode_legacy(x, inv) : fp8_encode_ref_scaled(x, inv);
}
__device__ __noinline__ uint32_t fp8_encode_ocp_scaled(float x, float inv) {
  uint16_t r;
  const float y = scaled(x, inv);
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(y));
  return r & 0xFFu;
}

// Fast form of the same encoder for a lane's worth of magnitudes, two at a time,
// on the conversion hardware.  For 2^-6 <= |y| < 248 the reference rounds the
// mantissa half-UP; the hardware converter rounds half-to-even.  Truncating |y|
// to FP16 and setting the lowest mantissa bit moves every value strictly off
// the rounding boundaries (they are FP16 numbers with a zero low bit) without
// crossing one, and puts exact ties just above: round-to-nearest-even of that
// equals round-half-up of |y|.  |y| >= 248 must give 0x7F: those lanes are made
// NaN, which the converter encodes as 0x7F.  Zero gives 0.  `min_all` collects the
// smallest magnitude seen, for the element-wise entry point (see
// fp8_encode_words_ref; the block codecs do not read it and the compiler drops it).
template <bool kNanPropagates = false>
__device__ __forceinline__ uint32_t fp8_encode_pair_fast(float ylo_abs, float yhi_abs, __half2& min_all) {
  uint32_t h;
  asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(yhi_abs), "f"(ylo_abs));
  const __half2 hh = *reinterpret_cast<const __half2*>(&h);
  min_all = kNanPropagates ? __hmin2_nan(min_all, hh) : __hmin2(min_all, hh);  // default: a NaN lane is ignored
  // (The same NaN can be made on the FMA pipe, clamp(8h - 1983, 0, 1) * 65504 added to h and the infinity turned into NaN
  // by z*0 + z: identical bytes, three half-precision FMAs for one compare, measured no faster.)
  const uint32_t sat = __hge2_mask(hh, __half2half2(__ushort_as_half((unsigned short)0x5BC0)));  // 248.0
  const uint32_t h2 = h | 0x00010001u | sat;
  uint16_t c;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c) : "r"(h2));
  return c;  // low byte = code(ylo), high byte = code(yhi); bit 7 may be set on saturated lanes
}

// NW words (two BF16 each) of one lane with the reference encoder: codes of x * inv, inv finite and positive.
// The words carry the sign bits.  The hardware path gives every element its code and the sign bit of x; its
// sub-normal codes 1..7 are the reference's for every binary32 magnitude.  Two codes can differ and are looked at
// again:
//   0x08: the hardware rounds a magnitude in [7.5, 8) * 2^-9 up to the smallest normal code, the reference clamps
//         it to 7;
//   0x00: a zero product keeps sign 0 whatever the element's sign (`val < 0` is false for -0.0), and the float just
//         under 2^-10 gives 1 in the reference's `v * 512 + 0.5f` where exact half-up rounding gives 0.
// (code & 0x77) is zero for exactly those two codes: (that | 0x80) - 1 keeps bit 7 of every other byte, without
// borrowing across bytes, and the AND over a lane's words says whether any of its elements needs the second look.
// kLegacy (the element-wise entry point): a NaN element also needs it (the reference's 0x30); there a running FP16
// minimum that propagates NaN is the test, and code 0x7F counts as unsettled too.  The block codecs keep NaN on
// the fast path (saturation code, sign of x).
template <int NW, bool kLegacy = false>
__device__ __forceinline__ void fp8_encode_words_ref(const uint32_t* raw, float inv, uint32_t* out) {
  __half2 min_all = __half2half2(__ushort_as_half((unsigned short)0x7BFF));  // 65504; unused (and dropped) unless kLegacy
  uint32_t all_settled = 0x80808080u;
#pragma unroll
  for (int i = 0; i < NW / 2; ++i) {
    const uint32_t w0 = raw[2 * i], w1 = raw[2 * i + 1];
    const uint32_t c01 = fp8_encode_pair_fast<kLegacy>(__fmul_rn(fabsf(bf16lo(w0)), inv), __fmul_rn(fabsf(bf16hi(w0)), inv), min_all);
    const uint32_t c23 = fp8_encode_pair_fast<kLegacy>(__fmul_rn(fabsf(bf16lo(w1)), inv), __fmul_rn(fabsf(bf16hi(w1)), inv), min_all);
    const uint32_t mag = __byte_perm(c01, c23, 0x5410);
    const uint32_t sgn = __byte_perm(w0, w1, 0x7531);  // high bytes of the four BF16
    out[i] = (mag & 0x7F7F7F7Fu) | (sgn & 0x80808080u);
    if (!kLegacy) all_settled &= ((mag & 0x77777777u) | 0x80808080u) - 0x01010101u;
  }
  // kLegacy: anything below 2^-6 (0x2400 in FP16), zero included, or NaN?
  const bool careful = kLegacy ? !__hge(__hmin_nan(__low2half(min_all), __high2half(min_all)), __ushort_as_half((unsigned short)0x2400))
                               : (all_settled & 0x80808080u) != 0x80808080u;
  if (careful) {
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      uint32_t o = out[i];
      const uint32_t mag = o & 0x7F7F7F7Fu;
      uint32_t settled = (((mag & 0x77777777u) | 0x80808080u) - 0x01010101u) & 0x80808080u;
      if (kLegacy) settled &= ~((mag + 0x01010101u) & 0x80808080u);
      if (settled == 0x80808080u) continue;
      // A loop over the word's unsettled bytes with the exact restatement in its body: a loop is not turned into
      // predicated code (as straight-line code the 32 copies of this arm were, and every warp that met one small
      // element executed them all: 0.32 of the HBM rate on SwiGLU outputs), and a kernel without a call keeps its
      // registers (with the restatement out of line: 0.77 on the same data against 0.82 this way).
      uint32_t todo = (~settled >> 7) & 0x01010101u;   // one bit per unsettled byte, at the byte's lowest bit
      do {
        const int b = __ffs(todo) - 1;                 // 0, 8, 16 or 24
        todo &= todo - 1;
        const uint32_t rw = (b & 16) ? raw[2 * i + 1] : raw[2 * i];
        const float x = (b & 8) ? bf16hi(rw) : bf16lo(rw);
        const float y = __fmul_rn(fabsf(x), inv);
        if (kLegacy ? !(y >= 0.015625f) : (y < 0.015625f)) {
          const uint32_t code = kLegacy ? fp8_encode_legacy(x, inv) : fp8_encode_ref_scaled(x, inv);
          o = (o & ~(0xFFu << b)) | (code << b);
        }
      } while (todo);
      out[i] = o;
    }
  }
}

// OCP E4M3: round-to-nearest-even, saturate to +-448.  The hardware converter
// does exactly this (NaN -> 0x7F/0xFF).
__device__ __forceinline__ uint32_t fp8_encode_ocp_pair(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int NW, bool kOcp>
__device__ __forceinline__ void encode_fp8(const uint32_t* raw, float amax, float& scale, uint32_t* out) {
  scale = div_const<448>(amax);
  if (amax == 0.0f) {  // all-zero block: codes 0, scale 0
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) out[i] = 0u;
    return;
  }
  const float inv = __frcp_rn(scale);  // == RN(1/scale)
  if (!(inv < 3.0e38f)) {  // sub-normal scale: 1/scale overflowed; exact element-wise path
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      uint32_t w = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t rw = raw[2 * i + (k >> 1)];
        const float xv = (k & 1) ? bf16hi(rw) : bf16lo(rw);
        w |= (kOcp ? fp8_encode_ocp_scaled(xv, inv) : fp8_encode_exact<false>(xv, inv)) << (8 * k);
      }
      out[i] = w;
    }
    return;
  }
  if (kOcp) {
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) {
      const uint32_t w0 = raw[2 * i], w1 = raw[2 * i + 1];
      out[i] = fp8_encode_ocp_pair(__fmul_rn(bf16lo(w0), inv), __fmul_rn(bf16hi(w0), inv)) |
               (fp8_encode_ocp_pair(__fmul_rn(bf16lo(w1), inv), __fmul_rn(bf16hi(w1), inv)) << 16);
    }
    return;
  }
  fp8_encode_words_ref<NW>(raw, inv, out);
}

// NW words of one lane, whose block has absolute maximum `amax`: the block's scale and the lane's codes.
template <int kCodec, bool kFlag, int NW>
__device__ __forceinline__ void encode_block_part(const uint32_t* raw, float amax, float& scale, uint32_t* out) {
  if (kCodec == kCodecInt8) encode_int8<NW, kFlag>(raw, amax, scale, out);
  else encode_fp8<NW, kFlag>(raw, amax, scale, out);
}

// Where a block's output goes (see the header comment on packed chunks).
struct OutAddr {
  uint8_t* codes;
  float* scales;
};
__device__ __forceinline__ OutAddr locate(uint8_t* base, const PackedLayout& L, size_t elem0) {
  size_t c = 0, within = elem0;
  if (elem0 >= L.chunk_elems) { c = elem0 / L.chunk_elems; within = elem0 - c * L.chunk_elems; }
  uint8_t* cb = base + (int64_t)c * L.chunk_stride;
  const int64_t so = (c == L.last_chunk) ? L.scales_off_last : L.scales_off;
  return {cb + within, reinterpret_cast<float*>(cb + so) + within / 128};
}
__device__ __forceinline__ OutAddr locate(const uint8_t* base, const PackedLayout& L, size_t elem0) {
  return locate(const_cast<uint8_t*>(base), L, elem0);
}

// ---- job table ----------------------------------------------------------------
// One launch can serve several tensors (the saved activations of one checkpointed
// block are pushed together): the table lists them with the index of each one's
// first tile, and thread blocks walk the concatenated tile space.
struct CodecJob {
  const void* in;   // compress: BF16 source; dequantise: packed base
  void* out;        // compress: packed base; dequantise: BF16 destination
  size_t n;
  PackedLayout L;
  uint32_t tile0;   // first tile of this job in the launch's tile space
  uint32_t pad;
};
constexpr int kMaxJobs = 48;
struct JobTable {
  uint32_t count;
  uint32_t total_tiles;
  CodecJob jobs[kMaxJobs];
};
static_assert(sizeof(JobTable) <= 4000, "kernel parameters must stay under 4 KB");

// ---- compress kernel --------------------------------------------------------
// Requires per job: in 32-byte aligned; every chunk's codes and scales 16-byte
// aligned; chunk_elems a multiple of 16384 (or >= n).  A job's last tile may be
// ragged: it uses predicated loads and direct stores.

// 16 elements of a lane where eight lanes hold a block (the producers below): 16 codes out.
template <int kCodec, bool kFlag>
__device__ __forceinline__ uint4 compress_lane(const U32x8& raw, float& scale) {
  const float amax = absmax_8lanes(absmax_words<8>(raw.v));
  uint32_t c[kLaneElems / 4];
  encode_block_part<kCodec, kFlag, 8>(raw.v, amax, scale, c);
  return make_uint4(c[0], c[1], c[2], c[3]);
}

// 32 consecutive elements of a lane where four lanes hold a block: 32 codes out.
struct Lane32 { uint32_t w[16]; };
template <int kCodec, bool kFlag>
__device__ __forceinline__ void compress_lane32(const Lane32& raw, float& scale, uint4& c_lo, uint4& c_hi) {
  const float amax = absmax_4lanes(absmax_words<16>(raw.w));
  uint32_t c[kCompLaneElems / 4];
  encode_block_part<kCodec, kFlag, 16>(raw.w, amax, scale, c);
  c_lo = make_uint4(c[0], c[1], c[2], c[3]);
  c_hi = make_uint4(c[4], c[5], c[6], c[7]);
}

__device__ __forceinline__ Lane32 load_lane32(const uint16_t* p) {
  const U32x8 a = ld_stream32(p), b = ld_stream32(p + kLaneElems);
  Lane32 r;
#pragma unroll
  for (int i = 0; i < 8; ++i) { r.w[i] = a.v[i]; r.w[8 + i] = b.v[i]; }
  return r;
}

// Ragged last tile of a job: `rem` (< 8192) elements starting at tin / o.
template <int kCodec, bool kFlag>
__device__ __forceinline__ void compress_ragged_tile(const uint16_t* __restrict__ tin, const OutAddr o, size_t rem, int tid) {
  const size_t e0 = (size_t)tid * kCompLaneElems;
  // whole warps enter together so the shuffles stay converged
  if ((size_t)(tid & ~31) * kCompLaneElems >= rem) return;
  Lane32 r;
#pragma unroll
  for (int i = 0; i < 16; ++i) r.w[i] = 0u;
  if (e0 + kCompLaneElems <= rem) {
    r = load_lane32(tin + e0);
  } else if (e0 < rem) {
    for (size_t i = 0; e0 + i < rem; ++i) {
      const uint32_t h = tin[e0 + i];
      r.w[i >> 1] |= (i & 1) ? (h << 16) : h;
    }
  }
  float scale;
  uint4 c_lo, c_hi;
  compress_lane32<kCodec, kFlag>(r, scale, c_lo, c_hi);
  if (e0 + kCompLaneElems <= rem) {
    *reinterpret_cast<uint4*>(o.codes + e0) = c_lo;
    *reinterpret_cast<uint4*>(o.codes + e0 + 16) = c_hi;
  } else if (e0 < rem) {
    const uint32_t c[8] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w, c_hi.x, c_hi.y, c_hi.z, c_hi.w};
    for (size_t i = 0; e0 + i < rem; ++i) o.codes[e0 + i] = (uint8_t)(c[i >> 2] >> (8 * (i & 3)));
  }
  if ((tid & (kCompLanesPerBlock - 1)) == 0 && e0 < rem) o.scales[e0 / 128] = scale;
}

// One full tile: encode the lane's 32 elements and write codes and scale.
// kStaged = false: two 16-byte stores per lane, one lane in four stores the scale.
// kStaged = true : the warp's 1024 codes and 8 scales go to the warp's own shared-memory slice (two slices, taking
//                  turns) and lane 0 sends them out as two bulk asynchronous copies.  Only the warp synchronises:
//                  before a slice is written again, lane 0 waits until the bulk group issued from it two tiles ago
//                  has been read.
template <int kCodec, bool kFlag, bool kStaged>
__device__ __forceinline__ void compress_full_tile(const Lane32& raw, const OutAddr o, int tid, uint8_t* smem, int& buf) {
  float scale;
  uint4 c_lo, c_hi;
  compress_lane32<kCodec, kFlag>(raw, scale, c_lo, c_hi);
  if (!kStaged) {
    uint8_t* dst = o.codes + tid * kCompLaneElems;
    __stcs(reinterpret_cast<uint4*>(dst), c_lo);
    __stcs(reinterpret_cast<uint4*>(dst + 16), c_hi);
    if ((tid & (kCompLanesPerBlock - 1)) == 0) o.scales[tid / kCompLanesPerBlock] = scale;
  } else {
    const int lane = tid & 31, warp = tid >> 5;
    uint8_t* slice = smem + (warp * 2 + buf) * kWarpSliceBytes;
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
    *reinterpret_cast<uint4*>(slice + lane * kCompLaneElems) = c_lo;
    *reinterpret_cast<uint4*>(slice + lane * kCompLaneElems + 16) = c_hi;
    if ((lane & (kCompLanesPerBlock - 1)) == 0) reinterpret_cast<float*>(slice + kWarpCodes)[lane / kCompLanesPerBlock] = scale;
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      bulk_store(o.codes + warp * kWarpCodes, slice, kWarpCodes);
      bulk_store(o.scales + warp * kWarpScales, slice + kWarpCodes, kWarpScales * sizeof(float));
      bulk_commit();
    }
    buf ^= 1;
  }
}

// Round k of every thread block works on tile k*grid + block of the launch's
// tile space; the host sizes the grid so that all blocks run the same number of
// rounds (see grid_balanced).
// kForm 0: load a tile, encode it, store it; five resident blocks per SM (48 registers).
// kForm 1: software-pipelined: the loads of a block's next tile are issued before the current tile is encoded, so
//          a thread always has a tile's worth of loads in flight.  Twice the input registers: four resident blocks.
// kForm 2: as form 0 with four resident blocks (64 registers).
// Same tile order, same results.
constexpr int kCompressForms = 3;
template <int kForm>
struct CompressForm {
  static constexpr bool kPipelined = kForm == 1;
  static constexpr int kMinBlocks = kForm == 0 ? 5 : 4;
};

template <int kCodec, bool kFlag, bool kStaged, int kForm>
__global__ void __launch_bounds__(kThreads, CompressForm<kForm>::kMinBlocks)
compress_b128_kernel(const __grid_constant__ JobTable T, unsigned rounds, unsigned multi_ctas, unsigned multi_tiles) {
  pdl_prologue();
  // staged variant only: two slices of (codes | scales) per warp in dynamic shared memory
  extern __shared__ __align__(128) uint8_t smem_tiles[];
  constexpr bool kPipelined = CompressForm<kForm>::kPipelined;
  const int tid = threadIdx.x;
  int buf = 0;
  // Blocks below multi_ctas take `rounds` tiles each out of the first multi_tiles (tile k*multi_ctas + b in
  // round k, so blocks that run side by side read neighbouring tiles); the blocks after them take one tile
  // each of the rest.  Blocks start in index order, so the launch ends on short blocks and the SMs run dry
  // within one tile's time of each other instead of one long block's.
  const bool multi = blockIdx.x < multi_ctas;
  uint32_t j = 0;
  // tile of round k for this block, or false
  auto tile_of = [&](unsigned k, uint32_t& g) -> bool {
    if (k >= rounds) return false;
    if (multi) {
      g = k * multi_ctas + blockIdx.x;
      if (g >= multi_tiles) return false;
    } else {
      if (k) return false;
      g = multi_tiles + (blockIdx.x - multi_ctas);
    }
    return g < T.total_tiles;
  };
  // A tile is remembered as (job, tile within the job); the job's pointers and layout stay in the parameter bank.
  struct Where { uint32_t job, tile; bool ok, full; };
  auto resolve = [&](unsigned k) -> Where {
    Where w{0u, 0u, false, false};
    uint32_t g = 0;
    w.ok = tile_of(k, g);
    if (!w.ok) return w;
    while (j + 1 < T.count && g >= T.jobs[j + 1].tile0) ++j;
    w.job = j;
    w.tile = g - T.jobs[j].tile0;
    w.full = ((size_t)w.tile + 1) * kTileElems <= T.jobs[j].n;
    return w;
  };
  auto in_of = [&](const Where& w) { return static_cast<const uint16_t*>(T.jobs[w.job].in) + (size_t)w.tile * kTileElems; };
  Where cur = resolve(0);
  Lane32 nxt;
  if (kPipelined && cur.ok && cur.full) nxt = load_lane32(in_of(cur) + (size_t)tid * kCompLaneElems);
  for (unsigned k = 0; cur.ok; ++k) {
    Lane32 raw;
    Where next{0u, 0u, false, false};
    if (kPipelined) {
      raw = nxt;
      next = resolve(k + 1);
      if (next.ok && next.full) nxt = load_lane32(in_of(next) + (size_t)tid * kCompLaneElems);
    } else if (cur.full) {
      raw = load_lane32(in_of(cur) + (size_t)tid * kCompLaneElems);
    }
    const CodecJob& J = T.jobs[cur.job];
    const size_t e_tile = (size_t)cur.tile * kTileElems;
    const OutAddr o = locate(static_cast<uint8_t*>(J.out), J.L, e_tile);
    if (cur.full) compress_full_tile<kCodec, kFlag, kStaged>(raw, o, tid, smem_tiles, buf);
    else compress_ragged_tile<kCodec, kFlag>(in_of(cur), o, J.n - e_tile, tid);
    cur = kPipelined ? next : resolve(k + 1);
  }
  if (kStaged && (tid & 31) == 0) bulk_wait_all<0>();
}

// Any alignment, any n: one warp per 128-element block, scalar accesses.
template <int kCodec, bool kFlag>
__global__ void __launch_bounds__(kThreads)
compress_b128_generic_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, size_t n, PackedLayout L) {
  const size_t nblocks = (n + 127) / 128;
  const int lane = threadIdx.x & 31;
  const size_t warp0 = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (kThreads / 32);
  for (size_t blk = warp0; blk < nblocks; blk += nwarps) {
    const size_t e0 = blk * 128 + (size_t)lane * 4;
    uint32_t raw[2] = {0u, 0u};
    for (int i = 0; i < 4; ++i)
      if (e0 + i < n) raw[i >> 1] |= (uint32_t)in[e0 + i] << (16 * (i & 1));
    float m = absmax_words<2>(raw);
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 16));
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 8));
    const float amax = absmax_8lanes(m);
    float scale;
    uint32_t c[1];
    encode_block_part<kCodec, kFlag, 2>(raw, amax, scale, c);
    const OutAddr o = locate(out, L, blk * 128);
    for (int i = 0; i < 4; ++i)
      if (e0 + i < n) o.codes[(size_t)lane * 4 + i] = (uint8_t)(c[0] >> (8 * i));
    if (lane == 0) o.scales[0] = scale;
  }
}

// ---- dequantise -------------------------------------------------------------

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Signed byte k of w as a float, exactly: 2^23 + (code ^ 0x80) - (2^23 + 128).
template <int k>
__device__ __forceinline__ float s8_to_f32(uint32_t w_flipped) {
  const uint32_t bits = __byte_perm(w_flipped, 0x4B000000u, 0x7650 | k);
  return __fsub_rn(__uint_as_float(bits), 8388736.0f);
}

// Decoder of src/cuda/fp8_dequant.cu:20-36 without branches: the 7 magnitude
// bits placed at bit 20 form a binary32 whose value is dec * 2^-120, including
// the sub-normals and 0x7F (-> 480).  The sign is carried on the bits.
template <int k>
__device__ __forceinline__ float fp8_to_f32_scaled(uint32_t w) {
  const uint32_t byte = (w >> (8 * k)) & 0xFFu;
  const uint32_t bits = ((byte & 0x7Fu) << 20) | ((byte & 0x80u) << 24);
  return __fmul_rn(__uint_as_float(bits), 1.329227995784916e36f);  // * 2^120, exact
}

// Four codes in one word -> two words of BF16.
template <int kCodec>
__device__ __forceinline__ void decode4(uint32_t c, float scale, uint32_t& o0, uint32_t& o1) {
  float v0, v1, v2, v3;
  if (kCodec == kCodecInt8) {
    const uint32_t a = c ^ 0x80808080u;
    v0 = s8_to_f32<0>(a); v1 = s8_to_f32<1>(a); v2 = s8_to_f32<2>(a); v3 = s8_to_f32<3>(a);
  } else {
    v0 = fp8_to_f32_scaled<0>(c); v1 = fp8_to_f32_scaled<1>(c); v2 = fp8_to_f32_scaled<2>(c); v3 = fp8_to_f32_scaled<3>(c);
  }
  o0 = pack_bf16x2(__fmul_rn(v0, scale), __fmul_rn(v1, scale));
  o1 = pack_bf16x2(__fmul_rn(v2, scale), __fmul_rn(v3, scale));
}

template <int kCodec>
__device__ __forceinline__ uint16_t decode1(uint8_t c, float scale) {
  uint32_t o0, o1;
  decode4<kCodec>(c, scale, o0, o1);
  return (uint16_t)(o0 & 0xFFFFu);
}

// Requires per job: every chunk's codes 16-byte aligned, out 32-byte aligned.
// Each thread turns 16 codes (one 16-byte load) into 16 BF16 (one 32-byte
// store); the 8 lanes of a block read the same scale, which the L1 serves.
// Tiles are 16384 elements; a job's last tile is predicated per 16-element
// vector and its last (up to 15) elements are handled one per thread.
template <int kCodec>
__global__ void __launch_bounds__(kThreads, 5)
dequant_b128_kernel(const __grid_constant__ JobTable T, unsigned rounds) {
  pdl_prologue();
  constexpr int kDU = kDequantUnroll;
  const int tid = threadIdx.x;
  uint32_t j = 0;
  for (unsigned k = 0; k < rounds; ++k) {
    const uint32_t g = k * gridDim.x + blockIdx.x;
    if (g >= T.total_tiles) break;
    while (j + 1 < T.count && g >= T.jobs[j + 1].tile0) ++j;
    const CodecJob& J = T.jobs[j];
    const size_t e_tile = (size_t)(g - J.tile0) * kDequantTileElems;
    const size_t nvec = (J.n - e_tile) / kLaneElems;  // whole vectors from here to the end of the job
    const OutAddr A = locate(static_cast<const uint8_t*>(J.in), J.L, e_tile);  // a tile never straddles chunks
    uint16_t* out = static_cast<uint16_t*>(J.out) + e_tile;
    uint4 c[kDU];
    float s[kDU];
#pragma unroll
    for (int u = 0; u < kDU; ++u) {
      const int lv = u * kThreads + tid;
      if ((size_t)lv < nvec) {
        c[u] = __ldcs(reinterpret_cast<const uint4*>(A.codes + (size_t)lv * kLaneElems));
        s[u] = __ldg(A.scales + lv / kLanesPerBlock);
      }
    }
#pragma unroll
    for (int u = 0; u < kDU; ++u) {
      const int lv = u * kThreads + tid;
      if ((size_t)lv < nvec) {
        U32x8 o;
        decode4<kCodec>(c[u].x, s[u], o.v[0], o.v[1]);
        decode4<kCodec>(c[u].y, s[u], o.v[2], o.v[3]);
        decode4<kCodec>(c[u].z, s[u], o.v[4], o.v[5]);
        decode4<kCodec>(c[u].w, s[u], o.v[6], o.v[7]);
        st_stream32(out + (size_t)lv * kLaneElems, o);
      }
    }
    // up to 15 trailing elements of the job, in its last tile
    if (nvec < (size_t)kThreads * kDU) {
      const size_t t0 = nvec * kLaneElems, left = J.n - e_tile - t0;
      if ((size_t)tid < left) {
        const size_t e = t0 + tid;
        out[e] = decode1<kCodec>(A.codes[e], A.scales[e / 128]);
      }
    }
  }
}

template <int kCodec>
__global__ void __launch_bounds__(kThreads)
dequant_b128_generic_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, size_t n, PackedLayout L) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride) {
    const OutAddr a = locate(in, L, e & ~(size_t)127);
    out[e] = decode1<kCodec>(a.codes[e & 127], a.scales[0]);
  }
}

// ---- element-wise FP8 with a caller-supplied scale --------------------------
// Same arithmetic as flame_bf16_to_fp8 / flame_fp8_to_bf16 in the reference; 16
// elements per thread per iteration with the fast encoder where it applies.

__global__ void __launch_bounds__(kThreads)
bf16_to_fp8_vec_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, float inv_scale, size_t n) {
  const size_t nvec = n / kLaneElems;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    const U32x8 r = ld_stream32(in + v * kLaneElems);
    uint32_t c[4];
    if ((inv_scale > 0.0f) && (inv_scale < 3.0e38f)) {  // the sign of x*inv_scale is the sign of x
      fp8_encode_words_ref<8, true>(r.v, inv_scale, c);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        c[i] = fp8_encode_legacy(bf16lo(r.v[2 * i]), inv_scale) | (fp8_encode_legacy(bf16hi(r.v[2 * i]), inv_scale) << 8) |
               (fp8_encode_legacy(bf16lo(r.v[2 * i + 1]), inv_scale) << 16) | (fp8_encode_legacy(bf16hi(r.v[2 * i + 1]), inv_scale) << 24);
    }
    __stcs(reinterpret_cast<uint4*>(out + v * kLaneElems), make_uint4(c[0], c[1], c[2], c[3]));
  }
  const size_t t0 = nvec * kLaneElems;
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - t0)) {
    const size_t e = t0 + threadIdx.x;
    out[e] = (uint8_t)fp8_encode_legacy(__uint_as_float((uint32_t)in[e] << 16), inv_scale);
  }
}

__global__ void __launch_bounds__(kThreads)
bf16_to_fp8_scalar_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, float inv_scale, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride)
    out[e] = (uint8_t)fp8_encode_legacy(__uint_as_float((uint32_t)in[e] << 16), inv_scale);
}

__global__ void __launch_bounds__(kThreads)
fp8_to_bf16_vec_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, size_t n) {
  const size_t nvec = n / kLaneElems;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    const uint4 c = __ldcs(reinterpret_cast<const uint4*>(in + v * kLaneElems));
    U32x8 o;
    decode4<kCodecFp8>(c.x, scale, o.v[0], o.v[1]);
    decode4<kCodecFp8>(c.y, scale, o.v[2], o.v[3]);
    decode4<kCodecFp8>(c.z, scale, o.v[4], o.v[5]);
    decode4<kCodecFp8>(c.w, scale, o.v[6], o.v[7]);
    st_stream32(out + v * kLaneElems, o);
  }
  const size_t t0 = nvec * kLaneElems;
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - t0)) {
    const size_t e = t0 + threadIdx.x;
    out[e] = decode1<kCodecFp8>(in[e], scale);
  }
}

__global__ void __launch_bounds__(kThreads)
fp8_to_bf16_scalar_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride)
    out[e] = decode1<kCodecFp8>(in[e], scale);
}

// ---- launch helpers ---------------------------------------------------------

int g_max_ctas = 0;  // 0 = default

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev] = v;
  }
  return cached[dev];
}

int grid_for(size_t work_items, int ctas_per_sm, int max_ctas) {
  size_t g = (size_t)sm_count() * (size_t)ctas_per_sm;
  const int cap = max_ctas > 0 ? max_ctas : g_max_ctas;
  if (cap > 0 && g > (size_t)cap) g = (size_t)cap;
  if (g > work_items) g = work_items;
  if (g < 1) g = 1;
  return (int)g;
}

// Resident thread blocks per SM of a kernel, from the occupancy query; remembered per (kernel, dynamic shared
// memory, device).  The key is the kernel's address: different instantiations of one template have the same
// function type, so a cache keyed by type would hand one kernel's answer to another.
int resident_ctas_per_sm(const void* kernel, size_t dyn_smem = 0) {
  struct Entry { const void* k; size_t smem; int dev; int v; };
  static std::mutex mu;
  static std::vector<Entry> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  std::lock_guard<std::mutex> lk(mu);
  for (const Entry& e : cache)
    if (e.k == kernel && e.smem == dyn_smem && e.dev == dev) return e.v;
  int v = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, kernel, kThreads, dyn_smem) != cudaSuccess || v <= 0) v = 4;
  cache.push_back({kernel, dyn_smem, dev, v});
  return v;
}

// What the last compress / dequantise launch of this thread chose (inspection hook for the tests).
thread_local LaunchRecord g_last_launch = {0, 0, 0, 0};

// A grid in which every thread block takes the same number of consecutive tiles
// and all blocks are resident at once: no second wave, no ragged last round.
struct Grid { int ctas; unsigned tiles_per_cta; };
constexpr int kTaperWaves = 2;
// waves of single-tile blocks at the end of an oversubscribed compress launch
// Measured on a B200, one DiT block per launch, 20 launches back to back (fraction of the 6552 GB/s copy rate):
// int8 form 0 / 1 / 2 = 0.95 / 0.91 / 0.98, FP8 = 0.86 / 0.71 / 0.85; with staged stores 0.91 / 0.95 / 0.89 and 0.78 / 0.66 / 0.78.
constexpr int kDefaultFormInt8 = 2, kDefaultFormFp8 = 0;  // see CompressForm
int env_int(const char* name) {
  const char* e = getenv(name);
  return e ? (atoi(e) < 1 ? 1 : atoi(e)) : 0;
}
// Small launches (at most `balance_limit` rounds per block): every block resident, the same number
// of rounds for all, no second wave and no ragged last round.  Large launches: `max_rounds` rounds
// per block and many more blocks than fit at once, so that the hardware block scheduler evens out
// SM speed differences, which add up over hundreds of rounds of a static assignment.  The two
// thresholds were swept on a B200 per kernel kind (compress 8 / 6 with two closing waves of single-tile
// blocks, dequantise 2 / 2);
// FLAME_ACT_BALANCE_LIMIT and FLAME_ACT_MAX_ROUNDS override them for tuning.
Grid grid_balanced(size_t tiles, int ctas_per_sm, int max_ctas, int balance_limit, int max_rounds) {
  static int env_limit = -1, env_rounds = -1;
  if (env_limit < 0) { env_limit = env_int("FLAME_ACT_BALANCE_LIMIT"); env_rounds = env_int("FLAME_ACT_MAX_ROUNDS"); }
  if (env_limit > 0) balance_limit = env_limit;
  if (env_rounds > 0) max_rounds = env_rounds;
  if (tiles == 0) tiles = 1;
  size_t cap = (size_t)sm_count() * (size_t)ctas_per_sm;
  const int lim = max_ctas > 0 ? max_ctas : g_max_ctas;
  const bool capped = lim > 0 && cap > (size_t)lim;
  if (capped) cap = (size_t)lim;
  size_t per = (tiles + cap - 1) / cap;
  if (!capped && per > (size_t)balance_limit) per = (size_t)max_rounds;
  return {(int)((tiles + per - 1) / per), (unsigned)per};
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline bool aligned(int64_t v, int64_t a) { return (v & (a - 1)) == 0; }

bool layout_fast(const void* base, const PackedLayout& L, size_t n) {
  if (!aligned(base, 16) || !aligned(L.scales_off, 16) || !aligned(L.scales_off_last, 16)) return false;
  if (L.chunk_elems >= n) return true;
  return (L.chunk_elems % kDequantTileElems) == 0 && aligned(L.chunk_stride, 16);  // 16384 covers both tile sizes
}

}  // namespace

int set_max_ctas(int v) { const int old = g_max_ctas; g_max_ctas = v < 0 ? 0 : v; return old; }

LaunchRecord last_launch() { return g_last_launch; }

PackedLayout single_chunk_layout(const void* codes, const void* scales, size_t n) {
  PackedLayout L;
  L.chunk_elems = n ? n : 1;
  L.chunk_stride = 0;
  L.scales_off = L.scales_off_last = static_cast<const uint8_t*>(scales) - static_cast<const uint8_t*>(codes);
  L.last_chunk = 0;
  return L;
}

PackedLayout packed_chunks_layout(size_t n, size_t chunk_elems, size_t chunk_stride) {
  PackedLayout L;
  L.chunk_elems = chunk_elems;
  L.chunk_stride = (int64_t)chunk_stride;
  L.last_chunk = n ? (n - 1) / chunk_elems : 0;
  const size_t last_elems = n - L.last_chunk * chunk_elems;
  L.scales_off = (int64_t)((chunk_elems + 255u) & ~(size_t)255u);
  L.scales_off_last = (int64_t)((last_elems + 255u) & ~(size_t)255u);
  return L;
}

namespace {

bool compress_job_fast(const TensorJob& j) { return aligned(j.bf16, 32) && layout_fast(j.packed, j.layout, j.n); }

template <int kTile>
void add_job(JobTable& T, const void* in, void* out, const TensorJob& j) {
  CodecJob& c = T.jobs[T.count++];
  c.in = in; c.out = out; c.n = j.n; c.L = j.layout; c.tile0 = T.total_tiles; c.pad = 0;
  T.total_tiles += (uint32_t)((j.n + kTile - 1) / kTile);
}

template <int kCodec, bool kFlag, bool kStaged, int kForm>
cudaError_t launch_compress_kernel(const JobTable& T, cudaStream_t stream, int max_ctas) {
  auto kern = compress_b128_kernel<kCodec, kFlag, kStaged, kForm>;
  const size_t smem = kStaged ? kStagedSmemBytes : 0;
  const int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(kern), smem);
  const Grid g = grid_balanced(T.total_tiles, per_sm, max_ctas, 8, 6);
  // Oversubscribed launches (several waves of blocks) end on single-tile blocks: `taper` waves of them.
  static int taper = -1;
  if (taper < 0) { const char* e = getenv("FLAME_ACT_TAPER_WAVES"); taper = e ? atoi(e) : kTaperWaves; if (taper < 0) taper = 0; }
  unsigned ctas = (unsigned)g.ctas, multi_ctas = (unsigned)g.ctas, multi_tiles = T.total_tiles;
  const size_t resident = (size_t)sm_count() * (size_t)per_sm;
  const size_t singles = (size_t)taper * resident;
  if (taper > 0 && g.tiles_per_cta > 1 && (size_t)g.ctas > 2 * resident && T.total_tiles > 2 * singles) {
    multi_tiles = T.total_tiles - (uint32_t)singles;
    multi_ctas = (multi_tiles + g.tiles_per_cta - 1) / g.tiles_per_cta;
    ctas = multi_ctas + (unsigned)singles;
  }
  g_last_launch = {(int)ctas, per_sm, (int)g.tiles_per_cta, kForm | (kStaged ? 4 : 0)};
  return launch_after(kern, ctas, kThreads, smem, stream, T, (unsigned)g.tiles_per_cta, multi_ctas, multi_tiles);
}

// Which form of the kernel a codec takes (defaults measured on a B200; FLAME_ACT_COMPRESS_FORM=0/1/2 or
// set_compress_form() override both codecs, for tuning and tests).
std::atomic<int> g_form_override{-2};  // -2: not read from the environment yet; -1: defaults
int compress_form(int codec) {
  int f = g_form_override.load(std::memory_order_relaxed);
  if (f == -2) {
    const char* e = getenv("FLAME_ACT_COMPRESS_FORM");
    f = (e && *e >= '0' && *e < '0' + kCompressForms && e[1] == 0) ? *e - '0' : -1;
    g_form_override.store(f, std::memory_order_relaxed);
  }
  if (f >= 0) return f;
  return codec == kCodecInt8 ? kDefaultFormInt8 : kDefaultFormFp8;
}

template <int kCodec, bool kFlag, bool kStaged>
cudaError_t launch_compress_table(const JobTable& T, cudaStream_t stream, int max_ctas) {
  switch (compress_form(kCodec)) {
    case 1: return launch_compress_kernel<kCodec, kFlag, kStaged, 1>(T, stream, max_ctas);
    case 2: return launch_compress_kernel<kCodec, kFlag, kStaged, 2>(T, stream, max_ctas);
    default: return launch_compress_kernel<kCodec, kFlag, kStaged, 0>(T, stream, max_ctas);
  }
}

cudaError_t launch_compress_table(int codec, unsigned flags, const JobTable& T, cudaStream_t stream, int max_ctas) {
  const bool f = (flags & 1u) != 0, st = (flags & kFlagStagedStores) != 0;
  if (codec == kCodecInt8) {
    if (f) return st ? launch_compress_table<kCodecInt8, true, true>(T, stream, max_ctas) : launch_compress_table<kCodecInt8, true, false>(T, stream, max_ctas);
    return st ? launch_compress_table<kCodecInt8, false, true>(T, stream, max_ctas) : launch_compress_table<kCodecInt8, false, false>(T, stream, max_ctas);
  }
  if (f) return st ? launch_compress_table<kCodecFp8, true, true>(T, stream, max_ctas) : launch_compress_table<kCodecFp8, true, false>(T, stream, max_ctas);
  return st ? launch_compress_table<kCodecFp8, false, true>(T, stream, max_ctas) : launch_compress_table<kCodecFp8, false, false>(T, stream, max_ctas);
}

cudaError_t launch_compress_generic(int codec, unsigned flags, const TensorJob& j, cudaStream_t stream, int max_ctas) {
  const bool flag = (flags & 1u) != 0;
  auto* i = static_cast<const uint16_t*>(j.bf16);
  auto* o = static_cast<uint8_t*>(j.packed);
  const size_t warps = (j.n + 127) / 128;
  const int grid = grid_for((warps + 7) / 8, 8, max_ctas);
  if (codec == kCodecInt8) {
    if (flag) compress_b128_generic_kernel<kCodecInt8, true><<<grid, kThreads, 0, stream>>>(i, o, j.n, j.layout);
    else compress_b128_generic_kernel<kCodecInt8, false><<<grid, kThreads, 0, stream>>>(i, o, j.n, j.layout);
  } else {
    if (flag) compress_b128_generic_kernel<kCodecFp8, true><<<grid, kThreads, 0, stream>>>(i, o, j.n, j.layout);
    else compress_b128_generic_kernel<kCodecFp8, false><<<grid, kThreads, 0, stream>>>(i, o, j.n, j.layout);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_compress_multi(int codec, const TensorJob* jobs, size_t count, unsigned flags, cudaStream_t stream, int max_ctas) {
  JobTable T;
  T.count = 0; T.total_tiles = 0;
  for (size_t k = 0; k < count; ++k) {
    const TensorJob& j = jobs[k];
    if (j.n == 0) continue;
    if (!j.bf16 || !j.packed) return cudaErrorInvalidValue;
    if (!compress_job_fast(j)) {
      cudaError_t e = launch_compress_generic(codec, flags, j, stream, max_ctas);
      if (e != cudaSuccess) return e;
      continue;
    }
    add_job<kTileElems>(T, j.bf16, j.packed, j);
    if (T.count == kMaxJobs) {
      cudaError_t e = launch_compress_table(codec, flags, T, stream, max_ctas);
      if (e != cudaSuccess) return e;
      T.count = 0; T.total_tiles = 0;
    }
  }
  return T.count ? launch_compress_table(codec, flags, T, stream, max_ctas) : cudaSuccess;
}

cudaError_t launch_dequant_multi(int codec, const TensorJob* jobs, size_t count, cudaStream_t stream, int max_ctas) {
  JobTable T;
  T.count = 0; T.total_tiles = 0;
  auto flush = [&]() -> cudaError_t {
    if (T.count == 0) return cudaSuccess;
    if (codec == kCodecInt8) {
      auto kern = dequant_b128_kernel<kCodecInt8>;
      const int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(kern));
      const Grid g = grid_balanced(T.total_tiles, per_sm, max_ctas, 2, 2);
      g_last_launch = {g.ctas, per_sm, (int)g.tiles_per_cta, 0};
      { const cudaError_t e = launch_after(kern, (unsigned)g.ctas, kThreads, 0, stream, T, (unsigned)g.tiles_per_cta); if (e != cudaSuccess) return e; }
    } else {
      auto kern = dequant_b128_kernel<kCodecFp8>;
      const int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(kern));
      const Grid g = grid_balanced(T.total_tiles, per_sm, max_ctas, 2, 2);
      g_last_launch = {g.ctas, per_sm, (int)g.tiles_per_cta, 0};
      { const cudaError_t e = launch_after(kern, (unsigned)g.ctas, kThreads, 0, stream, T, (unsigned)g.tiles_per_cta); if (e != cudaSuccess) return e; }
    }
    T.count = 0; T.total_tiles = 0;
    return cudaGetLastError();
  };
  for (size_t k = 0; k < count; ++k) {
    const TensorJob& j = jobs[k];
    if (j.n == 0) continue;
    if (!j.bf16 || !j.packed) return cudaErrorInvalidValue;
    if (!(aligned(j.bf16, 32) && layout_fast(j.packed, j.layout, j.n))) {
      auto* c = static_cast<const uint8_t*>(j.packed);
      auto* o = static_cast<uint16_t*>(j.bf16);
      const int grid = grid_for((j.n + kThreads - 1) / kThreads, 8, max_ctas);
      if (codec == kCodecInt8) dequant_b128_generic_kernel<kCodecInt8><<<grid, kThreads, 0, stream>>>(c, o, j.n, j.layout);
      else dequant_b128_generic_kernel<kCodecFp8><<<grid, kThreads, 0, stream>>>(c, o, j.n, j.layout);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      continue;
    }
    add_job<kDequantTileElems>(T, j.packed, j.bf16, j);
    if (T.count == kMaxJobs) {
      cudaError_t e = flush();
      if (e != cudaSuccess) return e;
    }
  }
  return flush();
}

cudaError_t launch_compress(int codec, const void* in, void* out, size_t n, const PackedLayout& L,
                            unsigned flags, cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  if (!in || !out) return cudaErrorInvalidValue;
  const TensorJob j{const_cast<void*>(in), out, n, L};
  return launch_compress_multi(codec, &j, 1, flags, stream, max_ctas);
}

cudaError_t launch_dequant(int codec, const void* in, void* out, size_t n, const PackedLayout& L,
                           cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  if (!in || !out) return cudaErrorInvalidValue;
  const TensorJob j{out, const_cast<void*>(in), n, L};
  return launch_dequant_multi(codec, &j, 1, stream, max_ctas);
}

// ---- producers that emit the packed form beside their BF16 output -----------
// The saved tensor of a checkpointed block is usually the output of a
// normalisation or the input of a gated activation.  These two kernels are those
// producers with the compress step built in: the codes and scales they write
// are, bit for bit, what compress_b128_kernel gives for the same BF16 tensor,
// and that tensor is never read again by a compress launch.

namespace {

__device__ __forceinline__ void st_plain32(void* p, const U32x8& r) {  // the next kernel reads it: no streaming hint
  uint4* q = reinterpret_cast<uint4*>(p);
  q[0] = make_uint4(r.v[0], r.v[1], r.v[2], r.v[3]);
  q[1] = make_uint4(r.v[4], r.v[5], r.v[6], r.v[7]);
}

// RMSNorm of src/cuda/fused_rms_norm.cu:26-80: rstd = rsqrt(mean(x^2) + eps), y = bf16((x * rstd) * w), fp32
// arithmetic.  A thread block takes rows blockIdx.x, blockIdx.x + gridDim.x, ...; lane t keeps elements
// [16t, 16t+16) of the row in registers from the one load to the stores, the weights stay in registers across rows,
// and the next row's load is issued before the current row is reduced, so that the row-wide reduction (shuffles,
// one barrier) runs beside a load in flight.  The two buffers of warp sums take turns: a buffer is written again
// only after every thread has passed the barrier of the row in between.  kCodec 0 writes y only.
template <int kCodec, bool kFlag>
__global__ void __launch_bounds__(1024)
rmsnorm_quant_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ y,
                     uint8_t* __restrict__ codes, float* __restrict__ scales, float* __restrict__ rstd_out, uint32_t rows, uint32_t cols, float eps) {
  __shared__ float warp_sums[2][32];
  const int tid = threadIdx.x;
  const bool live = (uint32_t)tid < cols / kLaneElems;
  const int nwarps = (int)(blockDim.x >> 5);
  U32x8 wr;
#pragma unroll
  for (int i = 0; i < 8; ++i) wr.v[i] = 0u;
  if (live) {
    const uint4* wp = reinterpret_cast<const uint4*>(w + (size_t)tid * kLaneElems);
    const uint4 a = __ldg(wp), b = __ldg(wp + 1);
    wr.v[0] = a.x; wr.v[1] = a.y; wr.v[2] = a.z; wr.v[3] = a.w; wr.v[4] = b.x; wr.v[5] = b.y; wr.v[6] = b.z; wr.v[7] = b.w;
  }
  uint32_t row = blockIdx.x;
  U32x8 nxt;
#pragma unroll
  for (int i = 0; i < 8; ++i) nxt.v[i] = 0u;
  if (live && row < rows) nxt = ld_stream32(x + (size_t)row * cols + (size_t)tid * kLaneElems);
  for (int parity = 0; row < rows; row += gridDim.x, parity ^= 1) {
    const U32x8 r = nxt;
    const uint32_t next_row = row + gridDim.x;
    if (live && next_row < rows) nxt = ld_stream32(x + (size_t)next_row * cols + (size_t)tid * kLaneElems);
    const size_t e0 = (size_t)row * cols + (size_t)tid * kLaneElems;
    float v[kLaneElems];
    unpack16(r, v);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < kLaneElems; ++i) s = __fmaf_rn(v[i], v[i], s);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, d);
    if ((tid & 31) == 0) warp_sums[parity][tid >> 5] = s;
    __syncthreads();
    float tot = 0.0f;  // every thread adds the warp sums in the same order: one value for the whole row
    for (int k = 0; k < nwarps; ++k) tot += warp_sums[parity][k];
    const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(tot, (float)cols), eps));
    if (rstd_out && tid == 0) rstd_out[row] = rstd;
    U32x8 o;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o.v[i] = pack_bf16x2(__fmul_rn(__fmul_rn(v[2 * i], rstd), bf16lo(wr.v[i])), __fmul_rn(__fmul_rn(v[2 * i + 1], rstd), bf16hi(wr.v[i])));
    if (live) st_plain32(y + e0, o);
    if (kCodec != 0) {
      float scale;
      const uint4 c = compress_lane<kCodec == 0 ? kCodecInt8 : kCodec, kFlag>(o, scale);  // dead lanes hold zeros and sit in groups of their own
      if (live) {
        __stcs(reinterpret_cast<uint4*>(codes + e0), c);
        if ((tid & (kLanesPerBlock - 1)) == 0) scales[e0 / 128] = scale;
      }
    }
  }
}

// SwiGLU: gate_up is [rows, 2*hidden] (gate columns, then up columns); h = bf16(silu(gate) * up) in fp32 arithmetic.
// The codes and scales are those of gate_up, the tensor the backward pass needs (src/autograd.rs:326-331).
// Four resident blocks per SM (64 registers): the launcher sizes the grid for four, and a fifth of the blocks waiting for a
// second wave costs more than the few registers do (measured: 84 µs against 70 µs with int8 codes at the DiT shape).
template <int kCodec, bool kFlag>
__global__ void __launch_bounds__(kThreads, 4)
swiglu_quant_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ h, uint8_t* __restrict__ codes,
                    float* __restrict__ scales, size_t rows, uint32_t hidden) {
  const uint32_t lanes_per_row = hidden / kLaneElems;
  const size_t total = rows * lanes_per_row;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const int tid = threadIdx.x;
  for (size_t base = (size_t)blockIdx.x * kThreads + (tid & ~31); base < total; base += stride) {  // whole warps together
    const size_t L = base + (tid & 31);
    const bool live = L < total;
    const size_t row = live ? L / lanes_per_row : 0;
    const uint32_t c0 = live ? (uint32_t)(L - row * lanes_per_row) * kLaneElems : 0;
    const size_t eg = row * 2 * (size_t)hidden + c0, eu = eg + hidden;
    U32x8 g, u;
#pragma unroll
    for (int i = 0; i < 8; ++i) g.v[i] = u.v[i] = 0u;
    if (live) { g = ld_stream32(gu + eg); u = ld_stream32(gu + eu); }
    float gv[kLaneElems], uv[kLaneElems];
    unpack16(g, gv);
    unpack16(u, uv);
    U32x8 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // sigmoid by the hardware exponential and reciprocal (each within a few units in the last place of fp32,
      // far below the BF16 rounding of the result)
      const float a = __fmul_rn(__fmul_rn(gv[2 * i], __fdividef(1.0f, 1.0f + __expf(-gv[2 * i]))), uv[2 * i]);
      const float b = __fmul_rn(__fmul_rn(gv[2 * i + 1], __fdividef(1.0f, 1.0f + __expf(-gv[2 * i + 1]))), uv[2 * i + 1]);
      o.v[i] = pack_bf16x2(a, b);
    }
    if (live) st_plain32(h + row * (size_t)hidden + c0, o);
    if (kCodec != 0) {
      float sg, su;
      const uint4 cg = compress_lane<kCodec == 0 ? kCodecInt8 : kCodec, kFlag>(g, sg);
      const uint4 cu = compress_lane<kCodec == 0 ? kCodecInt8 : kCodec, kFlag>(u, su);
      if (live) {
        __stcs(reinterpret_cast<uint4*>(codes + eg), cg);
        __stcs(reinterpret_cast<uint4*>(codes + eu), cu);
        if ((tid & (kLanesPerBlock - 1)) == 0) { scales[eg / 128] = sg; scales[eu / 128] = su; }
      }
    }
  }
}

template <typename F>
cudaError_t by_codec(int codec, unsigned flags, F&& f) {
  const bool fl = (flags & 1u) != 0;
  if (codec == 0) return f(std::integral_constant<int, 0>(), std::false_type());
  if (codec == kCodecInt8) return fl ? f(std::integral_constant<int, kCodecInt8>(), std::true_type()) : f(std::integral_constant<int, kCodecInt8>(), std::false_type());
  if (codec == kCodecFp8) return fl ? f(std::integral_constant<int, kCodecFp8>(), std::true_type()) : f(std::integral_constant<int, kCodecFp8>(), std::false_type());
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_rmsnorm_quant(int codec, unsigned flags, const void* x, const void* w, void* y, void* codes, void* scales,
                                 void* rstd_out, size_t rows, size_t cols, float eps, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  if (!x || !w || !y || (codec != 0 && (!codes || !scales))) return cudaErrorInvalidValue;
  if (cols % 128 != 0 || cols > 16384 || rows > 0x7FFFFFFFull) return cudaErrorInvalidValue;
  if (!aligned(x, 32) || !aligned(w, 16) || !aligned(y, 16) || (codec != 0 && (!aligned(codes, 16) || !aligned(scales, 4)))) return cudaErrorInvalidValue;
  const int threads = (int)((cols / kLaneElems + 31) / 32 * 32);
  return by_codec(codec, flags, [&](auto c, auto f) {
    auto kern = rmsnorm_quant_kernel<decltype(c)::value, decltype(f)::value>;
    // Every block resident at once and the same number of rows for each (as nearly as the row count allows).
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0) != cudaSuccess || per_sm <= 0) per_sm = 1;
    const size_t resident = (size_t)sm_count() * (size_t)per_sm;
    const size_t rows_per_block = (rows + resident - 1) / resident;
    const unsigned grid = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    kern<<<grid, threads, 0, stream>>>(
        static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w), static_cast<uint16_t*>(y),
        static_cast<uint8_t*>(codes), static_cast<float*>(scales), static_cast<float*>(rstd_out), (uint32_t)rows, (uint32_t)cols, eps);
    return cudaGetLastError();
  });
}

cudaError_t launch_swiglu_quant(int codec, unsigned flags, const void* gate_up, void* h, void* codes, void* scales,
                                size_t rows, size_t hidden, cudaStream_t stream, int max_ctas) {
  if (rows == 0 || hidden == 0) return cudaSuccess;
  if (!gate_up || !h || (codec != 0 && (!codes || !scales))) return cudaErrorInvalidValue;
  if (hidden % 128 != 0 || hidden > 0x7FFFFFFFull / 2) return cudaErrorInvalidValue;
  if (!aligned(gate_up, 32) || !aligned(h, 16) || (codec != 0 && (!aligned(codes, 16) || !aligned(scales, 4)))) return cudaErrorInvalidValue;
  const size_t lanes = rows * (hidden / kLaneElems);
  const int grid = grid_for((lanes + kThreads - 1) / kThreads, 4, max_ctas);
  return by_codec(codec, flags, [&](auto c, auto f) {
    swiglu_quant_kernel<decltype(c)::value, decltype(f)::value><<<grid, kThreads, 0, stream>>>(
        static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(h), static_cast<uint8_t*>(codes), static_cast<float*>(scales),
        rows, (uint32_t)hidden);
    return cudaGetLastError();
  });
}

cudaError_t launch_bf16_to_fp8(const void* in, void* out, float inv_scale, size_t n, cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  auto* i = static_cast<const uint16_t*>(in);
  auto* o = static_cast<uint8_t*>(out);
  if (aligned(in, 32) && aligned(out, 16)) {
    // as for the block codecs: a few rounds per thread block instead of hundreds of rounds of a fixed grid
    const int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(bf16_to_fp8_vec_kernel));
    const Grid g = grid_balanced((n / kLaneElems + kThreads - 1) / kThreads + 1, per_sm, max_ctas, 8, 6);
    bf16_to_fp8_vec_kernel<<<g.ctas, kThreads, 0, stream>>>(i, o, inv_scale, n);
  } else {
    const int grid = grid_for((n + kThreads - 1) / kThreads, 8, max_ctas);
    bf16_to_fp8_scalar_kernel<<<grid, kThreads, 0, stream>>>(i, o, inv_scale, n);
  }
  return cudaGetLastError();
}

cudaError_t launch_fp8_to_bf16(const void* in, void* out, float scale, size_t n, cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  auto* i = static_cast<const uint8_t*>(in);
  auto* o = static_cast<uint16_t*>(out);
  if (aligned(in, 16) && aligned(out, 32)) {
    const int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(fp8_to_bf16_vec_kernel));
    const Grid g = grid_balanced((n / kLaneElems + kThreads - 1) / kThreads + 1, per_sm, max_ctas, 2, 2);
    fp8_to_bf16_vec_kernel<<<g.ctas, kThreads, 0, stream>>>(i, o, scale, n);
  } else {
    const int grid = grid_for((n + kThreads - 1) / kThreads, 8, max_ctas);
    fp8_to_bf16_scalar_kernel<<<grid, kThreads, 0, stream>>>(i, o, scale, n);
  }
  return cudaGetLastError();
}

int default_compress_form(int codec) { return compress_form(codec); }
int set_compress_form(int form) {
  const int old = g_form_override.load(std::memory_order_relaxed);
  g_form_override.store((form >= 0 && form < kCompressForms) ? form : -1, std::memory_order_relaxed);
  return old < 0 ? -1 : old;
}

namespace {
template <int kCodec, bool kFlag, bool kStaged>
const void* compress_kernel_address(int form) {
  switch (form) {
    case 1: return reinterpret_cast<const void*>(compress_b128_kernel<kCodec, kFlag, kStaged, 1>);
    case 2: return reinterpret_cast<const void*>(compress_b128_kernel<kCodec, kFlag, kStaged, 2>);
    default: return reinterpret_cast<const void*>(compress_b128_kernel<kCodec, kFlag, kStaged, 0>);
  }
}
template <int kCodec>
const void* compress_kernel_address(bool f, bool st, int form) {
  if (f) return st ? compress_kernel_address<kCodec, true, true>(form) : compress_kernel_address<kCodec, true, false>(form);
  return st ? compress_kernel_address<kCodec, false, true>(form) : compress_kernel_address<kCodec, false, false>(form);
}
}  // namespace

int query_resident_ctas(int codec, unsigned flags, int form, bool compress) {
  const bool f = (flags & 1u) != 0, st = (flags & kFlagStagedStores) != 0;
  const void* k = nullptr;
  if (!compress) {
    k = codec == kCodecInt8 ? reinterpret_cast<const void*>(dequant_b128_kernel<kCodecInt8>) : reinterpret_cast<const void*>(dequant_b128_kernel<kCodecFp8>);
  } else {
    if (form < 0) form = compress_form(codec);
    k = codec == kCodecInt8 ? compress_kernel_address<kCodecInt8>(f, st, form) : compress_kernel_address<kCodecFp8>(f, st, form);
  }
  int v = 0;
  const size_t smem = (compress && st) ? kStagedSmemBytes : 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, k, kThreads, smem) != cudaSuccess) return -1;
  return v;
}

}  // namespace flame_b200
