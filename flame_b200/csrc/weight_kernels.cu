// FP8 E4M3 weights -> BF16 with the transpose built in, written for sm_100a.
//
// Takes the place of src/cuda/fused_dequant_transpose.cu in the reference (called from
// src/ops/fused_inference.rs:140-175): input [M, N] row-major FP8 bytes, output [N, M] row-major
// BF16, out[n][m] = bf16_rn(dec(in[m][n]) * scale).  The decoder is that file's: sub-normals
// mant * 2^-9, (1 + mant/8) * 2^(exp-7) for exponents 1..14, exponent 15 with a zero mantissa is 256
// and exponent 15 with any other mantissa is NaN (that file's reading of E4M3, not OCP's), the sign
// applied last, one fp32 multiply by the scale, round-to-nearest-even to BF16.
//
// HBM-bound byte work: 1 B read + 2 B written per element.  The reference stages a 32x32 tile in shared
// memory and moves one element per thread per access.  Here a warp owns a 32x32 tile and needs no
// shared memory: lane (rg, cg) = (lane / 8, lane % 8) loads the 4-byte pieces of rows 8rg..8rg+7 at
// columns 4cg..4cg+3 (a row's 32 bytes are one full sector across the eight lanes), transposes its
// 8x4 bytes in registers with byte permutes, decodes, and writes for each of its four columns the eight
// rows as one 16-byte store; the four row groups make 64 contiguous bytes (two full sectors) per
// output row.  Requires M % 8 == 0, N % 4 == 0 and 16-byte aligned pointers; anything else takes the
// element-per-thread kernel.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "codec_kernels.cuh"

namespace flame_b200 {
namespace {

constexpr int kWThreads = 256;

__device__ __forceinline__ uint32_t pack_bf16x2_w(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte k of w as the decoder's value times `s2`, where s2 = scale * 2^120 when that is finite: the seven
// magnitude bits placed at bit 20 are dec * 2^-120 as a binary32 (sub-normals included), so one multiply gives
// RN(dec * scale), the same rounding of the same real number as the reference's val *= scale.  `two_step`
// (scale * 2^120 overflows) multiplies by 2^120 first, which is exact, then by the scale.
template <int k>
__device__ __forceinline__ float fp8_weight_value(uint32_t w, float s2, float scale, bool two_step) {
  const uint32_t t = __byte_perm(w, 0u, 0x0444 | (k << 12));  // byte k at bits 24..31, zeros below
  const uint32_t bits = ((t & 0x7F000000u) >> 4) | (t & 0x80000000u);
  const float v = __uint_as_float(bits);
  return two_step ? __fmul_rn(__fmul_rn(v, 1.329227995784916e36f), scale) : __fmul_rn(v, s2);
}

// Four codes (one per byte of w) -> two words of BF16; `nan_bits` has bit 7 of byte k set when code k is one of
// the decoder's NaN codes (exponent 15, mantissa not zero).
__device__ __forceinline__ void decode4_weight(uint32_t w, uint32_t nan_bits, float s2, float scale, bool two_step, uint32_t& o0, uint32_t& o1) {
  float v0 = fp8_weight_value<0>(w, s2, scale, two_step), v1 = fp8_weight_value<1>(w, s2, scale, two_step);
  float v2 = fp8_weight_value<2>(w, s2, scale, two_step), v3 = fp8_weight_value<3>(w, s2, scale, two_step);
  if (nan_bits) {  // rare: weights do not normally hold NaN codes
    const float qnan = __uint_as_float(0x7FC00000u);
    if (nan_bits & 0x00000080u) v0 = qnan;
    if (nan_bits & 0x00008000u) v1 = qnan;
    if (nan_bits & 0x00800000u) v2 = qnan;
    if (nan_bits & 0x80000000u) v3 = qnan;
  }
  o0 = pack_bf16x2_w(v0, v1);
  o1 = pack_bf16x2_w(v2, v3);
}

// bit 7 of each byte: (code & 0x7F) > 0x78
__device__ __forceinline__ uint32_t nan_codes(uint32_t w) { return ((w & 0x7F7F7F7Fu) + 0x07070707u) & 0x80808080u; }

// rows r0..r3 (4 bytes each: columns c0..c3) -> columns c0..c3 (4 bytes each: rows r0..r3)
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t (&r)[4], uint32_t (&c)[4]) {
  const uint32_t a0 = __byte_perm(r[0], r[1], 0x5140), a1 = __byte_perm(r[0], r[1], 0x7362);  // (r0c0 r1c0 r0c1 r1c1), (r0c2 r1c2 r0c3 r1c3)
  const uint32_t b0 = __byte_perm(r[2], r[3], 0x5140), b1 = __byte_perm(r[2], r[3], 0x7362);
  c[0] = __byte_perm(a0, b0, 0x5410);
  c[1] = __byte_perm(a0, b0, 0x7632);
  c[2] = __byte_perm(a1, b1, 0x5410);
  c[3] = __byte_perm(a1, b1, 0x7632);
}

__global__ void __launch_bounds__(kWThreads)
fp8_dequant_transpose_tiles_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, float s2, int two_step_i,
                                   int M, int N, uint32_t tiles_n, uint64_t tiles) {
  const bool two_step = two_step_i != 0;
  const int lane = threadIdx.x & 31, rg = lane >> 3, cg = lane & 7;
  const uint64_t warp0 = (uint64_t)blockIdx.x * (kWThreads / 32) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (kWThreads / 32);
  for (uint64_t t = warp0; t < tiles; t += nwarps) {
    const int tm = (int)(t / tiles_n), tn = (int)(t - (uint64_t)tm * tiles_n);
    const int row0 = tm * 32 + rg * 8, col0 = tn * 32 + cg * 4;
    if (row0 >= M || col0 >= N) continue;       // M % 8 == 0 and N % 4 == 0: a lane's 8x4 piece is inside or outside as a whole
    uint32_t r[8];
    const uint8_t* src = in + (size_t)row0 * N + col0;
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __ldcs(reinterpret_cast<const uint32_t*>(src + (size_t)j * N));
    uint32_t lo[4], hi[4];                       // per column: rows 0..3 and rows 4..7 of the piece
    { const uint32_t a[4] = {r[0], r[1], r[2], r[3]}; transpose4x4_bytes(a, lo); }
    { const uint32_t a[4] = {r[4], r[5], r[6], r[7]}; transpose4x4_bytes(a, hi); }
    uint16_t* dst = out + (size_t)col0 * M + row0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 o;
      decode4_weight(lo[c], nan_codes(lo[c]), s2, scale, two_step, o.x, o.y);
      decode4_weight(hi[c], nan_codes(hi[c]), s2, scale, two_step, o.z, o.w);
      __stcs(reinterpret_cast<uint4*>(dst + (size_t)c * M), o);
    }
  }
}

// Any M, N and alignment: one element per thread, reads coalesced along N.
__global__ void __launch_bounds__(kWThreads)
fp8_dequant_transpose_generic_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, float s2, int two_step_i, int M, int N) {
  const bool two_step = two_step_i != 0;
  const size_t total = (size_t)M * N, stride = (size_t)gridDim.x * kWThreads;
  for (size_t e = (size_t)blockIdx.x * kWThreads + threadIdx.x; e < total; e += stride) {
    const size_t m = e / N, n = e - m * N;
    const uint32_t w = in[e];
    uint32_t o0, o1;
    decode4_weight(w, nan_codes(w) & 0x80u, s2, scale, two_step, o0, o1);
    out[n * M + m] = (uint16_t)(o0 & 0xFFFFu);
  }
}

}  // namespace

cudaError_t launch_fp8_dequant_transpose(const void* in, void* out, float scale, int M, int N, cudaStream_t stream, int max_ctas) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  if (!in || !out) return cudaErrorInvalidValue;
  // scale * 2^120 in one constant when it stays finite and normal (any practical weight scale); else two multiplies
  const float s2 = scale * 1.329227995784916e36f;
  uint32_t s2b;
  memcpy(&s2b, &s2, sizeof(s2b));
  const uint32_t ex = (s2b >> 23) & 0xFFu;
  const int two_step = (ex == 0u || ex == 0xFFu) ? 1 : 0;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool fast = (M % 8 == 0) && (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 3u) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  if (fast) {
    const uint32_t tiles_n = (uint32_t)((N + 31) / 32);
    const uint64_t tiles = (uint64_t)((M + 31) / 32) * tiles_n;
    uint64_t grid = (tiles + kWThreads / 32 - 1) / (kWThreads / 32);
    uint64_t cap = (uint64_t)sms * 8;
    if (max_ctas > 0 && (uint64_t)max_ctas < cap) cap = (uint64_t)max_ctas;
    if (grid > cap) grid = cap;
    fp8_dequant_transpose_tiles_kernel<<<(unsigned)grid, kWThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<uint16_t*>(out), scale, s2,
                                                                                 two_step, M, N, tiles_n, tiles);
  } else {
    const size_t total = (size_t)M * N;
    uint64_t grid = (total + kWThreads - 1) / kWThreads;
    if (grid > (uint64_t)sms * 8) grid = (uint64_t)sms * 8;
    fp8_dequant_transpose_generic_kernel<<<(unsigned)grid, kWThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<uint16_t*>(out), scale, s2,
                                                                                   two_step, M, N);
  }
  return cudaGetLastError();
}

}  // namespace flame_b200
