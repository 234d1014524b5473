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
// memory and moves one element per thread per access.  Here a warp owns a tile of 64 rows x 32 columns and
// needs no shared memory: lane (rg, cg) = (lane / 4, lane % 4) loads the 8-byte pieces of rows 8rg..8rg+7 at
// columns 8cg..8cg+7 (a row's 32 bytes are one full sector across the four lanes), transposes its 8x8
// bytes in registers with byte permutes, decodes on the conversion hardware, and writes for each of its
// eight columns the eight rows as one 16-byte store; the eight row groups make 128 contiguous bytes per
// output row.  Requires M % 8 == 0, N % 8 == 0, an 8-byte aligned input and a 16-byte aligned output;
// anything else takes the element-per-thread kernel.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "codec_kernels.cuh"

namespace flame_b200 {
namespace {

constexpr int kWThreads = 256;
constexpr int kTileRows = 64, kTileCols = 32;   // one warp: 8 row groups of 8 rows x 4 column groups of 8 columns

__device__ __forceinline__ uint32_t pack_bf16x2_w(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Four codes (one per byte of w) -> two words of BF16.  The conversion hardware turns two E4M3 bytes into two FP16
// values exactly (sub-normals, signed zero, exponent 15 with a zero mantissa = 256 included); FP16 -> FP32 is exact
// too, so one fp32 multiply by the scale and the rounding to BF16 are the reference's `val *= scale` and
// `__float2bfloat16`.  Where the hardware and the reference's decoder differ (exponent 15 with a mantissa of 1..6:
// 288..448 to the hardware, NaN to the reference), `nan_bits` says so: bit 7 of byte k is set when code k is one of
// the decoder's NaN codes.
__device__ __forceinline__ void decode4_weight(uint32_t w, uint32_t nan_bits, float scale, uint32_t& o0, uint32_t& o1) {
  uint32_t h01, h23;
  asm("{ .reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi; }" : "=r"(h01), "=r"(h23) : "r"(w));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h01)), b = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  float v0 = a.x, v1 = a.y, v2 = b.x, v3 = b.y;
  if (nan_bits) {  // rare: weights do not normally hold these codes
    const float qnan = __uint_as_float(0x7FC00000u);
    if (nan_bits & 0x00000080u) v0 = qnan;
    if (nan_bits & 0x00008000u) v1 = qnan;
    if (nan_bits & 0x00800000u) v2 = qnan;
    if (nan_bits & 0x80000000u) v3 = qnan;
  }
  o0 = pack_bf16x2_w(__fmul_rn(v0, scale), __fmul_rn(v1, scale));
  o1 = pack_bf16x2_w(__fmul_rn(v2, scale), __fmul_rn(v3, scale));
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
fp8_dequant_transpose_tiles_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale,
                                   int M, int N, uint32_t tiles_n, uint64_t tiles) {
  const int lane = threadIdx.x & 31, rg = lane >> 2, cg = lane & 3;
  const uint64_t warp0 = (uint64_t)blockIdx.x * (kWThreads / 32) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (kWThreads / 32);
  for (uint64_t t = warp0; t < tiles; t += nwarps) {
    const int tm = (int)(t / tiles_n), tn = (int)(t - (uint64_t)tm * tiles_n);
    const int row0 = tm * kTileRows + rg * 8, col0 = tn * kTileCols + cg * 8;
    if (row0 >= M || col0 >= N) continue;       // M % 8 == 0 and N % 8 == 0: a lane's 8x8 piece is inside or outside as a whole
    uint2 r[8];                                  // row j of the piece: columns 0..3 in .x, 4..7 in .y
    const uint8_t* src = in + (size_t)row0 * N + col0;
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __ldcs(reinterpret_cast<const uint2*>(src + (size_t)j * N));
    uint16_t* dst = out + (size_t)col0 * M + row0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {       // columns 0..3, then 4..7
      uint32_t lo[4], hi[4];                     // per column: rows 0..3 and rows 4..7 of the piece
      { const uint32_t a[4] = {half ? r[0].y : r[0].x, half ? r[1].y : r[1].x, half ? r[2].y : r[2].x, half ? r[3].y : r[3].x}; transpose4x4_bytes(a, lo); }
      { const uint32_t a[4] = {half ? r[4].y : r[4].x, half ? r[5].y : r[5].x, half ? r[6].y : r[6].x, half ? r[7].y : r[7].x}; transpose4x4_bytes(a, hi); }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 o;
        decode4_weight(lo[c], nan_codes(lo[c]), scale, o.x, o.y);
        decode4_weight(hi[c], nan_codes(hi[c]), scale, o.z, o.w);
        __stcs(reinterpret_cast<uint4*>(dst + (size_t)(4 * half + c) * M), o);
      }
    }
  }
}

// Any M, N and alignment: one element per thread, reads coalesced along N.
__global__ void __launch_bounds__(kWThreads)
fp8_dequant_transpose_generic_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, int M, int N) {
  const size_t total = (size_t)M * N, stride = (size_t)gridDim.x * kWThreads;
  for (size_t e = (size_t)blockIdx.x * kWThreads + threadIdx.x; e < total; e += stride) {
    const size_t m = e / N, n = e - m * N;
    const uint32_t w = in[e];
    uint32_t o0, o1;
    decode4_weight(w, nan_codes(w) & 0x80u, scale, o0, o1);
    out[n * M + m] = (uint16_t)(o0 & 0xFFFFu);
  }
}

}  // namespace

cudaError_t launch_fp8_dequant_transpose(const void* in, void* out, float scale, int M, int N, cudaStream_t stream, int max_ctas) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  if (!in || !out) return cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool fast = (M % 8 == 0) && (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(in) & 7u) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  if (fast) {
    const uint32_t tiles_n = (uint32_t)((N + kTileCols - 1) / kTileCols);
    const uint64_t tiles = (uint64_t)((M + kTileRows - 1) / kTileRows) * tiles_n;
    uint64_t grid = (tiles + kWThreads / 32 - 1) / (kWThreads / 32);
    uint64_t cap = (uint64_t)sms * 8;
    if (max_ctas > 0 && (uint64_t)max_ctas < cap) cap = (uint64_t)max_ctas;
    if (grid > cap) grid = cap;
    fp8_dequant_transpose_tiles_kernel<<<(unsigned)grid, kWThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<uint16_t*>(out), scale,
                                                                                 M, N, tiles_n, tiles);
  } else {
    const size_t total = (size_t)M * N;
    uint64_t grid = (total + kWThreads - 1) / kWThreads;
    if (grid > (uint64_t)sms * 8) grid = (uint64_t)sms * 8;
    fp8_dequant_transpose_generic_kernel<<<(unsigned)grid, kWThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<uint16_t*>(out), scale,
                                                                                   M, N);
  }
  return cudaGetLastError();
}

}  // namespace flame_b200
