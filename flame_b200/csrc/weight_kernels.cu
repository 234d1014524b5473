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
// anything else takes a kernel that moves 64 x 64 tiles through shared memory.  Several weights can share one launch (a job table in
// the kernel's parameters); the grid is one wave of resident blocks in which every warp takes the same
// number of tiles.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "codec_kernels.cuh"
#include "../../include/flame_offload.h"

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
template <bool kNanCodes>
__device__ __forceinline__ void decode4_weight(uint32_t w, uint32_t nan_bits, float scale, uint32_t& o0, uint32_t& o1) {
  uint32_t h01, h23;
  asm("{ .reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi; }" : "=r"(h01), "=r"(h23) : "r"(w));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h01)), b = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  float v0 = a.x, v1 = a.y, v2 = b.x, v3 = b.y;
  if (kNanCodes) {
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

// A lane's 8x8 piece (row j: columns 0..3 in r[j].x, 4..7 in r[j].y) transposed, decoded and written: column c of the
// piece is eight consecutive BF16 of output row c, one 16-byte store.
template <bool kNanCodes>
__device__ __forceinline__ void piece_out(const uint2 (&r)[8], float scale, uint16_t* dst, size_t M) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {       // columns 0..3, then 4..7
    uint32_t lo[4], hi[4];                     // per column: rows 0..3 and rows 4..7 of the piece
    { const uint32_t a[4] = {half ? r[0].y : r[0].x, half ? r[1].y : r[1].x, half ? r[2].y : r[2].x, half ? r[3].y : r[3].x}; transpose4x4_bytes(a, lo); }
    { const uint32_t a[4] = {half ? r[4].y : r[4].x, half ? r[5].y : r[5].x, half ? r[6].y : r[6].x, half ? r[7].y : r[7].x}; transpose4x4_bytes(a, hi); }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 o;
      decode4_weight<kNanCodes>(lo[c], kNanCodes ? nan_codes(lo[c]) : 0u, scale, o.x, o.y);
      decode4_weight<kNanCodes>(hi[c], kNanCodes ? nan_codes(hi[c]) : 0u, scale, o.z, o.w);
      __stcs(reinterpret_cast<uint4*>(dst + (size_t)(4 * half + c) * M), o);
    }
  }
}

// Up to kMaxWeightJobs weights in one launch: the tiles of all jobs form one range, which the warps of the grid share
// round-robin.  A block of a transformer has a handful of weights of 10-60 M elements; its caller issues one launch for
// them instead of one each (on the GPU the two measure the same within 3 %).
constexpr int kMaxWeightJobs = 16;
struct WeightJobs {
  const uint8_t* in[kMaxWeightJobs];
  uint16_t* out[kMaxWeightJobs];
  uint32_t first_tile[kMaxWeightJobs + 1];   // first_tile[count] = all tiles (the launcher keeps a table under 2^31 tiles)
  float scale[kMaxWeightJobs];
  int M[kMaxWeightJobs], N[kMaxWeightJobs];
  uint32_t tiles_n[kMaxWeightJobs];
  int count;
};

__global__ void __launch_bounds__(kWThreads, 6)
fp8_dequant_transpose_tiles_kernel(const __grid_constant__ WeightJobs T) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, rg = lane >> 2, cg = lane & 3;
  const uint32_t warp0 = blockIdx.x * (kWThreads / 32) + (threadIdx.x >> 5);
  const uint32_t nwarps = gridDim.x * (kWThreads / 32);
  const uint32_t tiles = T.first_tile[T.count];
  int job = 0;
  for (uint32_t t = warp0; t < tiles; t += nwarps) {
    while (t >= T.first_tile[job + 1]) ++job;    // tiles only move forward
    const uint8_t* __restrict__ in = T.in[job];
    uint16_t* __restrict__ out = T.out[job];
    const float scale = T.scale[job];
    const int M = T.M[job], N = T.N[job];
    const uint32_t tiles_n = T.tiles_n[job];
    const uint32_t tj = t - T.first_tile[job];
    const int tm = (int)(tj / tiles_n), tn = (int)(tj - (uint32_t)tm * tiles_n);
    const int row0 = tm * kTileRows + rg * 8, col0 = tn * kTileCols + cg * 8;
    if (row0 >= M || col0 >= N) continue;       // M % 8 == 0 and N % 8 == 0: a lane's 8x8 piece is inside or outside as a whole
    uint2 r[8];                                  // row j of the piece: columns 0..3 in .x, 4..7 in .y
    const uint8_t* src = in + (size_t)row0 * N + col0;
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __ldcs(reinterpret_cast<const uint2*>(src + (size_t)j * N));
    uint16_t* dst = out + (size_t)col0 * M + row0;
    // Does the piece hold one of the decoder's NaN codes?  Weights normally do not: the test is made once per piece and
    // the common path carries no per-element selects (as predicated code they were a quarter of all issued instructions).
    uint32_t any_nan = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) any_nan |= nan_codes(r[j].x) | nan_codes(r[j].y);
    if (any_nan == 0) piece_out<false>(r, scale, dst, (size_t)M);
    else piece_out<true>(r, scale, dst, (size_t)M);
  }
}

// Any M, N and alignment: a thread block moves a tile of 64 x 64 codes through shared memory, so that the reads run
// along N (32 consecutive bytes per warp and row) and the writes along M (32 consecutive BF16 per warp and output row).
constexpr int kGenTile = 64;
__global__ void __launch_bounds__(kWThreads)
fp8_dequant_transpose_generic_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, int M, int N,
                                     uint32_t tiles_n, uint32_t tiles) {
  __shared__ uint8_t tile[kGenTile][kGenTile + 1];
  for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const uint32_t tm = t / tiles_n, tn = t - tm * tiles_n;
    const size_t m0 = (size_t)tm * kGenTile, n0 = (size_t)tn * kGenTile;
#pragma unroll 4
    for (int i = threadIdx.x; i < kGenTile * kGenTile; i += kWThreads) {
      const int r = i / kGenTile, c = i % kGenTile;
      if (m0 + r < (size_t)M && n0 + c < (size_t)N) tile[r][c] = in[(m0 + r) * N + n0 + c];
    }
    __syncthreads();
#pragma unroll 4
    for (int i = threadIdx.x; i < kGenTile * kGenTile; i += kWThreads) {
      const int c = i / kGenTile, r = i % kGenTile;
      if (m0 + r < (size_t)M && n0 + c < (size_t)N) {
        const uint32_t w = tile[r][c];
        uint32_t o0, o1;
        decode4_weight<true>(w, nan_codes(w) & 0x80u, scale, o0, o1);
        out[(n0 + c) * M + m0 + r] = (uint16_t)(o0 & 0xFFFFu);
      }
    }
    __syncthreads();
  }
}

// Resident blocks per SM of the tile kernel, asked once per device.
int resident_tile_blocks_per_sm(int dev) {
  static std::atomic<int> cached[64];
  if (dev < 0 || dev >= 64) return 4;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, fp8_dequant_transpose_tiles_kernel, kWThreads, 0) != cudaSuccess || v <= 0) v = 4;
  cached[dev].store(v, std::memory_order_relaxed);
  return v;
}

}  // namespace

cudaError_t launch_fp8_dequant_transpose_jobs(const FlameWeightJob* jobs, int count, cudaStream_t stream, int max_ctas) {
  if (count <= 0) return cudaSuccess;
  if (!jobs) return cudaErrorInvalidValue;
  for (int i = 0; i < count; ++i) {
    if (jobs[i].M < 0 || jobs[i].N < 0) return cudaErrorInvalidValue;
    if (jobs[i].M > 0 && jobs[i].N > 0 && (!jobs[i].input_fp8 || !jobs[i].output_bf16)) return cudaErrorInvalidValue;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // One wave of resident blocks, every warp the same number of tiles (a grid of 8 blocks per SM where 6 fit ran a third of a
  // second wave on an otherwise idle GPU).
  uint64_t cap = (uint64_t)sms * (uint64_t)resident_tile_blocks_per_sm(dev);
  if (max_ctas > 0 && (uint64_t)max_ctas < cap) cap = (uint64_t)max_ctas;
  const uint64_t warps_per_block = kWThreads / 32;
  WeightJobs T;
  T.count = 0;
  T.first_tile[0] = 0;
  auto flush = [&]() -> cudaError_t {
    if (T.count == 0) return cudaSuccess;
    const uint64_t tiles = T.first_tile[T.count];
    const uint64_t rounds = (tiles + cap * warps_per_block - 1) / (cap * warps_per_block);
    uint64_t grid = (tiles + rounds * warps_per_block - 1) / (rounds * warps_per_block);
    if (grid > cap) grid = cap;
    const cudaError_t e = launch_after(fp8_dequant_transpose_tiles_kernel, (unsigned)grid, kWThreads, 0, stream, T);
    T.count = 0;
    return e;
  };
  for (int i = 0; i < count; ++i) {
    const int M = jobs[i].M, N = jobs[i].N;
    if (M == 0 || N == 0) continue;
    const uint8_t* in = static_cast<const uint8_t*>(jobs[i].input_fp8);
    uint16_t* out = static_cast<uint16_t*>(jobs[i].output_bf16);
    const uint64_t job_tiles = (uint64_t)((M + kTileRows - 1) / kTileRows) * (uint64_t)((N + kTileCols - 1) / kTileCols);
    const bool fast = (M % 8 == 0) && (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(in) & 7u) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) &&
                      job_tiles < (1ull << 30);
    if (!fast) {
      const uint64_t gt_n = ((uint64_t)N + kGenTile - 1) / kGenTile, gt = (((uint64_t)M + kGenTile - 1) / kGenTile) * gt_n;   // < 2^52 / 4096
      if (gt >= (1ull << 32)) return cudaErrorInvalidValue;
      uint64_t grid = gt;
      if (grid > (uint64_t)sms * 8) grid = (uint64_t)sms * 8;
      fp8_dequant_transpose_generic_kernel<<<(unsigned)grid, kWThreads, 0, stream>>>(in, out, jobs[i].scale, M, N, (uint32_t)gt_n, (uint32_t)gt);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      continue;
    }
    if (T.count > 0 && (uint64_t)T.first_tile[T.count] + job_tiles >= (1ull << 31)) {
      const cudaError_t e = flush();
      if (e != cudaSuccess) return e;
    }
    const int j = T.count++;
    T.in[j] = in; T.out[j] = out; T.scale[j] = jobs[i].scale; T.M[j] = M; T.N[j] = N;
    T.tiles_n[j] = (uint32_t)((N + kTileCols - 1) / kTileCols);
    T.first_tile[j + 1] = T.first_tile[j] + (uint32_t)job_tiles;
    if (T.count == kMaxWeightJobs) {
      const cudaError_t e = flush();
      if (e != cudaSuccess) return e;
    }
  }
  return flush();
}

cudaError_t launch_fp8_dequant_transpose(const void* in, void* out, float scale, int M, int N, cudaStream_t stream, int max_ctas) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  const FlameWeightJob job = {in, out, scale, M, N, 0};
  return launch_fp8_dequant_transpose_jobs(&job, 1, stream, max_ctas);
}

}  // namespace flame_b200
