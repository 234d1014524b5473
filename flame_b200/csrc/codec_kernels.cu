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
// an instruction count per element that stays under the issue budget.
//
// Compress tile: 256 threads x 4 x 16-byte loads = 8192 elements = 64 blocks of
// 128.  Sixteen consecutive lanes hold one block, so the block's absmax is four
// shuffles inside a half-warp.  Codes and scales are written into a shared
// memory tile (double buffered) and leave the SM as two bulk asynchronous
// copies (cp.async.bulk.global.shared::cta), so the store path costs one
// instruction per tile instead of one per thread.  Cluster size is 1 and no
// multicast is used anywhere.
//
// Arithmetic is IEEE binary32 throughout: this file must be compiled WITHOUT
// --use_fast_math and without -ftz; the operations whose rounding matters use
// the explicit _rn intrinsics so that no FMA contraction can change a result.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "codec_kernels.cuh"

namespace flame_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;                                   // BF16 per 16-byte load
constexpr int kUnroll = 4;                                // loads in flight per thread
constexpr int kTileElems = kThreads * kVec * kUnroll;     // 8192
constexpr int kTileBlocks = kTileElems / 128;             // 64 scales per tile
constexpr int kLanesPerBlock = 128 / kVec;                // 16

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

__device__ __forceinline__ uint4 ld_stream16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ld_stream8(const void* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ void unpack8(const uint4& r, float (&x)[8]) {
  x[0] = bf16lo(r.x); x[1] = bf16hi(r.x);
  x[2] = bf16lo(r.y); x[3] = bf16hi(r.y);
  x[4] = bf16lo(r.z); x[5] = bf16hi(r.z);
  x[6] = bf16lo(r.w); x[7] = bf16hi(r.w);
}

// fmaxf ignores a NaN operand, so a NaN element never becomes the absmax.
__device__ __forceinline__ float absmax8(const float (&x)[8]) {
  float m = fmaxf(fabsf(x[0]), fabsf(x[1]));
  m = fmaxf(m, fmaxf(fabsf(x[2]), fabsf(x[3])));
  m = fmaxf(m, fmaxf(fabsf(x[4]), fabsf(x[5])));
  m = fmaxf(m, fmaxf(fabsf(x[6]), fabsf(x[7])));
  return m;
}

// Max over the 16 lanes that hold one 128-element block.
__device__ __forceinline__ float absmax_halfwarp(float m) {
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 8));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
  m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  return m;
}

// ---- int8 -----------------------------------------------------------------

// round-to-nearest-even to a saturated signed byte; NaN gives 0.
__device__ __forceinline__ uint32_t f32_to_s8(float q) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(q));
  return static_cast<uint32_t>(r) & 0xFFu;
}

// The quotient x/scale, correctly rounded, decides the code.  A full IEEE
// division per element costs ~10 instructions; instead one correctly rounded
// reciprocal per block plus a residual correction per element gives the same
// correctly rounded quotient (Markstein: q0 = x*r, e = x - q0*s exactly by FMA,
// q = q0 + e*r is RN(x/s) when r = RN(1/s) and s's significand is not all
// ones).  Blocks whose scale is all-ones, tiny or huge (where e could
// underflow) take the plain division.
struct Int8Divider {
  float scale, inv;
  bool fast;
  __device__ __forceinline__ explicit Int8Divider(float s) : scale(s) {
    const uint32_t b = __float_as_uint(s);
    const uint32_t ex = (b >> 23) & 0xFFu;
    fast = (ex >= 64u) && (ex <= 190u) && ((b & 0x7FFFFFu) != 0x7FFFFFu);
    inv = __frcp_rn(s);
  }
  __device__ __forceinline__ float quotient(float x) const {
    if (fast) {
      const float q0 = __fmul_rn(x, inv);
      const float e = __fmaf_rn(-q0, scale, x);
      return __fmaf_rn(e, inv, q0);
    }
    return __fdiv_rn(x, scale);
  }
};

template <bool kMulInv>
__device__ __forceinline__ uint2 encode8_int8(const float (&x)[8], float scale) {
  uint32_t c[8];
  if (kMulInv) {
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = f32_to_s8(__fmul_rn(x[i], inv));
  } else {
    const Int8Divider d(scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = f32_to_s8(d.quotient(x[i]));
  }
  // scale == 0 (all-zero block): 0/0 and 0*inf are NaN, which encodes as 0.
  uint2 o;
  o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
  o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
  return o;
}

// ---- FP8 E4M3, the reference's encoder (src/cuda/fp8_quant.cu:19-57) --------
// Integer restatement: adding 1<<19 to the magnitude bits rounds the mantissa
// half-up to 3 bits with carry into the exponent; >>20 leaves exponent*8+mant;
// -960 re-biases (127-7)*8.  Anything that lands in exponent 15 (>= 248)
// becomes 0x7F.  Magnitudes under 2^-6 use the reference's float formula
// (int)(v*512 + 0.5f) clamped to 7.  The sign comes from `y < 0`, so -0.0
// encodes as 0x00 while a negative value that rounds to zero encodes as 0x80.
__device__ __forceinline__ uint32_t fp8_encode_ref(float y) {
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
  if (a > 0x7F800000u) { s = (b >> 24) & 0x80u; c = 0x7Fu; }  // NaN (undefined in the reference)
  return s | c;
}

// OCP E4M3: round-to-nearest-even, saturate to +-448.  The hardware converter
// does exactly this.
__device__ __forceinline__ uint32_t fp8_encode_ocp_pair(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

template <bool kOcp>
__device__ __forceinline__ uint2 encode8_fp8(const float (&x)[8], float amax, float scale) {
  uint2 o = make_uint2(0u, 0u);
  if (amax == 0.0f) return o;  // all-zero block: codes 0, scale 0
  const float inv = __fdiv_rn(1.0f, scale);
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(x[i], inv);
  if (kOcp) {
    o.x = fp8_encode_ocp_pair(y[0], y[1]) | (fp8_encode_ocp_pair(y[2], y[3]) << 16);
    o.y = fp8_encode_ocp_pair(y[4], y[5]) | (fp8_encode_ocp_pair(y[6], y[7]) << 16);
    // the converter turns NaN into 0x7F/0xFF already
  } else {
    uint32_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = fp8_encode_ref(y[i]);
    o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
  }
  return o;
}

template <int kCodec, bool kFlag>
__device__ __forceinline__ uint2 encode8(const float (&x)[8], float amax, float& scale) {
  if (kCodec == kCodecInt8) {
    scale = __fdiv_rn(amax, 127.0f);
    return encode8_int8<kFlag>(x, scale);
  } else {
    scale = __fdiv_rn(amax, 448.0f);
    return encode8_fp8<kFlag>(x, amax, scale);
  }
}

// ---- compress kernel --------------------------------------------------------
// Requires: in 16-byte aligned, codes 16-byte aligned, scales 16-byte aligned.
// Full tiles go through the shared-memory tiles and bulk stores; the last,
// partial tile uses predicated loads and direct stores.
template <int kCodec, bool kFlag>
__global__ void __launch_bounds__(kThreads)
compress_b128_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ codes,
                     float* __restrict__ scales, size_t n) {
  __shared__ __align__(128) uint8_t s_codes[2][kTileElems];
  __shared__ __align__(128) float s_scales[2][kTileBlocks];

  const int tid = threadIdx.x;
  const size_t full_tiles = n / kTileElems;
  int buf = 0;

  for (size_t tile = blockIdx.x; tile < full_tiles; tile += gridDim.x) {
    const uint16_t* tin = in + tile * kTileElems;
    uint4 raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) raw[u] = ld_stream16(tin + (size_t)(u * kThreads + tid) * kVec);

    // The bulk store issued two tiles ago read this buffer; it must be done.
    if (tid == 0) bulk_wait_read<1>();
    __syncthreads();

#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float x[8];
      unpack8(raw[u], x);
      const float amax = absmax_halfwarp(absmax8(x));
      float scale;
      const uint2 c = encode8<kCodec, kFlag>(x, amax, scale);
      const int v = u * kThreads + tid;
      *reinterpret_cast<uint2*>(&s_codes[buf][v * kVec]) = c;
      if ((tid & (kLanesPerBlock - 1)) == 0) s_scales[buf][v / kLanesPerBlock] = scale;
    }
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      bulk_store(codes + tile * kTileElems, s_codes[buf], kTileElems);
      bulk_store(scales + tile * kTileBlocks, s_scales[buf], kTileBlocks * sizeof(float));
      bulk_commit();
    }
    buf ^= 1;
  }

  // Ragged tail: owned by the block that would have taken tile `full_tiles`.
  const size_t tail0 = full_tiles * kTileElems;
  if (tail0 < n && (full_tiles % gridDim.x) == blockIdx.x) {
    const uint16_t* tin = in + tail0;
    const size_t rem = n - tail0;
#pragma unroll 1
    for (int u = 0; u < kUnroll; ++u) {
      const size_t e0 = (size_t)(u * kThreads + tid) * kVec;
      // whole warps enter together so the shuffles stay converged
      if (((size_t)(u * kThreads + (tid & ~31)) * kVec) >= rem) break;
      uint4 r = make_uint4(0u, 0u, 0u, 0u);
      if (e0 + kVec <= rem) {
        r = ld_stream16(tin + e0);
      } else if (e0 < rem) {
        uint16_t tmp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t i = 0; e0 + i < rem; ++i) tmp[i] = tin[e0 + i];
        r.x = tmp[0] | ((uint32_t)tmp[1] << 16); r.y = tmp[2] | ((uint32_t)tmp[3] << 16);
        r.z = tmp[4] | ((uint32_t)tmp[5] << 16); r.w = tmp[6] | ((uint32_t)tmp[7] << 16);
      }
      float x[8];
      unpack8(r, x);
      const float amax = absmax_halfwarp(absmax8(x));
      float scale;
      const uint2 c = encode8<kCodec, kFlag>(x, amax, scale);
      if (e0 + kVec <= rem) {
        *reinterpret_cast<uint2*>(codes + tail0 + e0) = c;
      } else if (e0 < rem) {
        const uint64_t cc = ((uint64_t)c.y << 32) | c.x;
        for (size_t i = 0; e0 + i < rem; ++i) codes[tail0 + e0 + i] = (uint8_t)(cc >> (8 * i));
      }
      if ((tid & (kLanesPerBlock - 1)) == 0 && e0 < rem) scales[(tail0 + e0) / 128] = scale;
    }
  }

  if (tid == 0) bulk_wait_all<0>();
}

// Any alignment, any n: one warp per 128-element block, scalar accesses.
template <int kCodec, bool kFlag>
__global__ void __launch_bounds__(kThreads)
compress_b128_generic_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ codes,
                             float* __restrict__ scales, size_t n) {
  const size_t nblocks = (n + 127) / 128;
  const int lane = threadIdx.x & 31;
  const size_t warp0 = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (kThreads / 32);
  for (size_t blk = warp0; blk < nblocks; blk += nwarps) {
    const size_t e0 = blk * 128 + (size_t)lane * 4;
    float x[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < 4; ++i)
      if (e0 + i < n) x[i] = __uint_as_float((uint32_t)in[e0 + i] << 16);
    float m = absmax8(x);
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 16));
    const float amax = absmax_halfwarp(m);
    float scale;
    const uint2 c = encode8<kCodec, kFlag>(x, amax, scale);
    for (int i = 0; i < 4; ++i)
      if (e0 + i < n) codes[e0 + i] = (uint8_t)(c.x >> (8 * i));
    if (lane == 0) scales[blk] = scale;
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
  const uint32_t bits = __byte_perm(w_flipped, 0x4B000000u, 0x7650 | k) ;
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

template <int kCodec>
__device__ __forceinline__ uint4 decode8(uint2 c, float scale) {
  float v[8];
  if (kCodec == kCodecInt8) {
    const uint32_t a = c.x ^ 0x80808080u, b = c.y ^ 0x80808080u;
    v[0] = s8_to_f32<0>(a); v[1] = s8_to_f32<1>(a); v[2] = s8_to_f32<2>(a); v[3] = s8_to_f32<3>(a);
    v[4] = s8_to_f32<0>(b); v[5] = s8_to_f32<1>(b); v[6] = s8_to_f32<2>(b); v[7] = s8_to_f32<3>(b);
  } else {
    v[0] = fp8_to_f32_scaled<0>(c.x); v[1] = fp8_to_f32_scaled<1>(c.x);
    v[2] = fp8_to_f32_scaled<2>(c.x); v[3] = fp8_to_f32_scaled<3>(c.x);
    v[4] = fp8_to_f32_scaled<0>(c.y); v[5] = fp8_to_f32_scaled<1>(c.y);
    v[6] = fp8_to_f32_scaled<2>(c.y); v[7] = fp8_to_f32_scaled<3>(c.y);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], scale);
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

// Requires: codes 8-byte aligned, out 16-byte aligned.  Each thread turns 8
// codes (one 8-byte load) into 8 BF16 (one 16-byte store); the 16 lanes of a
// block read the same scale, which the L1 serves.
template <int kCodec>
__global__ void __launch_bounds__(kThreads)
dequant_b128_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales,
                    uint16_t* __restrict__ out, size_t n) {
  const int tid = threadIdx.x;
  const size_t nvec = n / kVec;  // whole 8-element vectors
  const size_t tiles = (nvec + kThreads * kUnroll - 1) / (kThreads * kUnroll);
  for (size_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const size_t v0 = tile * (kThreads * kUnroll);
    uint2 c[kUnroll];
    float s[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const size_t v = v0 + (size_t)(u * kThreads + tid);
      if (v < nvec) {
        c[u] = ld_stream8(codes + v * kVec);
        s[u] = __ldg(scales + v / kLanesPerBlock);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const size_t v = v0 + (size_t)(u * kThreads + tid);
      if (v < nvec) __stcs(reinterpret_cast<uint4*>(out + v * kVec), decode8<kCodec>(c[u], s[u]));
    }
  }
  // up to 7 trailing elements
  const size_t t0 = nvec * kVec;
  if (blockIdx.x == 0 && tid < (int)(n - t0)) {
    const size_t e = t0 + tid;
    uint2 c = make_uint2(codes[e], 0u);
    const uint4 o = decode8<kCodec>(c, scales[e / 128]);
    out[e] = (uint16_t)(o.x & 0xFFFFu);
  }
}

template <int kCodec>
__global__ void __launch_bounds__(kThreads)
dequant_b128_generic_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales,
                            uint16_t* __restrict__ out, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride) {
    const uint4 o = decode8<kCodec>(make_uint2(codes[e], 0u), scales[e / 128]);
    out[e] = (uint16_t)(o.x & 0xFFFFu);
  }
}

// ---- element-wise FP8 with a caller-supplied scale --------------------------

__global__ void __launch_bounds__(kThreads)
bf16_to_fp8_vec_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, float inv_scale, size_t n) {
  const size_t nvec = n / kVec;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    float x[8];
    unpack8(ld_stream16(in + v * kVec), x);
    uint32_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = fp8_encode_ref(__fmul_rn(x[i], inv_scale));
    uint2 o;
    o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
    __stcs(reinterpret_cast<uint2*>(out + v * kVec), o);
  }
  const size_t t0 = nvec * kVec;
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - t0)) {
    const size_t e = t0 + threadIdx.x;
    out[e] = (uint8_t)fp8_encode_ref(__fmul_rn(__uint_as_float((uint32_t)in[e] << 16), inv_scale));
  }
}

__global__ void __launch_bounds__(kThreads)
bf16_to_fp8_scalar_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, float inv_scale, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride)
    out[e] = (uint8_t)fp8_encode_ref(__fmul_rn(__uint_as_float((uint32_t)in[e] << 16), inv_scale));
}

__global__ void __launch_bounds__(kThreads)
fp8_to_bf16_vec_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, size_t n) {
  const size_t nvec = n / kVec;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride)
    __stcs(reinterpret_cast<uint4*>(out + v * kVec), decode8<kCodecFp8>(ld_stream8(in + v * kVec), scale));
  const size_t t0 = nvec * kVec;
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - t0)) {
    const size_t e = t0 + threadIdx.x;
    out[e] = (uint16_t)(decode8<kCodecFp8>(make_uint2(in[e], 0u), scale).x & 0xFFFFu);
  }
}

__global__ void __launch_bounds__(kThreads)
fp8_to_bf16_scalar_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, float scale, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n; e += stride)
    out[e] = (uint16_t)(decode8<kCodecFp8>(make_uint2(in[e], 0u), scale).x & 0xFFFFu);
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

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

int set_max_ctas(int v) { const int old = g_max_ctas; g_max_ctas = v < 0 ? 0 : v; return old; }

cudaError_t launch_compress(int codec, const void* in, void* codes, void* scales, size_t n,
                            unsigned flags, cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  if (!in || !codes || !scales) return cudaErrorInvalidValue;
  const bool flag = (flags & 1u) != 0;
  auto* i = static_cast<const uint16_t*>(in);
  auto* c = static_cast<uint8_t*>(codes);
  auto* s = static_cast<float*>(scales);
  if (aligned(in, 16) && aligned(codes, 16) && aligned(scales, 16)) {
    const size_t tiles = (n + kTileElems - 1) / kTileElems;
    const int grid = grid_for(tiles, 6, max_ctas);
    if (codec == kCodecInt8) {
      if (flag) compress_b128_kernel<kCodecInt8, true><<<grid, kThreads, 0, stream>>>(i, c, s, n);
      else compress_b128_kernel<kCodecInt8, false><<<grid, kThreads, 0, stream>>>(i, c, s, n);
    } else {
      if (flag) compress_b128_kernel<kCodecFp8, true><<<grid, kThreads, 0, stream>>>(i, c, s, n);
      else compress_b128_kernel<kCodecFp8, false><<<grid, kThreads, 0, stream>>>(i, c, s, n);
    }
  } else {
    const size_t warps = (n + 127) / 128;
    const int grid = grid_for((warps + 7) / 8, 8, max_ctas);
    if (codec == kCodecInt8) {
      if (flag) compress_b128_generic_kernel<kCodecInt8, true><<<grid, kThreads, 0, stream>>>(i, c, s, n);
      else compress_b128_generic_kernel<kCodecInt8, false><<<grid, kThreads, 0, stream>>>(i, c, s, n);
    } else {
      if (flag) compress_b128_generic_kernel<kCodecFp8, true><<<grid, kThreads, 0, stream>>>(i, c, s, n);
      else compress_b128_generic_kernel<kCodecFp8, false><<<grid, kThreads, 0, stream>>>(i, c, s, n);
    }
  }
  return cudaGetLastError();
}

cudaError_t launch_dequant(int codec, const void* codes, const void* scales, void* out, size_t n,
                           cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  if (!codes || !scales || !out) return cudaErrorInvalidValue;
  auto* c = static_cast<const uint8_t*>(codes);
  auto* s = static_cast<const float*>(scales);
  auto* o = static_cast<uint16_t*>(out);
  if (aligned(codes, 8) && aligned(out, 16) && aligned(scales, 4)) {
    const size_t tiles = (n / kVec + kThreads * kUnroll - 1) / (kThreads * kUnroll);
    const int grid = grid_for(tiles ? tiles : 1, 8, max_ctas);
    if (codec == kCodecInt8) dequant_b128_kernel<kCodecInt8><<<grid, kThreads, 0, stream>>>(c, s, o, n);
    else dequant_b128_kernel<kCodecFp8><<<grid, kThreads, 0, stream>>>(c, s, o, n);
  } else {
    const int grid = grid_for((n + kThreads - 1) / kThreads, 8, max_ctas);
    if (codec == kCodecInt8) dequant_b128_generic_kernel<kCodecInt8><<<grid, kThreads, 0, stream>>>(c, s, o, n);
    else dequant_b128_generic_kernel<kCodecFp8><<<grid, kThreads, 0, stream>>>(c, s, o, n);
  }
  return cudaGetLastError();
}

cudaError_t launch_bf16_to_fp8(const void* in, void* out, float inv_scale, size_t n, cudaStream_t stream, int max_ctas) {
  if (n == 0) return cudaSuccess;
  auto* i = static_cast<const uint16_t*>(in);
  auto* o = static_cast<uint8_t*>(out);
  if (aligned(in, 16) && aligned(out, 8)) {
    const int grid = grid_for((n / kVec + kThreads - 1) / kThreads + 1, 8, max_ctas);
    bf16_to_fp8_vec_kernel<<<grid, kThreads, 0, stream>>>(i, o, inv_scale, n);
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
  if (aligned(in, 8) && aligned(out, 16)) {
    const int grid = grid_for((n / kVec + kThreads - 1) / kThreads + 1, 8, max_ctas);
    fp8_to_bf16_vec_kernel<<<grid, kThreads, 0, stream>>>(i, o, scale, n);
  } else {
    const int grid = grid_for((n + kThreads - 1) / kThreads, 8, max_ctas);
    fp8_to_bf16_scalar_kernel<<<grid, kThreads, 0, stream>>>(i, o, scale, n);
  }
  return cudaGetLastError();
}

}  // namespace flame_b200
