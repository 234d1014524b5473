// Internal launch interface of the codec kernels (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <stdlib.h>

struct FlameWeightJob;   // include/flame_offload.h

namespace flame_b200 {

// Programmatic dependent launch.  A kernel of this library that follows another one in a stream is launched with
// cudaLaunchAttributeProgrammaticStreamSerialization: its thread blocks may be placed on the SMs while the kernel
// before it drains, and they begin at once when it has finished, instead of after a launch's start-up time.
//   - A kernel launched this way begins with pdl_prologue(): `griddepcontrol.wait` returns when every kernel it depends
//     on has completed and its writes are visible, so nothing is read or written early; `griddepcontrol.launch_dependents`
//     lets the next such kernel be placed once every block of this one has started.  Without the attribute, and behind
//     anything that is not a kernel (a copy, an event wait), both instructions do nothing.
//   - Only launches of kernels that begin with the prologue go through launch_after().
// Measured on a B200, 20 launches of one DiT block back to back: int8 compress 0.971 -> 0.993 of the HBM copy rate,
// dequantise 0.958 -> 0.988, FP8 compress 0.868 -> 0.888.  FLAME_ACT_PDL=0 turns the attribute off.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("FLAME_ACT_PDL"); return !(e && e[0] == '0'); }();
  return on;
}
template <typename K, typename... A>
cudaError_t launch_after(K kernel, unsigned grid, unsigned block, size_t smem, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Same numbering as FLAME_OFFLOAD_COMPRESSION_INT8_B128 / _FP8_B128.
constexpr int kCodecInt8 = 2;
constexpr int kCodecFp8 = 3;

// Bits of `flags` for launch_compress.  Bit 0 is the public codec flag
// (FLAME_ACT_INT8_MUL_INV / FLAME_ACT_FP8_OCP); bit 1 picks the store path.
constexpr unsigned kFlagStagedStores = 2u;

// Addressing of compressed data as a run of self-contained chunks: chunk c holds
// elements [c*chunk_elems, (c+1)*chunk_elems) and starts at base + c*chunk_stride
// with its codes; its fp32 scales start scales_off bytes into the chunk
// (scales_off_last for the final, possibly shorter chunk).
struct PackedLayout {
  size_t chunk_elems;
  int64_t chunk_stride;
  int64_t scales_off;
  int64_t scales_off_last;
  size_t last_chunk;
};

// One chunk: codes at `codes`, scales at `scales` (any two buffers).
PackedLayout single_chunk_layout(const void* codes, const void* scales, size_t n);
// Chunks of `chunk_elems` (a multiple of 16384) every `chunk_stride` bytes, each
// in the packed layout codes | pad to 256 B | scales.
PackedLayout packed_chunks_layout(size_t n, size_t chunk_elems, size_t chunk_stride);

// One tensor of a multi-tensor launch: its BF16 memory (source of compress,
// destination of dequantise) and its compressed memory.
struct TensorJob {
  void* bf16;
  void* packed;
  size_t n;
  PackedLayout layout;
};

// Up to any number of tensors; tensors that qualify for the fast kernels are
// batched 48 to a launch, the others go one by one through the generic kernels.
cudaError_t launch_compress_multi(int codec, const TensorJob* jobs, size_t count, unsigned flags, cudaStream_t stream, int max_ctas);
cudaError_t launch_dequant_multi(int codec, const TensorJob* jobs, size_t count, cudaStream_t stream, int max_ctas);

// max_ctas: 0 = process default (see set_max_ctas), otherwise a cap on the grid.
cudaError_t launch_compress(int codec, const void* in_bf16, void* out_base, size_t n, const PackedLayout& layout,
                            unsigned flags, cudaStream_t stream, int max_ctas);
cudaError_t launch_dequant(int codec, const void* in_base, void* out_bf16, size_t n, const PackedLayout& layout,
                           cudaStream_t stream, int max_ctas);
cudaError_t launch_bf16_to_fp8(const void* in, void* out, float inv_scale, size_t n, cudaStream_t stream, int max_ctas);
cudaError_t launch_fp8_to_bf16(const void* in, void* out, float scale, size_t n, cudaStream_t stream, int max_ctas);
// Producers with the compress step built in (codec 0 = plain producer, no codes).
cudaError_t launch_rmsnorm_quant(int codec, unsigned flags, const void* x, const void* w, void* y, void* codes, void* scales,
                                 void* rstd_out, size_t rows, size_t cols, float eps, cudaStream_t stream);
cudaError_t launch_swiglu_quant(int codec, unsigned flags, const void* gate_up, void* h, void* codes, void* scales,
                                size_t rows, size_t hidden, cudaStream_t stream, int max_ctas);
// FP8 weights [M, N] -> BF16 [N, M] with the decoder of the reference's fused_dequant_transpose.cu (weight_kernels.cu).
cudaError_t launch_fp8_dequant_transpose(const void* in_fp8, void* out_bf16, float scale, int M, int N, cudaStream_t stream, int max_ctas);
cudaError_t launch_fp8_dequant_transpose_jobs(const ::FlameWeightJob* jobs, int count, cudaStream_t stream, int max_ctas);
int set_max_ctas(int v);

// Inspection hooks (tests): what the calling thread's last compress / dequantise launch chose, and a fresh
// occupancy query for the kernel a (codec, flags, form) combination selects.
struct LaunchRecord { int ctas, resident_per_sm, tiles_per_cta, form; };  // form: kernel form 0..2, +4 with staged stores
LaunchRecord last_launch();
int default_compress_form(int codec);
int set_compress_form(int form);  // 0..2, anything else = per-codec default; returns the old override (-1 = none)
// form < 0: the form the codec takes by default
int query_resident_ctas(int codec, unsigned flags, int form, bool compress);

}  // namespace flame_b200
