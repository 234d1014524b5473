// Internal launch interface of the codec kernels (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace flame_b200 {

// Same numbering as FLAME_OFFLOAD_COMPRESSION_INT8_B128 / _FP8_B128.
constexpr int kCodecInt8 = 2;
constexpr int kCodecFp8 = 3;

// max_ctas: 0 = process default (see set_max_ctas), otherwise a cap on the grid.
cudaError_t launch_compress(int codec, const void* in_bf16, void* codes, void* scales, size_t n,
                            unsigned flags, cudaStream_t stream, int max_ctas);
cudaError_t launch_dequant(int codec, const void* codes, const void* scales, void* out_bf16, size_t n,
                           cudaStream_t stream, int max_ctas);
cudaError_t launch_bf16_to_fp8(const void* in, void* out, float inv_scale, size_t n, cudaStream_t stream, int max_ctas);
cudaError_t launch_fp8_to_bf16(const void* in, void* out, float scale, size_t n, cudaStream_t stream, int max_ctas);
int set_max_ctas(int v);

}  // namespace flame_b200
