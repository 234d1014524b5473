// Host-side launcher for the reference's own int8 quantisation kernel, sage_quantize_tensor
// (src/sage_attention.rs:510-543: per-row scale = max|x| / 127, code = __float2int_rn(x / scale) clamped to
// [-128, 127]).  `make -C oracle refsage` streams those lines out of the reference's file in front of this one
// and compiles the two together into oracle/_ref; the kernel text itself is never stored here.  Used with
// row_size = 128 it is a per-128-block quantiser, which is what the int8 block codec is held against.
// Test infrastructure only.
#include <cuda_runtime.h>

extern "C" int sage_quantize_ref(const float* input, signed char* output, float* scales, int num_rows, int row_size, void* stream) {
  const long long n = (long long)num_rows * row_size;
  const int block = 256;
  // The kernel has a barrier inside its bounds check, so every thread of every block must pass the check:
  // the grid covers exactly n threads, and a row must not straddle two thread blocks.
  if (n <= 0 || n % block != 0 || block % row_size != 0) return (int)cudaErrorInvalidValue;
  sage_quantize_tensor<<<(unsigned)(n / block), block, 0, (cudaStream_t)stream>>>(input, output, scales, num_rows, row_size);
  return (int)cudaGetLastError();
}
