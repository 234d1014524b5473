// C ABI: error text, pinned host memory, async copies and the codec entry
// points.  The pool, the pinned cache and the policy live in their own files.
#include <atomic>
#include <cstring>
#include <vector>

#include "codec_kernels.cuh"
#include "common.h"

namespace flame_b200 {

namespace {
thread_local std::string t_last_error;
std::atomic<int> g_fault_kind{FLAME_OFFLOAD_FAULT_NONE};
std::atomic<int> g_fault_countdown{0};
}  // namespace

void set_last_error(const std::string& msg) { t_last_error = msg; }

FlameOffloadStatus fail(FlameOffloadStatus st, const std::string& msg) {
  t_last_error = msg;
  return st;
}

FlameOffloadStatus fail_cuda(cudaError_t e, const char* what) {
  t_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + std::to_string((int)e) + ")";
  return FLAME_OFFLOAD_ERR_CUDA;
}

bool fault_fires(int kind) {
  if (g_fault_kind.load(std::memory_order_relaxed) != kind) return false;
  if (g_fault_countdown.fetch_sub(1) == 1) {
    g_fault_kind.store(FLAME_OFFLOAD_FAULT_NONE);
    return true;
  }
  return false;
}

cudaError_t memcpy_async_checked(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t s) {
  if (fault_fires(FLAME_OFFLOAD_FAULT_MEMCPY)) return cudaErrorUnknown;
  return cudaMemcpyAsync(dst, src, bytes, kind, s);
}

cudaError_t host_alloc_checked(void** p, size_t bytes, unsigned flags) {
  if (fault_fires(FLAME_OFFLOAD_FAULT_HOST_ALLOC)) { *p = nullptr; return cudaErrorMemoryAllocation; }
  return cudaHostAlloc(p, bytes, flags);
}

}  // namespace flame_b200

using namespace flame_b200;

extern "C" {

const char* flame_offload_last_error(void) { return t_last_error.c_str(); }

void flame_offload_inject_fault(int kind, int countdown) {
  g_fault_countdown.store(countdown > 0 ? countdown : 1);
  g_fault_kind.store(kind);
}

// ---- pinned host memory (src/cuda/pinned_host.cu:4-45 in the reference) ------

void* flame_cuda_alloc_pinned_host(size_t size, unsigned int flags) {
  void* p = nullptr;
  return host_alloc_checked(&p, size, flags) == cudaSuccess ? p : nullptr;
}

int flame_cuda_free_pinned_host(void* ptr) { return (int)cudaFreeHost(ptr); }

int flame_cuda_memcpy_async(void* dst, const void* src, size_t bytes, int kind, void* stream) {
  cudaMemcpyKind k = cudaMemcpyDefault;
  if (kind == 1) k = cudaMemcpyHostToDevice;
  else if (kind == 2) k = cudaMemcpyDeviceToHost;
  else if (kind == 3) k = cudaMemcpyDeviceToDevice;
  return (int)memcpy_async_checked(dst, src, bytes, k, (cudaStream_t)stream);
}

int flame_cuda_host_register(void* ptr, size_t bytes, unsigned int flags) { return (int)cudaHostRegister(ptr, bytes, flags); }
int flame_cuda_host_unregister(void* ptr) { return (int)cudaHostUnregister(ptr); }

// ---- FlameCudaStatus-style copies (src/ffi/cuda_ffi.c:90-109) ------------------

static FlameOffloadStatus copy_status(void* dst, const void* src, uint64_t bytes, cudaMemcpyKind k, void* stream, const char* what) {
  if (!dst || !src || bytes == 0) return fail(FLAME_OFFLOAD_ERR_INVALID, std::string(what) + ": null pointer or zero bytes");
  cudaError_t e = memcpy_async_checked(dst, src, (size_t)bytes, k, (cudaStream_t)stream);
  return e == cudaSuccess ? FLAME_OFFLOAD_OK : fail_cuda(e, what);
}

FlameOffloadStatus flame_h2d_async(void* dst, const void* src, uint64_t bytes, void* stream) {
  return copy_status(dst, src, bytes, cudaMemcpyHostToDevice, stream, "flame_h2d_async");
}
FlameOffloadStatus flame_d2h_async(void* dst, const void* src, uint64_t bytes, void* stream) {
  return copy_status(dst, src, bytes, cudaMemcpyDeviceToHost, stream, "flame_d2h_async");
}
FlameOffloadStatus flame_d2d_async(void* dst, const void* src, uint64_t bytes, void* stream) {
  return copy_status(dst, src, bytes, cudaMemcpyDeviceToDevice, stream, "flame_d2d_async");
}

// ---- element-wise FP8 (src/cuda/fp8_quant.cu:74-93, src/cuda/fp8_dequant.cu:41-59)

int flame_bf16_to_fp8(const void* input, void* output, float inv_scale, size_t n, void* stream) {
  if (n == 0) return 0;
  if (fault_fires(FLAME_OFFLOAD_FAULT_KERNEL)) return (int)cudaErrorLaunchFailure;
  return (int)launch_bf16_to_fp8(input, output, inv_scale, n, (cudaStream_t)stream, 0);
}

int flame_fp8_to_bf16(const void* input, void* output, float scale, size_t n, void* stream) {
  if (n == 0) return 0;
  if (fault_fires(FLAME_OFFLOAD_FAULT_KERNEL)) return (int)cudaErrorLaunchFailure;
  return (int)launch_fp8_to_bf16(input, output, scale, n, (cudaStream_t)stream, 0);
}

// ---- FP8 weights with the transpose built in (src/cuda/fused_dequant_transpose.cu:104-126) ----

int flame_fused_dequant_transpose_bf16(const void* input, void* output, float scale, int M, int N, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0) return (int)cudaErrorInvalidValue;
  if (fault_fires(FLAME_OFFLOAD_FAULT_KERNEL)) return (int)cudaErrorLaunchFailure;
  return (int)launch_fp8_dequant_transpose(input, output, scale, M, N, (cudaStream_t)stream, 0);
}

int flame_fused_dequant_transpose_bf16_multi(const FlameWeightJob* jobs, int count, void* stream) {
  if (count <= 0) return 0;
  if (!jobs) return (int)cudaErrorInvalidValue;
  if (fault_fires(FLAME_OFFLOAD_FAULT_KERNEL)) return (int)cudaErrorLaunchFailure;
  return (int)launch_fp8_dequant_transpose_jobs(jobs, count, (cudaStream_t)stream, 0);
}

// ---- per-128-block codecs --------------------------------------------------------

static int quant_entry(int codec, const void* in, void* codes, void* scales, size_t n, unsigned flags, void* stream) {
  if (n == 0) return 0;
  if (!in || !codes || !scales) return (int)cudaErrorInvalidValue;
  return (int)launch_compress(codec, in, codes, n, single_chunk_layout(codes, scales, n), flags, (cudaStream_t)stream, 0);
}
static int dequant_entry(int codec, const void* codes, const void* scales, void* out, size_t n, void* stream) {
  if (n == 0) return 0;
  if (!codes || !scales || !out) return (int)cudaErrorInvalidValue;
  return (int)launch_dequant(codec, codes, out, n, single_chunk_layout(codes, scales, n), (cudaStream_t)stream, 0);
}

int flame_act_quant_int8_b128(const void* in, void* codes, void* scales, size_t n, unsigned int flags, void* stream) {
  return quant_entry(kCodecInt8, in, codes, scales, n, flags, stream);
}
int flame_act_dequant_int8_b128(const void* codes, const void* scales, void* out, size_t n, void* stream) {
  return dequant_entry(kCodecInt8, codes, scales, out, n, stream);
}
int flame_act_quant_fp8_b128(const void* in, void* codes, void* scales, size_t n, unsigned int flags, void* stream) {
  return quant_entry(kCodecFp8, in, codes, scales, n, flags, stream);
}
int flame_act_dequant_fp8_b128(const void* codes, const void* scales, void* out, size_t n, void* stream) {
  return dequant_entry(kCodecFp8, codes, scales, out, n, stream);
}

static int multi_entry(bool quant, int codec, const FlameActTensor* t, size_t count, unsigned flags, void* stream) {
  if (count == 0) return 0;
  if (!t || (codec != kCodecInt8 && codec != kCodecFp8)) return (int)cudaErrorInvalidValue;
  std::vector<TensorJob> jobs;
  jobs.reserve(count);
  for (size_t k = 0; k < count; ++k) {
    if (t[k].n == 0) continue;
    if (!t[k].bf16 || !t[k].codes || !t[k].scales) return (int)cudaErrorInvalidValue;
    jobs.push_back(TensorJob{t[k].bf16, t[k].codes, t[k].n, single_chunk_layout(t[k].codes, t[k].scales, t[k].n)});
  }
  return quant ? (int)launch_compress_multi(codec, jobs.data(), jobs.size(), flags, (cudaStream_t)stream, 0)
               : (int)launch_dequant_multi(codec, jobs.data(), jobs.size(), (cudaStream_t)stream, 0);
}

int flame_act_quant_b128_multi(int codec, const FlameActTensor* tensors, size_t count, unsigned int flags, void* stream) {
  return multi_entry(true, codec, tensors, count, flags, stream);
}
int flame_act_dequant_b128_multi(int codec, const FlameActTensor* tensors, size_t count, void* stream) {
  return multi_entry(false, codec, tensors, count, 0, stream);
}

int flame_act_rmsnorm_quant_b128(const void* x_bf16, const void* weight_bf16, void* y_bf16, void* codes_u8, void* scales_f32,
                                 void* rstd_f32, size_t rows, size_t cols, float eps, int codec, unsigned int flags, void* stream) {
  cudaError_t e = launch_rmsnorm_quant(codec, flags, x_bf16, weight_bf16, y_bf16, codes_u8, scales_f32, rstd_f32, rows, cols, eps, (cudaStream_t)stream);
  if (e == cudaErrorInvalidValue) set_last_error("flame_act_rmsnorm_quant_b128: needs cols % 128 == 0, cols <= 16384, 32-byte aligned rows and a known codec");
  return (int)e;
}

int flame_act_swiglu_quant_b128(const void* gate_up_bf16, void* h_bf16, void* codes_u8, void* scales_f32, size_t rows, size_t hidden,
                                int codec, unsigned int flags, void* stream) {
  cudaError_t e = launch_swiglu_quant(codec, flags, gate_up_bf16, h_bf16, codes_u8, scales_f32, rows, hidden, (cudaStream_t)stream, 0);
  if (e == cudaErrorInvalidValue) set_last_error("flame_act_swiglu_quant_b128: needs hidden % 128 == 0, 32-byte aligned rows and a known codec");
  return (int)e;
}

size_t flame_act_packed_scales_offset(size_t n) { return (n + 255u) & ~(size_t)255u; }
size_t flame_act_packed_bytes(size_t n) { return flame_act_packed_scales_offset(n) + 4u * ((n + 127u) / 128u); }

int flame_act_set_max_ctas(int max_ctas) { return set_max_ctas(max_ctas); }

int flame_act_set_compress_form(int form) { return set_compress_form(form); }

void flame_act_last_launch(FlameActLaunchInfo* out) {
  if (!out) return;
  const LaunchRecord r = last_launch();
  out->grid = r.ctas; out->resident_per_sm = r.resident_per_sm; out->tiles_per_block = r.tiles_per_cta; out->form = r.form;
}

int flame_act_query_resident_blocks(int codec, unsigned int flags, int form, int compress) {
  if (codec != kCodecInt8 && codec != kCodecFp8) return -1;
  return query_resident_ctas(codec, flags, form, compress != 0);
}

}  // extern "C"
