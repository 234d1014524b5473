// Compress-and-copy-out for callers that must not allocate.
//
// Some users of this library reach for an offload exactly when nothing can be
// allocated any more: an out-of-memory handler that has to move a saved
// activation off the device to make room, or a training loop whose memory
// plan was fixed at start-up and whose step must not call cudaMalloc/cudaFree
// (cudaFree stalls the whole device, and either call can fail once the job
// has claimed all memory).  The pool and the plain codec entry points need a
// device staging buffer from somebody.  This entry point brings its own: a
// fixed array that is part of the library image, so every GPU that uses the
// library holds kScratchBytes of it until the process exits.
//
// "Uses", not "opens": the CUDA runtime loads a library's kernels and static
// device arrays lazily, at the first cudaGetSymbolAddress, launch or occupancy
// query on a device, and that loading takes device memory.  A caller that needs
// the no-allocation property at the moment of need therefore makes one small
// warm-up call per device at start-up (each codec, an aligned and an unaligned
// input), while memory is still there to be had; from then on a call takes none.
//
// The price is a size limit and shared state: tensors of more than
// FLAME_ACT_NOALLOC_MAX_ELEMS elements are refused, and because every call
// uses the same array, two calls whose GPU work can overlap (different
// streams, or different threads without ordering between them) race on it.
// Calls on one stream are ordered and safe.
#include <mutex>

#include "codec_kernels.cuh"
#include "common.h"

namespace {

constexpr size_t kMaxElems = FLAME_ACT_NOALLOC_MAX_ELEMS;
// packed size of the largest accepted tensor: codes | pad to 256 B | one fp32 scale per 128 elements
constexpr size_t kScratchBytes = ((kMaxElems + 255) / 256) * 256 + 4 * ((kMaxElems + 127) / 128);

// Lives in device memory of every GPU on which this library has been used.  In host code
// this name is only a stand-in for the symbol, not a device address: kernels
// and copies must be given the address that cudaGetSymbolAddress returns.
static __device__ __align__(256) unsigned char g_spill_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device; looked up once per
// device, with that device current.
cudaError_t scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (g_scratch_addr[dev] == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_spill_scratch);
    if (e != cudaSuccess) return e;
    if (p == nullptr) return cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

using namespace flame_b200;

extern "C" int flame_act_offload_packed_noalloc(const void* in_bf16, void* packed_out, size_t n, int codec,
                                                unsigned int flags, void* stream_v) {
  if (n == 0) return 0;
  if (n > kMaxElems) {
    fail(FLAME_OFFLOAD_ERR_INVALID, "flame_act_offload_packed_noalloc: " + std::to_string(n) + " elements exceed the built-in scratch (" +
         std::to_string(kMaxElems) + " elements); use the pool or the plain codec entry points for larger tensors");
    return (int)cudaErrorInvalidValue;
  }
  if (!in_bf16 || !packed_out || (codec != kCodecInt8 && codec != kCodecFp8)) {
    fail(FLAME_OFFLOAD_ERR_INVALID, "flame_act_offload_packed_noalloc: null pointer or unknown codec");
    return (int)cudaErrorInvalidValue;
  }
  cudaStream_t stream = (cudaStream_t)stream_v;
  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) { fail_cuda(e, "flame_act_offload_packed_noalloc: cudaGetSymbolAddress"); return (int)e; }

  const size_t scales_off = (n + 255u) & ~(size_t)255u;
  const size_t total = scales_off + 4u * ((n + 127u) / 128u);
  // The array still holds the previous call's bytes; the padding between codes
  // and scales is part of the output and must read as zero.
  if (scales_off > n) {
    e = cudaMemsetAsync(scratch + n, 0, scales_off - n, stream);
    if (e != cudaSuccess) { fail_cuda(e, "flame_act_offload_packed_noalloc: cudaMemsetAsync"); return (int)e; }
  }
  e = launch_compress(codec, in_bf16, scratch, n, single_chunk_layout(scratch, scratch + scales_off, n), flags, stream, 0);
  if (e != cudaSuccess) { fail_cuda(e, "flame_act_offload_packed_noalloc: compress kernel"); return (int)e; }
  e = memcpy_async_checked(packed_out, scratch, total, cudaMemcpyDefault, stream);
  if (e != cudaSuccess) { fail_cuda(e, "flame_act_offload_packed_noalloc: copy out"); return (int)e; }
  return 0;
}
