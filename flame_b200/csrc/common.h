// Shared host-side helpers of the offload library (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <string>

#include "../../include/flame_offload.h"

namespace flame_b200 {

// Per-thread text returned by flame_offload_last_error().
void set_last_error(const std::string& msg);
FlameOffloadStatus fail(FlameOffloadStatus st, const std::string& msg);
FlameOffloadStatus fail_cuda(cudaError_t e, const char* what);

// Host-side fault injection (tests only): returns true when the call of this
// kind that is now being made was chosen to fail.
bool fault_fires(int kind);

// cudaMemcpyAsync / cudaHostAlloc behind the fault hook.
cudaError_t memcpy_async_checked(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t s);
cudaError_t host_alloc_checked(void** p, size_t bytes, unsigned flags);

}  // namespace flame_b200
