// Size-class cache of pinned host buffers.
// Mirrors PinnedPool in the reference (src/pinned_pool.rs:5-99): capacities are
// rounded up to 8 MiB classes (0 bytes asks for one class), checkout takes the
// smallest cached buffer that is large enough, checkin keeps a buffer only while
// the cache stays under max_cached_bytes (0 = cache nothing) and frees it
// otherwise.
#include <map>
#include <mutex>
#include <vector>

#include "common.h"

namespace {
constexpr size_t kSizeClassBytes = 8u << 20;
size_t round_up_class(size_t bytes) {
  if (bytes == 0) return kSizeClassBytes;
  return (bytes + kSizeClassBytes - 1) / kSizeClassBytes * kSizeClassBytes;
}
}  // namespace

struct FlamePinnedPool {
  std::mutex mu;
  unsigned flags = 0;
  size_t max_cached_bytes = 0;
  size_t cached_bytes = 0;
  std::map<size_t, std::vector<void*>> bins;
};

using namespace flame_b200;

extern "C" {

FlamePinnedPool* flame_pinned_pool_create(unsigned int alloc_flags, size_t max_cached_bytes) {
  auto* p = new FlamePinnedPool();
  p->flags = alloc_flags;
  p->max_cached_bytes = max_cached_bytes;
  return p;
}

void flame_pinned_pool_destroy(FlamePinnedPool* p) {
  if (!p) return;
  for (auto& kv : p->bins)
    for (void* b : kv.second) cudaFreeHost(b);
  delete p;
}

FlameOffloadStatus flame_pinned_pool_checkout(FlamePinnedPool* p, size_t min_bytes, void** out_ptr, size_t* out_capacity) {
  if (!p || !out_ptr || !out_capacity) return fail(FLAME_OFFLOAD_ERR_INVALID, "PinnedPool::checkout: null argument");
  const size_t needed = round_up_class(min_bytes);
  {
    std::lock_guard<std::mutex> lk(p->mu);
    auto it = p->bins.lower_bound(needed);
    if (it != p->bins.end() && !it->second.empty()) {
      *out_ptr = it->second.back();
      *out_capacity = it->first;
      it->second.pop_back();
      p->cached_bytes -= std::min(p->cached_bytes, it->first);
      if (it->second.empty()) p->bins.erase(it);
      return FLAME_OFFLOAD_OK;
    }
  }
  void* b = nullptr;
  cudaError_t e = host_alloc_checked(&b, needed, p->flags);
  if (e != cudaSuccess || !b) return fail(FLAME_OFFLOAD_ERR_CUDA, "cudaHostAlloc returned null (" + std::to_string(needed) + " bytes)");
  *out_ptr = b;
  *out_capacity = needed;
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_pinned_pool_checkin(FlamePinnedPool* p, void* ptr, size_t capacity) {
  if (!p || !ptr) return fail(FLAME_OFFLOAD_ERR_INVALID, "PinnedPool::checkin: null argument");
  {
    std::lock_guard<std::mutex> lk(p->mu);
    if (p->max_cached_bytes != 0 && p->cached_bytes + capacity <= p->max_cached_bytes) {
      p->cached_bytes += capacity;
      p->bins[capacity].push_back(ptr);
      return FLAME_OFFLOAD_OK;
    }
  }
  cudaFreeHost(ptr);  // not cached: dropped, as the Rust value would be
  return FLAME_OFFLOAD_OK;
}

void flame_pinned_pool_stats(const FlamePinnedPool* pc, size_t* cached_bytes, size_t* cached_buffers) {
  auto* p = const_cast<FlamePinnedPool*>(pc);
  if (!p) return;
  std::lock_guard<std::mutex> lk(p->mu);
  size_t n = 0;
  for (auto& kv : p->bins) n += kv.second.size();
  if (cached_bytes) *cached_bytes = p->cached_bytes;
  if (cached_buffers) *cached_buffers = n;
}

}  // extern "C"
