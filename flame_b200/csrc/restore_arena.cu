// Restore arena: ring bookkeeping over one device range reserved at set-up, so
// that the destinations of flame_offload_pool_pull_into() come from memory that
// is never allocated or freed while training runs.
//
// The reference allocates a fresh tensor in every pull
// (src/activation_offload.rs:655) and has a stream-keyed arena for other hot
// paths (src/staging.rs:219-297: arena_alloc / arena_record_and_release /
// arena_reset / arena_stats).  This arena follows that model: it belongs to ONE
// stream.  Every use of a region is queued on that stream, or ordered with it as
// pull_into() orders the pool's copies (it waits for the stream before the first
// write and makes the stream wait for the last), and release() is called once the
// last use has been queued.  Reuse is then ordered by the stream itself and the
// arena needs no CUDA call at all: it is host arithmetic over offsets.
//
// Restored activations live in ring order (restored first, consumed first), with
// some slack; release may come in any order, space is handed out again when the
// oldest regions have been released (or the newest: a region released straight
// after its allocation gives its space back at once).

#include <deque>
#include <mutex>

#include "common.h"

using namespace flame_b200;

struct FlameRestoreArena {
  std::mutex mu;
  uint8_t* base = nullptr;
  size_t cap = 0, align = 256;
  size_t head = 0;  // next offset handed out
  struct Region { size_t off, size; uint64_t ticket; bool live; };
  std::deque<Region> regions;  // ring order, oldest first
  uint64_t next_ticket = 1;
  FlameRestoreArenaStats st{};

  void trim() {
    while (!regions.empty() && !regions.front().live) regions.pop_front();
    while (!regions.empty() && !regions.back().live) regions.pop_back();
    head = regions.empty() ? 0 : regions.back().off + regions.back().size;
  }
};

extern "C" {

FlameRestoreArena* flame_restore_arena_create(void* base, size_t bytes, size_t alignment) {
  if (!base || bytes == 0) { fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena: null base or zero size"); return nullptr; }
  if (alignment == 0) alignment = 256;
  if (alignment & (alignment - 1)) { fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena: alignment must be a power of two"); return nullptr; }
  if (reinterpret_cast<uintptr_t>(base) % alignment) { fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena: base is not aligned"); return nullptr; }
  auto* a = new FlameRestoreArena();
  a->base = static_cast<uint8_t*>(base);
  a->cap = bytes - bytes % alignment;
  a->align = alignment;
  a->st.capacity_bytes = a->cap;
  if (a->cap == 0) { delete a; fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena: smaller than one aligned unit"); return nullptr; }
  return a;
}

void flame_restore_arena_destroy(FlameRestoreArena* a) { delete a; }

FlameOffloadStatus flame_restore_arena_alloc(FlameRestoreArena* a, size_t bytes, void** out_ptr, uint64_t* out_ticket) {
  if (!a || !out_ptr || !out_ticket) return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena alloc: null argument");
  if (bytes == 0) return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena alloc: zero bytes");
  std::lock_guard<std::mutex> lk(a->mu);
  const size_t need = (bytes + a->align - 1) & ~(a->align - 1);
  if (need < bytes || need > a->cap) {
    a->st.rejected++;
    return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena alloc: " + std::to_string(bytes) + " bytes exceed the arena (" + std::to_string(a->cap) + ")");
  }
  a->trim();
  size_t off = 0;
  bool ok = true;
  if (!a->regions.empty()) {
    const size_t tail = a->regions.front().off;  // oldest live byte
    if (a->head > tail) {                          // live bytes are [tail, head): free is [head, cap) and [0, tail)
      if (a->cap - a->head >= need) off = a->head;
      else if (tail >= need) off = 0;              // wrap; the unused end comes back with the regions before it
      else ok = false;
    } else {                                       // wrapped: free is [head, tail); head == tail means full
      if (tail - a->head >= need) off = a->head;
      else ok = false;
    }
  }
  if (!ok) {
    a->st.rejected++;
    return fail(FLAME_OFFLOAD_ERR_STATE, "restore arena full: " + std::to_string(a->st.in_use_bytes) + " of " + std::to_string(a->cap) +
                " bytes held by regions not yet released, " + std::to_string(need) + " wanted");
  }
  a->regions.push_back({off, need, a->next_ticket, true});
  a->head = off + need;
  a->st.allocs++;
  a->st.in_use_bytes += need;
  if (a->st.in_use_bytes > a->st.peak_in_use_bytes) a->st.peak_in_use_bytes = a->st.in_use_bytes;
  *out_ptr = a->base + off;
  *out_ticket = a->next_ticket++;
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_restore_arena_release(FlameRestoreArena* a, uint64_t ticket) {
  if (!a) return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena release: null arena");
  std::lock_guard<std::mutex> lk(a->mu);
  for (auto& r : a->regions) {
    if (r.ticket != ticket) continue;
    if (!r.live) break;
    r.live = false;
    a->st.releases++;
    a->st.in_use_bytes -= r.size;
    a->trim();
    return FLAME_OFFLOAD_OK;
  }
  return fail(FLAME_OFFLOAD_ERR_STATE, "restore arena release: ticket " + std::to_string(ticket) + " is not held (released twice, or reset since)");
}

FlameOffloadStatus flame_restore_arena_reset(FlameRestoreArena* a) {
  if (!a) return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena reset: null arena");
  std::lock_guard<std::mutex> lk(a->mu);
  a->regions.clear();
  a->head = 0;
  a->st.in_use_bytes = 0;
  a->st.resets++;
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_restore_arena_stats(const FlameRestoreArena* ac, FlameRestoreArenaStats* out) {
  auto* a = const_cast<FlameRestoreArena*>(ac);
  if (!a || !out) return fail(FLAME_OFFLOAD_ERR_INVALID, "restore arena stats: null argument");
  std::lock_guard<std::mutex> lk(a->mu);
  *out = a->st;
  out->live_regions = 0;
  for (auto& r : a->regions) out->live_regions += r.live;
  return FLAME_OFFLOAD_OK;
}

}  // extern "C"
