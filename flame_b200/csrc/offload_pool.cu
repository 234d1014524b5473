// Activation offload pool: host-side state machine and the chunked,
// double-buffered copy/codec pipeline behind flame_offload_pool_*.
//
// Semantics follow ActivationOffloadPool in the reference
// (src/activation_offload.rs:323-760): fixed number of slots, LIFO free stack,
// epoch-stamped handles, Idle/Pushed slot states, push never blocks the host,
// pool-full / stale-handle / double-pull are errors.  What differs is below the
// API:
//   * one pinned slab carved into equal chunks; a slot owns a list of chunks, so
//     pinned memory is consumed by what is stored, not by slots x max size;
//   * four non-blocking streams (compress, D2H, H2D, dequantise) so both copy
//     engines and the codec kernels run concurrently; a ring of device staging
//     tiles per direction; every hand-over between streams is an event, the
//     host never waits;
//   * restore writes into the caller's destination; in the compressed modes
//     the H2D of chunk k+1 overlaps the dequantise of chunk k;
//   * the source tensor is needed only until its D2H-complete event, which the
//     caller can query, instead of until pull.
//
// There is no device-side waiting anywhere in this design (no flags, no spin
// loops): ordering is CUDA events only, and every host wait is a bounded poll.
//
// Deferred offload (FlameOffloadPoolConfig.deferred_inflight_bytes > 0): push()
// records where the source becomes valid and queues the tensor; a thread owned by
// the pool enqueues the compress + D2H work of queued tensors in push order while
// the pinned bytes in flight stay under the budget.  A tensor still queued when
// backward reaches it has not left the device, so cancel() hands it back for use
// in place: the link then carries only what it can carry beside compute, instead
// of delaying backward with round trips that free nothing.  In that mode the
// offload side (compress stream, D2H stream, outgoing tile ring) is driven by the
// pool's thread only, the restore side by the caller's thread only.

#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "codec_kernels.cuh"
#include "common.h"

namespace flame_b200 {
namespace {

constexpr uint64_t kDefaultChunkBytes = 16ull << 20;
constexpr uint32_t kDefaultTiles = 2;
constexpr uint32_t kDefaultTileChunks = 8;
constexpr float kLegacyFp8Scale = 8.0f / 448.0f;  // src/activation_offload.rs:548

size_t packed_scales_offset(size_t n) { return (n + 255u) & ~(size_t)255u; }
size_t packed_bytes(size_t n) { return packed_scales_offset(n) + 4u * ((n + 127u) / 128u); }

struct Event {
  cudaEvent_t ev = nullptr;
  bool recorded = false;
  cudaError_t create() { return cudaEventCreateWithFlags(&ev, cudaEventDisableTiming); }
  cudaError_t record(cudaStream_t s) {
    cudaError_t e = cudaEventRecord(ev, s);
    if (e == cudaSuccess) recorded = true;
    return e;
  }
  // Makes `s` wait for the last record; a never-recorded event orders nothing.
  cudaError_t make_wait(cudaStream_t s) const { return recorded ? cudaStreamWaitEvent(s, ev, 0) : cudaSuccess; }
  void destroy() { if (ev) cudaEventDestroy(ev); ev = nullptr; }
};

enum class SlotState { Idle, Pushed };
enum class Issue { Done, Queued, Issuing };  // Done: the offload's work is enqueued (always so in the immediate mode)

// Everything the offload of one tensor needs, captured when push() is called.
struct PushPlan {
  std::vector<uint32_t> chunks;
  std::vector<cudaEvent_t> readers;  // restores that may still be reading these chunks
  const uint8_t* src = nullptr;
  const uint8_t* scales_src = nullptr;  // non-null: `src` holds codes and this the scales, already compressed on the device
  uint64_t numel = 0, bytes = 0;
  float fp8_scale = 0.0f;
  cudaEvent_t producer = nullptr, d2h_done = nullptr;
};
struct PushCounts { uint64_t link_bytes = 0, launches = 0; };

struct Slot {
  SlotState state = SlotState::Idle;
  Issue issue = Issue::Done;
  bool urgent = false;         // a restore is waiting for this queued offload
  bool failed = false;         // the deferred offload hit a CUDA error; `error` holds the text
  std::string error;
  std::unique_ptr<PushPlan> plan;
  uint64_t numel = 0, bytes = 0, stored_bytes = 0;
  int dtype = 0;
  float fp8_scale = 0.0f;
  std::vector<uint32_t> chunks;
  Event producer;  // compute stream, at push: the source is complete
  Event d2h_done;  // D2H stream: the source has been read, the pinned copy is complete
  Event consumer;  // compute stream, at pull: the destination may be written
  Event h2d_done;  // H2D stream: the pinned chunks have been read
  Event ready;     // the destination holds the restored tensor
};

struct Tile {
  uint8_t* dev = nullptr;
  Event full, free_;
};

// Asks the kernel to prefer `node` for this thread's next allocations.  Best
// effort: containers may forbid the call, in which case nothing changes.
void set_preferred_node(int node) {
#ifdef SYS_set_mempolicy
  if (node < 0) { syscall(SYS_set_mempolicy, 0 /*MPOL_DEFAULT*/, nullptr, 0); return; }
  unsigned long mask[16] = {0};
  if (node >= (int)(sizeof(mask) * 8)) return;
  mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
  syscall(SYS_set_mempolicy, 1 /*MPOL_PREFERRED*/, mask, sizeof(mask) * 8);
#else
  (void)node;
#endif
}

// FLAME_OFFLOAD_TRACE=1: one line per push / pull on stderr (the reference traces with env-gated
// eprintln!, e.g. FLAME_PROFILE and FLAME_COPY_TRACE, src/autograd.rs:1086-1089, src/staging.rs:382-415).
bool trace_on() {
  static const bool on = [] { const char* e = getenv("FLAME_OFFLOAD_TRACE"); return e && *e && *e != '0'; }();
  return on;
}

int gpu_numa_node(int device) {
  char bdf[32] = {0};
  if (cudaDeviceGetPCIBusId(bdf, sizeof(bdf), device) != cudaSuccess) return -1;
  for (char* p = bdf; *p; ++p) *p = (char)tolower(*p);
  char path[128];
  snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", bdf);
  FILE* f = fopen(path, "r");
  if (!f) return -1;
  int node = -1;
  if (fscanf(f, "%d", &node) != 1) node = -1;
  fclose(f);
  return node;
}

}  // namespace
}  // namespace flame_b200

using namespace flame_b200;

struct FlameOffloadPool {
  std::mutex mu;
  int device = 0;
  int compression = 0;
  size_t num_slots = 0, slot_bytes = 0;
  uint64_t chunk_src_bytes = 0;   // source bytes covered by one chunk
  uint64_t chunk_elems = 0;       // BF16 elements per chunk (compressed modes)
  uint64_t host_chunk_bytes = 0;  // pinned bytes per chunk
  uint32_t tile_chunks = 1;       // chunks per device staging tile = per codec launch
  uint64_t d2h_piece = 0, h2d_piece = 0;  // copies are issued in pieces of this size (0 = whole chunk)
  uint32_t codec_flags = 0;
  int codec_max_ctas = 0;

  uint8_t* slab = nullptr;
  size_t slab_bytes = 0;
  // Queue, not stack: a push takes the chunks that were released longest ago.  A chunk just released by a restore may
  // still be read by that restore's host-to-device copy, and the offload that takes it has to wait for that copy; with
  // first-in first-out reuse an offload issued beside restores (weights streaming in, the next step's forward) does
  // not queue up behind them.  Slots, which callers see, stay last in first out as in the reference.
  std::deque<uint32_t> free_chunks;
  std::vector<int32_t> chunk_last_reader;  // slot whose restore last read the chunk, -1 = none
  size_t total_chunks = 0;

  std::vector<Slot> slots;
  std::vector<size_t> free_stack;
  uint64_t epoch = 1;

  cudaStream_t s_quant = nullptr, s_d2h = nullptr, s_h2d = nullptr, s_dequant = nullptr;
  std::vector<Tile> out_tiles, in_tiles;
  uint64_t out_next = 0, in_next = 0;

  FlameOffloadStats stats{};

  // Optional timing (FlameOffloadPoolConfig.collect_timing): spans between two timing-enabled events, added to the
  // statistics once the device has passed them.  Offload spans are opened by whichever thread enqueues the offload
  // (the pool's own thread in the deferred mode), so the list has a lock of its own.
  struct Span { cudaEvent_t a, b; int kind; };     // kind 0: offload on the D2H stream, 1: restore on the H2D stream, 2: a wait for a restore
  bool timing = false;
  std::mutex timing_mu;
  std::vector<Span> spans;
  std::vector<cudaEvent_t> spare_events;
  uint64_t span_ns[3] = {0, 0, 0};
  uint64_t spans_done = 0;

  cudaEvent_t timing_event() {      // with timing_mu held
    if (!spare_events.empty()) { cudaEvent_t e = spare_events.back(); spare_events.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    return cudaEventCreate(&e) == cudaSuccess ? e : nullptr;
  }
  // Opens a span on `st`; returns its first event (nullptr when timing is off or no event could be made).
  cudaEvent_t span_open(cudaStream_t st) {
    if (!timing) return nullptr;
    std::lock_guard<std::mutex> lk(timing_mu);
    cudaEvent_t a = timing_event();
    if (a && cudaEventRecord(a, st) != cudaSuccess) { spare_events.push_back(a); a = nullptr; }
    return a;
  }
  void span_close(cudaEvent_t a, cudaStream_t st, int kind) {
    if (!a) return;
    std::lock_guard<std::mutex> lk(timing_mu);
    cudaEvent_t b = timing_event();
    if (!b || cudaEventRecord(b, st) != cudaSuccess) { spare_events.push_back(a); if (b) spare_events.push_back(b); return; }
    spans.push_back({a, b, kind});
  }
  // Adds every span the device has finished to the totals and takes its events back.
  void harvest_spans(size_t only_if_at_least = 0) {
    if (!timing) return;
    std::lock_guard<std::mutex> lk(timing_mu);
    if (spans.size() < only_if_at_least) return;
    size_t keep = 0;
    for (size_t i = 0; i < spans.size(); ++i) {
      const Span sp = spans[i];
      const cudaError_t q = cudaEventQuery(sp.b);
      if (q == cudaErrorNotReady) { spans[keep++] = sp; continue; }
      float ms = 0.0f;
      if (q == cudaSuccess && cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess && ms >= 0.0f) {
        span_ns[sp.kind] += (uint64_t)((double)ms * 1e6);
        spans_done++;
      }
      spare_events.push_back(sp.a);
      spare_events.push_back(sp.b);
    }
    spans.resize(keep);
  }

  // deferred offload
  bool deferred = false;
  uint64_t inflight_budget = 0, inflight_bytes = 0;
  std::deque<size_t> queue;                                // slots whose offload has not been enqueued, push order
  std::deque<std::pair<cudaEvent_t, uint64_t>> inflight;   // (d2h_done, pinned bytes) of enqueued offloads, oldest first
  bool hold = false, stop = false;
  Event hold_after;          // the hold begins when this event (recorded on the caller's stream) has completed
  bool hold_armed = false;
  std::thread worker;
  std::condition_variable cv_work, cv_issued;

  bool compressed() const { return compression != FLAME_OFFLOAD_COMPRESSION_NONE; }
  uint8_t* chunk_ptr(uint32_t c) const { return slab + (size_t)c * host_chunk_bytes; }

  // Pinned bytes one chunk of `e` elements (or `b` raw bytes) occupies.
  size_t stored_for(uint64_t e_or_bytes) const {
    switch (compression) {
      case FLAME_OFFLOAD_COMPRESSION_NONE: return e_or_bytes;
      case FLAME_OFFLOAD_COMPRESSION_FP8: return e_or_bytes;
      default: return packed_bytes(e_or_bytes);
    }
  }

  // A queued offload that never ran wrote nothing: whoever read these chunks last is still their last reader.
  void release_chunks_unwritten(Slot& s) {
    // they go back to the FRONT, in order: nothing was written and nobody reads them, so they are the best to take next
    for (auto it = s.chunks.rbegin(); it != s.chunks.rend(); ++it) free_chunks.push_front(*it);
    s.chunks.clear();
  }

  void release_chunks(Slot& s, int32_t reader) {
    for (uint32_t c : s.chunks) {
      chunk_last_reader[c] = reader;
      free_chunks.push_back(c);
    }
    s.chunks.clear();
  }

  FlameOffloadStatus check_handle(FlameOffloadHandle h, const char* who) const {
    if (h.epoch != epoch)
      return fail(FLAME_OFFLOAD_ERR_STATE, std::string(who) + ": handle epoch " + std::to_string(h.epoch) +
                  " is stale (current " + std::to_string(epoch) + "); was clear() called between push and pull?");
    if (h.slot >= slots.size())
      return fail(FLAME_OFFLOAD_ERR_STATE, std::string(who) + ": slot " + std::to_string(h.slot) + " out of range (" +
                  std::to_string(slots.size()) + " slots)");
    if (slots[h.slot].state != SlotState::Pushed)
      return fail(FLAME_OFFLOAD_ERR_STATE, std::string(who) + ": slot " + std::to_string(h.slot) +
                  " is Idle, expected Pushed; double pull, or handle reuse after clear?");
    return FLAME_OFFLOAD_OK;
  }
};

namespace {

#define POOL_TRY(expr, what)                                  \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) { fail_cuda(_e, what); return _e; } \
  } while (0)

// One chunk's copy, optionally cut into pieces so that the copy engine leaves gaps on the link.
cudaError_t copy_in_pieces(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t st, uint64_t piece) {
  if (piece == 0 || piece >= bytes) return memcpy_async_checked(dst, src, bytes, kind, st);
  for (size_t off = 0; off < bytes; off += piece) {
    cudaError_t e = memcpy_async_checked(static_cast<uint8_t*>(dst) + off, static_cast<const uint8_t*>(src) + off,
                                         std::min<size_t>(piece, bytes - off), kind, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t kernel_guard() { return fault_fires(FLAME_OFFLOAD_FAULT_KERNEL) ? cudaErrorLaunchFailure : cudaSuccess; }

// Captures what the offload of slot `s` needs.  Called with the pool locked.
PushPlan make_plan(FlameOffloadPool& p, const Slot& s, const uint8_t* src) {
  PushPlan plan;
  plan.chunks = s.chunks;
  plan.src = src;
  plan.numel = s.numel;
  plan.bytes = s.bytes;
  plan.fp8_scale = s.fp8_scale;
  plan.producer = s.producer.ev;
  plan.d2h_done = s.d2h_done.ev;
  // A chunk that an earlier restore is still reading must not be overwritten.
  std::vector<int32_t> seen;
  for (uint32_t c : s.chunks) {
    const int32_t r = p.chunk_last_reader[c];
    if (r < 0 || std::find(seen.begin(), seen.end(), r) != seen.end()) continue;
    seen.push_back(r);
    if (p.slots[r].h2d_done.recorded) plan.readers.push_back(p.slots[r].h2d_done.ev);
  }
  return plan;
}

// Enqueue the offload of one tensor; `plan.producer` has been recorded on the caller's compute stream.
// Touches the compress and D2H streams and the outgoing tile ring, which belong to the calling thread
// (the caller's thread in the immediate mode, the pool's thread in the deferred mode), and nothing else
// that changes.  Returns the first CUDA error.
cudaError_t issue_push(FlameOffloadPool& p, const PushPlan& plan, PushCounts& n) {
  for (cudaEvent_t ev : plan.readers) POOL_TRY(cudaStreamWaitEvent(p.s_d2h, ev, 0), "push: wait(h2d_done)");
  const size_t nchunks = plan.chunks.size();
  cudaEvent_t span = nullptr;   // opened when the D2H stream has the source (or the first tile) in front of it
  if (plan.scales_src) {
    // Compressed by its producer: each chunk's codes and scales go straight to their places in the pinned chunk.
    POOL_TRY(cudaStreamWaitEvent(p.s_d2h, plan.producer, 0), "push: wait(producer)");
    span = p.span_open(p.s_d2h);
    for (size_t k = 0; k < nchunks; ++k) {
      const uint64_t e0 = k * p.chunk_elems;
      const uint64_t ec = std::min<uint64_t>(p.chunk_elems, plan.numel - e0);
      const uint64_t sb = 4u * ((ec + 127u) / 128u);
      uint8_t* dst = p.chunk_ptr(plan.chunks[k]);
      POOL_TRY(copy_in_pieces(dst, plan.src + e0, ec, cudaMemcpyDeviceToHost, p.s_d2h, p.d2h_piece), "push: D2H(codes)");
      POOL_TRY(memcpy_async_checked(dst + packed_scales_offset(ec), plan.scales_src + 4u * (e0 / 128u), sb, cudaMemcpyDeviceToHost, p.s_d2h),
               "push: D2H(scales)");
      n.link_bytes += ec + sb;
    }
  } else if (!p.compressed()) {
    POOL_TRY(cudaStreamWaitEvent(p.s_d2h, plan.producer, 0), "push: wait(producer)");
    span = p.span_open(p.s_d2h);
    for (size_t k = 0; k < nchunks; ++k) {
      const uint64_t off = k * p.chunk_src_bytes;
      const uint64_t len = std::min<uint64_t>(p.chunk_src_bytes, plan.bytes - off);
      POOL_TRY(copy_in_pieces(p.chunk_ptr(plan.chunks[k]), plan.src + off, len, cudaMemcpyDeviceToHost, p.s_d2h, p.d2h_piece), "push: D2H");
      n.link_bytes += len;
    }
  } else {
    POOL_TRY(cudaStreamWaitEvent(p.s_quant, plan.producer, 0), "push: wait(producer)");
    // One codec launch fills a staging tile of up to tile_chunks self-contained
    // chunks; each chunk then crosses the link as one copy.
    for (size_t k0 = 0; k0 < nchunks; k0 += p.tile_chunks) {
      const size_t kn = std::min<size_t>(p.tile_chunks, nchunks - k0);
      const uint64_t e0 = k0 * p.chunk_elems;
      const uint64_t e = std::min<uint64_t>(kn * p.chunk_elems, plan.numel - e0);
      Tile& t = p.out_tiles[p.out_next++ % p.out_tiles.size()];
      POOL_TRY(t.free_.make_wait(p.s_quant), "push: wait(tile free)");
      POOL_TRY(kernel_guard(), "push: compress kernel");
      const void* in = plan.src + 2 * e0;
      if (p.compression == FLAME_OFFLOAD_COMPRESSION_FP8)
        POOL_TRY(launch_bf16_to_fp8(in, t.dev, 1.0f / plan.fp8_scale, e, p.s_quant, p.codec_max_ctas), "push: bf16_to_fp8");
      else
        POOL_TRY(launch_compress(p.compression, in, t.dev, e, packed_chunks_layout(e, p.chunk_elems, p.host_chunk_bytes),
                                 p.codec_flags, p.s_quant, p.codec_max_ctas), "push: compress");
      n.launches++;
      POOL_TRY(t.full.record(p.s_quant), "push: record(tile full)");
      POOL_TRY(t.full.make_wait(p.s_d2h), "push: wait(tile full)");
      if (k0 == 0) span = p.span_open(p.s_d2h);
      for (size_t j = 0; j < kn; ++j) {
        const uint64_t ec = std::min<uint64_t>(p.chunk_elems, e - j * p.chunk_elems);
        const size_t link = p.stored_for(ec);
        POOL_TRY(copy_in_pieces(p.chunk_ptr(plan.chunks[k0 + j]), t.dev + j * p.host_chunk_bytes, link,
                                cudaMemcpyDeviceToHost, p.s_d2h, p.d2h_piece), "push: D2H");
        n.link_bytes += link;
      }
      POOL_TRY(t.free_.record(p.s_d2h), "push: record(tile free)");
    }
  }
  POOL_TRY(cudaEventRecord(plan.d2h_done, p.s_d2h), "push: record(d2h_done)");
  p.span_close(span, p.s_d2h, 0);
  return cudaSuccess;
}

void count_push(FlameOffloadPool& p, const PushPlan& plan, const PushCounts& n) {
  p.stats.bytes_link_out += n.link_bytes;
  p.stats.codec_launches += n.launches;
  p.stats.chunks_out += plan.chunks.size();
}

// The pool's thread in the deferred mode: enqueues queued offloads in push order while the pinned bytes
// in flight are under the budget (a tensor that a restore is waiting for goes first and always runs).
void deferred_worker(FlameOffloadPool* p) {
  cudaSetDevice(p->device);
  std::unique_lock<std::mutex> lk(p->mu);
  while (!p->stop) {
    while (!p->inflight.empty() && cudaEventQuery(p->inflight.front().first) != cudaErrorNotReady) {
      p->inflight_bytes -= p->inflight.front().second;
      p->inflight.pop_front();
    }
    if (p->hold_armed && cudaEventQuery(p->hold_after.ev) != cudaErrorNotReady) {
      p->hold = true;
      p->hold_armed = false;
    }
    bool take = false;
    if (!p->queue.empty()) {
      const Slot& c = p->slots[p->queue.front()];
      take = c.urgent || (!p->hold && p->inflight_bytes < p->inflight_budget);
    }
    if (!take) {
      if (p->queue.empty() && p->inflight.empty() && !p->hold_armed) p->cv_work.wait(lk);
      else p->cv_work.wait_for(lk, std::chrono::microseconds(100));
      continue;
    }
    const size_t slot = p->queue.front();
    p->queue.pop_front();
    Slot& s = p->slots[slot];
    s.issue = Issue::Issuing;
    std::unique_ptr<PushPlan> plan = std::move(s.plan);
    lk.unlock();
    PushCounts n;
    const cudaError_t e = issue_push(*p, *plan, n);
    std::string text = e == cudaSuccess ? std::string() : std::string(flame_offload_last_error());
    lk.lock();
    if (e == cudaSuccess) {
      s.d2h_done.recorded = true;
      count_push(*p, *plan, n);
      p->inflight.emplace_back(plan->d2h_done, n.link_bytes);
      p->inflight_bytes += n.link_bytes;
    } else {
      s.failed = true;
      s.error = text;
    }
    s.issue = Issue::Done;
    s.urgent = false;
    p->stats.pushes_queued = p->queue.size();
    p->cv_issued.notify_all();
  }
}

// Waits (bounded) until the offload of slot `s` has been enqueued, moving it to the head of the queue.
// Called with `lk` held.
FlameOffloadStatus wait_issued(FlameOffloadPool* p, std::unique_lock<std::mutex>& lk, size_t slot, const char* who) {
  Slot& s = p->slots[slot];
  if (s.issue == Issue::Queued) {
    auto it = std::find(p->queue.begin(), p->queue.end(), slot);
    if (it != p->queue.end()) { p->queue.erase(it); p->queue.push_front(slot); }
    s.urgent = true;
    p->cv_work.notify_all();
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30);
  while (s.issue != Issue::Done) {
    if (p->cv_issued.wait_until(lk, deadline) == std::cv_status::timeout && s.issue != Issue::Done)
      return fail(FLAME_OFFLOAD_ERR_TIMEOUT, std::string(who) + ": the pool's thread did not enqueue the offload within 30 s");
  }
  return FLAME_OFFLOAD_OK;
}

cudaError_t enqueue_pull(FlameOffloadPool& p, Slot& s, uint8_t* dst, uint8_t* scales_dst, cudaStream_t compute, unsigned flags) {
  POOL_TRY(s.consumer.record(compute), "pull: cudaEventRecord(consumer)");
  POOL_TRY(s.d2h_done.make_wait(p.s_h2d), "pull: wait(d2h_done)");
  const size_t nchunks = s.chunks.size();
  cudaEvent_t span = p.span_open(p.s_h2d);
  if (scales_dst) {
    // The compressed form itself is wanted (the caller dequantises it, several tensors to a launch): each chunk's
    // codes and scales go straight to their places in the caller's two buffers; no staging tile, no kernel.
    POOL_TRY(s.consumer.make_wait(p.s_h2d), "pull: wait(consumer)");
    for (size_t k = 0; k < nchunks; ++k) {
      const uint64_t e0 = k * p.chunk_elems;
      const uint64_t ec = std::min<uint64_t>(p.chunk_elems, s.numel - e0);
      const uint64_t sb = 4u * ((ec + 127u) / 128u);
      const uint8_t* src = p.chunk_ptr(s.chunks[k]);
      POOL_TRY(copy_in_pieces(dst + e0, src, ec, cudaMemcpyHostToDevice, p.s_h2d, p.h2d_piece), "pull: H2D(codes)");
      POOL_TRY(memcpy_async_checked(scales_dst + 4u * (e0 / 128u), src + packed_scales_offset(ec), sb, cudaMemcpyHostToDevice, p.s_h2d),
               "pull: H2D(scales)");
      p.stats.bytes_link_in += ec + sb;
    }
    POOL_TRY(s.h2d_done.record(p.s_h2d), "pull: record(h2d_done)");
    POOL_TRY(s.ready.record(p.s_h2d), "pull: record(ready)");
  } else if (!p.compressed()) {
    POOL_TRY(s.consumer.make_wait(p.s_h2d), "pull: wait(consumer)");
    for (size_t k = 0; k < nchunks; ++k) {
      const uint64_t off = k * p.chunk_src_bytes;
      const uint64_t len = std::min<uint64_t>(p.chunk_src_bytes, s.bytes - off);
      POOL_TRY(copy_in_pieces(dst + off, p.chunk_ptr(s.chunks[k]), len, cudaMemcpyHostToDevice, p.s_h2d, p.h2d_piece), "pull: H2D");
      p.stats.bytes_link_in += len;
    }
    POOL_TRY(s.h2d_done.record(p.s_h2d), "pull: record(h2d_done)");
    POOL_TRY(s.ready.record(p.s_h2d), "pull: record(ready)");
  } else {
    POOL_TRY(s.consumer.make_wait(p.s_dequant), "pull: wait(consumer)");
    for (size_t k0 = 0; k0 < nchunks; k0 += p.tile_chunks) {
      const size_t kn = std::min<size_t>(p.tile_chunks, nchunks - k0);
      const uint64_t e0 = k0 * p.chunk_elems;
      const uint64_t e = std::min<uint64_t>(kn * p.chunk_elems, s.numel - e0);
      Tile& t = p.in_tiles[p.in_next++ % p.in_tiles.size()];
      POOL_TRY(t.free_.make_wait(p.s_h2d), "pull: wait(tile free)");
      for (size_t j = 0; j < kn; ++j) {
        const uint64_t ec = std::min<uint64_t>(p.chunk_elems, e - j * p.chunk_elems);
        const size_t link = p.stored_for(ec);
        POOL_TRY(copy_in_pieces(t.dev + j * p.host_chunk_bytes, p.chunk_ptr(s.chunks[k0 + j]), link,
                                cudaMemcpyHostToDevice, p.s_h2d, p.h2d_piece), "pull: H2D");
        p.stats.bytes_link_in += link;
      }
      POOL_TRY(t.full.record(p.s_h2d), "pull: record(tile full)");
      POOL_TRY(t.full.make_wait(p.s_dequant), "pull: wait(tile full)");
      POOL_TRY(kernel_guard(), "pull: dequantise kernel");
      void* out = dst + 2 * e0;
      if (p.compression == FLAME_OFFLOAD_COMPRESSION_FP8)
        POOL_TRY(launch_fp8_to_bf16(t.dev, out, s.fp8_scale, e, p.s_dequant, p.codec_max_ctas), "pull: fp8_to_bf16");
      else
        POOL_TRY(launch_dequant(p.compression, t.dev, out, e, packed_chunks_layout(e, p.chunk_elems, p.host_chunk_bytes),
                                p.s_dequant, p.codec_max_ctas), "pull: dequantise");
      p.stats.codec_launches++;
      POOL_TRY(t.free_.record(p.s_dequant), "pull: record(tile free)");
    }
    POOL_TRY(s.h2d_done.record(p.s_h2d), "pull: record(h2d_done)");
    POOL_TRY(s.ready.record(p.s_dequant), "pull: record(ready)");
  }
  p.span_close(span, p.s_h2d, 1);
  if (!(flags & FLAME_OFFLOAD_PULL_DEFER_WAIT)) {
    cudaEvent_t w = p.span_open(compute);
    POOL_TRY(s.ready.make_wait(compute), "pull: wait(ready)");
    p.span_close(w, compute, 2);
  }
  p.stats.chunks_in += nchunks;
  return cudaSuccess;
}

void destroy_pool(FlameOffloadPool* p) {
  for (auto& sp : p->spans) { cudaEventDestroy(sp.a); cudaEventDestroy(sp.b); }
  for (cudaEvent_t e : p->spare_events) cudaEventDestroy(e);
  p->hold_after.destroy();
  for (auto& s : p->slots) { s.producer.destroy(); s.d2h_done.destroy(); s.consumer.destroy(); s.h2d_done.destroy(); s.ready.destroy(); }
  for (auto* ring : {&p->out_tiles, &p->in_tiles})
    for (auto& t : *ring) { t.full.destroy(); t.free_.destroy(); if (t.dev) cudaFree(t.dev); }
  for (cudaStream_t s : {p->s_quant, p->s_d2h, p->s_h2d, p->s_dequant}) if (s) cudaStreamDestroy(s);
  if (p->slab) cudaFreeHost(p->slab);
  delete p;
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

FlameOffloadStatus poll_streams(FlameOffloadPool* p, double timeout_s) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  for (;;) {
    bool busy = false;
    for (cudaStream_t s : {p->s_quant, p->s_d2h, p->s_h2d, p->s_dequant}) {
      cudaError_t e = cudaStreamQuery(s);
      if (e == cudaErrorNotReady) busy = true;
      else if (e != cudaSuccess) return fail_cuda(e, "synchronize: cudaStreamQuery");
    }
    if (!busy) return FLAME_OFFLOAD_OK;
    if (std::chrono::steady_clock::now() >= deadline)
      return fail(FLAME_OFFLOAD_ERR_TIMEOUT, "synchronize: pool streams still busy after the timeout");
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

FlameOffloadStatus poll_event(cudaEvent_t ev, double timeout_s, const char* what) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  for (;;) {
    cudaError_t e = cudaEventQuery(ev);
    if (e == cudaSuccess) return FLAME_OFFLOAD_OK;
    if (e != cudaErrorNotReady) return fail_cuda(e, what);
    if (std::chrono::steady_clock::now() >= deadline) return fail(FLAME_OFFLOAD_ERR_TIMEOUT, std::string(what) + ": timed out");
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

}  // namespace

extern "C" {

FlameOffloadPool* flame_offload_pool_create(size_t num_slots, size_t max_bytes, int compression, const FlameOffloadPoolConfig* cfg_in) {
  // Argument checks of src/activation_offload.rs:371-380.
  if (num_slots == 0) { fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::new: num_slots must be > 0"); return nullptr; }
  if (max_bytes == 0) { fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::new: max_bytes must be > 0"); return nullptr; }
  if (compression < 0 || compression > FLAME_OFFLOAD_COMPRESSION_FP8_B128) {
    fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::new: unknown compression mode");
    return nullptr;
  }
  FlameOffloadPoolConfig cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.device = -1;
  cfg.numa_node = -2;  // look the GPU's node up in sysfs
  if (cfg_in) {
    if (cfg_in->struct_size == 0 || cfg_in->struct_size > sizeof(cfg)) {
      fail(FLAME_OFFLOAD_ERR_INVALID, "FlameOffloadPoolConfig.struct_size is not set");
      return nullptr;
    }
    memcpy(&cfg, cfg_in, cfg_in->struct_size);
  }
  int device = cfg.device;
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { fail(FLAME_OFFLOAD_ERR_CUDA, "cudaGetDevice failed"); return nullptr; }
  uint64_t chunk = cfg.chunk_bytes ? cfg.chunk_bytes : kDefaultChunkBytes;
  if (chunk % (64u << 10) != 0) { fail(FLAME_OFFLOAD_ERR_INVALID, "chunk_bytes must be a multiple of 64 KiB"); return nullptr; }

  DeviceGuard guard(device);
  auto* p = new FlameOffloadPool();
  p->device = device;
  p->compression = compression;
  p->num_slots = num_slots;
  p->slot_bytes = max_bytes;
  p->codec_flags = cfg.codec_flags;
  p->codec_max_ctas = cfg.codec_max_ctas;
  p->d2h_piece = cfg.d2h_piece_bytes;
  p->h2d_piece = cfg.h2d_piece_bytes;
  p->timing = cfg.collect_timing != 0;

  // A slot that fits in one chunk gets a chunk of exactly its stored size, so a
  // pool of small slots holds num_slots * stored(max_bytes) pinned bytes like
  // the reference (src/activation_offload.rs:383-399, 441-449).
  const bool single = max_bytes <= chunk;
  p->chunk_src_bytes = single ? max_bytes : chunk;
  const size_t chunks_per_slot = single ? 1 : (max_bytes + chunk - 1) / chunk;
  if (compression == FLAME_OFFLOAD_COMPRESSION_NONE) {
    p->host_chunk_bytes = p->chunk_src_bytes;
  } else {
    p->chunk_elems = single ? (max_bytes + 1) / 2 : chunk / 2;
    p->host_chunk_bytes = p->stored_for(p->chunk_elems);
  }
  p->tile_chunks = single ? 1 : std::max<uint32_t>(1, cfg.tile_chunks ? cfg.tile_chunks : kDefaultTileChunks);
  p->tile_chunks = (uint32_t)std::min<size_t>(p->tile_chunks, chunks_per_slot);
  size_t total = num_slots * chunks_per_slot;
  if (cfg.host_budget_bytes) total = std::max<size_t>(1, cfg.host_budget_bytes / p->host_chunk_bytes);
  p->total_chunks = total;
  p->slab_bytes = total * p->host_chunk_bytes;

  int node = cfg.numa_node == -2 ? gpu_numa_node(device) : cfg.numa_node;
  if (node >= 0) set_preferred_node(node);
  void* slab = nullptr;
  cudaError_t e = host_alloc_checked(&slab, p->slab_bytes, cfg.host_alloc_flags);
  if (node >= 0) set_preferred_node(-1);
  if (e != cudaSuccess || !slab) {
    fail_cuda(e, "ActivationOffloadPool::new: cudaHostAlloc of the pinned slab");
    destroy_pool(p);
    return nullptr;
  }
  p->slab = static_cast<uint8_t*>(slab);
  p->chunk_last_reader.assign(total, -1);
  for (size_t c = 0; c < total; ++c) p->free_chunks.push_back((uint32_t)c);

  bool ok = true;
  auto chk = [&](cudaError_t err, const char* what) { if (ok && err != cudaSuccess) { fail_cuda(err, what); ok = false; } };
  int lo = 0, hi = 0;
  chk(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
  // Codec kernels are short and feed the copy engines: highest priority, so they
  // are scheduled ahead of queued compute blocks.
  chk(cudaStreamCreateWithPriority(&p->s_quant, cudaStreamNonBlocking, hi), "cudaStreamCreate(quant)");
  chk(cudaStreamCreateWithPriority(&p->s_dequant, cudaStreamNonBlocking, hi), "cudaStreamCreate(dequant)");
  chk(cudaStreamCreateWithFlags(&p->s_d2h, cudaStreamNonBlocking), "cudaStreamCreate(d2h)");
  chk(cudaStreamCreateWithFlags(&p->s_h2d, cudaStreamNonBlocking), "cudaStreamCreate(h2d)");

  p->slots.resize(num_slots);
  for (auto& s : p->slots) {
    chk(s.producer.create(), "cudaEventCreate"); chk(s.d2h_done.create(), "cudaEventCreate");
    chk(s.consumer.create(), "cudaEventCreate"); chk(s.h2d_done.create(), "cudaEventCreate");
    chk(s.ready.create(), "cudaEventCreate");
  }
  p->free_stack.reserve(num_slots);
  for (size_t i = num_slots; i-- > 0;) p->free_stack.push_back(i);  // slot 0 on top

  if (p->compressed()) {
    const uint32_t tiles = cfg.staging_tiles ? cfg.staging_tiles : kDefaultTiles;
    for (auto* ring : {&p->out_tiles, &p->in_tiles}) {
      ring->resize(tiles);
      for (auto& t : *ring) {
        void* d = nullptr;
        chk(cudaMalloc(&d, p->host_chunk_bytes * p->tile_chunks), "cudaMalloc(staging tile)");
        t.dev = static_cast<uint8_t*>(d);
        chk(t.full.create(), "cudaEventCreate"); chk(t.free_.create(), "cudaEventCreate");
      }
    }
  }
  if (!ok) { destroy_pool(p); return nullptr; }
  if (cfg.deferred_inflight_bytes) {
    if (p->hold_after.create() != cudaSuccess) { fail(FLAME_OFFLOAD_ERR_CUDA, "cudaEventCreate(hold_after)"); destroy_pool(p); return nullptr; }
    p->deferred = true;
    p->inflight_budget = cfg.deferred_inflight_bytes;
    p->worker = std::thread(deferred_worker, p);
  }
  p->stats.host_chunks_total = total;
  p->stats.host_chunks_free = total;
  return p;
}

void flame_offload_pool_destroy(FlameOffloadPool* p) {
  if (!p) return;
  if (p->worker.joinable()) {
    { std::lock_guard<std::mutex> lk(p->mu); p->stop = true; }
    p->cv_work.notify_all();
    p->worker.join();
  }
  DeviceGuard guard(p->device);
  poll_streams(p, 30.0);
  destroy_pool(p);
}

size_t flame_offload_pool_num_slots(const FlameOffloadPool* p) { return p ? p->num_slots : 0; }
size_t flame_offload_pool_slot_bytes(const FlameOffloadPool* p) { return p ? p->slot_bytes : 0; }
size_t flame_offload_pool_host_bytes(const FlameOffloadPool* p) { return p ? p->slab_bytes : 0; }
int flame_offload_pool_compression(const FlameOffloadPool* p) { return p ? p->compression : -1; }

size_t flame_offload_pool_in_flight(const FlameOffloadPool* pc) {
  auto* p = const_cast<FlameOffloadPool*>(pc);
  if (!p) return 0;
  std::lock_guard<std::mutex> lk(p->mu);
  size_t n = 0;
  for (auto& s : p->slots) n += s.state == SlotState::Pushed;
  return n;
}

static FlameOffloadStatus push_impl(FlameOffloadPool* p, const void* src, const void* packed_scales, size_t numel, int dtype, void* compute_stream, FlameOffloadHandle* out);

FlameOffloadStatus flame_offload_pool_push(FlameOffloadPool* p, const void* src, size_t numel, int dtype, void* compute_stream, FlameOffloadHandle* out) {
  return push_impl(p, src, nullptr, numel, dtype, compute_stream, out);
}

FlameOffloadStatus flame_offload_pool_push_packed(FlameOffloadPool* p, const void* codes, const void* scales, size_t numel, void* compute_stream, FlameOffloadHandle* out) {
  if (!p || !out) return fail(FLAME_OFFLOAD_ERR_INVALID, "push_packed: null pool or handle pointer");
  if (p->compression != FLAME_OFFLOAD_COMPRESSION_INT8_B128 && p->compression != FLAME_OFFLOAD_COMPRESSION_FP8_B128)
    return fail(FLAME_OFFLOAD_ERR_UNSUPPORTED, "push_packed: the pool is not in a per-128-block mode");
  if (!scales) return fail(FLAME_OFFLOAD_ERR_INVALID, "push_packed: null scales pointer");
  return push_impl(p, codes, scales, numel, FLAME_OFFLOAD_DTYPE_BF16, compute_stream, out);
}

static FlameOffloadStatus push_impl(FlameOffloadPool* p, const void* src, const void* packed_scales, size_t numel, int dtype, void* compute_stream, FlameOffloadHandle* out) {
  if (!p || !out) return fail(FLAME_OFFLOAD_ERR_INVALID, "push: null pool or handle pointer");
  // Dtype gate, src/activation_offload.rs:467-476.
  if (dtype != FLAME_OFFLOAD_DTYPE_BF16 && dtype != FLAME_OFFLOAD_DTYPE_F32)
    return fail(FLAME_OFFLOAD_ERR_UNSUPPORTED, "ActivationOffloadPool::push: dtype not supported (BF16/F32 only)");
  const size_t esz = dtype == FLAME_OFFLOAD_DTYPE_BF16 ? 2 : 4;
  const size_t bytes = numel * esz;
  if (bytes == 0) return fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::push: tensor is empty");
  if (!src) return fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::push: null source pointer");
  if (bytes > p->slot_bytes)
    return fail(FLAME_OFFLOAD_ERR_INVALID, "ActivationOffloadPool::push: tensor " + std::to_string(bytes) +
                " bytes exceeds slot capacity " + std::to_string(p->slot_bytes) + " bytes");

  std::lock_guard<std::mutex> lk(p->mu);
  DeviceGuard guard(p->device);
  if (p->free_stack.empty()) {
    p->stats.push_rejected_full++;
    return fail(FLAME_OFFLOAD_ERR_STATE, "ActivationOffloadPool full: " + std::to_string(p->num_slots) +
                " slots all in-flight. Increase num_slots.");
  }
  // Compression applies to BF16 only (src/activation_offload.rs:537-542).
  if (p->compressed() && dtype != FLAME_OFFLOAD_DTYPE_BF16)
    return fail(FLAME_OFFLOAD_ERR_UNSUPPORTED, "compressed offload only supports BF16 activations");

  const size_t nchunks = p->compressed() ? (numel + p->chunk_elems - 1) / p->chunk_elems
                                         : (bytes + p->chunk_src_bytes - 1) / p->chunk_src_bytes;
  if (nchunks > p->free_chunks.size()) {
    p->stats.push_rejected_full++;
    return fail(FLAME_OFFLOAD_ERR_STATE, "ActivationOffloadPool full: pinned slab exhausted (" +
                std::to_string(p->free_chunks.size()) + " chunks free, " + std::to_string(nchunks) + " needed)");
  }
  const size_t slot = p->free_stack.back();
  p->free_stack.pop_back();
  Slot& s = p->slots[slot];
  s.numel = numel; s.bytes = bytes; s.dtype = dtype;
  s.fp8_scale = p->compression == FLAME_OFFLOAD_COMPRESSION_FP8 ? kLegacyFp8Scale : 0.0f;
  s.chunks.clear();
  s.stored_bytes = 0;
  for (size_t k = 0; k < nchunks; ++k) {
    s.chunks.push_back(p->free_chunks.front());
    p->free_chunks.pop_front();
    if (p->compressed()) s.stored_bytes += p->stored_for(std::min<uint64_t>(p->chunk_elems, numel - k * p->chunk_elems));
  }
  if (!p->compressed()) s.stored_bytes = bytes;

  s.failed = false;
  s.error.clear();
  s.urgent = false;
  s.d2h_done.recorded = false;
  cudaError_t e = s.producer.record((cudaStream_t)compute_stream);
  if (e != cudaSuccess) fail_cuda(e, "push: cudaEventRecord(producer)");
  if (e == cudaSuccess) {
    PushPlan plan = make_plan(*p, s, static_cast<const uint8_t*>(src));
    plan.scales_src = static_cast<const uint8_t*>(packed_scales);
    if (p->deferred) {
      s.plan.reset(new PushPlan(std::move(plan)));
      s.issue = Issue::Queued;
      p->queue.push_back(slot);
      p->stats.pushes_queued = p->queue.size();
      p->cv_work.notify_one();
    } else {
      PushCounts n;
      e = issue_push(*p, plan, n);
      if (e == cudaSuccess) { s.d2h_done.recorded = true; count_push(*p, plan, n); }
    }
  }
  if (e != cudaSuccess) {
    // As the reference does on a failed copy (src/activation_offload.rs:528-533): the slot goes back.
    p->release_chunks(s, -1);
    p->free_stack.push_back(slot);
    return FLAME_OFFLOAD_ERR_CUDA;
  }
  s.state = SlotState::Pushed;
  if (trace_on())
    fprintf(stderr, "[flame_offload] push slot=%zu epoch=%llu numel=%zu dtype=%d bytes=%zu stored=%llu chunks=%zu free_chunks=%zu\n", slot,
            (unsigned long long)p->epoch, numel, dtype, bytes, (unsigned long long)s.stored_bytes, nchunks, p->free_chunks.size());
  p->harvest_spans(512);   // keeps the list of open spans short when nobody reads the statistics
  p->stats.pushes++;
  p->stats.bytes_logical_out += bytes;
  p->stats.host_chunks_free = p->free_chunks.size();
  out->slot = slot;
  out->epoch = p->epoch;
  return FLAME_OFFLOAD_OK;
}

static FlameOffloadStatus pull_impl(FlameOffloadPool* p, FlameOffloadHandle h, void* dst, size_t dst_bytes, void* scales_dst, void* compute_stream, unsigned int flags);

FlameOffloadStatus flame_offload_pool_pull_into(FlameOffloadPool* p, FlameOffloadHandle h, void* dst, size_t dst_bytes, void* compute_stream, unsigned int flags) {
  return pull_impl(p, h, dst, dst_bytes, nullptr, compute_stream, flags);
}

FlameOffloadStatus flame_offload_pool_pull_packed(FlameOffloadPool* p, FlameOffloadHandle h, void* codes_dst, void* scales_dst, void* compute_stream, unsigned int flags) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "pull_packed: null pool");
  if (p->compression != FLAME_OFFLOAD_COMPRESSION_INT8_B128 && p->compression != FLAME_OFFLOAD_COMPRESSION_FP8_B128)
    return fail(FLAME_OFFLOAD_ERR_UNSUPPORTED, "pull_packed: the pool is not in a per-128-block mode");
  if (!scales_dst) return fail(FLAME_OFFLOAD_ERR_INVALID, "pull_packed: null scales destination");
  return pull_impl(p, h, codes_dst, (size_t)-1, scales_dst, compute_stream, flags);
}

static FlameOffloadStatus pull_impl(FlameOffloadPool* p, FlameOffloadHandle h, void* dst, size_t dst_bytes, void* scales_dst, void* compute_stream, unsigned int flags) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "pull: null pool");
  std::unique_lock<std::mutex> lk(p->mu);
  FlameOffloadStatus st = p->check_handle(h, "ActivationOffloadPool::pull");
  if (st != FLAME_OFFLOAD_OK) return st;
  Slot& s = p->slots[h.slot];
  if (!dst) return fail(FLAME_OFFLOAD_ERR_INVALID, "pull: null destination");
  if (dst_bytes < s.bytes)
    return fail(FLAME_OFFLOAD_ERR_INVALID, "pull: destination holds " + std::to_string(dst_bytes) + " bytes, tensor needs " + std::to_string(s.bytes));
  if (s.issue != Issue::Done) {  // deferred and not enqueued yet: it jumps the queue, then the restore follows it
    st = wait_issued(p, lk, h.slot, "pull");
    if (st != FLAME_OFFLOAD_OK) return st;
  }
  if (s.failed) {  // the deferred offload itself failed: the data never reached the host; the slot is given up
    const std::string text = "pull: the deferred offload of this slot failed: " + s.error;
    s.state = SlotState::Idle;
    p->release_chunks(s, -1);
    p->free_stack.push_back(h.slot);
    p->stats.host_chunks_free = p->free_chunks.size();
    return fail(FLAME_OFFLOAD_ERR_CUDA, text);
  }
  DeviceGuard guard(p->device);
  cudaError_t e = enqueue_pull(*p, s, static_cast<uint8_t*>(dst), static_cast<uint8_t*>(scales_dst), (cudaStream_t)compute_stream, flags);
  if (e != cudaSuccess) return FLAME_OFFLOAD_ERR_CUDA;  // slot stays Pushed (src/activation_offload.rs:704-711)
  if (trace_on())
    fprintf(stderr, "[flame_offload] pull slot=%llu bytes=%llu chunks=%zu deferred_wait=%u keep=%u\n", (unsigned long long)h.slot,
            (unsigned long long)s.bytes, s.chunks.size(), flags & FLAME_OFFLOAD_PULL_DEFER_WAIT, (flags & FLAME_OFFLOAD_PULL_KEEP) >> 1);
  if (!(flags & FLAME_OFFLOAD_PULL_KEEP)) {
    s.state = SlotState::Idle;
    p->release_chunks(s, (int32_t)h.slot);
    p->free_stack.push_back(h.slot);
  }
  p->stats.pulls++;
  p->stats.bytes_logical_in += s.bytes;
  p->stats.host_chunks_free = p->free_chunks.size();
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_prefetch(FlameOffloadPool* p, FlameOffloadHandle h, void* dst, size_t dst_bytes, void* compute_stream) {
  return flame_offload_pool_pull_into(p, h, dst, dst_bytes, compute_stream, FLAME_OFFLOAD_PULL_DEFER_WAIT);
}

int flame_offload_pool_cancel(FlameOffloadPool* p, FlameOffloadHandle h) {
  if (!p) return -(int)fail(FLAME_OFFLOAD_ERR_INVALID, "cancel: null pool");
  std::lock_guard<std::mutex> lk(p->mu);
  FlameOffloadStatus st = p->check_handle(h, "ActivationOffloadPool::cancel");
  if (st != FLAME_OFFLOAD_OK) return -(int)st;
  Slot& s = p->slots[h.slot];
  if (s.issue != Issue::Queued) return 0;
  p->queue.erase(std::find(p->queue.begin(), p->queue.end(), (size_t)h.slot));
  s.plan.reset();
  s.issue = Issue::Done;
  s.state = SlotState::Idle;
  p->release_chunks_unwritten(s);
  p->free_stack.push_back(h.slot);
  p->stats.pushes_cancelled++;
  p->stats.pushes_queued = p->queue.size();
  p->stats.host_chunks_free = p->free_chunks.size();
  if (trace_on()) fprintf(stderr, "[flame_offload] cancel slot=%llu (still on the device)\n", (unsigned long long)h.slot);
  return 1;
}

FlameOffloadStatus flame_offload_pool_hold(FlameOffloadPool* p, int on) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "hold: null pool");
  std::lock_guard<std::mutex> lk(p->mu);
  p->hold = on != 0;
  p->hold_armed = false;
  p->cv_work.notify_all();
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_hold_after(FlameOffloadPool* p, void* stream) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "hold_after: null pool");
  std::lock_guard<std::mutex> lk(p->mu);
  if (!p->deferred) return FLAME_OFFLOAD_OK;
  DeviceGuard guard(p->device);
  cudaError_t e = p->hold_after.record((cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(e, "hold_after: cudaEventRecord");
  p->hold_armed = true;
  p->cv_work.notify_all();
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_discard(FlameOffloadPool* p, FlameOffloadHandle h) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "discard: null pool");
  std::unique_lock<std::mutex> lk(p->mu);
  FlameOffloadStatus st = p->check_handle(h, "ActivationOffloadPool::discard");
  if (st != FLAME_OFFLOAD_OK) return st;
  Slot& s = p->slots[h.slot];
  if (s.issue == Issue::Queued) {  // never enqueued: nothing was written
    p->queue.erase(std::find(p->queue.begin(), p->queue.end(), (size_t)h.slot));
    s.plan.reset();
    s.issue = Issue::Done;
    s.state = SlotState::Idle;
    p->release_chunks_unwritten(s);
    p->free_stack.push_back(h.slot);
    p->stats.pushes_cancelled++;
    p->stats.pushes_queued = p->queue.size();
    p->stats.host_chunks_free = p->free_chunks.size();
    return FLAME_OFFLOAD_OK;
  }
  if (s.issue == Issue::Issuing) {
    st = wait_issued(p, lk, h.slot, "discard");
    if (st != FLAME_OFFLOAD_OK) return st;
  }
  s.state = SlotState::Idle;
  // An offload that is still writing these chunks runs on the D2H stream, the
  // stream every later offload into them is queued on, so reuse stays ordered.
  // A restore that kept the slot (FLAME_OFFLOAD_PULL_KEEP) may still be reading
  // them: the next writer waits for this slot's last host-to-device copy.
  p->release_chunks(s, s.h2d_done.recorded ? (int32_t)h.slot : -1);
  p->free_stack.push_back(h.slot);
  p->stats.host_chunks_free = p->free_chunks.size();
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_wait_ready(FlameOffloadPool* p, size_t slot, void* stream) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "wait_ready: null pool");
  std::lock_guard<std::mutex> lk(p->mu);
  if (slot >= p->slots.size()) return fail(FLAME_OFFLOAD_ERR_STATE, "wait_ready: slot out of range");
  DeviceGuard guard(p->device);
  cudaEvent_t w = p->span_open((cudaStream_t)stream);
  cudaError_t e = p->slots[slot].ready.make_wait((cudaStream_t)stream);
  p->span_close(w, (cudaStream_t)stream, 2);
  return e == cudaSuccess ? FLAME_OFFLOAD_OK : fail_cuda(e, "wait_ready: cudaStreamWaitEvent");
}

FlameOffloadStatus flame_offload_pool_clear(FlameOffloadPool* p) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "clear: null pool");
  std::unique_lock<std::mutex> lk(p->mu);
  for (size_t i = 0; i < p->slots.size(); ++i) {  // an offload the pool's thread is enqueueing right now finishes first
    if (p->slots[i].issue == Issue::Issuing) {
      FlameOffloadStatus st = wait_issued(p, lk, i, "clear");
      if (st != FLAME_OFFLOAD_OK) return st;
    }
  }
  for (size_t i = 0; i < p->slots.size(); ++i) {
    Slot& s = p->slots[i];
    s.state = SlotState::Idle;
    if (s.issue == Issue::Queued) {
      s.plan.reset();
      s.issue = Issue::Done;
      p->release_chunks_unwritten(s);
      p->stats.pushes_cancelled++;
    } else {
      p->release_chunks(s, s.h2d_done.recorded ? (int32_t)i : -1);
    }
  }
  p->queue.clear();
  p->stats.pushes_queued = 0;
  p->free_stack.clear();
  for (size_t i = p->num_slots; i-- > 0;) p->free_stack.push_back(i);
  p->epoch += 1;
  if (p->epoch == 0) p->epoch = 1;
  p->stats.host_chunks_free = p->free_chunks.size();
  return FLAME_OFFLOAD_OK;
}

int flame_offload_pool_source_released(FlameOffloadPool* p, FlameOffloadHandle h) {
  if (!p) return -(int)FLAME_OFFLOAD_ERR_INVALID;
  std::lock_guard<std::mutex> lk(p->mu);
  if (h.epoch != p->epoch || h.slot >= p->slots.size()) {
    fail(FLAME_OFFLOAD_ERR_STATE, "source_released: stale or invalid handle");
    return -(int)FLAME_OFFLOAD_ERR_STATE;
  }
  Slot& s = p->slots[h.slot];
  if (s.issue != Issue::Done) return 0;  // deferred and not enqueued yet: the source has not been read
  if (s.failed) {
    fail(FLAME_OFFLOAD_ERR_CUDA, "source_released: the deferred offload of this slot failed: " + s.error);
    return -(int)FLAME_OFFLOAD_ERR_CUDA;
  }
  if (!s.d2h_done.recorded) return 1;
  DeviceGuard guard(p->device);
  cudaError_t e = cudaEventQuery(s.d2h_done.ev);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  fail_cuda(e, "source_released: cudaEventQuery");
  return -(int)FLAME_OFFLOAD_ERR_CUDA;
}

FlameOffloadStatus flame_offload_pool_slot_info(FlameOffloadPool* p, FlameOffloadHandle h, FlameOffloadSlotInfo* out) {
  if (!p || !out) return fail(FLAME_OFFLOAD_ERR_INVALID, "slot_info: null argument");
  std::lock_guard<std::mutex> lk(p->mu);
  FlameOffloadStatus st = p->check_handle(h, "slot_info");
  if (st != FLAME_OFFLOAD_OK) return st;
  const Slot& s = p->slots[h.slot];
  out->numel = s.numel; out->dtype = s.dtype; out->compression = p->compression;
  out->bytes = s.bytes; out->stored_bytes = s.stored_bytes; out->chunks = s.chunks.size();
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_synchronize(FlameOffloadPool* p, double timeout_s) {
  if (!p) return fail(FLAME_OFFLOAD_ERR_INVALID, "synchronize: null pool");
  const auto t0 = std::chrono::steady_clock::now();
  if (p->deferred) {  // queued offloads first (unless they are being held back), then what the streams hold
    std::unique_lock<std::mutex> lk(p->mu);
    const auto deadline = t0 + std::chrono::duration_cast<std::chrono::steady_clock::duration>(std::chrono::duration<double>(timeout_s));
    auto busy = [&] {
      if (!p->hold && !p->queue.empty()) return true;
      for (auto& s : p->slots) if (s.issue == Issue::Issuing) return true;
      return false;
    };
    while (busy()) {
      if (std::chrono::steady_clock::now() >= deadline)
        return fail(FLAME_OFFLOAD_ERR_TIMEOUT, "synchronize: deferred offloads still queued after the timeout");
      p->cv_issued.wait_for(lk, std::chrono::milliseconds(1));
    }
  }
  const double left = timeout_s - std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  DeviceGuard guard(p->device);
  return poll_streams(p, std::max(left, 0.001));
}

FlameOffloadStatus flame_offload_pool_read_slot(FlameOffloadPool* p, FlameOffloadHandle h, void* codes_out, void* scales_out, double timeout_s) {
  if (!p || !codes_out) return fail(FLAME_OFFLOAD_ERR_INVALID, "read_slot: null argument");
  std::unique_lock<std::mutex> lk(p->mu);
  FlameOffloadStatus st = p->check_handle(h, "read_slot");
  if (st != FLAME_OFFLOAD_OK) return st;
  Slot& s = p->slots[h.slot];
  if (s.issue != Issue::Done) {
    st = wait_issued(p, lk, h.slot, "read_slot");
    if (st != FLAME_OFFLOAD_OK) return st;
  }
  if (s.failed) return fail(FLAME_OFFLOAD_ERR_CUDA, "read_slot: the deferred offload of this slot failed: " + s.error);
  DeviceGuard guard(p->device);
  st = poll_event(s.d2h_done.ev, timeout_s, "read_slot: waiting for the offload");
  if (st != FLAME_OFFLOAD_OK) return st;
  auto* co = static_cast<uint8_t*>(codes_out);
  auto* so = static_cast<float*>(scales_out);
  for (size_t k = 0; k < s.chunks.size(); ++k) {
    const uint8_t* c = p->chunk_ptr(s.chunks[k]);
    if (!p->compressed()) {
      const uint64_t off = k * p->chunk_src_bytes;
      memcpy(co + off, c, std::min<uint64_t>(p->chunk_src_bytes, s.bytes - off));
      continue;
    }
    const uint64_t e0 = k * p->chunk_elems;
    const uint64_t e = std::min<uint64_t>(p->chunk_elems, s.numel - e0);
    memcpy(co + e0, c, e);
    if (p->compression != FLAME_OFFLOAD_COMPRESSION_FP8 && so)
      memcpy(so + e0 / 128, c + packed_scales_offset(e), 4 * ((e + 127) / 128));
  }
  if (p->compression == FLAME_OFFLOAD_COMPRESSION_FP8 && so) so[0] = s.fp8_scale;
  return FLAME_OFFLOAD_OK;
}

FlameOffloadStatus flame_offload_pool_stats(const FlameOffloadPool* pc, FlameOffloadStats* out) {
  auto* p = const_cast<FlameOffloadPool*>(pc);
  if (!p || !out) return fail(FLAME_OFFLOAD_ERR_INVALID, "stats: null argument");
  std::lock_guard<std::mutex> lk(p->mu);
  if (p->timing) {
    DeviceGuard guard(p->device);
    p->harvest_spans();
    std::lock_guard<std::mutex> tl(p->timing_mu);
    p->stats.offload_span_us = p->span_ns[0] / 1000u;
    p->stats.restore_span_us = p->span_ns[1] / 1000u;
    p->stats.ready_wait_us = p->span_ns[2] / 1000u;
    p->stats.spans_timed = p->spans_done;
    p->stats.spans_pending = p->spans.size();
  }
  *out = p->stats;
  return FLAME_OFFLOAD_OK;
}

}  // extern "C"
