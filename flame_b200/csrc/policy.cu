// Bandwidth probe and the recompute-vs-offload policy.
//
// The reference decides with a fixed rule (offload every BF16 requires_grad
// saved tensor, src/autograd.rs:1721-1725) and keeps an unused
// CheckpointPolicy::Adaptive { memory_threshold, prefer_recompute }
// (src/gradient_checkpointing.rs:70-74, 201-232).  Here the decision is made
// from measured numbers: how many bytes each direction of the host link can
// move while forward / backward compute runs, how much may stay resident, and
// what a recompute would cost instead.
#include <algorithm>
#include <numeric>
#include <vector>

#include "codec_kernels.cuh"
#include "common.h"

using namespace flame_b200;

namespace {

struct ProbeBuffers {
  void *host = nullptr, *dev_a = nullptr, *dev_b = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  cudaStream_t s = nullptr;
  ~ProbeBuffers() {
    if (host) cudaFreeHost(host);
    if (dev_a) cudaFree(dev_a);
    if (dev_b) cudaFree(dev_b);
    if (t0) cudaEventDestroy(t0);
    if (t1) cudaEventDestroy(t1);
    if (s) cudaStreamDestroy(s);
  }
};

}  // namespace

extern "C" {

FlameOffloadStatus flame_offload_probe(size_t bytes, int reps, FlameLinkProbe* out) {
  if (!out) return fail(FLAME_OFFLOAD_ERR_INVALID, "probe: null output");
  if (bytes == 0) bytes = 256u << 20;
  bytes &= ~(size_t)0xFFFF;
  if (bytes == 0) return fail(FLAME_OFFLOAD_ERR_INVALID, "probe: bytes must be at least 64 KiB");
  if (reps <= 0) reps = 5;
  ProbeBuffers b;
#define PROBE_TRY(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) return fail_cuda(_e, "probe: " #expr); } while (0)
  PROBE_TRY(cudaHostAlloc(&b.host, bytes, cudaHostAllocDefault));
  PROBE_TRY(cudaMalloc(&b.dev_a, bytes));
  PROBE_TRY(cudaMalloc(&b.dev_b, bytes));
  PROBE_TRY(cudaStreamCreateWithFlags(&b.s, cudaStreamNonBlocking));
  PROBE_TRY(cudaEventCreate(&b.t0));
  PROBE_TRY(cudaEventCreate(&b.t1));
  PROBE_TRY(cudaMemsetAsync(b.dev_a, 0x3c, bytes, b.s));  // BF16 0x3c3c ~ 0.0115: finite values
  memset(b.host, 0, bytes);

  auto timed = [&](auto&& body, double& ms_best) -> cudaError_t {
    ms_best = 1e30;
    for (int r = 0; r < reps + 1; ++r) {  // first pass is the warm-up
      cudaError_t e = cudaEventRecord(b.t0, b.s);
      if (e != cudaSuccess) return e;
      if ((e = body()) != cudaSuccess) return e;
      if ((e = cudaEventRecord(b.t1, b.s)) != cudaSuccess) return e;
      if ((e = cudaEventSynchronize(b.t1)) != cudaSuccess) return e;
      float ms = 0;
      if ((e = cudaEventElapsedTime(&ms, b.t0, b.t1)) != cudaSuccess) return e;
      if (r > 0) ms_best = std::min<double>(ms_best, ms);
    }
    return cudaSuccess;
  };
  double ms = 0;
  PROBE_TRY(timed([&] { return cudaMemcpyAsync(b.host, b.dev_a, bytes, cudaMemcpyDeviceToHost, b.s); }, ms));
  out->d2h_gbs = bytes / ms * 1e-6;
  PROBE_TRY(timed([&] { return cudaMemcpyAsync(b.dev_b, b.host, bytes, cudaMemcpyHostToDevice, b.s); }, ms));
  out->h2d_gbs = bytes / ms * 1e-6;
  PROBE_TRY(timed([&] { return cudaMemcpyAsync(b.dev_b, b.dev_a, bytes, cudaMemcpyDeviceToDevice, b.s); }, ms));
  out->hbm_copy_gbs = 2.0 * bytes / ms * 1e-6;
  // int8 block codec over as many elements as fit: in = dev_a (2 B/elem), packed out = dev_b.
  const size_t n = (bytes / 2) & ~(size_t)8191;
  auto* packed = static_cast<uint8_t*>(b.dev_b);
  const size_t so = (n + 255u) & ~(size_t)255u;
  PROBE_TRY(timed([&] { return launch_compress(kCodecInt8, b.dev_a, packed, n, single_chunk_layout(packed, packed + so, n), 0, b.s, 0); }, ms));
  out->quant_gbs = (3.03125 * n) / ms * 1e-6;
  PROBE_TRY(timed([&] { return launch_dequant(kCodecInt8, packed, b.dev_a, n, single_chunk_layout(packed, packed + so, n), b.s, 0); }, ms));
  out->dequant_gbs = (3.03125 * n) / ms * 1e-6;
#undef PROBE_TRY
  return FLAME_OFFLOAD_OK;
}

// Greedy, deterministic plan.
//  1. The resident budget goes to the tensors saved LAST in forward (highest
//     group first): backward needs them first, so a restore has the least
//     compute to hide behind.
//  2. Everything else is offloaded, lossy codec where allowed (payload
//     bytes * (1/2 + 1/64)), BF16 otherwise.
//  3. Each direction of the link can move rate * utilisation * window bytes for
//     free: D2H behind forward (and, for what is still queued, backward), H2D
//     behind backward.  While the payload exceeds the smaller of the two, the
//     tensor with the cheapest recompute per payload byte is switched to
//     recompute, as long as recomputing costs less than its exposed transfer.
//  4. What still does not fit is reported as estimated exposed time.
FlameOffloadStatus flame_offload_policy_plan(const FlamePolicyInput* in, const FlamePolicyTensor* t, size_t n, int32_t* dec, double* est_overhead_ms) {
  if (!in || (!t && n) || (!dec && n)) return fail(FLAME_OFFLOAD_ERR_INVALID, "policy_plan: null argument");
  if (in->d2h_gbs <= 0 || in->h2d_gbs <= 0) return fail(FLAME_OFFLOAD_ERR_INVALID, "policy_plan: link rates must be positive");
  const int lossy = in->lossy_codec == FLAME_POLICY_OFFLOAD_FP8 ? FLAME_POLICY_OFFLOAD_FP8 : FLAME_POLICY_OFFLOAD_INT8;
  const double util = in->link_utilisation > 0 && in->link_utilisation <= 1.0 ? in->link_utilisation : 0.9;

  std::vector<size_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return t[a].group > t[b].group; });
  uint64_t resident = 0;
  std::vector<double> payload(n, 0.0);
  for (size_t i : order) {
    if (resident + t[i].bytes <= in->device_budget_bytes) {
      dec[i] = FLAME_POLICY_RESIDENT;
      resident += t[i].bytes;
    } else if (t[i].allow_lossy) {
      dec[i] = lossy;
      payload[i] = (double)t[i].bytes * (0.5 + 1.0 / 64.0);
    } else {
      dec[i] = FLAME_POLICY_OFFLOAD_BF16;
      payload[i] = (double)t[i].bytes;
    }
  }
  const double fwd = std::max(0.0, in->fwd_ms), bwd = std::max(0.0, in->bwd_ms);
  // bytes per ms = GB/s * 1e6
  const double free_out = in->d2h_gbs * 1e6 * util * (fwd + 0.5 * bwd);
  const double free_in = in->h2d_gbs * 1e6 * util * bwd;
  double total = std::accumulate(payload.begin(), payload.end(), 0.0);
  double recompute_ms = 0.0;
  auto exposed_ms = [&](double bytes) {
    return std::max(0.0, bytes - free_out) / (in->d2h_gbs * 1e6) + std::max(0.0, bytes - free_in) / (in->h2d_gbs * 1e6);
  };
  for (;;) {
    const double over = exposed_ms(total);
    if (over <= 0.0) break;
    size_t best = n;
    double best_cost = 0.0;
    for (size_t i = 0; i < n; ++i) {
      if (payload[i] <= 0.0 || t[i].recompute_ms < 0.0) continue;
      const double cost = t[i].recompute_ms / payload[i];
      if (best == n || cost < best_cost) { best = i; best_cost = cost; }
    }
    if (best == n) break;
    const double saved = over - exposed_ms(total - payload[best]);
    if (t[best].recompute_ms >= saved) break;  // recomputing would cost more than it hides
    total -= payload[best];
    payload[best] = 0.0;
    recompute_ms += t[best].recompute_ms;
    dec[best] = FLAME_POLICY_RECOMPUTE;
  }
  if (est_overhead_ms) *est_overhead_ms = exposed_ms(total) + recompute_ms;
  return FLAME_OFFLOAD_OK;
}

}  // extern "C"

namespace {

struct SimResult { double stall_ms, recompute_ms; uint64_t resident, link; double busy_ms; };

// Timeline of one step under a given plan (see the header comment).
SimResult simulate(const FlamePolicyInput& in, const FlamePolicyBlock* b, size_t n, const std::vector<int32_t>& dec, double payload_ratio) {
  const double out_rate = in.d2h_gbs * 1e6, in_rate = in.h2d_gbs * 1e6;  // bytes per ms
  SimResult r{0.0, 0.0, 0, 0, 0.0};
  std::vector<double> d2h_done(n, 0.0);
  double t = 0.0, q_out = 0.0;
  for (size_t g = 0; g < n; ++g) {  // forward
    t += b[g].fwd_ms;
    if (dec[g] == FLAME_POLICY_RESIDENT) { r.resident += b[g].saved_bytes; continue; }
    if (dec[g] == FLAME_POLICY_RECOMPUTE) continue;
    const double payload = (double)b[g].saved_bytes * (dec[g] == FLAME_POLICY_OFFLOAD_BF16 ? 1.0 : payload_ratio);
    r.link += (uint64_t)payload;
    q_out = std::max(q_out, t) + payload / out_rate;
    d2h_done[g] = q_out;
    r.busy_ms += payload / out_rate;
  }
  // backward: restores are issued one block ahead of their consumer, in reverse order
  double q_in = t;
  std::vector<double> ready(n, 0.0);
  auto issue = [&](size_t g, double now) {
    if (dec[g] != FLAME_POLICY_OFFLOAD_BF16 && dec[g] != FLAME_POLICY_OFFLOAD_INT8 && dec[g] != FLAME_POLICY_OFFLOAD_FP8) return;
    const double payload = (double)b[g].saved_bytes * (dec[g] == FLAME_POLICY_OFFLOAD_BF16 ? 1.0 : payload_ratio);
    q_in = std::max(std::max(q_in, now), d2h_done[g]) + payload / in_rate;
    ready[g] = q_in;
    r.busy_ms += payload / in_rate;
  };
  if (n) issue(n - 1, t);
  for (size_t k = 0; k < n; ++k) {
    const size_t g = n - 1 - k;
    if (g > 0) issue(g - 1, t);  // prefetch the next block to be consumed
    if (ready[g] > t) { r.stall_ms += ready[g] - t; t = ready[g]; }
    if (dec[g] == FLAME_POLICY_RECOMPUTE) { t += b[g].fwd_ms; r.recompute_ms += b[g].fwd_ms; }
    t += b[g].bwd_ms;
  }
  return r;
}

}  // namespace

extern "C" {

FlameOffloadStatus flame_offload_policy_plan_blocks(const FlamePolicyInput* in, const FlamePolicyBlock* blocks, size_t n,
                                                              int offload_decision, int32_t* decisions, FlamePolicyBlockPlan* out) {
  if (!in || (!blocks && n) || (!decisions && n)) return fail(FLAME_OFFLOAD_ERR_INVALID, "policy_plan_blocks: null argument");
  if (in->d2h_gbs <= 0 || in->h2d_gbs <= 0) return fail(FLAME_OFFLOAD_ERR_INVALID, "policy_plan_blocks: link rates must be positive");
  if (offload_decision != FLAME_POLICY_OFFLOAD_BF16 && offload_decision != FLAME_POLICY_OFFLOAD_INT8 && offload_decision != FLAME_POLICY_OFFLOAD_FP8)
    return fail(FLAME_OFFLOAD_ERR_INVALID, "policy_plan_blocks: offload_decision must be one of the OFFLOAD_* values");
  const double ratio = 0.5 + 1.0 / 64.0;
  std::vector<int32_t> best;
  SimResult best_r{};
  double best_cost = 0.0;
  std::vector<int32_t> dec(n);
  const bool capped = in->overhead_cap_ms > 0.0;
  for (size_t resident = 0; resident <= n; ++resident) {
    uint64_t res_bytes = 0;
    for (size_t g = n - resident; g < n; ++g) res_bytes += blocks[g].saved_bytes;
    if (!capped && res_bytes > in->device_budget_bytes) break;  // more trailing blocks only cost more memory
    bool feasible = false;
    for (size_t recompute = 0; recompute + resident <= n; ++recompute) {
      for (size_t g = 0; g < n; ++g)
        dec[g] = g >= n - resident ? FLAME_POLICY_RESIDENT : (g < recompute ? FLAME_POLICY_RECOMPUTE : offload_decision);
      const SimResult r = simulate(*in, blocks, n, dec, ratio);
      const double cost = r.stall_ms + r.recompute_ms + std::max(0.0, in->interference) * r.busy_ms;
      if (capped) {
        // the first resident count (fewest resident bytes) with a plan under the cap wins; among its plans, the cheapest
        if (cost > in->overhead_cap_ms) continue;
        if (!feasible || cost < best_cost - 0.01) { best = dec; best_r = r; best_cost = cost; }
        feasible = true;
        continue;
      }
      // strictly better time wins; within 0.01 ms prefer fewer resident bytes (earlier in the search)
      if (best.empty() || cost < best_cost - 0.01) { best = dec; best_r = r; best_cost = cost; }
    }
    if (capped && feasible) break;
  }
  for (size_t g = 0; g < n; ++g) decisions[g] = best.empty() ? offload_decision : best[g];
  if (out) { out->est_stall_ms = best_r.stall_ms; out->est_recompute_ms = best_r.recompute_ms; out->resident_bytes = best_r.resident; out->link_bytes = best_r.link;
             out->est_interference_ms = std::max(0.0, in->interference) * best_r.busy_ms; }
  return FLAME_OFFLOAD_OK;
}

}  // extern "C"
