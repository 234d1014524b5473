"""Benchmark of the activation offload+restore path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--codec int8|fp8|none] [--impl reference]

One *step* is one pass of the hot path over the saved activations of one DiT
training step (20 blocks x {2 norm outputs, QKV, attention output, SwiGLU
gate+up} at 4608 tokens, hidden 3072; 6.79 GB of BF16): every tensor is
offloaded in forward order, then every tensor is restored in reverse order.

Reported, for the whole job (all N replicas; the slowest replica sets the time):

* ``value``  BF16-equivalent GB/s (bytes offloaded + bytes restored, per second)
  of the path itself: ``push`` of every tensor (compress, D2H into the pinned
  slab), then ``pull_into`` of every tensor (H2D, dequantise into the
  destination).  Inputs are resident in HBM when the timed region starts, as
  activations are; CUDA events; ``value_per_gpu`` = value / N.
* ``e2e``    the same step through the reference's own signatures, ``push`` and
  the allocating ``pull``, plus a device-to-host read of a number computed from
  what came back, timed on the host clock around a device synchronise.
* ``roofline``  achieved algorithmic GB/s of the compress kernel (3.03125 B per
  element) with inputs and outputs in HBM, against the measured HBM copy rate;
  ``roofline_dequant`` likewise.  No host link in that leg: it is what bounds
  the kernels, not the metric.
* ``link``   D2H / H2D GB/s of the pool per replica, measured one direction at a
  time (a barrier between) and both at once, beside plain pinned copies issued
  by all replicas at the same moment and the PCIe Gen5 x16 bound (63.0 GB/s);
  ``link.pcie`` is what sysfs says about each GPU's link and its bridges.
* ``fp8_mixed``  (N=1) the FP8 per-128 codec over the mixed activation set
  (GELU outputs, heavy-tailed attention outputs, SwiGLU hidden states).
* ``cpu_baseline``  the CPU oracle's quantise+pack / unpack+dequantise on this
  box's host cores over a bounded sample (rank 0, N=1 only).
* ``overhead``  step time of a 20-block DiT training step with activations
  offloaded, relative to keeping them resident.  N=1: every arm.  N>1: on every
  replica at once, the link probed with all replicas copying, and the plan that
  keeps the estimated overhead under a cap at that link rate.

``--impl reference`` times the reference's CPU arm instead: the reference crate
is GPU-only Rust and has no CPU quantise/pack path of its own, so the timed code
is the C oracle (a port), on all host threads, over a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "activation offload+restore GB/s (BF16-equiv), sum over the N replicas (value_per_gpu = value / N)"
UNIT = "GB/s"
ALG_BYTES_PER_ELEM = 3.03125  # 2 B read + 1 B code + 4/128 B scale (and the mirror image for dequantise)
# dram__bytes_read.sum + dram__bytes_write.sum per element from the ncu captures summarised under profiles/
# (one launch = one DiT block, 169,869,312 elements: 483.1 MB int8 / 490.0 MB FP8 compress, 458.1 MB dequantise); traffic grows in
# proportion to the elements of a launch.  Below the algorithmic figure because the L2 still holds part of the
# output when the kernel ends.
NCU_TRAFFIC_PER_ELEM = {"compress": {"int8": 483.1e6 / 169869312, "fp8": 490.0e6 / 169869312}, "dequant": 458.1e6 / 169869312}
# the FP8 weight kernel on an [18432, 3072] weight: 56.64 MB read + 57.5 MB written inside the launch (the other half of the
# 113 MB output was still in the L2 when it ended)
NCU_TRAFFIC_PER_WEIGHT_ELEM = (56.64e6 + 57.5e6) / 56623104
PCIE_GEN5_X16_GBS = 63.0      # 32 GT/s x 16 lanes x 128/130 / 8
TOKENS, HIDDEN, BLOCKS = 4608, 3072, 20
# saved set of one block, as last dims: norm1 out, QKV, attention out, norm2 out, SwiGLU gate+up
BLOCK_SAVED = (HIDDEN, 3 * HIDDEN, HIDDEN, HIDDEN, 6 * HIDDEN)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs (read-only NVML, else nvidia-smi)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index, self.sm, self.sm_max, self.reasons, self._stop, self._t = index, [], None, set(), threading.Event(), None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and all(v.strip().isdigit() for v in visible.split(",")) else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.sm.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        for name, bit in (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4)):
            if r & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        if out:
            c = [x.strip() for x in out.split(",")]
            if c[0].isdigit():
                self.sm.append(int(c[0]))
            if c[1].isdigit():
                self.sm_max = int(c[1])
            for i, name in enumerate(self.NAMES):
                if len(c) > 2 + i and c[2 + i] == "Active":
                    self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._sample_nvml() if self._nvml else self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.002 if self._nvml else 0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no clock samples"]}
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons), "samples": len(sm)}


C4_TENSORS, C4_SHAPE = 200, (8, 4096, 3072)  # 200 x 201.3 MB = 40.27 GB of BF16 per GPU per step


def make_workload(torch, dev, seed: int, blocks: int = BLOCKS, kind: str = "dit"):
    """The saved activations of one step: N(0,1) with 0.1 % of entries replaced by +-U(20,60), BF16.

    kind "dit": 20 blocks x the five saved tensors of a DiT block.  kind "c4": the 40 GB-per-GPU case, 200 tensors
    of [8,4096,3072] (25 distinct ones, each used 8 times: the bytes moved are what matters here)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    tensors = []
    if kind == "c4":
        distinct = []
        for _ in range(25):
            x = torch.randn(C4_SHAPE, device=dev, dtype=torch.float32, generator=g)
            mask = torch.rand(C4_SHAPE, device=dev, generator=g) < 1e-3
            x = torch.where(mask, x.sign() * (20.0 + 40.0 * torch.rand(C4_SHAPE, device=dev, generator=g)), x)
            distinct.append(x.to(torch.bfloat16).contiguous())
            del x, mask
        return [distinct[i % 25] for i in range(C4_TENSORS)]
    for _ in range(blocks):
        for last in BLOCK_SAVED:
            x = torch.randn(1, TOKENS, last, device=dev, dtype=torch.float32, generator=g)
            mask = torch.rand(x.shape, device=dev, generator=g) < 1e-3
            mag = torch.empty_like(x).uniform_(20.0, 60.0, generator=g) * torch.where(torch.rand(x.shape, device=dev, generator=g) < 0.5, -1.0, 1.0)
            tensors.append(torch.where(mask, mag, x).to(torch.bfloat16).contiguous())
            del x, mask, mag
    return tensors


def verify_against_oracle(torch, lib, x, codec: str) -> bool:
    """One tensor through the C ABI, compared bit for bit with the CPU oracle (the checker, not the product)."""
    import numpy as np
    from oracle import capi

    n = min(x.numel(), 1 << 22)
    xs = x.reshape(-1)[:n].contiguous()
    codes = torch.empty(n, dtype=torch.uint8, device=x.device)
    scales = torch.empty((n + 127) // 128, dtype=torch.float32, device=x.device)
    out = torch.empty(n, dtype=torch.bfloat16, device=x.device)
    s = torch.cuda.current_stream().cuda_stream
    q, d = (lib.flame_act_quant_int8_b128, lib.flame_act_dequant_int8_b128) if codec == "int8" else \
           (lib.flame_act_quant_fp8_b128, lib.flame_act_dequant_fp8_b128)
    assert q(xs.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, 0, s) == 0
    assert d(codes.data_ptr(), scales.data_ptr(), out.data_ptr(), n, s) == 0
    torch.cuda.synchronize()
    bits = xs.view(torch.int16).cpu().numpy().view(np.uint16)
    wc, ws = (capi.quant_int8_b128 if codec == "int8" else capi.quant_fp8_b128)(bits)
    wo = (capi.dequant_int8_b128 if codec == "int8" else capi.dequant_fp8_b128)(wc, ws)
    return (np.array_equal(codes.cpu().numpy(), wc.view(np.uint8)) and np.array_equal(scales.cpu().numpy().view(np.uint32), ws.view(np.uint32))
            and np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), wo))


def plain_copy_rates(torch, lib, dev, barrier):
    """(D2H, H2D, duplex D2H, duplex H2D) GB/s of plain 1 GiB pinned cudaMemcpyAsync on this replica, every phase started
    together with the other replicas; the duplex pair runs both directions at once on two streams."""
    nb = 1 << 30
    d = torch.empty(nb, dtype=torch.uint8, device=dev)
    d2 = torch.empty(nb, dtype=torch.uint8, device=dev)
    h = torch.empty(nb, dtype=torch.uint8).pin_memory()
    h2 = torch.empty(nb, dtype=torch.uint8).pin_memory()
    st = torch.cuda.current_stream()
    side = torch.cuda.Stream(dev)
    rates = []
    for kind, dst, src in ((2, h, d), (1, d, h)):
        lib.flame_cuda_memcpy_async(dst.data_ptr(), src.data_ptr(), nb, kind, st.cuda_stream)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(2):
            lib.flame_cuda_memcpy_async(dst.data_ptr(), src.data_ptr(), nb, kind, st.cuda_stream)
        e1.record(st)
        torch.cuda.synchronize()
        rates.append(2 * nb / (e0.elapsed_time(e1) * 1e-3) * 1e-9)
    lib.flame_cuda_memcpy_async(d2.data_ptr(), h2.data_ptr(), nb, 1, side.cuda_stream)
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record(st); ev[2].record(side)
    for _ in range(2):
        lib.flame_cuda_memcpy_async(h.data_ptr(), d.data_ptr(), nb, 2, st.cuda_stream)
        lib.flame_cuda_memcpy_async(d2.data_ptr(), h2.data_ptr(), nb, 1, side.cuda_stream)
    ev[1].record(st); ev[3].record(side)
    torch.cuda.synchronize()
    rates.append(2 * nb / (ev[0].elapsed_time(ev[1]) * 1e-3) * 1e-9)
    rates.append(2 * nb / (ev[2].elapsed_time(ev[3]) * 1e-3) * 1e-9)
    return rates


def cpu_leg(seconds_target: float = 12.0, codec_name: str = "int8"):
    """CPU oracle pack+unpack on all host threads over a bounded sample of the workload. Returns (GB/s bf16-equiv, cores, sample)."""
    import numpy as np
    from flame_b200 import synthetic
    from oracle import capi

    codec = {"int8": capi.CODEC_INT8, "fp8": capi.CODEC_FP8, "none": capi.CODEC_NONE}[codec_name]
    cores = os.cpu_count() or 1
    n = TOKENS * HIDDEN  # one [1,4608,3072] norm output
    x = synthetic.normal_with_outliers(n, seed=0)
    capi.roundtrip_mt(x, codec, cores)  # warm-up, page in
    t0 = time.perf_counter()
    reps = 0
    while True:
        capi.roundtrip_mt(x, codec, cores)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_target or reps >= 400:
            break
    gbs = (2 * 2 * n * reps) / dt * 1e-9  # bytes offloaded + bytes restored
    return gbs, cores, f"{reps} x one [1,{TOKENS},{HIDDEN}] BF16 tensor ({2 * n / 1e6:.1f} MB), quantise+pack then unpack+dequantise, {cores} threads, {dt:.1f} s", dt / reps


def reference_gpu_path(args):
    """The reference's GPU path for the same workload, as far as it can be run here: its three CUDA files of this
    path (src/cuda/fp8_quant.cu, fp8_dequant.cu, pinned_host.cu) compiled unmodified into oracle/_ref, driven in the
    order its pool drives them (src/activation_offload.rs:465-611 push, :619-731 pull): one pinned buffer and one
    device staging buffer per slot, ONE transfer stream, whole-tensor copies, a fixed FP8 scale of 8/448, a fresh
    destination per pull, the compute stream waiting on each pull's ready event.  The Rust host code itself cannot
    be built on this image, so the sequence is issued from this function; none of this library's code is on it.
    Returns None when the compiled reference or a GPU is absent."""
    try:
        import torch
        from oracle import capi
        ref = capi.load_ref_cuda()
        if ref is None or not torch.cuda.is_available():
            return None
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        tensors = make_workload(torch, dev, seed=0, blocks=args.blocks, kind="dit")
        step_bytes = sum(t.numel() * 2 for t in tensors)
        step_elems = sum(t.numel() for t in tensors)
        max_bytes = max(t.numel() * 2 for t in tensors)
        compute = torch.cuda.current_stream()
        transfer = torch.cuda.Stream(dev)
        tp = transfer.cuda_stream
        out = {"sources": "src/cuda/fp8_quant.cu, fp8_dequant.cu, pinned_host.cu compiled unmodified (nvcc, sm_100a); push/pull order of "
                          "src/activation_offload.rs:465-731 issued by bench.py", "unit": UNIT}
        hbm_peak, _ = measured_peaks()
        # kernels alone, device-resident, events on the launching stream
        codes = [torch.empty(t.numel(), dtype=torch.uint8, device=dev) for t in tensors]
        back = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=dev)
        inv, scale = 448.0 / 8.0, 8.0 / 448.0
        for phase in range(2):
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record(transfer)
            for t, c in zip(tensors, codes):
                assert ref.flame_bf16_to_fp8(t.data_ptr(), c.data_ptr(), inv, t.numel(), tp) == 0
            e1.record(transfer)
            for t, c in zip(tensors, codes):
                assert ref.flame_fp8_to_bf16(c.data_ptr(), back.data_ptr(), scale, t.numel(), tp) == 0
            e2.record(transfer)
            torch.cuda.synchronize()
        alg = 3.0 * step_elems
        qg, dg = alg / (e0.elapsed_time(e1) * 1e-3) * 1e-9, alg / (e1.elapsed_time(e2) * 1e-3) * 1e-9
        out["kernels"] = {"bf16_to_fp8_kernel_gbs": round(qg, 1), "fp8_to_bf16_kernel_gbs": round(dg, 1), "alg_bytes_per_elem": 3.0,
                          "frac_of_hbm": [round(qg / hbm_peak, 3), round(dg / hbm_peak, 3)],
                          "device_roundtrip_bf16eq_gbs": round(2 * step_bytes / (e0.elapsed_time(e2) * 1e-3) * 1e-9, 1)}
        del codes, back
        if hasattr(ref, "flame_fused_rms_norm_bf16"):      # the producer of two of a block's saved tensors (src/cuda/fused_rms_norm.cu)
            xr = tensors[0].view(TOKENS, HIDDEN)
            wr = torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev)
            yr = torch.empty_like(xr)
            flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
            ts = []
            for k in range(25):
                flush.zero_()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(transfer)
                assert ref.flame_fused_rms_norm_bf16(xr.data_ptr(), wr.data_ptr(), yr.data_ptr(), TOKENS, HIDDEN, 1e-6, tp) == 0
                a1.record(transfer)
                torch.cuda.synchronize()
                if k >= 5:
                    ts.append(a0.elapsed_time(a1) * 1e3)
            ts.sort()
            us = ts[len(ts) // 2]
            out["kernels"]["fused_rms_norm_bf16_us"] = round(us, 2)
            out["kernels"]["fused_rms_norm_bf16_gbs"] = round(4.0 * TOKENS * HIDDEN / us * 1e-3, 1)
            del flush, yr
        if hasattr(ref, "flame_fused_dequant_transpose_bf16"):   # its FP8 weight kernel (src/cuda/fused_dequant_transpose.cu) at the QKV weight's shape
            m, n = 3 * HIDDEN, HIDDEN
            wc = torch.randint(0, 0x78, (m, n), dtype=torch.uint8, device=dev)
            wo = torch.empty(n, m, dtype=torch.bfloat16, device=dev)
            flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
            ts = []
            for k in range(25):
                flush.zero_()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(transfer)
                assert ref.flame_fused_dequant_transpose_bf16(wc.data_ptr(), wo.data_ptr(), 0.0123, m, n, tp) == 0
                a1.record(transfer)
                torch.cuda.synchronize()
                if k >= 5:
                    ts.append(a0.elapsed_time(a1) * 1e3)
            ts.sort()
            us = ts[len(ts) // 2]
            out["kernels"]["fused_dequant_transpose_bf16_us"] = round(us, 2)
            out["kernels"]["fused_dequant_transpose_bf16_gbs"] = round(3.0 * m * n / us * 1e-3, 1)
            del flush, wc, wo
        for mode in ("fp8", "none"):
            slot_bytes = (max_bytes + 1) // 2 if mode == "fp8" else max_bytes
            host = [ref.flame_cuda_alloc_pinned_host(slot_bytes, 0) for _ in tensors]       # cudaHostAllocDefault, as the pool does
            if any(h is None for h in host):
                for h in host:
                    if h is not None:
                        ref.flame_cuda_free_pinned_host(h)
                out[mode] = {"unavailable": "cudaHostAlloc failed"}
                continue
            staging = [torch.empty(slot_bytes, dtype=torch.uint8, device=dev) for _ in tensors] if mode == "fp8" else None
            done = [torch.cuda.Event() for _ in tensors]
            ready = [torch.cuda.Event() for _ in tensors]

            def step():
                for i, t in enumerate(tensors):                      # push
                    done[i].record(compute)
                    transfer.wait_event(done[i])
                    if mode == "fp8":
                        assert ref.flame_bf16_to_fp8(t.data_ptr(), staging[i].data_ptr(), inv, t.numel(), tp) == 0
                        assert ref.flame_cuda_memcpy_async(host[i], staging[i].data_ptr(), t.numel(), 2, tp) == 0
                    else:
                        assert ref.flame_cuda_memcpy_async(host[i], t.data_ptr(), t.numel() * 2, 2, tp) == 0
                for i in reversed(range(len(tensors))):             # pull, last pushed first
                    t = tensors[i]
                    fresh = torch.empty_like(t)
                    if mode == "fp8":
                        assert ref.flame_cuda_memcpy_async(staging[i].data_ptr(), host[i], t.numel(), 1, tp) == 0
                        assert ref.flame_fp8_to_bf16(staging[i].data_ptr(), fresh.data_ptr(), scale, t.numel(), tp) == 0
                    else:
                        assert ref.flame_cuda_memcpy_async(fresh.data_ptr(), host[i], t.numel() * 2, 1, tp) == 0
                    ready[i].record(transfer)
                    compute.wait_event(ready[i])
                    fresh.record_stream(transfer)

            for _ in range(max(1, min(args.warmup, 3))):
                step()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k = max(1, min(args.steps, 5))
            a.record(compute)
            for _ in range(k):
                step()
            b.record(compute)
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / k
            link_bytes = step_elems if mode == "fp8" else step_bytes
            out[mode] = {"e2e_gbs": round(2 * step_bytes / (ms * 1e-3) * 1e-9, 2), "ms_per_step": round(ms, 3), "steps": k,
                         "d2h_bytes_per_step": int(link_bytes), "h2d_bytes_per_step": int(link_bytes),
                         "pinned_bytes": int(slot_bytes * len(tensors)), "device_staging_bytes": int(slot_bytes * len(tensors)) if mode == "fp8" else 0}
            for h in host:
                ref.flame_cuda_free_pinned_host(h)
            del staging
            torch.cuda.empty_cache()
        return out
    except Exception as exc:  # the CPU line below stands on its own
        return {"error": f"{type(exc).__name__}: {exc}"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps_rates, cores, sample, step_s = [], 0, "", []
    per = max(2.0, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        gbs, cores, sample, _ = cpu_leg(per, args.codec)
        if i >= args.warmup:
            steps_rates.append(gbs)
            step_s.append(time.perf_counter() - t0)
    value = sum(steps_rates) / len(steps_rates)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(sum(step_s) / len(step_s) * 1e3, 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 codes + f32 scales" if args.codec == "int8" else args.codec, "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": "each step: " + sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference crate is GPU-only Rust with no CPU quantise/pack path; this arm times the C oracle (a port of its formulas) on the host cores",
    }
    if args.gpus == 1 and not args.no_ref_gpu:
        gpu = reference_gpu_path(args)
        if gpu is not None:
            line["reference_gpu_path"] = gpu
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    if getattr(args, "workload", "dit") == "c4":
        return {"workload": f"{C4_TENSORS} x {list(C4_SHAPE)} BF16 per GPU per step = {C4_TENSORS * 8 * 4096 * 3072 * 2 / 1e9:.2f} GB; offload all, restore all in reverse",
                "codec": args.codec + ("-b128" if args.codec != "none" else ""), "chunk_bytes": args.chunk_mb << 20, "tile_chunks": args.tile_chunks,
                "l2": "inputs larger than L2", "replicas": world, "parallelism": f"dp{world} independent replicas, no collective"}
    return {"workload": f"DiT saved activations: {BLOCKS} blocks x [norm1 3072, QKV 9216, attn 3072, norm2 3072, gate+up 18432] x {TOKENS} tokens, BF16, "
                        f"{BLOCKS * sum(BLOCK_SAVED) * TOKENS * 2 / 1e9:.2f} GB per step per GPU; offload all in forward order, restore all in reverse",
            "codec": args.codec + ("-b128" if args.codec != "none" else ""), "chunk_bytes": args.chunk_mb << 20, "tile_chunks": args.tile_chunks,
            "l2": "inputs larger than L2 (6.79 GB of distinct tensors per step)", "replicas": world, "parallelism": f"dp{world} independent replicas, no collective"}


def _event_ms(torch, stream, fn, reps: int, warmup: int = 1, spread: bool = False):
    """Median CUDA-event milliseconds of fn() on `stream` after `warmup` calls; with `spread`, (median, p10, p90)."""
    for _ in range(max(1, warmup)):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    if spread:
        return ts[len(ts) // 2], ts[len(ts) // 10], ts[min(len(ts) - 1, (9 * len(ts)) // 10)]
    return ts[len(ts) // 2]


def run_sweep(args, torch, lib, dev, rank):
    """Config 5: one contiguous BF16 N(0,1) tensor of 1 MB .. 4 GB, offload + restore through the pool with no
    compression, int8 and fp8, chunk sizes 2 / 8 / 32 MB.  One JSON line per point: BF16-equivalent GB/s of the
    round trip, link GB/s against the PCIe Gen5 x16 bound, and the codec kernels' share against the HBM peak."""
    from flame_b200 import ActivationOffloadPool, OffloadCompression

    hbm_peak, peak_kind = measured_peaks()
    stream = torch.cuda.current_stream()
    modes = {"none": OffloadCompression.NONE, "int8": OffloadCompression.INT8_B128, "fp8": OffloadCompression.FP8_B128}
    g = torch.Generator(device=dev).manual_seed(0)
    mb = 1
    while mb <= args.sweep_max_mb:
        nbytes = mb << 20
        n = nbytes // 2
        x = torch.randn(n, device=dev, dtype=torch.float32, generator=g).to(torch.bfloat16) if n <= (1 << 28) else \
            torch.randn(n // 8, device=dev, dtype=torch.float32, generator=g).to(torch.bfloat16).repeat(8)
        dst = torch.empty_like(x)
        for codec, mode in modes.items():
            for chunk_mb in (2, 8, 32):
                pool = ActivationOffloadPool(dev, 1, nbytes, mode, chunk_bytes=chunk_mb << 20)

                def round_trip():
                    pool.pull_into(pool.push(x), dst)

                # the reference's own convention (benches/activation_bwd.rs:16-18: 20 warm-up, 100 timed, median with
                # p10/p90) where a round trip is short; fewer repetitions where one takes tens of milliseconds
                reps, warm = (100, 20) if mb <= 64 else (20, 3) if mb <= 512 else (5, 1)
                ms, p10, p90 = _event_ms(torch, stream, round_trip, reps, warm, spread=True)
                st = pool.stats()
                link_bytes = st["bytes_link_out"] // st["pushes"]
                point = {"mode": "sweep", "tensor_mb": mb, "codec": codec, "chunk_mb": chunk_mb, "round_trip_ms": round(ms, 4),
                         "round_trip_ms_p10": round(p10, 4), "round_trip_ms_p90": round(p90, 4), "reps": reps, "warmup": warm,
                         "gbs_bf16_equiv": round(2 * nbytes / (ms * 1e-3) * 1e-9, 2),
                         # the round trip is one offload followed by one restore: each direction gets about half the time
                         "link_gbs_per_direction": round(link_bytes / (ms * 1e-3 / 2) * 1e-9, 2),
                         "link_frac_of_pcie_gen5_x16": round(link_bytes / (ms * 1e-3 / 2) * 1e-9 / PCIE_GEN5_X16_GBS, 3)}
                if codec != "none":
                    q = lib.flame_act_quant_int8_b128 if codec == "int8" else lib.flame_act_quant_fp8_b128
                    d = lib.flame_act_dequant_int8_b128 if codec == "int8" else lib.flame_act_dequant_fp8_b128
                    codes = torch.empty(n, dtype=torch.uint8, device=dev)
                    scales = torch.empty((n + 127) // 128, dtype=torch.float32, device=dev)
                    sp = stream.cuda_stream
                    qms = _event_ms(torch, stream, lambda: q(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, 0, sp), reps, warm)
                    dms = _event_ms(torch, stream, lambda: d(codes.data_ptr(), scales.data_ptr(), dst.data_ptr(), n, sp), reps, warm)
                    alg = ALG_BYTES_PER_ELEM * n
                    point["compress_gbs"] = round(alg / (qms * 1e-3) * 1e-9, 1)
                    point["dequant_gbs"] = round(alg / (dms * 1e-3) * 1e-9, 1)
                    point["compress_frac_of_hbm"] = round(point["compress_gbs"] / hbm_peak, 3)
                    point["dequant_frac_of_hbm"] = round(point["dequant_gbs"] / hbm_peak, 3)
                    point["hbm_peak_kind"] = peak_kind
                    del codes, scales
                if rank == 0:
                    print(json.dumps(point), flush=True)
                pool.close()
        del x, dst
        torch.cuda.empty_cache()
        mb *= 2


def run_interference(args, torch, lib, dev):
    """How much a host-link copy slows kernels that run beside it.  An HBM-bound loop (SiLU over 28 MB tensors)
    and a compute-bound loop (BF16 GEMM) are timed alone and while 1 GiB crosses the link on another stream,
    device-to-host and host-to-device, issued as one copy or in pieces."""
    import torch.nn.functional as F

    xs = [torch.randn(1, TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16) for _ in range(8)]
    a = torch.randn(TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16)
    w = torch.randn(HIDDEN, 3 * HIDDEN, device=dev, dtype=torch.bfloat16)
    nb = 256 << 20
    src = torch.randn(nb // 2, device=dev).to(torch.bfloat16)
    back = torch.empty_like(src)
    host = torch.empty(nb, dtype=torch.uint8).pin_memory()
    side = torch.cuda.Stream(dev)

    def elementwise():
        for i in range(300):
            F.silu(xs[i % 8])

    def gemm():
        for _ in range(60):
            torch.matmul(a, w)

    def copies(kind, piece):
        def issue():
            for _ in range(4):
                for off in range(0, nb, piece):
                    if kind == 2:
                        lib.flame_cuda_memcpy_async(host.data_ptr() + off, src.data_ptr() + off, piece, 2, side.cuda_stream)
                    else:
                        lib.flame_cuda_memcpy_async(back.data_ptr() + off, host.data_ptr() + off, piece, 1, side.cuda_stream)
        return issue

    def run(fg, bg):
        torch.cuda.synchronize()
        e0, e1, s0, s1 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        s0.record(side)
        if bg is not None:
            bg()
        s1.record(side)
        e0.record()
        fg()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), (4 * nb / (s0.elapsed_time(s1) * 1e-3) * 1e-9 if bg is not None else None)

    for fg in (elementwise, gemm):
        run(fg, None)
    base = {"elementwise": min(run(elementwise, None)[0] for _ in range(3)), "gemm": min(run(gemm, None)[0] for _ in range(3))}
    print(json.dumps({"mode": "interference", "alone_ms": {k: round(v, 3) for k, v in base.items()}}), flush=True)
    for direction, kind in (("d2h", 2), ("h2d", 1)):
        for piece_mb in (1, 2, 4, 16, 256):
            row = {"mode": "interference", "copy": direction, "piece_mb": piece_mb}
            for name, fg in (("elementwise", elementwise), ("gemm", gemm)):
                ms, gbs = run(fg, copies(kind, piece_mb << 20))
                row[name + "_ms"] = round(ms, 3)
                row[name + "_slowdown_pct"] = round(100.0 * (ms - base[name]) / base[name], 1)
                row[name + "_copy_gbs"] = round(gbs, 1)
            print(json.dumps(row), flush=True)


def run_weights(args, torch, dev):
    """Block weights streamed host -> device through the pool (BlockOffloader): every block once forward, once backward."""
    from flame_b200 import BlockOffloader, OffloadCompression

    mode = {"int8": OffloadCompression.INT8_B128, "fp8": OffloadCompression.FP8_B128, "none": OffloadCompression.NONE}[args.codec]
    g = torch.Generator(device=dev).manual_seed(0)
    shapes = {"attn.qkv.weight": (3 * HIDDEN, HIDDEN), "attn.out.weight": (HIDDEN, HIDDEN),
              "mlp.up.weight": (6 * HIDDEN, HIDDEN), "mlp.down.weight": (HIDDEN, 3 * HIDDEN),
              "norm1.weight": (HIDDEN,), "norm2.weight": (HIDDEN,)}
    blocks = [{k: (torch.randn(v, device=dev, generator=g) * 0.02).to(torch.bfloat16) for k, v in shapes.items()} for _ in range(args.blocks)]
    block_bytes = sum(t.numel() * 2 for t in blocks[0].values())
    off = BlockOffloader(dev, blocks, mode, chunk_bytes=args.chunk_mb << 20)
    del blocks
    torch.cuda.empty_cache()
    order = list(range(args.blocks)) + list(reversed(range(args.blocks)))
    stream = torch.cuda.current_stream()

    def step():
        off.prefetch_block(order[0])
        for i, idx in enumerate(order):
            w = off.await_block(idx)
            if i + 1 < len(order):
                off.prefetch_block(order[i + 1])
            w["norm1.weight"].add_(0)      # a consumer on the compute stream, so each block is really waited for
    for _ in range(max(1, args.warmup)):
        step()
    torch.cuda.synchronize()
    st0 = off.stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clk:
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    st1 = off.stats()
    link = (st1["bytes_link_in"] - st0["bytes_link_in"]) / args.steps
    # consecutive equal indices (the turn-around block) are served from the slot that already holds them
    loaded = sum(1 for i, idx in enumerate(order) if i == 0 or order[i - 1] != idx)
    print(json.dumps({
        "mode": "weights", "metric": "block weights streamed host->device, BF16-equivalent GB/s", "unit": "GB/s",
        "value": round(loaded * block_bytes / (ms * 1e-3) * 1e-9, 2), "ms_per_step": round(ms, 3), "steps": args.steps, "warmup": args.warmup,
        "codec": args.codec, "blocks": args.blocks, "block_bytes": block_bytes, "blocks_loaded_per_step": loaded,
        "h2d_link_gbs": round(link / (ms * 1e-3) * 1e-9, 2), "h2d_frac_of_bound": round(link / (ms * 1e-3) * 1e-9 / PCIE_GEN5_X16_GBS, 3),
        "pinned_bytes": off.pinned_bytes(), "device_slot_bytes": off.device_bytes(), "codec_launches": st1["codec_launches"] - st0["codec_launches"],
        "clocks": clk.summary()}), flush=True)
    off.close()


def run_producers(args, torch, lib, dev):
    """RMSNorm and SwiGLU with the compress step built in, at the DiT block's shapes: CUDA-event time per launch with
    and without codes, against the PyTorch ops they replace and against the separate compress launch they save."""
    import torch.nn.functional as F

    hbm_peak, peak_kind = measured_peaks()
    st = torch.cuda.current_stream()
    sp = st.cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=30):
        for _ in range(5):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()                                  # cold L2: the inputs come from HBM, as in a training step
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st); fn(); e1.record(st)
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    out = {"mode": "producers", "unit": "GB/s of algorithmic bytes", "peak": hbm_peak, "peak_kind": f"of {peak_kind}", "l2": "flushed before every launch"}
    rows, cols, hidden = TOKENS, HIDDEN, 3 * HIDDEN
    x = torch.randn(rows, cols, device=dev, generator=g).to(torch.bfloat16)
    w = torch.ones(cols, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    codes = torch.empty(rows * 2 * hidden, dtype=torch.uint8, device=dev)
    scales = torch.empty(rows * 2 * hidden // 128, dtype=torch.float32, device=dev)
    gu = torch.randn(rows, 2 * hidden, device=dev, generator=g).to(torch.bfloat16)
    h = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)

    def rms(codec):
        assert lib.flame_act_rmsnorm_quant_b128(x.data_ptr(), w.data_ptr(), y.data_ptr(), codes.data_ptr(), scales.data_ptr(), rstd.data_ptr(),
                                                rows, cols, 1e-6, codec, 0, sp) == 0

    def swi(codec):
        assert lib.flame_act_swiglu_quant_b128(gu.data_ptr(), h.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, hidden, codec, 0, sp) == 0

    def torch_rms():
        r = torch.rsqrt(x.pow(2).sum(-1, keepdim=True, dtype=torch.float32) / cols + 1e-6).to(x.dtype)
        return x * r * w

    def torch_swiglu():
        a, b = gu.chunk(2, dim=-1)
        return F.silu(a) * b

    n_r, n_s = rows * cols, rows * 2 * hidden
    for name, fn, alg in (("rmsnorm", lambda: rms(0), 4.0 * n_r), ("rmsnorm+int8", lambda: rms(2), (4.0 + 1.03125) * n_r),
                          ("rmsnorm+fp8", lambda: rms(3), (4.0 + 1.03125) * n_r), ("rmsnorm, PyTorch ops", torch_rms, 4.0 * n_r),
                          ("compress int8 of the norm output, separate launch", lambda: lib.flame_act_quant_int8_b128(y.data_ptr(), codes.data_ptr(), scales.data_ptr(), n_r, 0, sp), 3.03125 * n_r),
                          ("swiglu", lambda: swi(0), 3.0 * n_s), ("swiglu+int8", lambda: swi(2), (3.0 + 1.03125) * n_s),
                          ("swiglu+fp8", lambda: swi(3), (3.0 + 1.03125) * n_s), ("swiglu, PyTorch ops", torch_swiglu, 3.0 * n_s),
                          ("compress int8 of gate+up, separate launch", lambda: lib.flame_act_quant_int8_b128(gu.data_ptr(), codes.data_ptr(), scales.data_ptr(), n_s, 0, sp), 3.03125 * n_s)):
        us = timed(fn)
        out[name] = {"us": round(us, 2), "gbs": round(alg / us * 1e-3, 1), "frac": round(alg / us * 1e-3 / hbm_peak, 3), "alg_bytes": int(alg)}
    out["shapes"] = {"rmsnorm": [rows, cols], "swiglu gate_up": [rows, 2 * hidden]}
    print(json.dumps(out), flush=True)


def pcie_info(torch, index: int) -> dict:
    """What sysfs says about the host link of CUDA device `index`: negotiated and maximum speed and width of the GPU's
    own PCIe function and of every bridge above it, up to the root.  Plain file reads; absent files are left out."""
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}

    def read(path):
        try:
            with open(path) as f:
                return f.read().strip()
        except OSError:
            return None

    def link(dev_path):
        d = {k: read(os.path.join(dev_path, k)) for k in ("current_link_speed", "current_link_width", "max_link_speed", "max_link_width")}
        return {k: v for k, v in d.items() if v is not None}

    out = {"bdf": bdf}
    try:        # the driver's own view of the link (read-only NVML queries)
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bdf.encode() if hasattr(bdf, "encode") else bdf)
        out["nvml"] = {"gen_current": pynvml.nvmlDeviceGetCurrPcieLinkGeneration(h), "gen_max": pynvml.nvmlDeviceGetMaxPcieLinkGeneration(h),
                       "width_current": pynvml.nvmlDeviceGetCurrPcieLinkWidth(h), "width_max": pynvml.nvmlDeviceGetMaxPcieLinkWidth(h)}
    except Exception as exc:
        out["nvml"] = f"unavailable: {type(exc).__name__}"
    node = os.path.realpath(os.path.join("/sys/bus/pci/devices", bdf))
    if not os.path.isdir(node):
        out["sysfs"] = "no such device directory"
        return out
    own = link(node)
    out.update(own if own else {"link_attributes": "sysfs has no current_link_speed / current_link_width for this function"})
    numa = read(os.path.join(node, "numa_node"))
    if numa is not None:
        out["numa_node"] = numa
    chain = []
    parent = os.path.dirname(node)
    while os.path.basename(parent).count(":") == 2:          # 0000:17:00.0 style names: bridges above the GPU
        chain.append({"bdf": os.path.basename(parent), **link(parent)})
        parent = os.path.dirname(parent)
    out["bridges_to_root"] = chain
    out["root"] = os.path.basename(parent)
    return out


def verify_restored(torch, tensors, dst, codec: str, picks=(0, 2, 3)) -> bool:
    """A few restored tensors of the pool round trip against the CPU oracle's dequantise-of-quantise of their sources
    (bit for bit; for the uncompressed mode, against the sources themselves).  The checker, not the product."""
    import numpy as np
    from oracle import capi

    ok = True
    for i in picks:
        if i >= len(tensors):
            continue
        got = dst[i].reshape(-1).view(torch.int16).cpu().numpy().view(np.uint16)
        bits = tensors[i].reshape(-1).view(torch.int16).cpu().numpy().view(np.uint16)
        if codec == "none":
            ok &= bool(np.array_equal(got, bits))
            continue
        wc, ws = (capi.quant_int8_b128 if codec == "int8" else capi.quant_fp8_b128)(bits)
        ok &= bool(np.array_equal(got, (capi.dequant_int8_b128 if codec == "int8" else capi.dequant_fp8_b128)(wc, ws)))
    return ok


def codec_leg(torch, lib, dev, tensors, dst, codec: str, steps: int, warmup: int, groups, sampler_index: int):
    """Compress into packed device buffers and dequantise back, HBM in and HBM out, one launch per group of tensors.
    Returns (ms per step compress, ms per step dequantise, launches per step, clock summary)."""
    from flame_b200 import _lib

    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    codec_id = 2 if codec == "int8" else 3
    packed = [torch.empty(lib.flame_act_packed_bytes(t.numel()), dtype=torch.uint8, device=dev) for t in tensors]
    so = [lib.flame_act_packed_scales_offset(t.numel()) for t in tensors]

    def table(bf16):
        return [((_lib.ActTensor * len(g))(*[_lib.ActTensor(bf16[i].data_ptr(), packed[i].data_ptr(), packed[i].data_ptr() + so[i],
                                                              bf16[i].numel()) for i in g]), len(g)) for g in groups]
    q_tables, d_tables = table(tensors), table(dst)

    def offload_all():
        for arr, n in q_tables:
            rc = lib.flame_act_quant_b128_multi(codec_id, arr, n, 0, sp)
            assert rc == 0, rc

    def restore_all():
        for arr, n in reversed(d_tables):
            rc = lib.flame_act_dequant_b128_multi(codec_id, arr, n, sp)
            assert rc == 0, rc

    for _ in range(max(warmup, 1)):
        offload_all(); restore_all()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1)]
    with ClockSampler(sampler_index) as clk:
        ev[0].record(stream)
        for k in range(steps):
            offload_all(); ev[2 * k + 1].record(stream)
            restore_all(); ev[2 * k + 2].record(stream)
        torch.cuda.synchronize()
    q_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(steps)) / steps
    d_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(steps)) / steps
    return q_ms, d_ms, len(groups), clk.summary()


def roofline_entries(codec: str, q_ms: float, d_ms: float, elems: int, launches: int):
    hbm_peak, peak_kind = measured_peaks()
    alg = ALG_BYTES_PER_ELEM * elems
    qa, da = alg / (q_ms * 1e-3) * 1e-9, alg / (d_ms * 1e-3) * 1e-9
    comp = {"bound": "hbm", "kernel": "compress_b128_kernel", "achieved": round(qa, 1), "peak": hbm_peak, "unit": "GB/s",
            "frac": round(qa / hbm_peak, 4), "peak_kind": f"of {peak_kind}",
            "traffic": int(NCU_TRAFFIC_PER_ELEM["compress"][codec] * elems / launches),
            "alg_bytes_per_launch": int(alg / launches), "avg_launch_us": round(q_ms * 1e3 / launches, 2), "launches_per_step": launches,
            "leg": "device-resident: packed codes written to HBM, no host link"}
    deq = {"bound": "hbm", "kernel": "dequant_b128_kernel", "achieved": round(da, 1), "peak": hbm_peak, "unit": "GB/s",
           "frac": round(da / hbm_peak, 4), "peak_kind": f"of {peak_kind}",
           "traffic": int(NCU_TRAFFIC_PER_ELEM["dequant"] * elems / launches),
           "alg_bytes_per_launch": int(alg / launches), "avg_launch_us": round(d_ms * 1e3 / launches, 2)}
    return comp, deq


def run_fp8_mixed(torch, lib, dev, steps: int, warmup: int) -> dict:
    """FP8 e4m3 per-128 (scale = absmax/448) over the mixed activation set: GELU outputs of an N(0,1) input
    [1,4608,9216], heavy-tailed attention outputs 2*t(nu=3) [1,4608,3072], SwiGLU hidden states [1,4608,9216].
    Codes and scales of a sample are checked against the oracle; the kernels are timed device-resident, the pool end
    to end.  The three tensors are replicated to six so that one pass is larger than the L2."""
    import numpy as np
    from flame_b200 import ActivationOffloadPool, OffloadCompression, synthetic
    from oracle import capi

    base = [synthetic.gelu_of_normal(TOKENS * 3 * HIDDEN, seed=0), synthetic.student_t3_times2(TOKENS * HIDDEN, seed=0),
            synthetic.swiglu_hidden(TOKENS * 3 * HIDDEN, seed=0)]
    names = ["gelu(N(0,1)) [1,4608,9216]", "2*t(nu=3) [1,4608,3072]", "silu(g)*u [1,4608,9216]"]
    tensors = [torch.from_numpy(b.view(np.int16)).to(dev).view(torch.bfloat16) for b in base]
    tensors = tensors + [t.clone() for t in tensors]
    dst = [torch.empty_like(t) for t in tensors]
    step_bytes = sum(t.numel() * 2 for t in tensors)
    step_elems = sum(t.numel() for t in tensors)
    ok = True
    for b in base:                                           # the first 4 Mi elements of each distribution against the oracle
        ok &= verify_against_oracle(torch, lib, torch.from_numpy(b[:1 << 22].view(np.int16)).to(dev).view(torch.bfloat16), "fp8")
    groups = [[0, 1, 2], [3, 4, 5]]
    q_ms, d_ms, launches, clk = codec_leg(torch, lib, dev, tensors, dst, "fp8", steps, warmup, groups, dev.index or 0)
    comp, deq = roofline_entries("fp8", q_ms, d_ms, step_elems, launches)
    pool = ActivationOffloadPool(dev, len(tensors), max(t.numel() * 2 for t in tensors), OffloadCompression.FP8_B128,
                                 host_budget_bytes=ActivationOffloadPool.host_bytes_needed([t.numel() * 2 for t in tensors], OffloadCompression.FP8_B128))
    stream = torch.cuda.current_stream()

    def step():
        hs = [pool.push(t) for t in tensors]
        for h, d in zip(reversed(hs), reversed(dst)):
            pool.pull_into(h, d)
    for _ in range(max(1, warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ok &= verify_restored(torch, tensors, dst, "fp8", picks=(1,))
    # Error of the round trip per distribution, relative to the block maximum.  The reference's encoder sends every
    # magnitude from 248 up (0.55 of the block maximum, which sits at 448) to code 0x7F, and its decoder reads 0x7F as
    # 480: the top of every block comes back as 1.07 x the maximum.  The same tensors through the OCP encoder
    # (FLAME_ACT_FP8_OCP: round to nearest even, saturate at 448) for contrast.
    def worst(a, b):
        x, y = a.float().view(-1, 128), b.float().view(-1, 128)
        return round(float(((x - y).abs().amax(1) / x.abs().amax(1).clamp_min(1e-30)).max()), 4)
    err, err_ocp = {}, {}
    sp = stream.cuda_stream
    for n, t, d in zip(names, tensors, dst):
        err[n] = worst(t, d)
        codes = torch.empty(t.numel(), dtype=torch.uint8, device=dev)
        scales = torch.empty(t.numel() // 128, dtype=torch.float32, device=dev)
        back = torch.empty_like(t)
        assert lib.flame_act_quant_fp8_b128(t.data_ptr(), codes.data_ptr(), scales.data_ptr(), t.numel(), 1, sp) == 0
        assert lib.flame_act_dequant_fp8_b128(codes.data_ptr(), scales.data_ptr(), back.data_ptr(), t.numel(), sp) == 0
        torch.cuda.synchronize()
        err_ocp[n] = worst(t, back)
        del codes, scales, back
    pool.close()
    return {"workload": "FP8 e4m3 per 128 over " + ", ".join(names) + " (each twice: 339.7 MB per pass)", "verified_against_oracle": bool(ok),
            "value": round(2 * step_bytes / (ms * 1e-3) * 1e-9, 2), "unit": UNIT, "ms_per_step": round(ms, 3), "steps": steps,
            "roofline": comp, "roofline_dequant": deq, "max_abs_err_over_block_absmax": err,
            "max_abs_err_over_block_absmax_ocp_encoder": err_ocp, "clocks": clk}


def run_overhead_replicas(torch, dev, rank: int, world: int, barrier, gather, steps: int) -> dict:
    """N > 1: the DiT step on every replica at the same moment.  The link is probed with all replicas copying at
    once, the block planner gets those rates and a cap on the estimated overhead, and the planned arm runs beside
    the resident one."""
    from flame_b200.dit_workload import measure_overhead

    o = measure_overhead(dev, steps=steps, warmup=2, arms=("capped", "deferred_int8"), sync=barrier)
    keys = ("ms_per_step", "overhead_pct", "overhead_pct_vs_mean_baseline", "held_after_forward_gb", "peak_mem_gb")
    mine = o.get("offload_int8_capped", {})
    out = {"replicas": world, "model": o["model"], "cap_pct": o.get("cap_pct"), "interference": o.get("interference"),
           "note": "every replica probes its link, plans and runs the step at the same moment; lists are in rank order"}
    out["probe_d2h_gbs"] = [round(v, 2) for v in gather(o["probe"]["d2h_gbs"])]
    out["probe_h2d_gbs"] = [round(v, 2) for v in gather(o["probe"]["h2d_gbs"])]
    out["resident_ms_per_step"] = [round(v, 3) for v in gather(o["resident"]["ms_per_step"])]
    out["resident_held_after_forward_gb"] = o["resident"]["held_after_forward_gb"]
    for k in keys:
        out["planned_" + k] = [round(v, 3) for v in gather(float(mine.get(k, float("nan"))))]
    offl = gather(float(mine.get("blocks", "").count("O")))
    reco = gather(float(mine.get("blocks", "").count("C")))
    out["planned_blocks_offloaded"] = [int(v) for v in offl]
    out["planned_blocks_recomputed"] = [int(v) for v in reco]
    out["planned_freed_after_forward_gb"] = [round(out["resident_held_after_forward_gb"] - v, 3) for v in out["planned_held_after_forward_gb"]]
    dfr = o.get("offload_int8_all_deferred", {})
    # the other adaptive arm: every block handed to a deferred pool, which sends out what the link carries beside forward
    out["deferred_ms_per_step"] = [round(v, 3) for v in gather(float(dfr.get("ms_per_step", float("nan"))))]
    out["deferred_overhead_pct_vs_mean_baseline"] = [round(v, 2) for v in gather(float(dfr.get("overhead_pct_vs_mean_baseline", float("nan"))))]
    out["deferred_freed_after_forward_gb"] = [round(out["resident_held_after_forward_gb"] - v, 3) for v in gather(float(dfr.get("held_after_forward_gb", float("nan"))))]
    out["deferred_tensors_sent_out_per_step"] = [round(v, 1) for v in gather(float(dfr.get("tensors_pushed_per_step", 0.0)) - float(dfr.get("tensors_used_in_place_per_step", 0.0)))]
    out["rank0"] = {"plan": mine.get("blocks"), "plan_est_ms": mine.get("plan_est_ms"), "offloaded_gb_per_step": mine.get("offloaded_gb_per_step"),
                    "link_gb_per_step": mine.get("link_gb_per_step")}
    out["overhead_pct_worst_replica"] = max(out["planned_overhead_pct_vs_mean_baseline"])
    return out


def host_mem_available_bytes():
    """MemAvailable of /proc/meminfo, or None."""
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return None


LINKSWEEP = (  # (label, chunk MiB, cudaHostAlloc flags, D2H piece MiB, tile chunks)
    ("default: 16 MiB chunks, cudaHostAllocDefault, whole-chunk copies", 16, 0, 0.0, 8),
    ("2 MiB chunks", 2, 0, 0.0, 8),
    ("8 MiB chunks", 8, 0, 0.0, 8),
    ("32 MiB chunks", 32, 0, 0.0, 4),
    ("write-combined slab (cudaHostAllocWriteCombined)", 16, 4, 0.0, 8),
    ("portable slab (cudaHostAllocPortable)", 16, 1, 0.0, 8),
    ("device-to-host copies in 2 MiB pieces", 16, 0, 2.0, 8),
    ("staging tiles of 2 chunks", 16, 0, 0.0, 2),
)


def run_linksweep(args, torch, dev, rank, world, barrier, max_over_ranks, gather):
    """What the pool exposes that could matter when replicas share host links: chunk size, the slab's allocation flags,
    the size of the copy pieces, the staging tile.  One workload, one pool per setting, all replicas in step; one JSON
    line per setting with the whole-job and per-replica figures of the offload+restore step."""
    from flame_b200 import ActivationOffloadPool, OffloadCompression, replicas

    mode = {"int8": OffloadCompression.INT8_B128, "fp8": OffloadCompression.FP8_B128, "none": OffloadCompression.NONE}[args.codec]
    tensors = make_workload(torch, dev, seed=replicas.workload_seed(rank), blocks=args.blocks, kind="dit")
    dst = [torch.empty_like(t) for t in tensors]
    step_bytes = sum(t.numel() * 2 for t in tensors)
    stream = torch.cuda.current_stream()
    for label, chunk_mb, flags, piece_mb, tile_chunks in LINKSWEEP:
        pool = ActivationOffloadPool(dev, len(tensors), max(t.numel() * 2 for t in tensors), mode, chunk_bytes=chunk_mb << 20, tile_chunks=tile_chunks,
                                     d2h_piece_bytes=int(piece_mb * (1 << 20)), host_alloc_flags=flags,
                                     host_budget_bytes=ActivationOffloadPool.host_bytes_needed([t.numel() * 2 for t in tensors], mode, chunk_mb << 20))

        def step():
            hs = [pool.push(t) for t in tensors]
            for h, d in zip(reversed(hs), reversed(dst)):
                pool.pull_into(h, d)
        step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        mine = e0.elapsed_time(e1) / args.steps
        slowest = max_over_ranks(mine)
        per = gather(mine)
        pinned = pool.host_bytes()
        pool.close()
        if rank == 0:
            print(json.dumps({"mode": "linksweep", "setting": label, "replicas": world, "codec": args.codec, "steps": args.steps,
                              "value": round(world * 2 * step_bytes / (slowest * 1e-3) * 1e-9, 2), "value_per_gpu": round(2 * step_bytes / (slowest * 1e-3) * 1e-9, 2),
                              "unit": UNIT, "ms_per_step": round(slowest, 2), "ms_per_step_per_replica": [round(v, 1) for v in per],
                              "gbs_per_replica": [round(2 * step_bytes / (v * 1e-3) * 1e-9, 1) for v in per], "pinned_bytes": pinned}), flush=True)


def run_weight_stream(torch, lib, dev, steps: int, warmup: int) -> dict:
    """The weight-side reuse of the pool in short form, for the default line: FP8 E4M3 weights of DiT blocks (one byte per
    element over the link, through an uncompressed pool) handed out as transposed BF16 by BlockOffloader, every block once in
    forward and once in reverse order; and the expansion kernel alone on a block's four weights, back to back.  One expanded
    weight is compared with the CPU restatement of the reference's decoder after the timed region."""
    from flame_b200 import BlockOffloader, OffloadCompression
    from flame_b200._lib import WeightJob
    hbm_peak, peak_kind = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(7)
    shapes = {"attn.qkv.weight": (3 * HIDDEN, HIDDEN), "attn.out.weight": (HIDDEN, HIDDEN),
              "mlp.up.weight": (6 * HIDDEN, HIDDEN), "mlp.down.weight": (HIDDEN, 3 * HIDDEN)}
    scale, nblocks = 0.0123, 6
    blocks = [{k: torch.randint(0, 0x78, v, dtype=torch.uint8, device=dev, generator=g) | (torch.randint(0, 2, v, dtype=torch.uint8, device=dev, generator=g) << 7)
               for k, v in shapes.items()} for _ in range(nblocks)]
    probe = blocks[2]["attn.out.weight"].cpu().numpy()
    elems = sum(m * n for m, n in shapes.values())
    off = BlockOffloader(dev, blocks, OffloadCompression.NONE, chunk_bytes=32 << 20, fp8_weights={k: (scale, True) for k in shapes})
    del blocks
    torch.cuda.empty_cache()
    order = list(range(nblocks)) + list(reversed(range(nblocks)))
    stream = torch.cuda.current_stream()
    sink = torch.zeros(1, dtype=torch.float32, device=dev)

    def step():
        off.prefetch_block(order[0])
        for i, idx in enumerate(order):
            w = off.await_block(idx)
            if i + 1 < len(order):
                off.prefetch_block(order[i + 1])
            sink.add_(w["attn.out.weight"][0, 0].float())      # a consumer on the compute stream, so each block is really waited for
    for _ in range(max(1, warmup)):
        step()
    torch.cuda.synchronize()
    st0 = off.stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    st1 = off.stats()
    link = (st1["bytes_link_in"] - st0["bytes_link_in"]) / steps
    loaded = sum(1 for i, idx in enumerate(order) if i == 0 or order[i - 1] != idx)
    got = off.ensure_block(2)["attn.out.weight"]
    torch.cuda.synchronize()
    from oracle import capi as oracle
    m, n = shapes["attn.out.weight"]
    ok = bool((got.view(torch.int16).cpu().numpy().view("uint16") == oracle.fp8_dequant_transpose(probe, scale, m, n)).all())
    off.close()
    # the expansion kernel alone: a block's four weights in one launch, 20 blocks back to back over four buffer sets (1.1 GB each way)
    sets = [[(torch.randint(0, 0x78, s, dtype=torch.uint8, device=dev, generator=g), torch.empty(s[1], s[0], dtype=torch.bfloat16, device=dev)) for s in shapes.values()]
            for _ in range(4)]
    tables = [(WeightJob * 4)(*[WeightJob(c.data_ptr(), d.data_ptr(), scale, c.shape[0], c.shape[1], 0) for c, d in ws]) for ws in sets]
    sp = stream.cuda_stream
    for k in range(8):
        assert lib.flame_fused_dequant_transpose_bf16_multi(tables[k % 4], 4, sp) == 0
    torch.cuda.synchronize()
    e0.record(stream)
    for k in range(20):
        assert lib.flame_fused_dequant_transpose_bf16_multi(tables[k % 4], 4, sp) == 0
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 20
    return {"workload": f"{nblocks} DiT blocks of FP8 E4M3 weights (qkv, out, up, down: {elems / 1e6:.1f} M codes per block), streamed host->device and "
                        "expanded to transposed BF16; every block once forward and once in reverse per step",
            "value": round(loaded * elems * 2 / (ms * 1e-3) * 1e-9, 2), "unit": "GB/s BF16-equivalent", "ms_per_step": round(ms, 3), "steps": steps,
            "blocks_loaded_per_step": loaded, "h2d_link_gbs": round(link / (ms * 1e-3) * 1e-9, 2),
            "h2d_frac_of_bound": round(link / (ms * 1e-3) * 1e-9 / PCIE_GEN5_X16_GBS, 3), "verified_against_oracle": ok,
            "roofline": {"bound": "hbm", "kernel": "fp8_dequant_transpose_tiles_kernel", "achieved": round(3.0 * elems / us * 1e-3, 1), "peak": hbm_peak,
                         "unit": "GB/s", "frac": round(3.0 * elems / us * 1e-3 / hbm_peak, 4), "peak_kind": f"of {peak_kind}", "traffic": int(elems * NCU_TRAFFIC_PER_WEIGHT_ELEM),
                         "alg_bytes_per_launch": int(3 * elems), "avg_launch_us": round(us, 2),
                         "leg": "a block's four weights in one launch, 20 launches back to back over four buffer sets"}}


def run_weight_kernel(args, torch, lib, dev):
    """flame_fused_dequant_transpose_bf16 (FP8 weights [M,N] -> BF16 [N,M]) at the DiT block's weight shapes, 1 B read +
    2 B written per element against the measured HBM rate.  Per shape: one launch between two CUDA events with the L2
    flushed before it (`us`; the events of this GPU tick in steps of about 2 us and the figure holds the launch's own
    start-up), and 20 launches back to back over rotating buffer sets that together exceed twice the L2 (`us_back_to_back`).
    Then a block's four weights, 20 blocks back to back: one call per weight, and all four in one launch."""
    from flame_b200._lib import WeightJob
    hbm_peak, peak_kind = measured_peaks()
    st = torch.cuda.current_stream()
    sp = st.cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    out = {"mode": "weightkernel", "unit": "GB/s of algorithmic bytes (3 per element)", "peak": hbm_peak, "peak_kind": f"of {peak_kind}",
           "l2": "us: flushed before every launch; us_back_to_back: buffer sets rotate, more than 2 x L2 between two uses of one"}

    def entry(us, alg):
        return {"us": round(us, 2), "gbs": round(alg / us * 1e-3, 1), "frac": round(alg / us * 1e-3 / hbm_peak, 3)}

    def timed(fn, reps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for k in range(reps):
            fn(k)
        e1.record(st)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    for name, (m, n) in (("attn.qkv.weight [9216,3072]", (3 * HIDDEN, HIDDEN)), ("attn.out.weight [3072,3072]", (HIDDEN, HIDDEN)),
                         ("mlp.up.weight [18432,3072]", (6 * HIDDEN, HIDDEN)), ("mlp.down.weight [3072,9216]", (HIDDEN, 3 * HIDDEN)),
                         ("odd shape [3001,1537] (shared-memory fallback kernel)", (3001, 1537))):
        alg = 3.0 * m * n
        nsets = max(2, int(2 * 126e6 // alg) + 2)
        sets = [(torch.randint(0, 0x78, (m, n), dtype=torch.uint8, device=dev, generator=g), torch.empty(n, m, dtype=torch.bfloat16, device=dev))
                for _ in range(nsets)]

        def fn(k):
            c, d = sets[k % nsets]
            assert lib.flame_fused_dequant_transpose_bf16(c.data_ptr(), d.data_ptr(), 0.0123, m, n, sp) == 0
        for k in range(5):
            fn(k)
        ts = []
        for k in range(30):
            flush.zero_()
            ts.append(timed(fn, 1))
        ts.sort()
        out[name] = dict(entry(ts[len(ts) // 2], alg), alg_bytes=int(alg))
        b2b = entry(timed(fn, 20 * nsets), alg)
        out[name].update(us_back_to_back=b2b["us"], gbs_back_to_back=b2b["gbs"], frac_back_to_back=b2b["frac"], buffer_sets=nsets)
        del sets
    # all four weights of a block back to back, as a block's expansion after its bytes have arrived
    shapes = [(3 * HIDDEN, HIDDEN), (HIDDEN, HIDDEN), (6 * HIDDEN, HIDDEN), (HIDDEN, 3 * HIDDEN)]
    sets = [[(torch.randint(0, 0x78, s, dtype=torch.uint8, device=dev, generator=g), torch.empty(s[1], s[0], dtype=torch.bfloat16, device=dev)) for s in shapes]
            for _ in range(4)]
    tables = [(WeightJob * 4)(*[WeightJob(c.data_ptr(), d.data_ptr(), 0.0123, m, n, 0) for (c, d), (m, n) in zip(ws, shapes)]) for ws in sets]

    def block(k):
        for (c, d), (m, n) in zip(sets[k % 4], shapes):
            assert lib.flame_fused_dequant_transpose_bf16(c.data_ptr(), d.data_ptr(), 0.0123, m, n, sp) == 0

    def block_multi(k):
        assert lib.flame_fused_dequant_transpose_bf16_multi(tables[k % 4], 4, sp) == 0
    elems = sum(m * n for m, n in shapes)
    for label, fn in (("one block's four weights, 20 blocks back to back", block), ("the same, one launch per block (_multi)", block_multi)):
        for k in range(8):
            fn(k)
        out[label] = dict(entry(timed(fn, 20), 3.0 * elems), alg_bytes=int(3 * elems))
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--codec", choices=["int8", "fp8", "none"], default="int8")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--chunk-mb", type=int, default=32, help="pipeline chunk in MiB of source; 32 measured 2 percent above 16 on the DiT step's tensors at one GPU, no different at two")
    ap.add_argument("--tile-chunks", type=int, default=4)
    ap.add_argument("--d2h-piece-mb", type=float, default=0.0, help="issue device-to-host copies in pieces of this size (0 = whole chunks)")
    ap.add_argument("--host-alloc-flags", type=int, default=0, help="cudaHostAlloc flags of the pinned slab (4 = write-combined)")
    ap.add_argument("--waves", type=int, default=0, help="offload and restore a step's tensors in this many waves (0 = as few as the host's memory allows)")
    ap.add_argument("--blocks", type=int, default=BLOCKS, help="fewer blocks = smaller case (profiling only)")
    ap.add_argument("--no-dit", action="store_true", help="skip the DiT training-step overhead measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-fp8-mixed", action="store_true", help="skip the FP8 mixed-activation-set block")
    ap.add_argument("--no-weights", action="store_true", help="skip the FP8 weight-streaming block")
    ap.add_argument("--no-ref-gpu", action="store_true", help="--impl reference: skip timing the reference's own compiled CUDA files")
    ap.add_argument("--only", choices=["all", "value", "codec", "e2e"], default="all",
                    help="profiling: run only one timed region (codec = the device-resident compress/dequantise leg)")
    ap.add_argument("--mode", choices=["bench", "sweep", "interference", "weights", "producers", "linksweep", "weightkernel"], default="bench",
                    help="sweep: 1 MB..4 GB single tensor x codec x chunk size; interference: copies against HBM-bound kernels; "
                         "weights: block weights streamed host->device through the same pool")
    ap.add_argument("--sweep-max-mb", type=int, default=4096)
    ap.add_argument("--workload", choices=["dit", "c4"], default="dit",
                    help="c4: 200 x [8,4096,3072] BF16 = 40 GB per GPU per step (the replica-contention case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from flame_b200 import ActivationOffloadPool, OffloadCompression, _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a replica that failed never reaches the next barrier: the others give up after three minutes instead of ten
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    lib = _lib.lib()  # raises if the CUDA library is missing: there is no fallback

    from flame_b200 import replicas

    def barrier():
        replicas.barrier(world)
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        return replicas.max_over_ranks(ms, world, dev)

    def gather(v: float) -> list:
        return replicas.gather_over_ranks(v, world, dev)

    if args.mode != "bench":
        if args.mode == "sweep":
            run_sweep(args, torch, lib, dev, rank)
        elif args.mode == "linksweep":
            run_linksweep(args, torch, dev, rank, world, barrier, max_over_ranks, gather)
        elif rank == 0:
            {"producers": lambda: run_producers(args, torch, lib, dev), "weights": lambda: run_weights(args, torch, dev),
             "weightkernel": lambda: run_weight_kernel(args, torch, lib, dev),
             "interference": lambda: run_interference(args, torch, lib, dev)}[args.mode]()
        if world > 1:
            dist.destroy_process_group()
        return

    tensors = make_workload(torch, dev, seed=replicas.workload_seed(rank), blocks=args.blocks, kind=args.workload)
    step_bytes = sum(t.numel() * 2 for t in tensors)
    step_elems = sum(t.numel() for t in tensors)
    max_bytes = max(t.numel() * 2 for t in tensors)
    mode = {"int8": OffloadCompression.INT8_B128, "fp8": OffloadCompression.FP8_B128, "none": OffloadCompression.NONE}[args.codec]
    stream = torch.cuda.current_stream()
    verified = verify_against_oracle(torch, lib, tensors[1], args.codec) if args.codec != "none" else True
    dst = [torch.empty_like(t) for t in tensors]
    hbm_peak, peak_kind = measured_peaks()
    line = {
        "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"int8": "int8 codes + f32 scales", "fp8": "fp8-e4m3 codes + f32 scales", "none": "bf16"}[args.codec],
        "data": "synthetic", "config": workload_config(args, world),
    }
    launches = 0

    # ---- the path: the pool, through pinned host memory; inputs resident in HBM, CUDA events -----------------------
    if args.only in ("all", "value", "e2e"):
        # Pinned memory for one step of every replica must fit in the host's memory.  Where it does not (the 40 GB
        # case on a box with little RAM), the step runs in `waves`: a wave's tensors go out and come back before the
        # next wave starts, through a slab sized for one wave.  The bytes moved per step are the same.
        need = ActivationOffloadPool.host_bytes_needed([t.numel() * 2 for t in tensors], mode, args.chunk_mb << 20)
        avail = host_mem_available_bytes()
        waves = args.waves if args.waves > 0 else (max(1, -(-(world * need) // int(0.45 * avail))) if avail else 1)
        waves = int(max_over_ranks(float(waves)))
        per_wave = -(-len(tensors) // waves)
        wave_sets = [list(range(i, min(i + per_wave, len(tensors)))) for i in range(0, len(tensors), per_wave)]
        budget = max(ActivationOffloadPool.host_bytes_needed([tensors[i].numel() * 2 for i in ws], mode, args.chunk_mb << 20) for ws in wave_sets)
        line["config"]["waves_per_step"] = waves
        line["config"]["host_mem_available_gb"] = round(avail / 1e9, 1) if avail else None
        pool = ActivationOffloadPool(dev, per_wave, max_bytes, mode, chunk_bytes=args.chunk_mb << 20, tile_chunks=args.tile_chunks,
                                     d2h_piece_bytes=int(args.d2h_piece_mb * (1 << 20)), host_alloc_flags=args.host_alloc_flags,
                                     host_budget_bytes=budget)

        def path_step():
            for ws in wave_sets:
                handles = [pool.push(tensors[i]) for i in ws]
                for h, i in zip(reversed(handles), reversed(ws)):
                    pool.pull_into(h, dst[i])

    if args.only in ("all", "value"):
        for _ in range(max(args.warmup, 1)):
            path_step()
        barrier()
        st0 = pool.stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk_value:
            wall0 = time.perf_counter()
            e0.record(stream)
            for _ in range(args.steps):
                path_step()
            e1.record(stream)
            barrier()
            wall = (time.perf_counter() - wall0) / args.steps
        my_ms = e0.elapsed_time(e1) / args.steps
        value_ms = max_over_ranks(my_ms)
        st1 = pool.stats()
        d2h_b = (st1["bytes_link_out"] - st0["bytes_link_out"]) // args.steps
        h2d_b = (st1["bytes_link_in"] - st0["bytes_link_in"]) // args.steps
        launches += st1["codec_launches"] - st0["codec_launches"]
        # what came back, against the oracle's dequantise-of-quantise of what went out
        restored_ok = verify_restored(torch, tensors, dst, args.codec) if args.workload == "dit" else verify_restored(torch, tensors, dst, args.codec, picks=(0,))
        verified = bool(verified and restored_ok)
        value = world * 2 * step_bytes / (value_ms * 1e-3) * 1e-9
        line.update({"value": round(value, 2), "value_per_gpu": round(value / world, 2), "ms_per_step": round(value_ms, 3),
                     "ms_per_step_per_replica": [round(v, 2) for v in gather(my_ms)], "wall_ms_per_step": round(wall * 1e3, 3),
                     "pinned_bytes": pool.host_bytes(), "d2h_bytes_per_step": int(d2h_b), "h2d_bytes_per_step": int(h2d_b),
                     "api": "flame_offload_pool_push / flame_offload_pool_pull_into", "clocks": clk_value.summary()})

    # ---- end to end through the reference's signatures: push, allocating pull, a result read back on the host ------
    if args.only in ("all", "e2e"):
        def e2e_step():
            acc = torch.zeros((), dtype=torch.float32, device=dev)
            for ws in wave_sets:
                handles = [pool.push(tensors[i]) for i in ws]
                for h in reversed(handles):
                    y = pool.pull(h)                    # a fresh tensor per pull, as src/activation_offload.rs:655
                    acc += y.view(-1)[:: max(1, y.numel() // 64)].float().sum()
                    del y
            return float(acc.item())                    # device-to-host read of the step's result

        k_e2e = max(1, min(args.steps, 10))
        for _ in range(max(1, min(args.warmup, 2))):
            e2e_step()
        barrier()
        sa = pool.stats()
        with ClockSampler(local) as clk_e2e:
            t0 = time.perf_counter()
            for _ in range(k_e2e):
                result = e2e_step()
            torch.cuda.synchronize()
            my_s = (time.perf_counter() - t0) / k_e2e
            barrier()
        sb = pool.stats()
        launches_e2e = sb["codec_launches"] - sa["codec_launches"]
        e2e_ms = max_over_ranks(my_s * 1e3)
        line["e2e"] = {"value": round(world * 2 * step_bytes / (e2e_ms * 1e-3) * 1e-9, 2), "unit": UNIT,
                       "h2d_bytes_per_step": int((sb["bytes_link_in"] - sa["bytes_link_in"]) // k_e2e),
                       "d2h_bytes_per_step": int((sb["bytes_link_out"] - sa["bytes_link_out"]) // k_e2e) + 4,   # + the result read back
                       "ms_per_step": round(e2e_ms, 3), "steps": k_e2e, "timed": "host clock around the steps and a device synchronise",
                       "result_read_back": result, "gpu_launches": int(launches_e2e),
                       "api": "ActivationOffloadPool.push / pull (fresh destination per pull) + .item() of a checksum"}
        line["clocks_e2e"] = clk_e2e.summary()
        if "value" not in line:
            line.update({"value": line["e2e"]["value"], "ms_per_step": line["e2e"]["ms_per_step"], "clocks": line["clocks_e2e"]})

    # ---- per-direction link rates, apart from the headline ------------------------------------------------------------
    if args.only == "all" and waves == 1:
        barrier()
        w0 = time.perf_counter()
        handles = [pool.push(t) for t in tensors]
        pool.synchronize(300.0)          # bounded wait for the pool's own streams
        d2h_s = time.perf_counter() - w0
        barrier()                        # every replica has finished offloading before any starts restoring
        a1, a2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a1.record(stream)
        for h, d in zip(reversed(handles), reversed(dst)):
            pool.pull_into(h, d)          # the compute stream waits for each restore
        a2.record(stream)
        torch.cuda.synchronize()
        d2h_all = gather(d2h_b / d2h_s * 1e-9)
        h2d_all = gather(h2d_b / (a1.elapsed_time(a2) * 1e-3) * 1e-9)
        # both directions at once: the second half of the tensors goes out while the first half comes back
        half = len(tensors) // 2
        first = [pool.push(t) for t in tensors[:half]]
        pool.synchronize(300.0)
        barrier()
        sa = pool.stats()
        w0 = time.perf_counter()
        second = []
        for i in range(half):
            second.append(pool.push(tensors[half + i]))
            pool.pull_into(first[half - 1 - i], dst[half - 1 - i])
        pool.synchronize(300.0)
        torch.cuda.synchronize()
        dup_s = time.perf_counter() - w0
        sb = pool.stats()
        dup_out = gather((sb["bytes_link_out"] - sa["bytes_link_out"]) / dup_s * 1e-9)
        dup_in = gather((sb["bytes_link_in"] - sa["bytes_link_in"]) / dup_s * 1e-9)
        for h in second:
            pool.discard(h)
        # the practical ceiling at this replica count: plain 1 GiB pinned copies, all replicas at the same moment
        plain = plain_copy_rates(torch, lib, dev, barrier)
        plain_d2h, plain_h2d = gather(plain[0]), gather(plain[1])
        plain_dup_out, plain_dup_in = gather(plain[2]), gather(plain[3])
        r1 = lambda xs: [round(v, 1) for v in xs]
        link = {"bound_gbs": PCIE_GEN5_X16_GBS, "d2h_gbs": round(min(d2h_all), 2), "h2d_gbs": round(min(h2d_all), 2),
                "d2h_gbs_per_replica": r1(d2h_all), "h2d_gbs_per_replica": r1(h2d_all),
                "plain_copy_d2h_gbs_per_replica": r1(plain_d2h), "plain_copy_h2d_gbs_per_replica": r1(plain_h2d),
                "duplex_d2h_gbs_per_replica": r1(dup_out), "duplex_h2d_gbs_per_replica": r1(dup_in),
                "plain_copy_duplex_d2h_gbs_per_replica": r1(plain_dup_out), "plain_copy_duplex_h2d_gbs_per_replica": r1(plain_dup_in),
                "sum_d2h_gbs": round(sum(d2h_all), 1), "sum_h2d_gbs": round(sum(h2d_all), 1),
                "sum_plain_copy_d2h_gbs": round(sum(plain_d2h), 1), "sum_plain_copy_h2d_gbs": round(sum(plain_h2d), 1),
                "note": "d2h_gbs / h2d_gbs are the slowest replica's, one direction at a time with a barrier between the phases; duplex_* is "
                        "offload of one half of the tensors beside restore of the other half; plain_copy_* is cudaMemcpyAsync of 1 GiB "
                        "from all replicas at once (duplex: both directions at once on two streams)"}
        link["d2h_frac_of_bound"] = round(link["d2h_gbs"] / PCIE_GEN5_X16_GBS, 3)
        link["h2d_frac_of_bound"] = round(link["h2d_gbs"] / PCIE_GEN5_X16_GBS, 3)
        link["d2h_frac_of_plain_copy"] = round(min(a / b for a, b in zip(d2h_all, plain_d2h)), 3)
        link["h2d_frac_of_plain_copy"] = round(min(a / b for a, b in zip(h2d_all, plain_h2d)), 3)
        link["duplex_frac_of_plain_copy"] = round(min((a + b) / (c + d) for a, b, c, d in zip(dup_out, dup_in, plain_dup_out, plain_dup_in)), 3)
        # what sysfs knows about each replica's link: replica r uses CUDA device r, and every device is visible to rank 0
        link["pcie"] = [pcie_info(torch, i) for i in range(world)] if rank == 0 else None
        line["link"] = link
    if args.only in ("all", "value", "e2e"):
        pool.clear()
        pool.close()
        del pool

    # ---- the codec kernels alone: HBM in, HBM out, one launch per checkpointed block -----------------------------------
    if args.only in ("all", "codec") and args.codec != "none":
        per_block = len(BLOCK_SAVED) if args.workload == "dit" else 4
        groups = [list(range(b, min(b + per_block, len(tensors)))) for b in range(0, len(tensors), per_block)]
        k_codec = max(1, min(args.steps, 10))
        q_ms, d_ms, n_l, clk_codec = codec_leg(torch, lib, dev, tensors, dst, args.codec, k_codec, min(args.warmup, 3), groups, local)
        comp, deq = roofline_entries(args.codec, q_ms, d_ms, step_elems, n_l)
        comp["clocks"] = clk_codec
        line["roofline"], line["roofline_dequant"] = comp, deq
        line["device_resident"] = {"value": round(2 * step_bytes / ((q_ms + d_ms) * 1e-3) * 1e-9, 1), "unit": UNIT, "ms_per_step": round(q_ms + d_ms, 4),
                                   "steps": k_codec, "gpu_launches": 2 * n_l * k_codec,
                                   "note": "compress into packed device buffers and dequantise back; no host link, so not the metric"}
        if "value" not in line:
            line.update({"value": line["device_resident"]["value"], "ms_per_step": line["device_resident"]["ms_per_step"], "clocks": clk_codec})
            launches += 2 * n_l * k_codec
    line["verified_against_oracle"] = bool(verified)
    line["gpu_launches"] = int(launches)

    del tensors, dst
    torch.cuda.empty_cache()
    full = args.only == "all" and args.workload == "dit"
    if rank == 0 and world == 1 and full and not args.no_fp8_mixed:
        try:
            line["fp8_mixed"] = run_fp8_mixed(torch, lib, dev, steps=max(3, min(args.steps, 10)), warmup=3)
        except Exception as exc:
            line["fp8_mixed"] = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and full and not args.no_weights:
        try:
            line["weights_fp8"] = run_weight_stream(torch, lib, dev, steps=max(3, min(args.steps, 10)), warmup=3)
        except Exception as exc:
            line["weights_fp8"] = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, cores, sample, _ = cpu_leg(12.0, args.codec)
        line["cpu_baseline"] = {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    if full and not args.no_dit:
        try:
            if world == 1:
                from flame_b200.dit_workload import measure_overhead
                line["overhead"] = measure_overhead(dev, steps=max(3, min(args.steps, 5)), warmup=3)
            else:
                line["overhead"] = run_overhead_replicas(torch, dev, rank, world, barrier, gather, steps=3)
        except Exception as exc:  # the headline numbers above stand on their own
            line["overhead"] = {"error": f"{type(exc).__name__}: {exc}"}
            if world > 1:
                raise
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
