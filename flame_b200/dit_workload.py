"""DiT transformer-block training step used to measure step-time overhead of the offload path.

20 blocks, hidden 3072, 24 heads x 128, SwiGLU MLP with ratio 3 (hidden 9216),
RMSNorm, rotary embedding over a 64x64 latent grid (4096 image tokens) plus 512
text tokens, batch 1, BF16, random-init weights, fused AdamW.  The dense maths
(cuBLAS GEMMs, the library attention kernel) is PyTorch's: it is the compute the
copies have to hide behind, not part of this package's product.

Arms: activations resident (plain autograd), ``checkpoint_offload`` with the pool
in INT8_B128 or NONE mode, and ``checkpoint`` (full recompute).
"""
from __future__ import annotations

import math
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import checkpoint as ckpt
from . import fused_producers
from .activation_offload import ActivationOffloadPool, OffloadCompression
from .policy import Block, Decision, plan_blocks, probe

HIDDEN, HEADS, HEAD_DIM, MLP_HIDDEN = 3072, 24, 128, 9216
IMG_TOKENS, TXT_TOKENS, GRID = 4096, 512, 64
TOKENS = IMG_TOKENS + TXT_TOKENS
# True: RMSNorm and SwiGLU run as this library's kernels, which also emit the codes of the tensor the block saves
# while a block is being offloaded (flame_b200/fused_producers.py); False: PyTorch ops, compress launches read the tensors.
FUSED_PRODUCERS = False


def rope_tables(device):
    """cos/sin [T, HEAD_DIM/2]: axial (row, column) rotary angles for image tokens, 1-D positions for text tokens."""
    half = HEAD_DIM // 2
    freqs = 1.0 / (10000.0 ** (torch.arange(0, half // 2, device=device, dtype=torch.float32) / (half // 2)))
    ys, xs = torch.meshgrid(torch.arange(GRID, device=device), torch.arange(GRID, device=device), indexing="ij")
    img = torch.cat([ys.reshape(-1, 1).float() * freqs, xs.reshape(-1, 1).float() * freqs], dim=1)
    t = torch.arange(TXT_TOKENS, device=device).float().reshape(-1, 1)
    txt = torch.cat([t * freqs, t * freqs], dim=1)
    ang = torch.cat([txt, img], dim=0)
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def _rotate(x, cos, sin):
    """x [B, T, H, D]; rotates pairs (first half, second half) by the per-token angles."""
    x1, x2 = x[..., : HEAD_DIM // 2], x[..., HEAD_DIM // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


class RoPEFn(torch.autograd.Function):
    """Rotary embedding that saves nothing but the angle tables: backward rotates the gradient back."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _rotate(x, cos, sin)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _rotate(dy, cos, -sin), None, None


class RMSNormFn(torch.autograd.Function):
    """RMSNorm whose backward works from its OUTPUT (the tensor the next linear saves anyway) and 1/rms."""

    @staticmethod
    def forward(ctx, x, w, eps):
        if FUSED_PRODUCERS:
            y, rstd = fused_producers.rmsnorm(x, w, eps)
            rstd = rstd.view(*x.shape[:-1], 1).to(x.dtype)
        else:
            rstd = torch.rsqrt(x.pow(2).sum(-1, keepdim=True, dtype=torch.float32) / x.shape[-1] + eps).to(x.dtype)
            y = x * rstd * w
        ctx.save_for_backward(y, rstd, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        y, rstd, w = ctx.saved_tensors
        xhat = y / torch.where(w == 0, torch.ones_like(w), w)
        g = dy * w
        m = ((g * xhat).sum(-1, keepdim=True, dtype=torch.float32) / y.shape[-1]).to(y.dtype)
        dx = rstd * (g - xhat * m)
        dw = (dy * xhat).reshape(-1, y.shape[-1]).sum(0, dtype=torch.float32)
        return dx, dw.to(w.dtype), None


class SwiGLUDownFn(torch.autograd.Function):
    """down(silu(gate) * up) that saves only the gate+up tensor and rebuilds the hidden state in backward."""

    @staticmethod
    def forward(ctx, gu, wd):
        g, u = gu.chunk(2, dim=-1)
        ctx.save_for_backward(gu, wd)
        if FUSED_PRODUCERS:
            return fused_producers.swiglu(gu) @ wd.t()
        return (F.silu(g) * u) @ wd.t()

    @staticmethod
    def backward(ctx, dy):
        gu, wd = ctx.saved_tensors
        g, u = gu.chunk(2, dim=-1)
        sg = torch.sigmoid(g)
        silu = g * sg
        dwd = dy.reshape(-1, dy.shape[-1]).t() @ (silu * u).reshape(-1, g.shape[-1])
        dh = dy @ wd
        dgu = torch.empty_like(gu)
        dg, du = dgu.chunk(2, dim=-1)
        torch.mul(dh, silu, out=du)
        # d silu(g)/dg = sg * (1 + g * (1 - sg)) = sg + silu * (1 - sg)
        torch.mul(dh * u, torch.addcmul(sg, silu, 1 - sg), out=dg)
        return dgu, dwd


class DiTBlock(nn.Module):
    """Saves, per block, exactly: norm1 output, rotated Q/K and V, attention output, norm2 output, gate+up."""

    def __init__(self):
        super().__init__()
        self.norm1_w = nn.Parameter(torch.ones(HIDDEN))
        self.qkv = nn.Linear(HIDDEN, 3 * HIDDEN, bias=False)
        self.proj = nn.Linear(HIDDEN, HIDDEN, bias=False)
        self.norm2_w = nn.Parameter(torch.ones(HIDDEN))
        self.gate_up = nn.Linear(HIDDEN, 2 * MLP_HIDDEN, bias=False)
        self.down = nn.Linear(MLP_HIDDEN, HIDDEN, bias=False)

    def forward(self, x, cos, sin):
        b, t, _ = x.shape
        qkv = self.qkv(RMSNormFn.apply(x, self.norm1_w, 1e-6)).view(b, t, 3, HEADS, HEAD_DIM)
        q = RoPEFn.apply(qkv[:, :, 0], cos, sin)          # [B,T,H,D], contiguous
        k = RoPEFn.apply(qkv[:, :, 1], cos, sin)
        v = qkv[:, :, 2].contiguous()
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))  # views over [B,T,H,D]
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, HIDDEN))
        return x + SwiGLUDownFn.apply(self.gate_up(RMSNormFn.apply(x, self.norm2_w, 1e-6)), self.down.weight)


class DiT(nn.Module):
    def __init__(self, blocks: int = 20):
        super().__init__()
        self.blocks = nn.ModuleList(DiTBlock() for _ in range(blocks))
        self.decisions = None  # per block: Decision, or None = plain autograd

    def forward(self, x, cos, sin):
        for i, blk in enumerate(self.blocks):
            d = None if self.decisions is None else self.decisions[i]
            if d is None or d == Decision.RESIDENT:
                x = blk(x, cos, sin)
            elif d == Decision.RECOMPUTE:
                x = ckpt.checkpoint([x, cos, sin], blk)
            else:
                x = ckpt.checkpoint_offload([x, cos, sin], blk, decision=d)
        return x


def _time_steps(model, opt, x, cos, sin, steps, warmup):
    def one():
        loss = model(x, cos, sin).float().pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = one()
    e1.record()
    torch.cuda.synchronize()
    ms, peak = e0.elapsed_time(e1) / steps, torch.cuda.max_memory_allocated()
    # one more, untimed step to see how much the forward pass leaves on the device
    m0 = torch.cuda.memory_allocated()
    loss = model(x, cos, sin).float().pow(2).mean()
    torch.cuda.synchronize()
    pool = ckpt.activation_offload_pool()
    if pool is not None:
        if pool.stats()["pushes_queued"] == 0:  # nothing waits for its turn: only copies already on their way are awaited
            pool.synchronize(60.0)              # (a pool that holds tensors back keeps them back, as in the timed steps)
        pool.release_finished_sources()         # the pool lets go of a source when it next looks, which is at the next push
    held = torch.cuda.memory_allocated() - m0
    loss.backward()
    opt.step()
    opt.zero_grad(set_to_none=True)
    torch.cuda.synchronize()
    return ms, peak, held


def _block_times(model, x, cos, sin):
    """Forward and backward milliseconds of one block and the BF16 bytes checkpoint_offload would push for it."""
    blk = model.blocks[0]
    saved = ckpt.saved_bytes_of(blk, [x.detach().requires_grad_(True), cos, sin])
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    fwd = bwd = 0.0
    reps = 4
    for r in range(reps + 2):
        xin = x.detach().requires_grad_(True)
        ev[0].record()
        y = blk(xin, cos, sin)
        ev[1].record()
        y.backward(torch.ones_like(y))
        ev[2].record()
        torch.cuda.synchronize()
        if r > 1:  # the first passes warm up
            fwd += ev[0].elapsed_time(ev[1]) / reps
            bwd += ev[1].elapsed_time(ev[2]) / reps
    for p in blk.parameters():
        p.grad = None
    return fwd, bwd, saved


# Copies overlapped with training are issued in pieces (see FlameOffloadPoolConfig.d2h_piece_bytes): 2 MiB when the
# training thread issues them itself, 1 MiB for device-to-host copies that the pool's own thread issues (deferred pools).
COPY_PIECE_BYTES = 2 << 20
DEFERRED_D2H_PIECE_BYTES = 1 << 20
ISSUE_OFF_THREAD = 1 << 40   # a deferred pool with this in-flight budget never queues: it only moves the issuing off the training thread


# The capped plan's estimate of what a busy copy engine costs the compute beside it, per unit of busy time: a step
# with 12 of 20 blocks offloaded in int8 measured +4.2 to +5.3 ms for 75 ms of copy-engine time on a B200.
CAPPED_PLAN_INTERFERENCE = 0.065


def measure_overhead(device, steps: int = 3, warmup: int = 3, blocks: int = 20,
                     arms=("offload_int8", "capped", "timed", "deferred", "offload_bf16", "recompute", "fused"), custom=(),
                     resident_budget_blocks: int = 8, sync=None, cap_pct: float = 3.5) -> dict:
    """Step time of each arm relative to resident activations.  Returns a JSON-ready dict.

    ``sync``: called before the link probe and before every timed arm.  With several replicas it is a barrier, so
    that all of them probe, and later copy, at the same moment and see the link as it is when it is shared.
    Arm "capped": the plan that keeps as little resident as the probed link allows within ``cap_pct`` per cent of
    estimated extra step time (flame_offload_policy_plan_blocks with overhead_cap_ms)."""
    sync = sync or (lambda: None)
    torch.manual_seed(0)
    dev = torch.device(device)
    model = DiT(blocks).to(dev, torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5, fused=True)
    x = torch.randn(1, TOKENS, HIDDEN, device=dev, dtype=torch.bfloat16)
    cos, sin = rope_tables(dev)
    fwd_ms, bwd_ms, saved_bytes = _block_times(model, x, cos, sin)
    sync()
    link = probe(256 << 20, 3)
    out = {"model": f"DiT {blocks} blocks, hidden {HIDDEN}, {HEADS}x{HEAD_DIM} heads, SwiGLU {MLP_HIDDEN}, {TOKENS} tokens, batch 1, bf16, fused AdamW",
           "block_fwd_ms": round(fwd_ms, 3), "block_bwd_ms": round(bwd_ms, 3), "saved_bytes_per_block": int(saved_bytes),
           "probe": {"d2h_gbs": round(link.d2h_gbs, 2), "h2d_gbs": round(link.h2d_gbs, 2), "hbm_copy_gbs": round(link.hbm_copy_gbs, 1)}}

    model.decisions = None
    sync()
    base_ms, base_mem, base_held = _time_steps(model, opt, x, cos, sin, steps, warmup)
    out["resident"] = {"ms_per_step": round(base_ms, 3), "peak_mem_gb": round(base_mem / 1e9, 2),
                       "held_after_forward_gb": round(base_held / 1e9, 2)}

    def run_arm(name, decisions, mode, deferred_bytes=0, d2h_piece=COPY_PIECE_BYTES, base=None, **pool_kwargs):
        base = base_ms if base is None else base
        pool = None
        if mode is not None:
            # sized for every block offloaded at once; the plan decides how many really are
            sizes = [saved_bytes] * blocks
            pool = ActivationOffloadPool(dev, 16 * blocks, max(saved_bytes, 1 << 20), mode, d2h_piece_bytes=d2h_piece,
                                         h2d_piece_bytes=2 * COPY_PIECE_BYTES, deferred_inflight_bytes=deferred_bytes, **pool_kwargs,
                                         host_budget_bytes=int(ActivationOffloadPool.host_bytes_needed(sizes, mode) * 1.5))
            ckpt.set_activation_offload_pool(pool)
        model.decisions = decisions
        try:
            sync()
            ms, mem, held = _time_steps(model, opt, x, cos, sin, steps, warmup)
            res = {"ms_per_step": round(ms, 3), "overhead_pct": round(100.0 * (ms - base) / base, 2), "peak_mem_gb": round(mem / 1e9, 2),
                   "held_after_forward_gb": round(held / 1e9, 2),
                   "blocks": "".join({Decision.RESIDENT: "R", Decision.RECOMPUTE: "C"}.get(d, "O") for d in decisions)}
            if pool is not None:
                st = pool.stats()
                n = max(1, steps + warmup + 1)
                res["offloaded_gb_per_step"] = round(st["bytes_logical_out"] / n / 1e9, 3)
                res["link_gb_per_step"] = round(st["bytes_link_out"] / n / 1e9, 3)
                if st["push_rejected_full"]:      # a block that found the pool full was recomputed instead: the arm is not what it says
                    res["pushes_rejected_pool_full"] = int(st["push_rejected_full"])
                if st["spans_timed"]:      # the pool was asked to time itself: where the restores cost the step
                    res["timing_ms_per_step"] = {"offload_spans": round(st["offload_span_us"] / n / 1e3, 2),
                                                 "restore_spans": round(st["restore_span_us"] / n / 1e3, 2),
                                                 "compute_stream_waiting_for_restores": round(st["ready_wait_us"] / n / 1e3, 3)}
                if deferred_bytes:
                    res["tensors_used_in_place_per_step"] = round(st["pushes_cancelled"] / n, 1)
                    res["tensors_pushed_per_step"] = round(st["pushes"] / n, 1)
                    res["deferred_inflight_bytes"] = int(deferred_bytes)
        finally:
            model.decisions = None
            if pool is not None:
                torch.cuda.synchronize()
                ckpt.clear_activation_offload_pool()
                pool.close()
        return res

    blk = [Block(saved_bytes, fwd_ms, bwd_ms) for _ in range(blocks)]
    budget = resident_budget_blocks * saved_bytes
    if "offload_int8" in arms:
        p = plan_blocks(blk, d2h_gbs=link.d2h_gbs, h2d_gbs=link.h2d_gbs, device_budget_bytes=budget, offload=Decision.OFFLOAD_INT8)
        out["offload_int8_planned"] = run_arm("offload_int8_planned", p.decisions, OffloadCompression.INT8_B128,
                                              deferred_bytes=ISSUE_OFF_THREAD, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
        out["offload_int8_planned"]["plan_est_stall_ms"] = round(p.est_stall_ms, 2)
        out["offload_int8_planned"]["plan_est_interference_ms"] = round(p.est_interference_ms, 2)
        out["offload_int8_all"] = run_arm("offload_int8_all", [Decision.OFFLOAD_INT8] * blocks, OffloadCompression.INT8_B128)
        # overhead against how much is offloaded: the first k blocks go out, the rest stay resident
        curve = []
        for k in sorted({blocks * 2 // 5, blocks * 3 // 5, blocks * 3 // 4}):
            r = run_arm(f"int8_{k}", [Decision.OFFLOAD_INT8] * k + [Decision.RESIDENT] * (blocks - k), OffloadCompression.INT8_B128,
                        deferred_bytes=ISSUE_OFF_THREAD, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
            curve.append({"offloaded_blocks": k, "overhead_pct": r["overhead_pct"], "ms_per_step": r["ms_per_step"],
                          "held_after_forward_gb": r["held_after_forward_gb"], "offloaded_gb_per_step": r.get("offloaded_gb_per_step")})
        out["offload_int8_curve"] = curve
    if "capped" in arms:
        cap_ms = cap_pct / 100.0 * base_ms
        p = plan_blocks(blk, d2h_gbs=link.d2h_gbs, h2d_gbs=link.h2d_gbs, offload=Decision.OFFLOAD_INT8,
                        interference=CAPPED_PLAN_INTERFERENCE, overhead_cap_ms=cap_ms)
        capped_mode = OffloadCompression.INT8_B128 if Decision.OFFLOAD_INT8 in p.decisions else None
        r = run_arm("offload_int8_capped", p.decisions, capped_mode, deferred_bytes=ISSUE_OFF_THREAD, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
        if capped_mode is not None and "timed" in arms:
            # the same plan once more with the pool timing itself: where the restores cost the step (the event records
            # this takes are themselves work for the training thread, so the overhead figure is the untimed arm's)
            t = run_arm("offload_int8_capped_timed", p.decisions, capped_mode, deferred_bytes=ISSUE_OFF_THREAD,
                        d2h_piece=DEFERRED_D2H_PIECE_BYTES, collect_timing=True)
            r["timing_ms_per_step"] = t.get("timing_ms_per_step")
            r["timing_arm_ms_per_step"] = t["ms_per_step"]
        r["plan_est_ms"] = {"stall": round(p.est_stall_ms, 2), "recompute": round(p.est_recompute_ms, 2),
                            "interference": round(p.est_interference_ms, 2), "cap": round(cap_ms, 2)}
        r["plan_resident_gb"] = round(p.resident_bytes / 1e9, 3)
        out["offload_int8_capped"] = r
        out["cap_pct"], out["interference"] = cap_pct, CAPPED_PLAN_INTERFERENCE
    if "deferred" in arms or "deferred_int8" in arms:
        # Every block handed to the pool; a deferred pool sends out what the link carries beside the forward pass
        # and backward uses the rest where it is.  No plan, no budget: the link decides.
        one_block = int(saved_bytes * 0.52)
        out["offload_int8_all_deferred"] = run_arm("offload_int8_all_deferred", [Decision.OFFLOAD_INT8] * blocks,
                                                   OffloadCompression.INT8_B128, deferred_bytes=one_block, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
    if "deferred" in arms:
        out["offload_bf16_all_deferred"] = run_arm("offload_bf16_all_deferred", [Decision.OFFLOAD_BF16] * blocks,
                                                   OffloadCompression.NONE, deferred_bytes=saved_bytes, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
    if "offload_bf16" in arms:
        p = plan_blocks(blk, d2h_gbs=link.d2h_gbs, h2d_gbs=link.h2d_gbs, device_budget_bytes=budget, offload=Decision.OFFLOAD_BF16)
        out["offload_bf16_planned"] = run_arm("offload_bf16_planned", p.decisions, OffloadCompression.NONE,
                                              deferred_bytes=ISSUE_OFF_THREAD, d2h_piece=DEFERRED_D2H_PIECE_BYTES)
        out["offload_bf16_all"] = run_arm("offload_bf16_all", [Decision.OFFLOAD_BF16] * blocks, OffloadCompression.NONE)
    if "recompute" in arms:
        out["recompute"] = run_arm("recompute", [Decision.RECOMPUTE] * blocks, None)
    fused_names = ()
    if "fused" in arms:
        # The same step with RMSNorm and SwiGLU as this library's kernels (in the baseline too), which emit the codes of
        # the tensors a block saves while that block is being offloaded: three of seven tensors need no compress launch.
        global FUSED_PRODUCERS
        FUSED_PRODUCERS = True
        try:
            model.decisions = None
            f_ms, f_mem, f_held = _time_steps(model, opt, x, cos, sin, steps, warmup)
            out["resident_fused_producers"] = {"ms_per_step": round(f_ms, 3), "peak_mem_gb": round(f_mem / 1e9, 2),
                                               "held_after_forward_gb": round(f_held / 1e9, 2)}
            p = plan_blocks(blk, d2h_gbs=link.d2h_gbs, h2d_gbs=link.h2d_gbs, device_budget_bytes=budget, offload=Decision.OFFLOAD_INT8)
            out["offload_int8_planned_fused_producers"] = run_arm("offload_int8_planned_fused_producers", p.decisions, OffloadCompression.INT8_B128,
                                                                  deferred_bytes=ISSUE_OFF_THREAD, d2h_piece=DEFERRED_D2H_PIECE_BYTES, base=f_ms)
            model.decisions = None
            f_again, _, _ = _time_steps(model, opt, x, cos, sin, steps, 1)
            out["resident_fused_producers"]["ms_per_step_rerun"] = round(f_again, 3)
            fm = 0.5 * (f_ms + f_again)
            v = out["offload_int8_planned_fused_producers"]
            v["overhead_pct_vs_mean_baseline"] = round(100.0 * (v["ms_per_step"] - fm) / fm, 2)
            fused_names = ("offload_int8_planned_fused_producers",)
        finally:
            FUSED_PRODUCERS = False
    # experiments: (name, leading blocks offloaded, "int8" | "bf16", deferred_inflight_bytes, d2h_piece_bytes)
    for name, k, codec, deferred_bytes, piece, *rest in custom:
        dec = Decision.OFFLOAD_INT8 if codec == "int8" else Decision.OFFLOAD_BF16
        mode = OffloadCompression.INT8_B128 if codec == "int8" else OffloadCompression.NONE
        out[name] = run_arm(name, [dec] * k + [Decision.RESIDENT] * (blocks - k), mode, deferred_bytes=deferred_bytes, d2h_piece=piece,
                            **(rest[0] if rest else {}))
    out["resident_budget_blocks"] = resident_budget_blocks
    out["copy_piece_bytes"] = {"d2h": DEFERRED_D2H_PIECE_BYTES, "d2h_immediate_pools": COPY_PIECE_BYTES, "h2d": 2 * COPY_PIECE_BYTES}
    out["arms"] = {"planned / curve": "pool issues offloads from its own thread at once (deferred pool, unbounded in-flight budget)",
                   "all": "immediate pool: every block sent out and fetched back, as the reference's pool would",
                   "all_deferred": "deferred pool, one block in flight: sends out what the link carries beside the forward pass, the "
                                   "rest is used where it is (tensors_used_in_place_per_step)"}
    # the baseline again, last: run-to-run drift of the step time shows up as the difference to the first measurement
    model.decisions = None
    sync()
    again_ms, _, _ = _time_steps(model, opt, x, cos, sin, steps, 1)
    out["resident"]["ms_per_step_rerun"] = round(again_ms, 3)
    mean_base = 0.5 * (base_ms + again_ms)
    for k, v in list(out.items()) + [(None, c) for c in out.get("offload_int8_curve", [])]:
        if k in fused_names:
            continue
        if isinstance(v, dict) and "overhead_pct" in v:
            v["overhead_pct_vs_mean_baseline"] = round(100.0 * (v["ms_per_step"] - mean_base) / mean_base, 2)
    return out
