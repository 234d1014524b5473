"""autograd_v4 contexts through a real pool: every save mode, offloaded and restored in reverse, compared bit for bit
(uncompressed) or against the CPU oracle (int8 per 128)."""
import numpy as np
import pytest
import torch

from flame_b200 import ActivationOffloadPool, OffloadCompression
from flame_b200 import autograd_v4 as v4
from oracle import capi
from tests import gpu_util as G

pytestmark = pytest.mark.gpu
B, H, Q, K, D = 2, 4, 256, 384, 64


def _forward(dev, save):
    """What sdpa_forward computes and keeps (sdpa.rs:225-274), with the attention arithmetic left to torch."""
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(B, H, Q, D, device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, K, D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, K, D, device=dev, generator=g).to(torch.bfloat16)
    scale = D ** -0.5
    logits = (q.float() @ k.float().transpose(-1, -2)) * scale
    lse = torch.logsumexp(logits, dim=-1, keepdim=True)
    probs = torch.exp(logits - lse)
    kw = {v4.SdpaSave.SAVE_PROBS: dict(probs=probs.to(torch.bfloat16).contiguous()), v4.SdpaSave.SAVE_LSE: dict(lse=lse.contiguous()),
          v4.SdpaSave.RECOMPUTE: {}}[save]
    return v4.SdpaCtx.from_forward(q, k, v, scale=scale, save=save, **kw)


def _bits(t):
    return t.contiguous().view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32).cpu().numpy()


@pytest.mark.parametrize("save", list(v4.SdpaSave))
def test_context_round_trip_is_bit_exact_through_an_uncompressed_pool(cuda_device, save):
    ctx = _forward(cuda_device, save)
    names = [n for n in v4.SdpaCtx._OFFLOADABLE if getattr(ctx, n) is not None]
    assert names == {"SaveProbs": ["q", "k", "v", "probs"], "SaveLSE": ["q", "k", "v", "lse"], "Recompute": ["q", "k", "v"]}[save.value]
    want = {n: _bits(getattr(ctx, n)) for n in names}
    held = ctx.saved_bytes()
    pool = ActivationOffloadPool(cuda_device, 4, B * H * Q * K * 2, OffloadCompression.NONE, chunk_bytes=1 << 20)
    try:
        assert ctx.offload(pool) == held and ctx.saved_bytes() == 0 and pool.in_flight() == len(names)
        assert all(getattr(ctx, n) is None for n in names)
        ctx.restore(pool)
        torch.cuda.synchronize()
        assert pool.in_flight() == 0 and ctx.saved_bytes() == held
        for n in names:
            t = getattr(ctx, n)
            assert tuple(t.shape) == {"q": (B, H, Q, D), "k": (B, H, K, D), "v": (B, H, K, D), "probs": (B, H, Q, K), "lse": (B, H, Q, 1)}[n]
            assert np.array_equal(_bits(t), want[n]), n
        st = pool.stats()
        assert st["pushes"] == st["pulls"] == len(names)
    finally:
        pool.close()


@pytest.mark.parametrize("save", list(v4.SdpaSave))
def test_context_through_an_int8_pool_equals_the_oracle(cuda_device, save):
    ctx = _forward(cuda_device, save)
    bf16 = [n for n in ("q", "k", "v", "probs") if getattr(ctx, n) is not None]
    src = {n: G.bits_of(getattr(ctx, n)).reshape(-1) for n in bf16}
    lse_before = None if ctx.lse is None else _bits(ctx.lse)
    pool = ActivationOffloadPool(cuda_device, 4, B * H * Q * K * 2, OffloadCompression.INT8_B128, chunk_bytes=1 << 20)
    try:
        moved = ctx.offload(pool)
        assert moved == sum(2 * s.size for s in src.values()) and pool.in_flight() == len(bf16)
        assert (ctx.lse is None) == (lse_before is None)          # the FP32 log-sum-exp never enters a compressed pool
        ctx.restore(pool)
        torch.cuda.synchronize()
        for n in bf16:
            wc, ws = capi.quant_int8_b128(src[n])
            assert np.array_equal(G.bits_of(getattr(ctx, n)).reshape(-1), capi.dequant_int8_b128(wc, ws)), n
        if lse_before is not None:
            assert np.array_equal(_bits(ctx.lse), lse_before)
        assert pool.in_flight() == 0
    finally:
        pool.close()


def test_contexts_on_a_tape_restore_in_reverse_recording_order(cuda_device):
    """Three attention calls recorded on the tape and offloaded as they are recorded; backward walks the tape in
    reverse and restores each context when it reaches it: the pool's slot stack is used last in, first out."""
    v4.clear_tape()
    pool = ActivationOffloadPool(cuda_device, 16, B * H * Q * K * 2, OffloadCompression.NONE, chunk_bytes=1 << 20)
    try:
        want = {}
        for out_id, save in zip((11, 12, 13), v4.SdpaSave):
            ctx = _forward(cuda_device, save)
            want[out_id] = {n: _bits(getattr(ctx, n)) for n in v4.SdpaCtx._OFFLOADABLE if getattr(ctx, n) is not None}
            ctx.offload(pool)
            v4.record_node(v4.GradNode(out_id, (1, 2, 3), v4.SdpaOp(ctx, 1, 2, 3)))
        assert pool.in_flight() == 4 + 4 + 3
        for out_id in reversed(v4._tape().order()):
            node = v4.get_node(out_id)
            node.op.ctx.restore(pool)
            torch.cuda.synchronize()
            for n, w in want[out_id].items():
                assert np.array_equal(_bits(getattr(node.op.ctx, n)), w), (out_id, n)
        assert pool.in_flight() == 0
    finally:
        v4.clear_tape()
        pool.close()
