"""autograd_v4 mirror without a GPU: hook registration, tape order, what a context may hold per save mode, and the
order in which a context hands its tensors to a pool and takes them back
(src/autograd_v4/ops/sdpa.rs:48-96, 260-274; src/autograd_v4/graph.rs:12-66)."""
import threading

import pytest
import torch

from flame_b200 import autograd_v4 as v4


def _qkv(b=1, h=2, q=8, k=8, d=4):
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    return mk(b, h, q, d), mk(b, h, k, d), mk(b, h, k, d)


def test_hooks_register_once(monkeypatch):
    monkeypatch.setattr(v4, "_SDPA_HOOKS", None)
    seen = []
    hooks = v4.SdpaHooks(on_bwd_start=lambda: seen.append("bwd"))
    assert v4.register_sdpa_hooks(hooks) is True
    assert v4.register_sdpa_hooks(v4.SdpaHooks()) is False          # OnceCell::set on a full cell
    assert v4._SDPA_HOOKS is hooks
    v4._SDPA_HOOKS.on_bwd_start()
    v4._SDPA_HOOKS.on_fwd_end(v4.SdpaStats())                      # the defaults are callable no-ops
    assert seen == ["bwd"]


def test_tape_keeps_recording_order_and_is_thread_local():
    v4.clear_tape()
    q, k, v = _qkv()
    ctx = v4.SdpaCtx.from_forward(q, k, v, scale=0.5, save=v4.SdpaSave.RECOMPUTE)
    for out_id in (5, 3, 9):
        v4.record_node(v4.GradNode(out_id, (1, 2), v4.SdpaOp(ctx, 1, 2, 2)))
    assert v4._tape().order() == [5, 3, 9]
    assert v4.get_node(3).parents == (1, 2) and v4.get_node(3).op.ctx is ctx and v4.get_node(4) is None
    v4.record_node(v4.GradNode(3, (7,), v4.SdpaOp(ctx, 7, 7, 7)))   # same id again: the map entry is replaced, the order grows
    assert v4._tape().order() == [5, 3, 9, 3] and v4.get_node(3).parents == (7,)
    other = {}
    t = threading.Thread(target=lambda: other.update(order=list(v4._tape().order()), node=v4.get_node(5)))
    t.start()
    t.join()
    assert other == {"order": [], "node": None}                     # another thread has its own tape
    v4.clear_tape()
    assert v4._tape().order() == [] and v4.get_node(5) is None


def test_context_holds_what_its_save_mode_says():
    q, k, v = _qkv()
    probs = torch.zeros(1, 2, 8, 8, dtype=torch.bfloat16)
    lse = torch.zeros(1, 2, 8, 1, dtype=torch.float32)
    a = v4.SdpaCtx.from_forward(q, k, v, scale=1.0, save=v4.SdpaSave.SAVE_PROBS, probs=probs)
    b = v4.SdpaCtx.from_forward(q, k, v, scale=1.0, save=v4.SdpaSave.SAVE_LSE, lse=lse, causal=True)
    c = v4.SdpaCtx.from_forward(q, k, v, scale=1.0, save=v4.SdpaSave.RECOMPUTE)
    assert a.shapes == b.shapes == c.shapes == (1, 2, 8, 8) and b.causal and not a.causal
    assert a.saved_bytes() == 3 * 64 * 2 + 128 * 2 and b.saved_bytes() == 3 * 64 * 2 + 16 * 4 and c.saved_bytes() == 3 * 64 * 2
    for bad in (dict(save=v4.SdpaSave.SAVE_PROBS), dict(save=v4.SdpaSave.SAVE_PROBS, probs=probs.float()),
                dict(save=v4.SdpaSave.SAVE_PROBS, probs=probs, lse=lse), dict(save=v4.SdpaSave.SAVE_LSE, lse=lse.view(1, 2, 8)),
                dict(save=v4.SdpaSave.SAVE_LSE, probs=probs), dict(save=v4.SdpaSave.RECOMPUTE, lse=lse)):
        with pytest.raises(ValueError):
            v4.SdpaCtx.from_forward(q, k, v, scale=1.0, **bad)


class _ListPool:
    """Stand-in with the pool's two calls: a stack of slots, last in first out."""

    def __init__(self, compression=0):
        self.compression, self.log, self._held = compression, [], {}

    def push(self, t):
        h = len(self.log)
        self.log.append(("push", tuple(t.shape), t.dtype))
        self._held[h] = t.clone()
        return h

    def pull(self, h):
        self.log.append(("pull", h))
        return self._held.pop(h)


@pytest.mark.parametrize("compressed", [False, True])
def test_offload_pushes_in_field_order_and_restore_pulls_in_reverse(compressed):
    q, k, v = _qkv()
    lse = torch.arange(16, dtype=torch.float32).view(1, 2, 8, 1)
    ctx = v4.SdpaCtx.from_forward(q, k, v.transpose(2, 3).contiguous().transpose(2, 3), scale=1.0, save=v4.SdpaSave.SAVE_LSE, lse=lse)
    want = {n: getattr(ctx, n).clone() for n in ("q", "k", "v", "lse")}
    pool = _ListPool(2 if compressed else 0)
    moved = ctx.offload(pool)
    # v is not contiguous and stays; the FP32 log-sum-exp leaves only through an uncompressed pool
    assert ctx.q is None and ctx.k is None and ctx.v is not None and (ctx.lse is None) == (not compressed)
    assert moved == 2 * 64 * 2 + (0 if compressed else 16 * 4)
    n_push = 2 if compressed else 3
    assert [e[0] for e in pool.log] == ["push"] * n_push
    ctx.restore(pool)
    assert pool.log[n_push:] == [("pull", h) for h in reversed(range(n_push))]
    for n, w in want.items():
        assert torch.equal(getattr(ctx, n), w)
    assert not ctx._handles
