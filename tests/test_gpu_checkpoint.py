"""checkpoint / checkpoint_offload on a GPU: gradients through the offload path equal the resident ones."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from flame_b200 import ActivationOffloadPool, InvalidOperation, OffloadCompression
from flame_b200 import checkpoint as ckpt
from flame_b200.gradient_checkpointing import CHECKPOINT_MANAGER, CheckpointPolicy
from flame_b200.policy import Decision

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    def __init__(self, d=512):
        super().__init__()
        self.norm = nn.RMSNorm(d)
        self.up = nn.Linear(d, 4 * d, bias=False)
        self.down = nn.Linear(2 * d, d, bias=False)

    def forward(self, x):
        g, u = self.up(self.norm(x)).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


def _grads(model, x, mode_per_block):
    for p in model.parameters():
        p.grad = None
    h = x.clone().requires_grad_(True)
    y = h
    for blk, mode in zip(model, mode_per_block):
        if mode == "resident":
            y = blk(y)
        elif mode == "recompute":
            y = ckpt.checkpoint([y], blk)
        else:
            y = ckpt.checkpoint_offload([y], blk, min_bytes=1 << 12)
    y.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    return [h.grad.clone()] + [p.grad.clone() for p in model.parameters()]


@pytest.fixture
def model_and_input(cuda_device):
    torch.manual_seed(0)
    model = nn.Sequential(*[Block() for _ in range(4)]).to(cuda_device, torch.bfloat16)
    x = torch.randn(2, 1024, 512, device=cuda_device, dtype=torch.bfloat16)
    yield model, x
    ckpt.clear_activation_offload_pool()


def test_uncompressed_offload_gives_bit_identical_gradients(cuda_device, model_and_input):
    model, x = model_and_input
    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.NONE, chunk_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    with pytest.raises(InvalidOperation, match="already set"):
        ckpt.set_activation_offload_pool(pool)
    for _ in range(2):  # two steps: slots and chunks are reused
        got = _grads(model, x, ["offload"] * 4)
        assert all(torch.equal(a, b) for a, b in zip(want, got))
        assert pool.in_flight() == 0
    st = pool.stats()
    assert st["pushes"] == st["pulls"] > 0
    # recompute arm and a mixed plan give the same gradients too
    assert all(torch.equal(a, b) for a, b in zip(want, _grads(model, x, ["recompute"] * 4)))
    assert all(torch.equal(a, b) for a, b in zip(want, _grads(model, x, ["offload", "recompute", "offload", "resident"])))


def test_int8_offload_gradients_are_close(cuda_device, model_and_input):
    model, x = model_and_input
    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.INT8_B128, chunk_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    got = _grads(model, x, ["offload"] * 4)
    for a, b in zip(want, got):
        rel = (a.float() - b.float()).norm() / a.float().norm().clamp_min(1e-12)
        assert rel < 0.05, float(rel)
    assert pool.stats()["bytes_link_out"] < 0.54 * pool.stats()["bytes_logical_out"] + (1 << 16)


def test_pool_exhaustion_falls_back_to_recompute(cuda_device, model_and_input, caplog):
    """A pool with too few slots: the block's handles are given back and the block is recomputed (autograd.rs:1742-1776)."""
    model, x = model_and_input
    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 2, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.NONE)
    ckpt.set_activation_offload_pool(pool)
    with caplog.at_level("WARNING"):
        got = _grads(model, x, ["offload"] * 4)
    assert any("falling back to recompute" in r.message for r in caplog.records)
    assert all(torch.equal(a, b) for a, b in zip(want, got))
    assert pool.in_flight() == 0


def test_a_graph_dropped_without_backward_gives_its_slots_back(cuda_device, model_and_input):
    model, x = model_and_input
    pool = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.INT8_B128, chunk_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    y = x.clone().requires_grad_(True)
    for blk in model:
        y = ckpt.checkpoint_offload([y], blk, min_bytes=1 << 12)
    assert pool.in_flight() > 0
    del y                      # no backward: the autograd graph and its packed entries die here
    import gc
    gc.collect()
    assert pool.in_flight() == 0
    st = pool.stats()
    assert st["host_chunks_free"] == st["host_chunks_total"]
    want = _grads(model, x, ["resident"] * 4)       # and the pool still works
    got = _grads(model, x, ["offload"] * 4)
    assert all((a.float() - b.float()).norm() / a.float().norm().clamp_min(1e-12) < 0.05 for a, b in zip(want, got))


def test_restore_arena_serves_destinations_and_gets_them_back(cuda_device, model_and_input):
    import gc

    from flame_b200.restore_arena import RestoreArena
    model, x = model_and_input
    arena = RestoreArena(cuda_device, 96 << 20)
    t = arena.empty((1000, 3), torch.bfloat16)
    assert t.shape == (1000, 3) and t.dtype == torch.bfloat16 and t.device == x.device and t.data_ptr() % 256 == 0
    t.fill_(1.5)
    v = t.view(-1)[10:20]
    del t
    gc.collect()
    assert arena.stats()["live_regions"] == 1          # a view keeps the storage, hence the region
    assert bool((v == 1.5).all())
    del v
    gc.collect()
    assert arena.stats()["live_regions"] == 0 and arena.stats()["releases"] == 1

    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.NONE, chunk_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    ckpt.set_restore_arena(arena)
    try:
        for _ in range(3):
            got = _grads(model, x, ["offload"] * 4)
            assert all(torch.equal(a, b) for a, b in zip(want, got))
        del got
        gc.collect()
        st = arena.stats()
        assert st["allocs"] > 10 and st["rejected"] == 0 and st["live_regions"] == 0 and st["in_use_bytes"] == 0
        assert st["peak_in_use_bytes"] <= st["capacity_bytes"]
        # an arena that is too small: restores fall back to fresh tensors, gradients unchanged
        small = RestoreArena(cuda_device, 1 << 20)
        ckpt.set_restore_arena(small)
        got = _grads(model, x, ["offload"] * 4)
        assert all(torch.equal(a, b) for a, b in zip(want, got))
        assert small.stats()["rejected"] > 0
    finally:
        ckpt.set_restore_arena(None)


def test_deferred_pool_uses_queued_activations_in_place(cuda_device, model_and_input):
    """A deferred pool with a tiny in-flight budget: most of the blocks' activations are still queued when backward
    reaches them and are used where they are; the rest come back from the host.  Gradients are bit-identical."""
    model, x = model_and_input
    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.NONE, chunk_bytes=1 << 20,
                                 deferred_inflight_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    for _ in range(3):
        got = _grads(model, x, ["offload"] * 4)
        assert all(torch.equal(a, b) for a, b in zip(want, got))
        assert pool.in_flight() == 0
    st = pool.stats()
    assert st["pushes_cancelled"] + st["pulls"] == st["pushes"] and st["pushes_queued"] == 0
    assert st["host_chunks_free"] == st["host_chunks_total"]
    # the same with int8: cancelled tensors are exact, restored ones quantised, so gradients are close
    ckpt.clear_activation_offload_pool()
    pool8 = ActivationOffloadPool(cuda_device, 64, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.INT8_B128, chunk_bytes=1 << 20,
                                  deferred_inflight_bytes=8 << 20)
    ckpt.set_activation_offload_pool(pool8)
    got = _grads(model, x, ["offload"] * 4)
    for a, b in zip(want, got):
        assert (a.float() - b.float()).norm() / a.float().norm().clamp_min(1e-12) < 0.05
    # a graph dropped without backward gives queued slots back as well
    y = x.clone().requires_grad_(True)
    for blk in model:
        y = ckpt.checkpoint_offload([y], blk, min_bytes=1 << 12)
    del y
    import gc
    gc.collect()
    assert pool8.in_flight() == 0


def test_without_a_pool_checkpoint_offload_is_checkpoint(cuda_device, model_and_input):
    model, x = model_and_input
    ckpt.clear_activation_offload_pool()
    want = _grads(model, x, ["resident"] * 4)
    assert all(torch.equal(a, b) for a, b in zip(want, _grads(model, x, ["offload"] * 4)))
    with torch.no_grad():
        y = ckpt.checkpoint_offload([x], model[0])      # autograd off: just runs the closure
    assert not y.requires_grad


def test_offloading_frees_device_memory(cuda_device):
    """The source of an offloaded activation is released once its device-to-host copy is done."""
    torch.manual_seed(0)
    model = nn.Sequential(*[Block(1024) for _ in range(6)]).to(cuda_device, torch.bfloat16)
    x = torch.randn(4, 2048, 1024, device=cuda_device, dtype=torch.bfloat16)

    def peak(modes):
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        _grads(model, x, modes)
        return torch.cuda.max_memory_allocated()

    resident = peak(["resident"] * 6)
    pool = ActivationOffloadPool(cuda_device, 128, 4 * 2048 * 4096 * 2, OffloadCompression.INT8_B128, chunk_bytes=4 << 20)
    ckpt.set_activation_offload_pool(pool)
    ckpt.set_prefetch_blocks(1)
    try:
        peak(["offload"] * 6)
        offloaded = peak(["offload"] * 6)
    finally:
        ckpt.set_prefetch_blocks(2)
        ckpt.clear_activation_offload_pool()
    assert offloaded < 0.8 * resident, (offloaded, resident)


def test_checkpoint_manager_cpu_offload_policy_uses_the_pool(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 4, 1 << 20, OffloadCompression.NONE)
    ckpt.set_activation_offload_pool(pool)
    try:
        CHECKPOINT_MANAGER.clear()
        CHECKPOINT_MANAGER.set_policy(CheckpointPolicy.cpu_offload())
        CHECKPOINT_MANAGER.set_device(cuda_device)
        assert CHECKPOINT_MANAGER.stats().checkpointed_tensors == 0 and CHECKPOINT_MANAGER.stats().memory_saved == 0
        t = torch.randn(1000, device=cuda_device).to(torch.bfloat16)
        CHECKPOINT_MANAGER.checkpoint_saved_tensor(7, t)
        assert pool.in_flight() == 1 and CHECKPOINT_MANAGER.stats().checkpointed_tensors == 1
        back = CHECKPOINT_MANAGER.fetch_saved(7)
        torch.cuda.synchronize()
        assert torch.equal(back, t) and CHECKPOINT_MANAGER.fetch_saved(8) is None
        assert torch.equal(CHECKPOINT_MANAGER.restore_tensor(7), t)
        with pytest.raises(InvalidOperation):
            CHECKPOINT_MANAGER.restore_tensor(7)
        CHECKPOINT_MANAGER.set_policy(CheckpointPolicy.recompute())
        CHECKPOINT_MANAGER.set_recompute_for(9, (1000,), torch.bfloat16, lambda: t * 2)
        assert torch.equal(CHECKPOINT_MANAGER.restore_tensor(9), t * 2) and CHECKPOINT_MANAGER.stats().recompute_count == 1
    finally:
        CHECKPOINT_MANAGER.clear()
        ckpt.clear_activation_offload_pool()


def test_save_and_restore_hooks_consult_the_manager_once_it_has_entries(cuda_device, model_and_input):
    """src/autograd.rs:894-907 and 1867-1892: with CHECKPOINT_HAS_ENTRIES set, every tensor a block saves is offered
    to the manager, and backward takes the manager's copy (made contiguous) where it has one."""
    from flame_b200 import gradient_checkpointing as gc_mod

    model, x = model_and_input
    want = _grads(model, x, ["resident"] * 4)
    pool = ActivationOffloadPool(cuda_device, 256, 2 * 1024 * 2048 * 2 * 2, OffloadCompression.NONE, chunk_bytes=1 << 20)
    ckpt.set_activation_offload_pool(pool)
    mgr = gc_mod.CHECKPOINT_MANAGER
    fetched, offered = [], []
    real_fetch, real_offer = mgr.fetch_saved, mgr.checkpoint_saved_tensor
    mgr.fetch_saved = lambda tid, device=None: (fetched.append(tid), real_fetch(tid, device))[1]
    mgr.checkpoint_saved_tensor = lambda tid, t: (offered.append(tid), real_offer(tid, t))[1]
    try:
        mgr.clear()
        assert gc_mod.CHECKPOINT_HAS_ENTRIES is False
        _grads(model, x, ["offload"] * 4)
        assert not offered and not fetched                     # the fast path: no entry, the manager is never asked
        mgr.set_policy(CheckpointPolicy.cpu_offload())
        marker = torch.ones(8, device=cuda_device, dtype=torch.bfloat16)
        mgr.checkpoint_saved_tensor("marker", marker)          # the first entry raises the flag
        assert gc_mod.CHECKPOINT_HAS_ENTRIES is True
        offered.clear()
        got = _grads(model, x, ["offload"] * 4)
        assert len(offered) >= 4 * 3 and set(fetched) >= set(offered)          # every saved tensor went both ways
        assert mgr.stats().checkpointed_tensors == len(set(offered)) + 1
        for a, b in zip(want, got):
            assert torch.equal(a, b)                           # the manager's copies are the same bytes
        # a tensor whose manager entry is a recompute closure comes from that closure
        mgr.clear()
        mgr.set_policy(CheckpointPolicy.recompute())
        calls = []
        h = x.clone().requires_grad_(True)
        saved_ids = []
        real_offer2 = mgr.checkpoint_saved_tensor

        def spy(tid, t):
            saved_ids.append((tid, t))
            return real_offer2(tid, t)
        mgr.set_recompute_for("marker", (8,), torch.bfloat16, lambda: marker)
        mgr.checkpoint_saved_tensor = spy
        y = ckpt.checkpoint_offload([h], model[0], min_bytes=1 << 12)
        tid0, t0 = saved_ids[0]
        keep = t0.detach().clone()
        mgr.set_recompute_for(tid0, tuple(t0.shape), t0.dtype, lambda: (calls.append(tid0), keep.clone())[1])
        y.float().pow(2).mean().backward()
        torch.cuda.synchronize()
        assert calls and all(c == tid0 for c in calls)
    finally:
        mgr.fetch_saved, mgr.checkpoint_saved_tensor = real_fetch, real_offer
        mgr.clear()
        mgr.set_policy(CheckpointPolicy.recompute())
        ckpt.clear_activation_offload_pool()
        pool.close()
