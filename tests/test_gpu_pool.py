"""ActivationOffloadPool on a GPU: the reference's own four tests restated, then the new modes."""
import numpy as np
import pytest
import torch

from flame_b200 import (ActivationOffloadPool, InvalidInput, InvalidOperation, OffloadCompression, PinnedAllocFlags,
                        PinnedHostBuffer, PinnedPool, StagingDeviceBuf, Unsupported, CudaError, _lib, synthetic)
from oracle import capi
from tests import gpu_util as G

pytestmark = pytest.mark.gpu
NONE, FP8, INT8B, FP8B = (OffloadCompression.NONE, OffloadCompression.FP8, OffloadCompression.INT8_B128,
                          OffloadCompression.FP8_B128)


# ---- restated from src/activation_offload.rs:843-978 ---------------------------------------------

def test_push_pull_round_trip_bf16(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 2, 1024, NONE)
    assert pool.num_slots() == 2 and pool.slot_bytes() == 1024 and pool.host_bytes() == 2048
    src = (torch.arange(32, dtype=torch.float32) * 0.125 - 1.0).to(torch.bfloat16).view(4, 8).to(cuda_device)
    truth = G.bits_of(src)
    h = pool.push(src)
    assert pool.in_flight() == 1
    pulled = pool.pull(h)
    assert pool.in_flight() == 0
    assert pulled.dtype == torch.bfloat16 and tuple(pulled.shape) == (4, 8)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(pulled), truth)


def test_push_pull_lifo_two_slots_bf16(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 2, 2048, NONE)
    a = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.bfloat16, device=cuda_device)
    b = -a
    ha, hb = pool.push(a), pool.push(b)
    assert ha.slot != hb.slot and pool.in_flight() == 2
    pb, pa = pool.pull(hb), pool.pull(ha)
    assert pool.in_flight() == 0
    torch.cuda.synchronize()
    assert torch.equal(pb, b) and torch.equal(pa, a)


def test_push_when_full_errors(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 1, 512, NONE)
    pool.push(torch.ones(8, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(InvalidOperation, match="full"):
        pool.push(torch.full((8,), 2.0, dtype=torch.bfloat16, device=cuda_device))


def test_clear_invalidates_handles(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 2, 256, NONE)
    h = pool.push(torch.full((4,), 5.0, dtype=torch.bfloat16, device=cuda_device))
    assert pool.in_flight() == 1
    pool.clear()
    assert pool.in_flight() == 0
    with pytest.raises(InvalidOperation, match="stale"):
        pool.pull(h)


# ---- remaining error cases of push/pull -----------------------------------------------------------

def test_error_cases(cuda_device):
    with pytest.raises(InvalidInput):
        ActivationOffloadPool(cuda_device, 0, 1024, NONE)
    with pytest.raises(InvalidInput):
        ActivationOffloadPool(cuda_device, 1, 0, NONE)
    pool = ActivationOffloadPool(cuda_device, 2, 1024, NONE)
    with pytest.raises(Unsupported):
        pool.push(torch.ones(4, dtype=torch.float16, device=cuda_device))
    with pytest.raises(InvalidInput, match="empty"):
        pool.push(torch.empty(0, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(InvalidInput, match="exceeds slot capacity"):
        pool.push(torch.ones(513, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(InvalidInput, match="contiguous"):
        pool.push(torch.ones(8, 8, dtype=torch.bfloat16, device=cuda_device).t()[:2])
    h = pool.push(torch.ones(4, dtype=torch.bfloat16, device=cuda_device))
    pool.pull(h)
    with pytest.raises(InvalidOperation, match="double pull"):
        pool.pull(h)
    from flame_b200.activation_offload import OffloadHandle
    with pytest.raises(InvalidOperation, match="out of range"):
        pool.pull(OffloadHandle(99, h.epoch))
    cpool = ActivationOffloadPool(cuda_device, 2, 1024, INT8B)
    with pytest.raises(Unsupported, match="only supports BF16"):
        cpool.push(torch.ones(4, dtype=torch.float32, device=cuda_device))
    assert cpool.in_flight() == 0
    # F32 passes through the uncompressed pool bit exactly
    f = torch.randn(100, device=cuda_device)
    g = pool.pull(pool.push(f))
    torch.cuda.synchronize()
    assert torch.equal(f, g)


def test_lifo_slot_reuse_and_epoch(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 3, 64, NONE)
    t = torch.ones(4, dtype=torch.bfloat16, device=cuda_device)
    h0, h1 = pool.push(t), pool.push(t)
    assert (h0.slot, h1.slot) == (0, 1) and h0.epoch == 1
    pool.pull(h0)
    assert pool.push(t).slot == 0           # freed slot is on top of the stack
    pool.clear()
    assert pool.push(t).epoch == 2


# ---- compressed modes: what is in pinned memory equals the oracle's packing ---------------------

@pytest.mark.parametrize("mode", [INT8B, FP8B, FP8, NONE])
@pytest.mark.parametrize("n,chunk", [(1000, 0), (128 * 1024 + 77, 64 << 10), (1 << 20, 256 << 10), (3 * (1 << 20) + 5, 1 << 20)])
def test_stored_bytes_and_round_trip(cuda_device, mode, n, chunk):
    bits = synthetic.normal_with_outliers(n, seed=n)
    x = G.to_dev(bits, cuda_device)
    pool = ActivationOffloadPool(cuda_device, 2, 2 * n, mode, chunk_bytes=chunk, staging_tiles=2)
    h = pool.push(x)
    info = pool.slot_info(h)
    codes, scales = pool.read_slot(h)
    if mode == INT8B:
        wc, ws = capi.quant_int8_b128(bits)
        want_out = capi.dequant_int8_b128(wc, ws)
    elif mode == FP8B:
        wc, ws = capi.quant_fp8_b128(bits)
        want_out = capi.dequant_fp8_b128(wc, ws)
    elif mode == FP8:
        s = np.float32(8.0) / np.float32(448.0)
        wc, ws = capi.bf16_to_fp8(bits, np.float32(1.0) / s), np.array([s], np.float32)
        want_out = capi.fp8_to_bf16(wc, s)
    else:
        wc, ws, want_out = bits.view(np.uint8), None, bits
    assert np.array_equal(codes, wc.view(np.uint8))
    if ws is not None:
        assert np.array_equal(scales.view(np.uint32), ws.view(np.uint32))
    if chunk and 2 * n > chunk:
        assert info["chunks"] == -(-2 * n // chunk)
    y = pool.pull(h)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(y), want_out)
    st = pool.stats()
    assert st["pushes"] == 1 and st["pulls"] == 1 and st["bytes_logical_out"] == 2 * n
    assert st["bytes_link_out"] == st["bytes_link_in"] == info["stored_bytes"]
    if mode in (INT8B, FP8B):
        assert st["bytes_link_out"] < 0.54 * 2 * n + 4096
    pool.close()


@pytest.mark.parametrize("mode", [INT8B, NONE])
def test_config1_tensor_one_round_trip_through_the_pool(cuda_device, mode):
    """[1,4096,3072] BF16, N(0,1) with 0.1 % +-U(20,60) outliers, seed 0: what lands in pinned memory is the oracle's
    packing, what comes back is the oracle's dequantisation (int8) or the source bit for bit (uncompressed)."""
    bits = synthetic.normal_with_outliers(4096 * 3072, 0)
    x = G.to_dev(bits, cuda_device).view(1, 4096, 3072)
    pool = ActivationOffloadPool(cuda_device, 1, bits.size * 2, mode, chunk_bytes=8 << 20)
    h = pool.push(x)
    codes, scales = pool.read_slot(h)
    y = pool.pull(h)
    torch.cuda.synchronize()
    assert tuple(y.shape) == (1, 4096, 3072)
    if mode == INT8B:
        wc, ws = capi.quant_int8_b128(bits)
        assert np.array_equal(codes, wc.view(np.uint8)) and np.array_equal(scales.view(np.uint32), ws.view(np.uint32))
        assert np.array_equal(G.bits_of(y).reshape(-1), capi.dequant_int8_b128(wc, ws))
        err = (y.float() - x.float()).abs().view(-1, 128).amax(dim=1)
        assert bool((err <= torch.from_numpy(ws).to(cuda_device)).all())   # |err| <= absmax/127 per block
        assert pool.slot_bytes() == 25165824 and pool.stats()["bytes_link_out"] == 12976128
    else:
        assert np.array_equal(codes.view(np.uint16), bits) and np.array_equal(G.bits_of(y).reshape(-1), bits)
    pool.close()


def test_pull_into_deferred_wait_and_source_release(cuda_device):
    n = 1 << 20
    bits = synthetic.normal(n, 1)
    x = G.to_dev(bits, cuda_device)
    pool = ActivationOffloadPool(cuda_device, 4, 2 * n, INT8B, chunk_bytes=256 << 10)
    h = pool.push(x)
    pool.synchronize()
    assert pool.source_released(h)
    dst = torch.full((n,), 7.0, dtype=torch.bfloat16, device=cuda_device)
    pool.pull_into(h, dst, defer_wait=True)
    pool.wait_ready(h.slot)
    torch.cuda.synchronize()
    wc, ws = capi.quant_int8_b128(bits)
    assert np.array_equal(G.bits_of(dst), capi.dequant_int8_b128(wc, ws))
    h = pool.push(x)                      # the same through the entry point named for it
    dst.fill_(3.0)
    pool.prefetch(h, dst)
    pool.wait_ready(h.slot)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(dst), capi.dequant_int8_b128(wc, ws)) and pool.in_flight() == 0
    with pytest.raises(InvalidInput, match="destination"):
        pool.pull_into(pool.push(x), torch.empty(n - 1, dtype=torch.bfloat16, device=cuda_device))


def test_many_tensors_reverse_order_with_slot_and_chunk_reuse(cuda_device):
    """Forward pushes, backward pulls in reverse, three 'steps' over the same small pool; destinations are
    poisoned first so a missing event edge shows up as stale bytes."""
    sizes = [70000, 8192 * 5, 300001, 128, 99999, 1 << 18]
    pool = ActivationOffloadPool(cuda_device, len(sizes), 2 * max(sizes), INT8B, chunk_bytes=64 << 10, staging_tiles=2)
    for step in range(3):
        tensors, handles = [], []
        for i, n in enumerate(sizes):
            bits = synthetic.normal_with_outliers(n, seed=100 * step + i)
            x = G.to_dev(bits, cuda_device)
            handles.append(pool.push(x))
            tensors.append(bits)
            del x                                  # the pool alone keeps the source alive until D2H completes
        outs = []
        for h, n in zip(reversed(handles), reversed(sizes)):
            dst = torch.full((n,), float("nan"), dtype=torch.bfloat16, device=cuda_device)
            pool.pull_into(h, dst)
            outs.append(dst)
        torch.cuda.synchronize()
        for dst, bits in zip(outs, reversed(tensors)):
            wc, ws = capi.quant_int8_b128(bits)
            assert np.array_equal(G.bits_of(dst), capi.dequant_int8_b128(wc, ws))
        assert pool.in_flight() == 0
    st = pool.stats()
    assert st["host_chunks_free"] == st["host_chunks_total"]


@pytest.mark.parametrize("mode", [INT8B, FP8B, NONE])
def test_random_interleaving_of_pushes_and_pulls(cuda_device, mode):
    """Seeded random schedule: pushes and pulls in any order (not only LIFO), deferred waits, a two-tile staging
    ring, chunks far smaller than the tensors, a pinned slab that is nearly full, while the compute stream is kept
    busy overwriting freed sources.  Every restore must equal the oracle's result for its own tensor."""
    rng = np.random.default_rng(2024)
    sizes = [int(v) for v in rng.integers(1000, 600000, size=24)]
    pool = ActivationOffloadPool(cuda_device, 8, 2 * max(sizes), mode, chunk_bytes=64 << 10, staging_tiles=2, tile_chunks=3,
                                 host_budget_bytes=ActivationOffloadPool.host_bytes_needed([2 * s for s in sorted(sizes)[-6:]], mode, 64 << 10))
    want = {}
    live = {}      # handle -> index
    pending = []   # (dst, index, slot, deferred)
    scratch = torch.empty(1 << 22, dtype=torch.bfloat16, device=cuda_device)
    next_i = 0
    for step in range(200):
        do_push = next_i < len(sizes) and (not live or rng.random() < 0.55)
        if do_push:
            n = sizes[next_i]
            bits = synthetic.normal_with_outliers(n, seed=3000 + next_i)
            x = G.to_dev(bits, cuda_device)
            try:
                h = pool.push(x)
            except InvalidOperation:
                do_push = False        # slab or slots full: pull something instead
            else:
                if mode == INT8B:
                    want[next_i] = capi.dequant_int8_b128(*capi.quant_int8_b128(bits))
                elif mode == FP8B:
                    want[next_i] = capi.dequant_fp8_b128(*capi.quant_fp8_b128(bits))
                else:
                    want[next_i] = bits
                live[h] = next_i
                next_i += 1
                del x
                scratch.normal_()      # the allocator may hand the freed source to this kernel
        if not do_push and live:
            h = list(live)[int(rng.integers(0, len(live)))]
            i = live.pop(h)
            dst = torch.full((sizes[i],), float("nan"), dtype=torch.bfloat16, device=cuda_device)
            deferred = bool(rng.random() < 0.5)
            pool.pull_into(h, dst, defer_wait=deferred)
            pending.append((dst, i, h.slot, deferred))
        if not live and next_i >= len(sizes):
            break
    for dst, i, slot, deferred in pending:
        if deferred:
            pool.wait_ready(slot)
    torch.cuda.synchronize()
    assert len(pending) == len(sizes)
    for dst, i, _, _ in pending:
        assert np.array_equal(G.bits_of(dst), want[i]), i
    assert pool.in_flight() == 0


# ---- deferred offload: queued tensors, cancel, hold ---------------------------------------------------

def test_deferred_offload_queue_cancel_and_hold(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 6, 1 << 20, INT8B, chunk_bytes=64 << 10, deferred_inflight_bytes=1 << 20)
    bits = [synthetic.normal_with_outliers(40000 + 1000 * i, seed=50 + i) for i in range(6)]
    want = [capi.dequant_int8_b128(*capi.quant_int8_b128(b)) for b in bits]
    xs = [G.to_dev(b, cuda_device) for b in bits]
    assert pool.cancel(pool.push(xs[0])) is None or True      # may or may not have been enqueued yet: both are legal
    pool.synchronize(10.0)
    pool.clear()
    base = pool.stats()["pushes_cancelled"]                      # 0 or 1, depending on who was faster above
    pool.hold_offloads(True)                                    # nothing is enqueued from here on
    hs = [pool.push(x) for x in xs]
    st = pool.stats()
    assert st["pushes_queued"] == 6 and pool.in_flight() == 6
    assert not pool.source_released(hs[0])
    pool.synchronize(5.0)                                       # held tensors do not count as pending work
    # cancel: the source comes back untouched, the slot and its chunks are free
    src = pool.cancel(hs[5])
    assert src is not None and src.data_ptr() == xs[5].data_ptr() and pool.in_flight() == 5
    with pytest.raises(InvalidOperation):
        pool.pull(hs[5])
    # a pull of a queued tensor sends it out at once, hold or not
    out = pool.pull(hs[4])
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(out), want[4])
    assert pool.cancel(hs[3]) is not None
    pool.discard(hs[2])                                         # a queued tensor can be discarded too
    st = pool.stats()
    assert st["pushes_cancelled"] == base + 3 and st["pushes_queued"] == 2 and pool.in_flight() == 2
    # release the hold: the rest goes out in push order
    pool.hold_offloads(False)
    pool.synchronize(10.0)
    assert pool.stats()["pushes_queued"] == 0 and pool.source_released(hs[0]) and pool.source_released(hs[1])
    assert pool.cancel(hs[0]) is None                           # too late: it is on the host now
    for i in (1, 0):
        out = pool.pull(hs[i])
        torch.cuda.synchronize()
        assert np.array_equal(G.bits_of(out), want[i])
    st = pool.stats()
    assert pool.in_flight() == 0 and st["host_chunks_free"] == st["host_chunks_total"]
    # clear() with queued tensors
    pool.hold_offloads(True)
    hs = [pool.push(x) for x in xs[:3]]
    pool.clear()
    assert pool.in_flight() == 0 and pool.stats()["pushes_queued"] == 0
    with pytest.raises(InvalidOperation):
        pool.pull(hs[0])
    pool.hold_offloads(False)
    h = pool.push(xs[0])
    out = pool.pull(h)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(out), want[0])
    pool.close()


@pytest.mark.parametrize("mode", [INT8B, NONE])
def test_deferred_random_interleaving_with_cancels(cuda_device, mode):
    """The random schedule above on a deferred pool with a small in-flight budget; a third of the restores try
    cancel() first.  A cancelled tensor must be the source itself; everything else must equal the oracle."""
    rng = np.random.default_rng(7)
    sizes = [int(v) for v in rng.integers(1000, 400000, size=32)]
    pool = ActivationOffloadPool(cuda_device, 8, 2 * max(sizes), mode, chunk_bytes=64 << 10, staging_tiles=2, tile_chunks=3,
                                 deferred_inflight_bytes=256 << 10)
    want, live, done = {}, {}, []
    next_i = cancelled = 0
    for step in range(400):
        do_push = next_i < len(sizes) and (not live or rng.random() < 0.55)
        if do_push:
            bits = synthetic.normal_with_outliers(sizes[next_i], seed=4000 + next_i)
            x = G.to_dev(bits, cuda_device)
            try:
                h = pool.push(x)
            except InvalidOperation:
                do_push = False
            else:
                want[next_i] = (bits, capi.dequant_int8_b128(*capi.quant_int8_b128(bits)) if mode == INT8B else bits)
                live[h] = next_i
                next_i += 1
                del x
        if not do_push and live:
            h = list(live)[int(rng.integers(0, len(live)))]
            i = live.pop(h)
            src = pool.cancel(h) if rng.random() < 0.34 else None
            if src is not None:
                cancelled += 1
                done.append((src, i, True))
            else:
                dst = torch.full((sizes[i],), float("nan"), dtype=torch.bfloat16, device=cuda_device)
                pool.pull_into(h, dst)
                done.append((dst, i, False))
        if step % 50 == 25:
            pool.hold_offloads(bool((step // 50) % 2))
        if not live and next_i >= len(sizes):
            break
    pool.hold_offloads(False)
    torch.cuda.synchronize()
    assert len(done) == len(sizes)
    for t, i, was_cancelled in done:
        assert np.array_equal(G.bits_of(t), want[i][0] if was_cancelled else want[i][1]), (i, was_cancelled)
    st = pool.stats()
    assert st["pushes_cancelled"] == cancelled and st["pulls"] + cancelled == st["pushes"] == len(sizes)
    assert pool.in_flight() == 0 and st["host_chunks_free"] == st["host_chunks_total"]
    pool.close()


def test_host_budget_smaller_than_slots_rejects_then_recovers(cuda_device):
    n = 1 << 18
    x = torch.randn(n, device=cuda_device).to(torch.bfloat16)
    one = _lib.lib().flame_act_packed_bytes(32768)  # pinned bytes of one 64 KiB chunk
    pool = ActivationOffloadPool(cuda_device, 8, 2 * n, INT8B, chunk_bytes=64 << 10, host_budget_bytes=one * 10)
    h = pool.push(x)                      # 8 chunks
    with pytest.raises(InvalidOperation, match="pinned slab exhausted"):
        pool.push(x)
    assert pool.in_flight() == 1 and pool.stats()["push_rejected_full"] == 1
    pool.pull(h)
    pool.pull(pool.push(x))
    torch.cuda.synchronize()


# ---- failures injected on the host --------------------------------------------------------------

def test_injected_copy_failure_returns_slot(cuda_device):
    lib = _lib.lib()
    pool = ActivationOffloadPool(cuda_device, 1, 4096, NONE)
    x = torch.ones(16, dtype=torch.bfloat16, device=cuda_device)
    lib.flame_offload_inject_fault(1, 1)   # the next copy fails with an error code
    with pytest.raises(CudaError):
        pool.push(x)
    assert pool.in_flight() == 0
    h = pool.push(x)                        # the slot went back to the free stack
    lib.flame_offload_inject_fault(1, 1)
    with pytest.raises(CudaError):
        pool.pull(h)
    assert pool.in_flight() == 1            # slot stays Pushed; a retry succeeds
    y = pool.pull(h)
    torch.cuda.synchronize()
    assert torch.equal(x, y)


def test_injected_kernel_and_alloc_failures(cuda_device):
    lib = _lib.lib()
    pool = ActivationOffloadPool(cuda_device, 1, 1 << 16, INT8B)
    x = torch.randn(1000, device=cuda_device).to(torch.bfloat16)
    lib.flame_offload_inject_fault(2, 1)
    with pytest.raises(CudaError):
        pool.push(x)
    assert pool.in_flight() == 0
    pool.pull(pool.push(x))
    lib.flame_offload_inject_fault(3, 1)
    with pytest.raises(CudaError):
        ActivationOffloadPool(cuda_device, 1, 1 << 16, NONE)
    lib.flame_offload_inject_fault(0, 1)
    torch.cuda.synchronize()


def test_deferred_offload_failure_is_reported_by_the_next_call(cuda_device):
    """A deferred offload fails on the pool's thread after push() has returned OK (host-side injection): the slot is
    marked, source_released and pull report it, the slot is given up and the pool goes on working."""
    lib = _lib.lib()
    pool = ActivationOffloadPool(cuda_device, 2, 1 << 16, INT8B, deferred_inflight_bytes=1 << 20)
    bits = synthetic.normal_with_outliers(1000, seed=1)
    x = G.to_dev(bits, cuda_device)
    for kind in (2, 1):                             # the compress launch, then a copy
        pool.hold_offloads(True)
        h = pool.push(x)                            # queued: nothing has run yet
        lib.flame_offload_inject_fault(kind, 1)
        pool.hold_offloads(False)                   # the pool's thread picks it up and hits the injected error
        pool.synchronize(10.0)
        with pytest.raises(CudaError, match="deferred offload"):
            pool.source_released(h)
        with pytest.raises(CudaError, match="deferred offload"):
            pool.pull(h)
        assert pool.in_flight() == 0
        st = pool.stats()
        assert st["host_chunks_free"] == st["host_chunks_total"]
        out = pool.pull(pool.push(x))
        torch.cuda.synchronize()
        assert np.array_equal(G.bits_of(out), capi.dequant_int8_b128(*capi.quant_int8_b128(bits)))
    lib.flame_offload_inject_fault(0, 1)
    pool.close()


def test_synchronize_times_out_instead_of_hanging(cuda_device):
    """A bounded host wait: with a long copy queued, a zero timeout reports TIMEOUT and the pool stays usable."""
    from flame_b200.errors import Timeout

    n = 1 << 27
    x = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
    pool = ActivationOffloadPool(cuda_device, 1, 2 * n, NONE)
    h = pool.push(x)
    try:
        pool.synchronize(0.0)
        finished_early = True
    except Timeout:
        finished_early = False
    pool.synchronize(60.0)
    y = pool.pull(h)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    assert finished_early in (True, False)


# ---- pinned.rs / pinned_pool.rs ---------------------------------------------------------------------

def test_pinned_alloc_and_async_copy(cuda_device):
    """tests/pinned_smoke.rs:5-37 restated, plus the read-back the reference test leaves out."""
    n = 1 << 20
    host = PinnedHostBuffer.with_capacity_elems(n, PinnedAllocFlags.WRITE_COMBINED, np.uint32)
    host.as_mut_capacity_slice()[:] = np.arange(n, dtype=np.uint32)
    host.set_len(n)
    dev = StagingDeviceBuf(cuda_device, n, np.uint32)
    stream = torch.cuda.Stream(cuda_device)
    dev.async_upload_from(host, stream)
    torch.cuda.synchronize()
    got = dev.slice().cpu().numpy().view(np.uint32)
    assert np.array_equal(got, np.arange(n, dtype=np.uint32))
    assert host.flags().contains(PinnedAllocFlags.WRITE_COMBINED) and PinnedAllocFlags().bits() == 4


def test_pinned_host_buffer_api(cuda_device):
    with pytest.raises(InvalidInput):
        PinnedHostBuffer.with_capacity_elems(0, PinnedAllocFlags.DEFAULT)
    b = PinnedHostBuffer.with_capacity_elems(16, PinnedAllocFlags.DEFAULT, np.uint8)
    assert (b.capacity(), b.capacity_bytes(), len(b)) == (16, 16, 0)
    b.copy_from_slice(np.arange(8, dtype=np.uint8))
    assert b.len_bytes() == 8 and list(b.as_slice()) == list(range(8))
    assert b.reinterpret(np.uint32).size == 2
    b.set_len(7)
    with pytest.raises(InvalidOperation):
        b.reinterpret(np.uint32)
    b.set_len(8)
    w = b.into_reinterpret(np.uint16)
    assert w.capacity() == 8 and len(w) == 4 and b.as_ptr() is None
    with pytest.raises(OverflowError):
        w.copy_from_slice(np.zeros(9, np.uint16))
    w.free()


def test_pinned_pool_size_classes_and_cache_cap(cuda_device):
    MiB = 1 << 20
    pool = PinnedPool(PinnedAllocFlags.DEFAULT, 24 * MiB)
    a = pool.checkout(1)
    assert a.capacity_bytes() == 8 * MiB and len(a) == 0
    b = pool.checkout(9 * MiB)
    assert b.capacity_bytes() == 16 * MiB
    assert pool.checkout(0).capacity_bytes() == 8 * MiB
    ptr_a = a.as_ptr()
    pool.checkin(a)
    pool.checkin(b)
    assert pool.stats() == (24 * MiB, 2)
    c = pool.checkout(8 * MiB + 1)         # smallest cached buffer that is large enough
    assert c.capacity_bytes() == 16 * MiB and pool.stats() == (8 * MiB, 1)
    d = pool.checkout(100)
    assert d.as_ptr() == ptr_a and pool.stats() == (0, 0)
    big = pool.checkout(32 * MiB)
    pool.checkin(big)                      # over the cap: freed, not cached
    assert pool.stats() == (0, 0)
    nocache = PinnedPool(PinnedAllocFlags.DEFAULT, 0)
    nocache.checkin(nocache.checkout(1))
    assert nocache.stats() == (0, 0)


def test_probe_reports_positive_rates(cuda_device):
    from flame_b200.policy import probe

    p = probe(64 << 20, 2)
    assert p.d2h_gbs > 1 and p.h2d_gbs > 1 and p.hbm_copy_gbs > 100 and p.quant_gbs > 100 and p.dequant_gbs > 100


def test_plain_c_caller_round_trips(cuda_device, tmp_path):
    """tests/helpers/abi_roundtrip.c: the reference's pool tests and an int8 round trip from a caller written in C."""
    import os
    import subprocess

    from tests.test_abi import ROOT, build_c_caller
    exe = str(tmp_path / "abi_roundtrip")
    r = build_c_caller(exe)
    assert r.returncode == 0, r.stderr
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.pathsep.join([os.path.join(ROOT, "flame_b200"), os.path.join(ROOT, "oracle"),
                                              "/usr/local/cuda/lib64", env.get("LD_LIBRARY_PATH", "")])
    env["CUDA_VISIBLE_DEVICES"] = str(cuda_device.index or 0)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and "abi_roundtrip: ok" in r.stdout, (r.stdout, r.stderr)


def test_collect_timing_reports_offload_restore_and_wait_spans(cuda_device):
    """FlameOffloadPoolConfig.collect_timing: device time of every offload, restore and wait for a restore."""
    n = 32 << 20                                        # 64 MB of BF16: a few milliseconds each way
    x = torch.randn(n, device=cuda_device).to(torch.bfloat16)
    dst = torch.empty_like(x)
    for mode in (OffloadCompression.NONE, OffloadCompression.INT8_B128):
        pool = ActivationOffloadPool(cuda_device, 4, 2 * n, mode, collect_timing=True)
        quiet = ActivationOffloadPool(cuda_device, 4, 2 * n, mode)
        try:
            for _ in range(3):
                pool.pull_into(pool.push(x), dst)                     # the wait is inside pull_into
                h = pool.push(x)
                pool.prefetch(h, dst)
                pool.wait_ready(h.slot)                               # the wait is a call of its own
                quiet.pull_into(quiet.push(x), dst)
            torch.cuda.synchronize()
            st, q = pool.stats(), quiet.stats()
            assert st["spans_pending"] == 0 and st["spans_timed"] == 3 * 2 * 3          # offload + restore + wait, six round trips
            link_ms = st["bytes_link_out"] / 6 / 63.0e9 * 1e3                           # one direction at the PCIe Gen5 x16 bound
            for key in ("offload_span_us", "restore_span_us"):
                per_trip_ms = st[key] / 6 / 1e3
                assert link_ms * 0.9 < per_trip_ms < link_ms * 20, (key, per_trip_ms, link_ms)
            # nothing else runs on the stream, so it waits for about as long as offload and restore take
            assert st["ready_wait_us"] > 0.5 * st["restore_span_us"]
            assert q["spans_timed"] == 0 and q["offload_span_us"] == 0 and q["ready_wait_us"] == 0
        finally:
            pool.close()
            quiet.close()


@pytest.mark.parametrize("mode", [INT8B, NONE])
def test_one_tensor_of_more_than_4_gib_through_the_pool(cuda_device, mode):
    """2^31 + 128 * 77 + 5 BF16 elements (4.3 GB) in one push: byte offsets beyond 32 bits in the slab, the chunk list and
    the restore.  What comes back equals the codec applied on the device without the pool (int8), or the source."""
    n = (1 << 31) + 128 * 77 + 5
    free, _ = torch.cuda.mem_get_info(cuda_device)
    if free < (30 << 30):
        pytest.skip("needs 30 GB of free device memory")
    x = torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
    g = torch.Generator(device=cuda_device).manual_seed(9)
    for lo in range(0, n, 1 << 27):
        hi = min(n, lo + (1 << 27))
        x[lo:hi] = torch.randn(hi - lo, device=cuda_device, dtype=torch.float32, generator=g).to(torch.bfloat16)
    pool = ActivationOffloadPool(cuda_device, 1, 2 * n, mode, chunk_bytes=32 << 20)
    h = pool.push(x)
    dst = torch.empty_like(x)
    pool.pull_into(h, dst)
    torch.cuda.synchronize()
    if mode == INT8B:
        codes, scales = G.quant("int8", x)
        want = G.dequant("int8", codes, scales, n)
        del codes, scales
    else:
        want = x
    assert torch.equal(dst.view(torch.int16), want.view(torch.int16))
    st = pool.stats()
    assert st["bytes_logical_out"] == 2 * n and st["bytes_link_out"] == st["bytes_link_in"]
    assert st["bytes_link_out"] == (capi.packed_bytes(n) if mode == INT8B else 2 * n)
    pool.close()
