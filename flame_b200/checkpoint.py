"""Save / restore hooks: ``checkpoint`` and ``checkpoint_offload``.

Mirror of the hooks in the reference's tape engine:

* ``set_activation_offload_pool``      <- src/autograd.rs:63-74 (global pool, set once)
* ``checkpoint(inputs, f)``            <- src/autograd.rs:1584-1647 + the ``Op::Checkpoint`` arm, 2271-2435
  (forward without a tape, recompute in backward)
* ``checkpoint_offload(inputs, f)``    <- src/autograd.rs:1659-1798 + the ``Op::CheckpointOffload`` arm, 2437-2510
  (forward once with the tape on, every saved BF16 activation pushed to the pool,
  pulled back in reverse during backward; no pool -> ``checkpoint``; pool full
  mid-block -> handles given back and the block falls back to ``checkpoint``)

The tape here is PyTorch's: ``torch.autograd.graph.saved_tensors_hooks`` sees
every tensor an op saves for backward, which is what the reference walks in
``sub_tape[*].saved_tensors``.  Because a Python closure cannot be re-run on
detached inputs the way the Rust closure is re-run on tensor ids, ``f`` takes the
inputs as arguments: ``f(*inputs)``.

One thing is added on top of the reference's just-in-time pulls (its restore sits
on the critical path, src/autograd.rs:2470-2479): blocks register in forward
order, and when backward first touches block k the restores of block k-1 are
issued into freshly allocated destinations (``pull_into`` with a deferred wait),
so the host link works one block ahead of the VJPs.
"""
from __future__ import annotations

import logging
import weakref
from typing import Callable, Optional, Sequence

import torch
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from . import fused_producers
from .activation_offload import ActivationOffloadPool, OffloadCompression
from .errors import InvalidInput, InvalidOperation, OffloadError
from .policy import Decision

log = logging.getLogger("flame_b200.checkpoint")

_ACTIVATION_POOL: Optional[ActivationOffloadPool] = None


def set_activation_offload_pool(pool: ActivationOffloadPool) -> None:
    """Install the pool ``checkpoint_offload`` uses.  Once; a second call is an error (autograd.rs:70-74)."""
    global _ACTIVATION_POOL
    if _ACTIVATION_POOL is not None:
        raise InvalidOperation("Activation offload pool already set")
    _ACTIVATION_POOL = pool


def clear_activation_offload_pool() -> None:
    """Uninstall the pool (the reference's OnceLock cannot be reset; tests and benchmarks need to)."""
    global _ACTIVATION_POOL
    _SCHEDULER.reset()       # while the pool is still installed: a deferred pool is released from its hold
    _ACTIVATION_POOL = None


def activation_offload_pool() -> Optional[ActivationOffloadPool]:
    return _ACTIVATION_POOL


_RESTORE_ARENA = None
_BATCHED_CODEC = False


def set_batched_codec(on: bool) -> None:
    """Per-128-block pools: compress a block's saved tensors with one launch when its forward ends and expand them
    with one launch when its backward begins (the pool then moves compressed bytes only, `push_packed` /
    `pull_packed`), instead of one launch per tensor and staging tile inside the pool."""
    global _BATCHED_CODEC
    _BATCHED_CODEC = bool(on)


def set_restore_arena(arena) -> None:
    """Restored activations are written into `arena` (a RestoreArena made on the stream backward runs on) instead
    of freshly allocated tensors (src/activation_offload.rs:655); None switches back.  When the arena has no
    released space next in its ring, the restore falls back to a fresh tensor."""
    global _RESTORE_ARENA
    _RESTORE_ARENA = arena


def _destination(shape, dtype, device) -> torch.Tensor:
    if _RESTORE_ARENA is not None:
        t = _RESTORE_ARENA.empty(shape, dtype)
        if t is not None:
            return t
    return torch.empty(shape, dtype=dtype, device=device)


def checkpoint(inputs: Sequence[torch.Tensor], f: Callable[..., torch.Tensor]) -> torch.Tensor:
    """Recompute arm: run ``f(*inputs)`` without saving activations, re-run it in backward."""
    if not inputs:
        raise InvalidInput("checkpoint requires at least one input")
    if not torch.is_grad_enabled():
        return f(*inputs)
    return _torch_checkpoint(f, *inputs, use_reentrant=False)


def dense_permutation(t: torch.Tensor):
    """Permutation p with ``t.permute(p)`` contiguous, or None.

    A saved tensor is often a transposed view of dense memory (attention inputs in [B,H,T,D]
    order over [B,T,H,D] storage).  The pool moves flat contiguous memory, so such a view is
    offloaded through its contiguous permutation and re-viewed after the restore.
    """
    if t.is_contiguous():
        return tuple(range(t.dim()))
    perm = tuple(sorted(range(t.dim()), key=lambda d: (-t.stride(d), d)))
    return perm if t.permute(perm).is_contiguous() else None


def offloadable(t: torch.Tensor, min_bytes: int) -> bool:
    """The rule of src/autograd.rs:1721-1725 (BF16 activations that require grad), plus: on the GPU,
    not a parameter, not tiny, and backed by dense memory."""
    if isinstance(t, torch.nn.Parameter) or isinstance(getattr(t, "_base", None), torch.nn.Parameter):
        return False  # weights and views of weights (a linear saves weight.t()) are not activations
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.requires_grad
            and t.numel() * 2 >= min_bytes and dense_permutation(t) is not None)


def saved_bytes_of(f: Callable[..., torch.Tensor], inputs: Sequence[torch.Tensor], min_bytes: int = 1 << 20) -> int:
    """BF16 bytes ``checkpoint_offload(inputs, f)`` would push: a dry run of ``f`` with counting hooks."""
    seen, total = {}, 0

    def pack(t):
        nonlocal total
        if offloadable(t, min_bytes):
            key = (t.data_ptr(), t.numel(), t._version)
            if key not in seen:
                seen[key] = t          # held, so that its address cannot be given to another tensor during the run
                total += t.numel() * 2
        return t

    with torch.enable_grad(), torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        f(*inputs)
    return total


class _Entry:
    """One offloaded saved tensor (OffloadedTapeEntry's handle plus what restore needs)."""

    __slots__ = ("handle", "shape", "dtype", "restored", "waited", "block", "packed", "__weakref__")

    def __init__(self, handle, shape, dtype, block):
        self.handle, self.shape, self.dtype, self.block = handle, shape, dtype, block
        self.restored = None
        self.waited = False
        self.packed = None      # (codes, scales) on the device while a batched restore waits to be expanded

    def __del__(self):
        # The graph was dropped without a backward pass (an evaluation step, an exception): the
        # slot must not stay Pushed for ever.
        if self.restored is None and self.packed is None and self.handle is not None:
            try:
                self.block.pool.discard(self.handle)
            except Exception:
                pass


def _manager():
    """The legacy side channel (gradient_checkpointing.CHECKPOINT_MANAGER), or None while it holds no entry.

    The reference consults its manager for every saved tensor behind one relaxed atomic load
    (src/autograd.rs:894-907 when an op is recorded, 1867-1880 when backward fetches a saved tensor); the flag is
    False until an entry exists, so a step that never uses the manager pays one attribute read per saved tensor."""
    from . import gradient_checkpointing as gc_mod   # imported late: that module imports this one

    return gc_mod if gc_mod.CHECKPOINT_HAS_ENTRIES else None


class _Managed:
    """A saved tensor that was also handed to the legacy manager when it was recorded."""

    __slots__ = ("tid", "inner")

    def __init__(self, tid, inner):
        self.tid, self.inner = tid, inner


class _View:
    """A saved tensor that is a reshaped and/or permuted view of an offloaded entry's flat memory."""

    __slots__ = ("entry", "shape", "inverse")

    def __init__(self, entry, shape, inverse):
        self.entry, self.shape, self.inverse = entry, shape, inverse


class _Block:
    """The offloaded sub-tape of one ``checkpoint_offload`` call."""

    def __init__(self, pool: ActivationOffloadPool, index: int, min_bytes: int):
        self.pool, self.index, self.min_bytes = pool, index, min_bytes
        # weak: an entry, and the restored tensor it caches, must die as soon as the last
        # graph node that saved it has run its backward
        self.entries: list = []
        self._by_key: dict = {}
        self._handles: list = []
        self.failed = False
        self.bytes_offloaded = 0
        self.restores_issued = False
        # per-128-block pools: producers that can emit codes beside their output do so while this block runs
        self.emit = int(pool.compression) if pool.compression in (OffloadCompression.INT8_B128, OffloadCompression.FP8_B128) else 0
        # batched codec: the block's tensors are compressed by ONE launch when its forward ends and expanded by ONE
        # launch when its backward begins, instead of one small launch per tensor and staging tile inside the pool
        self.batch = bool(self.emit) and _BATCHED_CODEC
        self._pending: list = []    # (entry, contiguous source) waiting for that one compress launch

    # -- forward -----------------------------------------------------------------------------
    def pack(self, t: torch.Tensor):
        inner = self._pack(t)
        mgr = _manager()
        if mgr is None:
            return inner
        # src/autograd.rs:894-907: with entries present, every saved tensor of a recorded op is offered to the
        # manager (which keeps it under its CPUOffload policy and ignores it otherwise); the tape keeps its own
        tid = mgr.tensor_id(t)
        with mgr.CHECKPOINT_MANAGER_LOCK:
            mgr.CHECKPOINT_MANAGER.checkpoint_saved_tensor(tid, t)
        return _Managed(tid, inner)

    def _pack(self, t: torch.Tensor):
        # Only BF16 activations that take part in the gradient are offloaded; weights, non-BF16
        # tensors and small tensors stay resident (autograd.rs:1721-1739).
        if self.failed or not offloadable(t, self.min_bytes):
            # A tensor that stays resident is kept detached: autograd hands the hook tensors with their
            # grad_fn, and a saved OUTPUT held that way (attention's log-sum-exp, a norm's 1/rms) would keep
            # its own node alive for ever if the graph is dropped without a backward pass.
            return t.detach() if t.grad_fn is not None else t
        perm = dense_permutation(t)
        inverse = tuple(perm.index(d) for d in range(t.dim()))
        base = t.permute(perm)  # contiguous view of the same memory
        # the same memory is often saved several times under different shapes (a norm output
        # and its 2-D view in the following linear): one offload, many views
        key = (t.data_ptr(), t.numel(), t._version)
        hit = self._by_key.get(key)
        if hit is not None:
            return _View(hit[0], tuple(base.shape), inverse)
        try:
            pre = fused_producers.take(t) if self.emit else None
            if pre is None and self.batch:
                e = _Entry(None, (t.numel(),), t.dtype, self)      # pushed by finish_forward, with the rest of the block
                self.entries.append(weakref.ref(e))
                self._by_key[key] = (e, base)
                self._pending.append((e, base))
                self.bytes_offloaded += t.numel() * 2
                return _View(e, tuple(base.shape), inverse)
            # a producer with the compress step built in already wrote this tensor's codes: no compress launch
            h = self.pool.push_packed(pre[0], pre[1], (t.numel(),)) if pre is not None else self.pool.push(base)
        except OffloadError as exc:  # pool exhausted: abandon offload for this block
            log.warning("checkpoint_offload: pool push failed (%s), falling back to recompute; %d handles already pushed",
                        exc, len(self.entries))
            self.failed = True
            return t.detach() if t.grad_fn is not None else t
        e = _Entry(h, (t.numel(),), t.dtype, self)
        self.entries.append(weakref.ref(e))
        # The source is held until the block's forward ends: if it were freed earlier (the pool lets go of it once
        # it has been copied out), the allocator could give its address to another tensor of the same size, which
        # would then be taken for a view of this one.
        self._by_key[key] = (e, base)
        self._handles.append(h)
        self.bytes_offloaded += t.numel() * 2
        return _View(e, tuple(base.shape), inverse)

    def finish_forward(self) -> None:
        if self._pending and not self.failed:
            try:
                self._compress_pending()
            except OffloadError as exc:
                log.warning("checkpoint_offload: pool push failed (%s), falling back to recompute", exc)
                self.failed = True
        self._pending = []
        self._by_key.clear()

    def _compress_pending(self) -> None:
        """One compress launch for every tensor of the block that no producer compressed, then their pushes."""
        from . import _lib
        lib = _lib.lib()
        dev = self.pool.device
        bufs = []
        for e, base in self._pending:
            n = base.numel()
            bufs.append((torch.empty(n, dtype=torch.uint8, device=dev), torch.empty((n + 127) // 128, dtype=torch.float32, device=dev)))
        arr = (_lib.ActTensor * len(bufs))(*[_lib.ActTensor(base.data_ptr(), c.data_ptr(), s_.data_ptr(), base.numel())
                                             for (e, base), (c, s_) in zip(self._pending, bufs)])
        rc = lib.flame_act_quant_b128_multi(self.emit, arr, len(bufs), 0, torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise OffloadError(f"flame_act_quant_b128_multi failed ({rc}): {_lib.last_error()}")
        for (e, base), (c, s_) in zip(self._pending, bufs):
            e.handle = self.pool.push_packed(c, s_, (base.numel(),))
            self._handles.append(e.handle)

    def abandon(self) -> None:
        handles, self._handles = self._handles, []
        for h in handles:
            try:
                self.pool.discard(h)
            except OffloadError:
                pass
        # the entries must not discard these handles a second time when they die: a (slot, epoch) pair is not
        # unique per push, and by then the slot may hold another tensor
        for ref in self.entries:
            e = ref()
            if e is not None:
                e.handle = None
        self.entries.clear()

    # -- backward ------------------------------------------------------------------------------
    def issue_restores(self) -> None:
        """Start the restore of every entry that has not been started yet (deferred wait)."""
        self.restores_issued = True
        for ref in reversed(self.entries):
            e = ref()
            if e is not None and e.restored is None and e.packed is None:
                self._restore(e)

    def _restore(self, e: "_Entry") -> None:
        # A deferred pool may not have started this tensor's offload yet: then it never left the device and is
        # used where it is, instead of being sent out and fetched back while backward waits.
        src = self.pool.cancel(e.handle)
        if src is not None:
            e.restored = src.reshape(e.shape)
            e.waited = True
            return
        if self.batch:     # the compressed form comes back now; it is expanded with the rest of the block, when first needed
            n = e.shape[0]
            codes = torch.empty(n, dtype=torch.uint8, device=self.pool.device)
            scales = torch.empty((n + 127) // 128, dtype=torch.float32, device=self.pool.device)
            self.pool.pull_packed(e.handle, codes, scales, defer_wait=True)
            e.packed = (codes, scales)
            return
        dst = _destination(e.shape, e.dtype, self.pool.device)
        self.pool.pull_into(e.handle, dst, defer_wait=True)
        e.restored = dst

    def _expand(self) -> None:
        """One dequantise launch for every entry of the block whose compressed form has come back."""
        from . import _lib
        live = [e for e in (r() for r in self.entries) if e is not None and e.packed is not None and e.restored is None]
        if not live:
            return
        for e in live:
            self.pool.wait_ready(e.handle.slot)
        dsts = [_destination(e.shape, e.dtype, self.pool.device) for e in live]
        arr = (_lib.ActTensor * len(live))(*[_lib.ActTensor(d.data_ptr(), e.packed[0].data_ptr(), e.packed[1].data_ptr(), d.numel())
                                             for e, d in zip(live, dsts)])
        rc = _lib.lib().flame_act_dequant_b128_multi(self.emit, arr, len(live), torch.cuda.current_stream(self.pool.device).cuda_stream)
        if rc != 0:
            raise OffloadError(f"flame_act_dequant_b128_multi failed ({rc}): {_lib.last_error()}")
        for e, d in zip(live, dsts):
            e.restored, e.waited, e.packed = d, True, None

    def unpack(self, obj):
        if isinstance(obj, _Managed):
            # src/autograd.rs:1867-1892: the manager's copy wins when it has one, and whatever comes back is made
            # contiguous; otherwise the tape's own saved tensor is used
            mgr = _manager()
            if mgr is not None:
                with mgr.CHECKPOINT_MANAGER_LOCK:
                    r = mgr.CHECKPOINT_MANAGER.fetch_saved(obj.tid)
                if r is not None:
                    return r if r.is_contiguous() else r.contiguous()
            return self.unpack(obj.inner)
        if isinstance(obj, _View):
            return self.unpack(obj.entry).view(obj.shape).permute(obj.inverse)
        if not isinstance(obj, _Entry):
            return obj
        if not self.restores_issued:   # the output-gradient hook normally got here first
            _SCHEDULER.on_backward_reach(self.index)
            if not self.restores_issued:
                self.issue_restores()
        if obj.restored is None and obj.packed is None:  # pushed after the block's restores were issued: cannot happen, but stay correct
            self._restore(obj)
        if obj.restored is None and obj.packed is not None:
            self._expand()
        if not obj.waited:
            self.pool.wait_ready(obj.handle.slot)
            obj.waited = True
        return obj.restored


class _Scheduler:
    """Keeps the checkpointed blocks of the current step in forward order and, as backward walks them in
    reverse, issues the restores of the offloaded blocks a few positions ahead of the VJPs."""

    def __init__(self):
        self.blocks: list = []      # per checkpoint_offload call of the step: weakref to its _Block, or None (resident / recompute)
        self.prefetch_blocks = 2
        self._backward_seen = False

    def reset(self):
        self.blocks.clear()
        if self._backward_seen:
            self._hold(False)
        self._backward_seen = False

    @staticmethod
    def _hold(on: bool) -> None:
        # deferred pools: nothing new goes out once the DEVICE has finished the forward pass (the host is ahead of
        # it when it gets here); what is still queued when backward reaches it is used in place
        pool = _ACTIVATION_POOL
        if pool is not None and getattr(pool, "deferred", False):
            try:
                if on:
                    pool.hold_offloads_after_current_work()
                else:
                    pool.hold_offloads(False)
            except OffloadError:
                pass

    def register(self, block: Optional[_Block]) -> int:
        if self._backward_seen:     # first forward call after a backward: a new step begins
            self.reset()
        self.blocks.append(weakref.ref(block) if block is not None else None)
        return len(self.blocks) - 1

    def on_backward_reach(self, position: int) -> None:
        """Backward is about to run the block registered at `position`."""
        if not self._backward_seen:
            self._hold(True)
        self._backward_seen = True
        # Sources whose copy out has finished are let go as backward proceeds (the pool itself only looks when
        # something is pushed, and nothing is pushed during backward): their memory is there for the gradients.
        pool = _ACTIVATION_POOL
        if pool is not None:
            try:
                pool.release_finished_sources()
            except OffloadError:
                pass
        for j in range(min(position, len(self.blocks) - 1), max(-1, position - 1 - self.prefetch_blocks), -1):
            ref = self.blocks[j]
            blk = ref() if ref is not None else None
            if blk is not None and not blk.restores_issued:
                blk.issue_restores()


_SCHEDULER = _Scheduler()


def set_prefetch_blocks(n: int) -> None:
    """How many block positions ahead of the VJPs restores are issued (0 = just in time, as the reference)."""
    _SCHEDULER.prefetch_blocks = max(0, int(n))


def checkpoint_offload(inputs: Sequence[torch.Tensor], f: Callable[..., torch.Tensor], *,
                       decision: Decision = Decision.OFFLOAD_INT8, min_bytes: int = 1 << 20) -> torch.Tensor:
    """Offload arm.  ``decision`` comes from the policy: RESIDENT runs ``f`` plainly, RECOMPUTE uses ``checkpoint``,
    any OFFLOAD_* value pushes the block's saved activations to the installed pool (whose own compression applies)."""
    if not inputs:
        raise InvalidInput("checkpoint_offload requires at least one input")
    pool = _ACTIVATION_POOL
    if pool is None or decision == Decision.RECOMPUTE:
        return checkpoint(inputs, f)
    if not torch.is_grad_enabled():
        return f(*inputs)
    if decision == Decision.RESIDENT:
        out = f(*inputs)
        if out.requires_grad:  # a resident block still tells the scheduler where backward is
            pos = _SCHEDULER.register(None)
            out.register_hook(lambda g, pos=pos: _SCHEDULER.on_backward_reach(pos))
        return out
    block = _Block(pool, len(_SCHEDULER.blocks), min_bytes)
    with torch.autograd.graph.saved_tensors_hooks(block.pack, block.unpack), fused_producers.emit_codes(block.emit):
        out = f(*inputs)
    block.finish_forward()
    if block.failed:
        log.warning("checkpoint_offload: falling back to recompute checkpoint (pool exhausted after %d tensors)", len(block.entries))
        block.abandon()
        del out
        return checkpoint(inputs, f)
    block.index = _SCHEDULER.register(block)  # the autograd graph keeps the block alive through the unpack hook
    if out.requires_grad:
        out.register_hook(lambda g, pos=block.index: _SCHEDULER.on_backward_reach(pos))
    return out
