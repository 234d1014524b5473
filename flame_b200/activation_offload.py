"""ActivationOffloadPool: mirror of src/activation_offload.rs:323-760.

Same constructor arguments, accessors, ``push`` / ``pull`` / ``clear`` and
error cases as the reference; the work happens in libflame_offload.so
(flame_offload_pool_*).  Tensors are torch CUDA tensors; only their data
pointer, element count and dtype cross the C ABI.

Differences from the reference, all additive:

* two more compression modes, ``INT8_B128`` and ``FP8_B128`` (per-128-element
  fp32 scales), next to ``NONE`` and the fixed-scale ``FP8``;
* ``pull_into`` restores into a tensor the caller already owns, optionally
  without making the current stream wait (``defer_wait``) so that a restore can
  be issued ahead of its consumer and joined later with ``wait_ready``;
* a non-contiguous source is refused (the reference copies from the storage
  base pointer and ignores view offsets, src/activation_offload.rs:771-800);
* the pool keeps the source tensor alive only until its device-to-host copy
  has finished (the reference holds it until pull,
  src/activation_offload.rs:600-605), so offloading actually frees device memory.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _lib
from .errors import (CudaError, InvalidInput, InvalidOperation, OffloadError, Timeout,  # noqa: F401
                     Unsupported, raise_for_status)


class OffloadCompression(enum.IntEnum):
    """src/activation_offload.rs:89-96 plus the two per-block codecs."""

    NONE = 0
    FP8 = 1          # reference mode: fixed per-tensor scale 8/448
    INT8_B128 = 2
    FP8_B128 = 3


@dataclass(frozen=True)
class OffloadHandle:
    """Copyable ticket returned by push (src/activation_offload.rs:292-303)."""

    slot: int
    epoch: int

    def _c(self) -> _lib.Handle:
        return _lib.Handle(self.slot, self.epoch)


def _dtype_tag(t) -> int:
    import torch

    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise Unsupported(f"ActivationOffloadPool::push: dtype {t.dtype} not supported (BF16/F32 only)")


class _Prepacked:
    """Keep-alive record of a tensor pushed in compressed form: its device codes and scales."""

    __slots__ = ("codes", "scales", "numel", "shape")

    def __init__(self, codes, scales, numel, shape):
        self.codes, self.scales, self.numel, self.shape = codes, scales, numel, shape


class ActivationOffloadPool:
    def __init__(self, device, num_slots: int, max_bytes: int,
                 compression: OffloadCompression = OffloadCompression.NONE, *,
                 chunk_bytes: int = 0, staging_tiles: int = 0, codec_flags: int = 0,
                 host_budget_bytes: int = 0, host_alloc_flags: int = 0, codec_max_ctas: int = 0,
                 numa_node: int = -2, tile_chunks: int = 0, d2h_piece_bytes: int = 0, h2d_piece_bytes: int = 0,
                 deferred_inflight_bytes: int = 0, collect_timing: bool = False):
        import torch

        self._torch = torch
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise Unsupported("ActivationOffloadPool needs a CUDA device; there is no CPU path")
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.device = torch.device("cuda", index)
        cfg = _lib.PoolConfig(C.sizeof(_lib.PoolConfig), index, chunk_bytes, staging_tiles, codec_flags,
                              host_budget_bytes, host_alloc_flags, codec_max_ctas, numa_node, tile_chunks,
                              d2h_piece_bytes, h2d_piece_bytes, deferred_inflight_bytes, 1 if collect_timing else 0, 0)
        self.deferred = deferred_inflight_bytes > 0
        self._lib = _lib.lib()
        with torch.cuda.device(index):
            self._h = self._lib.flame_offload_pool_create(num_slots, max_bytes, int(compression), C.byref(cfg))
        if not self._h:
            msg = _lib.last_error()
            if "must be > 0" in msg or "chunk_bytes" in msg or "unknown compression" in msg:
                raise InvalidInput(msg)
            raise CudaError(msg)
        self.compression = OffloadCompression(compression)
        self._meta: dict[int, tuple] = {}        # slot -> (shape, dtype)
        # Source tensors held until their device-to-host copy cannot be disturbed any more.  Keyed by a per-push
        # sequence number, not by slot: a slot is free again as soon as a restore with a deferred wait has been
        # issued from it, and a push that reuses it must not release (or be released with) the earlier tensor.
        self._keep_alive: dict[int, tuple] = {}  # push sequence number -> (handle, tensor)
        self._seq = 0
        self._seq_of_slot: dict[int, int] = {}   # slot -> sequence number of the push that holds it now
        self._awaiting: dict[int, int] = {}      # slot -> sequence number of the push whose deferred restore awaits wait_ready

    @staticmethod
    def host_bytes_needed(tensor_bytes, compression: OffloadCompression, chunk_bytes: int = 0) -> int:
        """Pinned bytes that hold all of `tensor_bytes` (BF16 byte sizes) at once: a value for `host_budget_bytes`.

        Every tensor occupies whole chunks, so the last chunk of each is partly empty.
        """
        chunk = chunk_bytes or (16 << 20)
        if compression == OffloadCompression.NONE:
            per_chunk = chunk
        elif compression == OffloadCompression.FP8:
            per_chunk = chunk // 2
        else:
            per_chunk = _lib.lib().flame_act_packed_bytes(chunk // 2)
        return sum(-(-int(b) // chunk) for b in tensor_bytes) * per_chunk

    # -- accessors (src/activation_offload.rs:429-455) ---------------------------------
    def num_slots(self) -> int:
        return self._lib.flame_offload_pool_num_slots(self._h)

    def slot_bytes(self) -> int:
        return self._lib.flame_offload_pool_slot_bytes(self._h)

    def host_bytes(self) -> int:
        return self._lib.flame_offload_pool_host_bytes(self._h)

    def in_flight(self) -> int:
        return self._lib.flame_offload_pool_in_flight(self._h)

    # -- push / pull -----------------------------------------------------------------------
    def _stream(self) -> int:
        return self._torch.cuda.current_stream(self.device).cuda_stream

    def release_finished_sources(self) -> None:
        """Lets go of every source tensor whose device-to-host copy has completed (push does this on its way in)."""
        self._sweep_keep_alive()

    def _sweep_keep_alive(self) -> None:
        """Drops source tensors whose device-to-host copy has completed.

        Offloads complete in the order they were pushed (one D2H stream), so the sweep walks from the
        oldest entry and stops at the first one that is still being read.
        """
        ka = self._keep_alive
        while ka:
            seq = next(iter(ka))
            if self._lib.flame_offload_pool_source_released(self._h, ka[seq][0]) == 0:
                break
            del ka[seq]

    def _hold_source(self, h, obj) -> None:
        self._seq += 1
        self._keep_alive[self._seq] = (h, obj)
        self._seq_of_slot[h.slot] = self._seq

    def _release_source(self, slot: int, deferred: bool) -> None:
        """After a restore from `slot` was issued.  Not deferred: the current stream already waits for the restore,
        which waited for the offload, so later work on that stream cannot disturb the source.  Deferred: the same
        holds only from wait_ready on, which looks the push up under `_awaiting`."""
        seq = self._seq_of_slot.pop(slot, None)
        if seq is None:
            return
        if deferred:
            self._awaiting[slot] = seq
        else:
            self._keep_alive.pop(seq, None)

    def push(self, tensor) -> OffloadHandle:
        """Asynchronously offload `tensor`; never blocks the host (activation_offload.rs:465-611)."""
        tag = _dtype_tag(tensor)
        if tensor.device != self.device:
            raise InvalidInput(f"ActivationOffloadPool::push: tensor on {tensor.device}, pool on {self.device}")
        if not tensor.is_contiguous():
            raise InvalidInput("ActivationOffloadPool::push: tensor must be contiguous")
        self._sweep_keep_alive()
        h = _lib.Handle()
        st = self._lib.flame_offload_pool_push(self._h, tensor.data_ptr() if tensor.numel() else None,
                                              tensor.numel(), tag, self._stream(), C.byref(h))
        if st != 0:
            raise_for_status(st, _lib.last_error())
        handle = OffloadHandle(h.slot, h.epoch)
        self._meta[h.slot] = (tuple(tensor.shape), tensor.dtype)
        self._hold_source(h, tensor.detach())
        return handle

    def push_packed(self, codes, scales, shape, dtype=None) -> OffloadHandle:
        """Offload a BF16 tensor of `shape` that its producer already compressed on the device (uint8 `codes`, one per
        element, and float32 `scales`, one per 128 elements, as flame_act_quant_*_b128 lay them out).  No compress launch;
        the restore gives BF16 as for any other slot."""
        torch = self._torch
        numel = 1
        for d in shape:
            numel *= int(d)
        if codes.dtype != torch.uint8 or scales.dtype != torch.float32 or not codes.is_contiguous() or not scales.is_contiguous():
            raise InvalidInput("ActivationOffloadPool::push_packed: codes must be contiguous uint8 and scales contiguous float32")
        if codes.numel() < numel or scales.numel() < (numel + 127) // 128 or codes.device != self.device or scales.device != self.device:
            raise InvalidInput("ActivationOffloadPool::push_packed: codes / scales do not cover the tensor or live on another device")
        self._sweep_keep_alive()
        h = _lib.Handle()
        st = self._lib.flame_offload_pool_push_packed(self._h, codes.data_ptr(), scales.data_ptr(), numel, self._stream(), C.byref(h))
        if st != 0:
            raise_for_status(st, _lib.last_error())
        self._meta[h.slot] = (tuple(shape), dtype or torch.bfloat16)
        self._hold_source(h, _Prepacked(codes, scales, numel, tuple(shape)))
        return OffloadHandle(h.slot, h.epoch)

    def pull_into(self, handle: OffloadHandle, dst, defer_wait: bool = False, keep: bool = False) -> None:
        """Restore into `dst` (contiguous, same dtype, at least as many bytes).

        keep=True leaves the slot Pushed with its pinned copy intact, so the same handle can be
        restored again (weights streamed in every step)."""
        if not dst.is_contiguous() or dst.device != self.device:
            raise InvalidInput("ActivationOffloadPool::pull_into: destination must be a contiguous tensor on the pool's device")
        st = self._lib.flame_offload_pool_pull_into(self._h, handle._c(), dst.data_ptr(), dst.numel() * dst.element_size(),
                                                   self._stream(), (1 if defer_wait else 0) | (2 if keep else 0))
        if st != 0:
            raise_for_status(st, _lib.last_error())
        if keep:
            return
        self._release_source(handle.slot, defer_wait)
        self._meta.pop(handle.slot, None)

    def pull_packed(self, handle: OffloadHandle, codes, scales, defer_wait: bool = False) -> None:
        """Restore the compressed form itself into `codes` (uint8, one per element) and `scales` (float32, one per 128
        elements): no dequantise launch; the caller expands it, e.g. several tensors with one launch."""
        torch = self._torch
        if codes.dtype != torch.uint8 or scales.dtype != torch.float32 or not codes.is_contiguous() or not scales.is_contiguous():
            raise InvalidInput("ActivationOffloadPool::pull_packed: codes must be contiguous uint8 and scales contiguous float32")
        info = self.slot_info(handle)
        if codes.numel() < info["numel"] or scales.numel() < (info["numel"] + 127) // 128:
            raise InvalidInput("ActivationOffloadPool::pull_packed: codes / scales are smaller than the tensor")
        st = self._lib.flame_offload_pool_pull_packed(self._h, handle._c(), codes.data_ptr(), scales.data_ptr(), self._stream(),
                                                     1 if defer_wait else 0)
        if st != 0:
            raise_for_status(st, _lib.last_error())
        self._release_source(handle.slot, defer_wait)
        self._meta.pop(handle.slot, None)

    def prefetch(self, handle: OffloadHandle, dst) -> None:
        """Start the restore into `dst` now; call wait_ready(handle.slot) before the first read."""
        self.pull_into(handle, dst, defer_wait=True)

    def pull(self, handle: OffloadHandle):
        """Restore into a freshly allocated tensor (activation_offload.rs:619-731)."""
        info = _lib.SlotInfo()
        raise_for_status(self._lib.flame_offload_pool_slot_info(self._h, handle._c(), C.byref(info)), _lib.last_error())
        shape, dtype = self._meta[handle.slot]
        out = self._torch.empty(shape, dtype=dtype, device=self.device)
        self.pull_into(handle, out)
        return out

    def cancel(self, handle: OffloadHandle):
        """Deferred pools: if the offload of `handle` has not been enqueued yet, takes it out of the queue and returns
        the source tensor, which never left the device (its slot is free again).  Otherwise None: restore it with
        pull / pull_into."""
        if not self.deferred:
            return None
        r = self._lib.flame_offload_pool_cancel(self._h, handle._c())
        if r < 0:
            raise_for_status(-r, _lib.last_error())
        if r == 0:
            return None
        self._meta.pop(handle.slot, None)
        src = self._keep_alive.pop(self._seq_of_slot.pop(handle.slot))[1]
        if isinstance(src, _Prepacked):
            # only the compressed form was kept on the device: dequantise it here, without a trip over the link
            out = self._torch.empty(src.numel, dtype=self._torch.bfloat16, device=self.device)
            fn = (self._lib.flame_act_dequant_int8_b128 if self.compression == OffloadCompression.INT8_B128
                  else self._lib.flame_act_dequant_fp8_b128)
            rc = fn(src.codes.data_ptr(), src.scales.data_ptr(), out.data_ptr(), src.numel, self._stream())
            if rc != 0:
                raise CudaError(f"dequantise of a cancelled pre-compressed tensor failed ({rc}): {_lib.last_error()}")
            src.codes.record_stream(self._torch.cuda.current_stream(self.device))
            src.scales.record_stream(self._torch.cuda.current_stream(self.device))
            return out.view(src.shape)
        return src

    def hold_offloads(self, on: bool) -> None:
        """Deferred pools: while on, queued offloads are not enqueued (backward has begun; they are about to be
        cancelled or pulled)."""
        raise_for_status(self._lib.flame_offload_pool_hold(self._h, 1 if on else 0), _lib.last_error())

    def hold_offloads_after_current_work(self) -> None:
        """Deferred pools: the hold begins when the device has finished what the current stream holds now (called when
        the host starts backward, it stops new offloads once the device has finished the forward pass)."""
        raise_for_status(self._lib.flame_offload_pool_hold_after(self._h, self._stream()), _lib.last_error())

    def discard(self, handle: OffloadHandle) -> None:
        """Frees the slot of `handle` without restoring it (an abandoned block, src/autograd.rs:1742-1769)."""
        raise_for_status(self._lib.flame_offload_pool_discard(self._h, handle._c()), _lib.last_error())
        self._meta.pop(handle.slot, None)
        self._seq_of_slot.pop(handle.slot, None)
        # the source stays referenced until its device-to-host copy, already queued, has finished
        self._sweep_keep_alive()

    def wait_ready(self, slot: int) -> None:
        """Makes the current stream wait for the latest restore issued from `slot`."""
        st = self._lib.flame_offload_pool_wait_ready(self._h, slot, self._stream())
        if st != 0:
            raise_for_status(st, _lib.last_error())
        seq = self._awaiting.pop(slot, None)
        if seq is not None:
            self._keep_alive.pop(seq, None)

    def clear(self) -> None:
        """Invalidate every handle, free every slot; does not synchronise (activation_offload.rs:742-760)."""
        raise_for_status(self._lib.flame_offload_pool_clear(self._h), _lib.last_error())
        self._meta.clear()
        self._keep_alive.clear()
        self._seq_of_slot.clear()
        self._awaiting.clear()

    # -- extras ------------------------------------------------------------------------------
    def synchronize(self, timeout_s: float = 60.0) -> None:
        raise_for_status(self._lib.flame_offload_pool_synchronize(self._h, timeout_s), _lib.last_error())

    def source_released(self, handle: OffloadHandle) -> bool:
        r = self._lib.flame_offload_pool_source_released(self._h, handle._c())
        if r < 0:
            raise_for_status(-r, _lib.last_error())
        return r == 1

    def slot_info(self, handle: OffloadHandle) -> dict:
        info = _lib.SlotInfo()
        raise_for_status(self._lib.flame_offload_pool_slot_info(self._h, handle._c(), C.byref(info)), _lib.last_error())
        return {n: getattr(info, n) for n, _ in _lib.SlotInfo._fields_}

    def read_slot(self, handle: OffloadHandle, timeout_s: float = 60.0):
        """What the pinned slab holds for `handle`, in canonical order: (codes, scales) numpy arrays."""
        info = self.slot_info(handle)
        if self.compression == OffloadCompression.NONE:
            codes = np.empty(info["bytes"], np.uint8)
            scales = None
        else:
            codes = np.empty(info["numel"], np.uint8)
            nsc = 1 if self.compression == OffloadCompression.FP8 else (info["numel"] + 127) // 128
            scales = np.empty(nsc, np.float32)
        st = self._lib.flame_offload_pool_read_slot(self._h, handle._c(), codes.ctypes.data,
                                                   scales.ctypes.data if scales is not None else None, timeout_s)
        raise_for_status(st, _lib.last_error())
        return codes, scales

    def stats(self) -> dict:
        s = _lib.Stats()
        raise_for_status(self._lib.flame_offload_pool_stats(self._h, C.byref(s)), _lib.last_error())
        return {n: getattr(s, n) for n, _ in _lib.Stats._fields_}

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._keep_alive.clear()
            self._lib.flame_offload_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
