"""Block weight streaming over the activation pool's pinned slab and chunked host-to-device pipeline.

The interface is the one the reference's trainers use for weights that do not fit on the device
(BlockOffloader of the flame-diffusion crate, described in docs/FLAME_MODULES.md:684-698, built on the pinned
staging helpers of src/pinned.rs:320-401): every block's weights live in pinned host memory, two device slots
alternate, ``prefetch_block(i + 1)`` runs while block ``i`` computes, ``await_block(i)`` hands out the tensors.

Here the host copy is a set of slots in an :class:`ActivationOffloadPool` (one per block and dtype) that are
restored with ``keep=True``, so the pinned copy stays and the same handle is restored again next step.  With a
compressed pool the host copy is int8 / FP8 codes with one scale per 128 elements and the restore dequantises
into the slot.

Weights that already are FP8 E4M3 bytes with one scale per tensor (the checkpoints the reference's inference path
loads, src/ops/fused_inference.rs:86-175) stream as they are through an uncompressed pool, one byte per element over
the link, and are expanded on the device when the block is awaited: ``flame_fp8_to_bf16`` for a weight used in its
stored [M, N] orientation, the kernel of ``flame_fused_dequant_transpose_bf16`` for those the GEMM wants as [N, M]
(src/cuda/fused_dequant_transpose.cu; one launch for all such weights of a block through the ``_multi`` entry point),
into BF16 buffers that belong to the device slot.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

from . import _lib, fused_inference
from .activation_offload import ActivationOffloadPool, OffloadCompression
from .errors import CudaError, InvalidInput, InvalidOperation, Unsupported

_ALIGN = 256


class BlockOffloader:
    def __init__(self, device, blocks: Sequence[Mapping[str, "object"]], compression: OffloadCompression = OffloadCompression.NONE,
                 chunk_bytes: int = 16 << 20, gpu_slots: int = 2, h2d_piece_bytes: int = 0,
                 fp8_weights: Optional[Mapping[str, tuple]] = None):
        """``fp8_weights``: name -> (scale, transpose) for the uint8 tensors of the blocks that hold FP8 E4M3 codes
        of a 2-D weight [M, N]; ``await_block`` hands them out as BF16, [N, M] when ``transpose`` is true."""
        import torch

        if not blocks:
            raise InvalidInput("BlockOffloader: no blocks")
        if gpu_slots < 1:
            raise InvalidInput("BlockOffloader: gpu_slots must be >= 1")
        self._torch = torch
        self.device = torch.device(device)
        # A block's tensors are laid out back to back in one flat buffer, BF16 tensors first, F32 after them, each
        # at a 256-byte boundary (128 BF16 elements, so no quantisation block spans two tensors and the padding,
        # being zero, changes no scale).  Each dtype group crosses the link as one pool slot.
        self._layout: List[List[tuple]] = []          # per block: (name, shape, dtype, offset, nbytes)
        self._groups: List[List[tuple]] = []          # per block: (dtype, offset, nbytes) of each dtype group
        self._fp8 = dict(fp8_weights or {})
        self._expand_bytes = 0                        # BF16 bytes the FP8 weights of the largest block expand to
        for blk in blocks:
            rows, groups, off = [], [], 0
            for name, t in blk.items():
                if t.dtype == torch.uint8:
                    if name not in self._fp8 or t.dim() != 2:
                        raise Unsupported(f"BlockOffloader: {name} is uint8; FP8 weights must be 2-D and named in fp8_weights")
                    if compression != OffloadCompression.NONE:
                        raise Unsupported("BlockOffloader: FP8 weight bytes stream through an uncompressed pool")
                    continue
                if t.dtype not in (torch.bfloat16, torch.float32):
                    raise Unsupported(f"BlockOffloader: {name} has dtype {t.dtype} (BF16/F32, or uint8 FP8 codes)")
                if compression != OffloadCompression.NONE and t.dtype != torch.bfloat16:
                    raise Unsupported(f"BlockOffloader: compressed streaming only supports BF16 weights ({name} is {t.dtype})")
                if t.numel() == 0:
                    raise InvalidInput(f"BlockOffloader: {name} is empty")
            for dtype in (torch.bfloat16, torch.float32, torch.uint8):
                g0 = off
                for name, t in blk.items():
                    if t.dtype != dtype:
                        continue
                    nbytes = t.numel() * t.element_size()
                    rows.append((name, tuple(t.shape), dtype, off, nbytes))
                    off = (off + nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
                if off > g0:
                    # FP8 bytes cross the link as they are: the uncompressed pool copies bytes, whatever the tag
                    groups.append((torch.bfloat16 if dtype == torch.uint8 else dtype, g0, off - g0))
            self._expand_bytes = max(self._expand_bytes, sum((2 * r[4] + _ALIGN - 1) // _ALIGN * _ALIGN for r in rows if r[2] == torch.uint8))
            self._layout.append(rows)
            self._groups.append(groups)
        self._slot_bytes = max(g[-1][1] + g[-1][2] for g in self._groups)
        sizes = [g[2] for gs in self._groups for g in gs]
        chunk = chunk_bytes or (16 << 20)
        # groups larger than a chunk: pin what they occupy; otherwise one chunk of the largest size per group
        budget = ActivationOffloadPool.host_bytes_needed(sizes, compression, chunk) if max(sizes) > chunk else 0
        self._pool = ActivationOffloadPool(self.device, len(sizes), max(sizes), compression, chunk_bytes=chunk,
                                           h2d_piece_bytes=h2d_piece_bytes, host_budget_bytes=budget)
        # host copy: each block passes through the device once (quantised there in the compressed modes)
        self._handles: List[List] = []
        for blk, rows, groups in zip(blocks, self._layout, self._groups):
            flat = torch.zeros(groups[-1][1] + groups[-1][2], dtype=torch.uint8, device=self.device)
            for name, shape, dtype, off, nbytes in rows:
                flat[off:off + nbytes].view(dtype).copy_(blk[name].detach().reshape(-1), non_blocking=True)
            self._handles.append([self._pool.push(flat[g0:g0 + gb].view(dtype)) for dtype, g0, gb in groups])
            del flat
        self._pool.synchronize(600.0)
        self._pool.release_finished_sources()
        self._n_slots = gpu_slots
        self._expanded: List[Optional[object]] = [None] * gpu_slots   # per device slot: BF16 forms of the block's FP8 weights
        self._bufs: List[Optional[object]] = [None] * gpu_slots
        self._resident: List[Optional[int]] = [None] * gpu_slots    # block index held (or being loaded) per device slot
        self._pending: List[bool] = [False] * gpu_slots              # its host-to-device copies have not been awaited yet
        self._active: Optional[int] = None                           # device slot of the block handed out last

    # -- accessors ---------------------------------------------------------------------------
    def block_count(self) -> int:
        return len(self._layout)

    def pinned_bytes(self) -> int:
        return self._pool.host_bytes()

    def device_bytes(self) -> int:
        return (self._slot_bytes + self._expand_bytes) * self._n_slots

    def stats(self) -> dict:
        return self._pool.stats()

    # -- streaming ----------------------------------------------------------------------------
    def _slot_of(self, idx: int) -> Optional[int]:
        for s, b in enumerate(self._resident):
            if b == idx:
                return s
        return None

    def _check(self, idx: int) -> None:
        if not 0 <= idx < len(self._layout):
            raise InvalidInput(f"BlockOffloader: block {idx} out of range ({len(self._layout)} blocks)")

    def prefetch_block(self, idx: int) -> None:
        """Starts the host-to-device copies of block `idx` into a device slot that is not the active one; returns at once.

        Work already queued on the current stream is ordered before the first write into that slot, so the block
        that used the slot before may still have kernels in flight."""
        self._check(idx)
        if self._slot_of(idx) is not None:
            return
        free = [s for s in range(self._n_slots) if self._resident[s] is None]
        others = [s for s in range(self._n_slots) if s != self._active]
        if free:
            slot = free[0]
        elif others:
            slot = next((s for s in others if not self._pending[s]), others[0])
        else:
            raise InvalidOperation("BlockOffloader: the only device slot holds the active block; evict_block() first")
        torch = self._torch
        if self._bufs[slot] is None:
            self._bufs[slot] = torch.empty(self._slot_bytes, dtype=torch.uint8, device=self.device)
        buf = self._bufs[slot]
        for (dtype, g0, gb), h in zip(self._groups[idx], self._handles[idx]):
            self._pool.pull_into(h, buf[g0:g0 + gb].view(dtype), defer_wait=True, keep=True)
        self._resident[slot] = idx
        self._pending[slot] = True

    def await_block(self, idx: int) -> Dict[str, "object"]:
        """Makes the current stream wait for block `idx` (prefetching it now if nobody did) and returns its tensors."""
        self._check(idx)
        slot = self._slot_of(idx)
        if slot is None:
            if self._n_slots == 1:
                self._active = None
            self.prefetch_block(idx)
            slot = self._slot_of(idx)
        if self._pending[slot]:
            for h in self._handles[idx]:
                self._pool.wait_ready(h.slot)
            self._pending[slot] = False
        self._active = slot
        buf = self._bufs[slot]
        torch = self._torch
        out, eoff = {}, 0
        jobs = []          # the block's transposed FP8 weights: one launch for all of them
        for name, shape, dtype, off, nbytes in self._layout[idx]:
            if dtype != torch.uint8:
                out[name] = buf[off:off + nbytes].view(dtype).view(shape)
                continue
            # FP8 codes [M, N] -> BF16 on the current stream, which already waits for the block's copies
            if self._expanded[slot] is None:
                self._expanded[slot] = torch.empty(self._expand_bytes, dtype=torch.uint8, device=self.device)
            scale, transpose = self._fp8[name]
            m, n = shape
            dst = self._expanded[slot][eoff:eoff + 2 * nbytes].view(torch.bfloat16)
            eoff += (2 * nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
            codes = buf[off:off + nbytes]
            try:
                if transpose:
                    jobs.append((codes, scale, dst, m, n))
                else:
                    fused_inference.dequant_fp8_to_bf16_into(codes, scale, dst)
            except CudaError as exc:
                raise CudaError(f"BlockOffloader: FP8 weight expansion of {name} failed: {exc}; {_lib.last_error()}") from exc
            out[name] = dst.view(n, m) if transpose else dst.view(m, n)
        if jobs:
            try:
                fused_inference.dequant_fp8_transpose_many(jobs)
            except CudaError as exc:
                raise CudaError(f"BlockOffloader: FP8 weight expansion of block {idx} failed: {exc}; {_lib.last_error()}") from exc
        return out

    def ensure_block(self, idx: int) -> Dict[str, "object"]:
        """prefetch_block + await_block."""
        self.prefetch_block(idx)
        return self.await_block(idx)

    def evict_block(self) -> None:
        """Drops the device copies in every slot; the pinned copies stay."""
        for slot, idx in enumerate(self._resident):
            if idx is not None and self._pending[slot]:
                # copies still in flight into a buffer that is about to be freed: the current stream, on which the
                # allocator will hand the memory out again, is ordered behind them first
                for h in self._handles[idx]:
                    self._pool.wait_ready(h.slot)
        self._bufs = [None] * self._n_slots
        self._expanded = [None] * self._n_slots
        self._resident = [None] * self._n_slots
        self._pending = [False] * self._n_slots
        self._active = None

    def close(self) -> None:
        self.evict_block()
        self._pool.close()
