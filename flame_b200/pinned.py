"""Pinned host memory: mirror of src/pinned.rs in the reference.

``PinnedAllocFlags``  <- pinned.rs:27-69 (DEFAULT 0, PORTABLE 1, WRITE_COMBINED 4; default = WC)
``PinnedHostBuffer``  <- pinned.rs:72-260 (typed owner of one cudaHostAlloc block)
``StagingDeviceBuf``  <- pinned.rs:320-401 (device buffer + H2D upload from a pinned buffer)
``register_slice_as_pinned`` / ``unregister_pinned`` / ``memcpy_async_*`` <- pinned.rs:403-455
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .errors import CudaError, InvalidInput, InvalidOperation

CUDA_MEMCPY_HOST_TO_DEVICE = 1
CUDA_MEMCPY_DEVICE_TO_HOST = 2


def _check_cuda(code: int, context: str) -> None:
    if code != 0:
        raise CudaError(f"{context} (cuda error {code})")


class PinnedAllocFlags:
    """Bit set of cudaHostAlloc flags (pinned.rs:27-69)."""

    __slots__ = ("_bits",)

    def __init__(self, bits: int | None = None):
        # Default::default() is WRITE_COMBINED in the reference (pinned.rs:51-55).
        self._bits = 0x04 if bits is None else int(bits)

    def bits(self) -> int:
        return self._bits

    def contains(self, other: "PinnedAllocFlags") -> bool:
        return (self._bits & other._bits) == other._bits

    @staticmethod
    def portable_write_combined() -> "PinnedAllocFlags":
        return PinnedAllocFlags.PORTABLE | PinnedAllocFlags.WRITE_COMBINED

    def __or__(self, rhs: "PinnedAllocFlags") -> "PinnedAllocFlags":
        return PinnedAllocFlags(self._bits | rhs._bits)

    def __eq__(self, other) -> bool:
        return isinstance(other, PinnedAllocFlags) and other._bits == self._bits

    def __hash__(self) -> int:
        return hash(self._bits)

    def __repr__(self) -> str:
        return f"PinnedAllocFlags({self._bits:#x})"


PinnedAllocFlags.DEFAULT = PinnedAllocFlags(0x00)
PinnedAllocFlags.PORTABLE = PinnedAllocFlags(0x01)
PinnedAllocFlags.WRITE_COMBINED = PinnedAllocFlags(0x04)


class PinnedHostBuffer:
    """Typed owner of one pinned allocation (pinned.rs:72-260).

    ``dtype`` plays the role of the Rust type parameter.  ``len`` counts
    initialised elements, ``capacity`` allocated ones.
    """

    def __init__(self, ptr: int, capacity: int, dtype, flags: PinnedAllocFlags, length: int = 0):
        self._ptr = ptr
        self._capacity = capacity
        self._dtype = np.dtype(dtype)
        self._flags = flags
        self._len = length

    @classmethod
    def with_capacity_elems(cls, capacity: int, flags: PinnedAllocFlags, dtype=np.uint8) -> "PinnedHostBuffer":
        if capacity == 0:
            raise InvalidInput("PinnedHostBuffer::with_capacity_elems requires capacity > 0")
        nbytes = capacity * np.dtype(dtype).itemsize
        if nbytes >= 1 << 63:
            raise InvalidInput("PinnedHostBuffer byte size overflow")
        ptr = _lib.lib().flame_cuda_alloc_pinned_host(nbytes, flags.bits())
        if not ptr:
            raise CudaError(f"cudaHostAlloc returned null ({nbytes} bytes)")
        return cls(ptr, capacity, dtype, flags)

    def capacity(self) -> int:
        return self._capacity

    def capacity_bytes(self) -> int:
        return self._capacity * self._dtype.itemsize

    def __len__(self) -> int:
        return self._len

    def len(self) -> int:
        return self._len

    def len_bytes(self) -> int:
        return self._len * self._dtype.itemsize

    def flags(self) -> PinnedAllocFlags:
        return self._flags

    def as_ptr(self) -> int:
        return self._ptr

    as_mut_ptr = as_ptr

    def _view(self, nelem: int, dtype=None) -> np.ndarray:
        dt = self._dtype if dtype is None else np.dtype(dtype)
        if self._ptr is None:
            raise InvalidOperation("PinnedHostBuffer used after it was freed")
        buf = (C.c_uint8 * (nelem * dt.itemsize)).from_address(self._ptr)
        return np.frombuffer(buf, dtype=dt, count=nelem)

    def as_slice(self) -> np.ndarray:
        return self._view(self._len)

    as_mut_slice = as_slice

    def as_mut_capacity_slice(self) -> np.ndarray:
        return self._view(self._capacity)

    def as_bytes(self) -> np.ndarray:
        return self._view(self.len_bytes(), np.uint8)

    def as_mut_bytes(self) -> np.ndarray:
        return self._view(self.capacity_bytes(), np.uint8)

    def copy_from_slice(self, src) -> None:
        src = np.ascontiguousarray(src, self._dtype).reshape(-1)
        if src.size > self._capacity:
            raise OverflowError("PinnedHostBuffer::copy_from_slice overflow")
        self.as_mut_capacity_slice()[: src.size] = src
        self.set_len(src.size)

    def clear(self) -> None:
        self._len = 0

    def set_len(self, length: int) -> None:
        if length > self._capacity:
            raise AssertionError("PinnedHostBuffer::set_len overflow")
        self._len = length

    def reinterpret(self, dtype) -> np.ndarray:
        """Read view of the initialised bytes as another element type (pinned.rs:190-200)."""
        dt = np.dtype(dtype)
        if self.len_bytes() % dt.itemsize != 0:
            raise InvalidOperation("PinnedHostBuffer::reinterpret requires aligned length")
        v = self._view(self.len_bytes() // dt.itemsize, dt)
        v.flags.writeable = False
        return v

    def reinterpret_mut(self, dtype) -> np.ndarray:
        dt = np.dtype(dtype)
        if self.len_bytes() % dt.itemsize != 0:
            raise InvalidOperation("PinnedHostBuffer::reinterpret_mut requires aligned length")
        return self._view(self.len_bytes() // dt.itemsize, dt)

    def into_reinterpret(self, dtype) -> "PinnedHostBuffer":
        """Consumes this buffer and returns the same allocation typed as `dtype` (pinned.rs:214-241)."""
        dt = np.dtype(dtype)
        if self.capacity_bytes() % dt.itemsize != 0:
            raise InvalidOperation("PinnedHostBuffer::into_reinterpret capacity misaligned")
        if self.len_bytes() % dt.itemsize != 0:
            raise InvalidOperation("PinnedHostBuffer::into_reinterpret length misaligned")
        out = PinnedHostBuffer(self._ptr, self.capacity_bytes() // dt.itemsize, dt, self._flags,
                               self.len_bytes() // dt.itemsize)
        self._ptr = None  # ownership moved
        return out

    def _release(self) -> int | None:
        """Gives up ownership without freeing (used when a pool takes the allocation)."""
        ptr, self._ptr = self._ptr, None
        return ptr

    def free(self) -> None:
        if self._ptr is not None:
            ptr, self._ptr = self._ptr, None
            _lib.lib().flame_cuda_free_pinned_host(ptr)

    def __del__(self):  # Drop (pinned.rs:244-250)
        try:
            self.free()
        except Exception:
            pass

    def __repr__(self) -> str:
        return f"PinnedHostBuffer(capacity={self._capacity}, len={self._len}, flags={self._flags})"


class StagingDeviceBuf:
    """Zero-initialised device buffer fed from a pinned buffer (pinned.rs:320-401)."""

    def __init__(self, device, length: int, dtype=np.uint8):
        import torch

        if length == 0:
            raise InvalidInput("StagingDeviceBuf::new len must be > 0")
        self._dtype = np.dtype(dtype)
        self._len = length
        self._device = torch.device(device)
        self._bytes = torch.zeros(length * self._dtype.itemsize, dtype=torch.uint8, device=self._device)

    def __len__(self) -> int:
        return self._len

    def len(self) -> int:
        return self._len

    def device(self):
        return self._device

    def slice(self):
        return self._bytes

    slice_mut = slice

    def into_inner(self):
        return self._bytes

    def async_upload_from(self, host: PinnedHostBuffer, stream) -> None:
        """H2D of the host buffer's initialised bytes on `stream` (a torch stream or a raw handle)."""
        nbytes = host.len_bytes()
        if nbytes > self._len * self._dtype.itemsize:
            raise InvalidInput("StagingDeviceBuf::async_upload_from host larger than device buffer")
        if nbytes == 0:
            return
        raw = getattr(stream, "cuda_stream", stream)
        memcpy_async_host_to_device(self._bytes.data_ptr(), host.as_ptr(), nbytes, raw)


def register_slice_as_pinned(array: np.ndarray, portable: bool) -> None:
    flags = 0x01 if portable else 0x00
    _check_cuda(_lib.lib().flame_cuda_host_register(array.ctypes.data, array.nbytes, flags), "cudaHostRegister")


def unregister_pinned(ptr: int | None) -> None:
    if not ptr:
        return
    _check_cuda(_lib.lib().flame_cuda_host_unregister(ptr), "cudaHostUnregister")


def memcpy_async_host_to_device(dst: int, src: int, nbytes: int, stream) -> None:
    _check_cuda(_lib.lib().flame_cuda_memcpy_async(dst, src, nbytes, CUDA_MEMCPY_HOST_TO_DEVICE, stream), "cudaMemcpyAsync H2D")


def memcpy_async_device_to_host(dst: int, src: int, nbytes: int, stream) -> None:
    _check_cuda(_lib.lib().flame_cuda_memcpy_async(dst, src, nbytes, CUDA_MEMCPY_DEVICE_TO_HOST, stream), "cudaMemcpyAsync D2H")
