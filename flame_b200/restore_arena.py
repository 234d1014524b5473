"""Destinations for restored activations out of one device range reserved at set-up.

The reference allocates a fresh tensor in every pull (src/activation_offload.rs:655); its stream-keyed arena for
other hot paths (src/staging.rs:219-297) is the model here.  ``RestoreArena`` owns one device buffer made at
set-up; ``empty(shape, dtype)`` hands out a tensor over the next free stretch of it without touching any
allocator, and the stretch goes back to the arena when the tensor's storage dies, whichever views of it were taken.

The arena belongs to the stream that is current when it is made: tensors from it must be used on that stream (as
``pull_into`` with that stream current does for the pool's copies).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

from . import _lib
from .errors import InvalidInput, raise_for_status


class _Region:
    """Exposes one stretch of the arena through the CUDA array interface; releasing it when the consumer drops it."""

    def __init__(self, arena: "RestoreArena", ptr: int, nbytes: int, ticket: int):
        self._arena, self._ticket = arena, ticket
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
                                         "strides": None}

    def __del__(self):
        try:
            self._arena._release(self._ticket)
        except Exception:
            pass


class RestoreArena:
    def __init__(self, device, nbytes: int, alignment: int = 256):
        import torch

        self._torch = torch
        self.device = torch.device(device)
        if nbytes <= 0:
            raise InvalidInput("RestoreArena: size must be > 0")
        self._lib = _lib.lib()
        self._buf = torch.empty(nbytes + alignment, dtype=torch.uint8, device=self.device)   # the one allocation
        base = (self._buf.data_ptr() + alignment - 1) // alignment * alignment
        self.stream = torch.cuda.current_stream(self.device)
        self._h = self._lib.flame_restore_arena_create(base, nbytes, alignment)
        if not self._h:
            raise InvalidInput(_lib.last_error())
        self.capacity = self.stats()["capacity_bytes"]

    def empty(self, shape, dtype) -> Optional["object"]:
        """A tensor of `shape` and `dtype` inside the arena, or None when the ring has no released space for it
        (or the request is larger than the whole arena)."""
        torch = self._torch
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype, device=self.device)
        ptr, ticket = C.c_void_p(), C.c_uint64()
        st = self._lib.flame_restore_arena_alloc(self._h, nbytes, C.byref(ptr), C.byref(ticket))
        if st != 0:
            if st == 5 or nbytes > self.capacity:      # full, or can never fit: the caller uses its own allocator
                return None
            raise_for_status(st, _lib.last_error())
        region = _Region(self, ptr.value, nbytes, ticket.value)
        flat = torch.as_tensor(region, device=self.device)       # keeps `region` alive until its storage dies
        return flat.view(dtype).view(tuple(shape))

    def _release(self, ticket: int) -> None:
        if getattr(self, "_h", None):
            self._lib.flame_restore_arena_release(self._h, ticket)

    def reset(self) -> None:
        raise_for_status(self._lib.flame_restore_arena_reset(self._h), _lib.last_error())

    def stats(self) -> dict:
        s = _lib.ArenaStats()
        raise_for_status(self._lib.flame_restore_arena_stats(self._h, C.byref(s)), _lib.last_error())
        return {n: getattr(s, n) for n, _ in _lib.ArenaStats._fields_}

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.flame_restore_arena_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
