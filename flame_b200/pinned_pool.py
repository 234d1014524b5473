"""PinnedPool: mirror of src/pinned_pool.rs:21-99 over flame_pinned_pool_*."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .errors import raise_for_status
from .pinned import PinnedAllocFlags, PinnedHostBuffer

SIZE_CLASS_BYTES = 8 * 1024 * 1024


class PinnedPool:
    """Cache of pinned buffers in 8 MiB size classes, capped at `max_cached_bytes`."""

    def __init__(self, flags: PinnedAllocFlags, max_cached_bytes: int):
        self._flags = flags
        self._h = _lib.lib().flame_pinned_pool_create(flags.bits(), max_cached_bytes)

    def checkout(self, min_bytes: int) -> PinnedHostBuffer:
        ptr, cap = C.c_void_p(), C.c_size_t()
        st = _lib.lib().flame_pinned_pool_checkout(self._h, min_bytes, C.byref(ptr), C.byref(cap))
        raise_for_status(st, _lib.last_error())
        return PinnedHostBuffer(ptr.value, cap.value, np.uint8, self._flags, 0)

    def checkin(self, buf: PinnedHostBuffer) -> None:
        cap = buf.capacity_bytes()
        ptr = buf._release()
        if ptr is None:
            return
        raise_for_status(_lib.lib().flame_pinned_pool_checkin(self._h, ptr, cap), _lib.last_error())

    def stats(self) -> tuple[int, int]:
        """(cached_bytes, cached_buffers), pinned_pool.rs:94-98."""
        b, n = C.c_size_t(), C.c_size_t()
        _lib.lib().flame_pinned_pool_stats(self._h, C.byref(b), C.byref(n))
        return b.value, n.value

    def close(self) -> None:
        if self._h:
            _lib.lib().flame_pinned_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
