"""Restore arena bookkeeping (no GPU: the arena is host arithmetic over a caller-owned range)."""
import ctypes as C

import pytest

from flame_b200 import _lib

BASE = 0x7F0000000000       # any aligned address: the arena never dereferences it


def _arena(nbytes=1024, align=256):
    lib = _lib.lib()
    h = lib.flame_restore_arena_create(BASE, nbytes, align)
    assert h
    return lib, h


def _alloc(lib, h, n):
    p, t = C.c_void_p(), C.c_uint64()
    st = lib.flame_restore_arena_alloc(h, n, C.byref(p), C.byref(t))
    return st, (p.value or 0) - BASE, t.value


def _stats(lib, h):
    s = _lib.ArenaStats()
    assert lib.flame_restore_arena_stats(h, C.byref(s)) == 0
    return {n: getattr(s, n) for n, _ in _lib.ArenaStats._fields_}


def test_ring_order_wrap_and_out_of_order_release():
    lib, h = _arena(1024)
    st, a, ta = _alloc(lib, h, 300)         # rounds to 512
    assert (st, a) == (0, 0)
    st, b, tb = _alloc(lib, h, 256)
    assert (st, b) == (0, 512)
    st, c, tc = _alloc(lib, h, 256)
    assert (st, c) == (0, 768)
    assert _alloc(lib, h, 1)[0] == 5        # full
    assert "restore arena full" in _lib.last_error()
    # releasing a region in the middle frees nothing yet: the oldest region is still held
    assert lib.flame_restore_arena_release(h, tb) == 0
    assert _alloc(lib, h, 1)[0] == 5
    # the oldest goes: its space and the middle one's come back, in ring order
    assert lib.flame_restore_arena_release(h, ta) == 0
    st, d, td = _alloc(lib, h, 700)         # 768 bytes at offset 0: wraps in front of the live region at 768
    assert (st, d) == (0, 0)
    assert _alloc(lib, h, 1)[0] == 5
    assert lib.flame_restore_arena_release(h, tc) == 0
    st, e, te = _alloc(lib, h, 256)
    assert (st, e) == (0, 768)
    s = _stats(lib, h)
    assert s["allocs"] == 5 and s["releases"] == 3 and s["rejected"] == 3 and s["live_regions"] == 2
    assert s["in_use_bytes"] == 1024 and s["peak_in_use_bytes"] == 1024 and s["capacity_bytes"] == 1024
    lib.flame_restore_arena_destroy(h)


def test_newest_region_released_first_gives_its_space_back_at_once():
    lib, h = _arena(1024)
    _, a, ta = _alloc(lib, h, 256)
    _, b, tb = _alloc(lib, h, 256)
    assert lib.flame_restore_arena_release(h, tb) == 0
    st, c, tc = _alloc(lib, h, 512)
    assert (st, c) == (0, 256)
    lib.flame_restore_arena_destroy(h)


def test_wrap_leaves_the_unused_end_behind_and_recovers_it():
    lib, h = _arena(1024)
    _, a, ta = _alloc(lib, h, 512)
    _, b, tb = _alloc(lib, h, 256)          # head at 768
    assert lib.flame_restore_arena_release(h, ta) == 0
    st, c, tc = _alloc(lib, h, 512)         # does not fit in [768, 1024): goes to 0
    assert (st, c) == (0, 0)
    assert _alloc(lib, h, 256)[0] == 5      # [512, 768) is live, [768, 1024) was skipped
    assert lib.flame_restore_arena_release(h, tb) == 0
    st, d, td = _alloc(lib, h, 512)         # the skipped end is free again behind region c
    assert (st, d) == (0, 512)
    lib.flame_restore_arena_destroy(h)


def test_errors_and_reset():
    lib = _lib.lib()
    assert not lib.flame_restore_arena_create(None, 1024, 256)
    assert not lib.flame_restore_arena_create(BASE, 0, 256)
    assert not lib.flame_restore_arena_create(BASE + 8, 1024, 256)
    assert not lib.flame_restore_arena_create(BASE, 1024, 96)
    lib, h = _arena(1024)
    assert _alloc(lib, h, 0)[0] == 1 and _alloc(lib, h, 4096)[0] == 1
    _, a, ta = _alloc(lib, h, 100)
    assert lib.flame_restore_arena_release(h, ta) == 0
    assert lib.flame_restore_arena_release(h, ta) == 5          # twice
    assert lib.flame_restore_arena_release(h, 999) == 5
    _, b, tb = _alloc(lib, h, 1024)
    assert lib.flame_restore_arena_reset(h) == 0
    assert lib.flame_restore_arena_release(h, tb) == 5          # tickets from before the reset are gone
    st, c, _ = _alloc(lib, h, 1024)
    assert (st, c) == (0, 0)
    assert _stats(lib, h)["resets"] == 1
    lib.flame_restore_arena_destroy(h)


def test_randomised_against_a_model():
    """Random alloc/release traffic: regions never overlap, stay in range and aligned; a rejected request really
    does not fit in ring order."""
    import random

    rng = random.Random(0)
    lib, h = _arena(1 << 16, 256)
    live = {}
    for _ in range(5000):
        if live and rng.random() < 0.5:
            # mostly release the oldest, sometimes any
            t = min(live) if rng.random() < 0.7 else rng.choice(list(live))
            assert lib.flame_restore_arena_release(h, t) == 0
            del live[t]
        else:
            n = rng.randrange(1, 9000)
            st, off, t = _alloc(lib, h, n)
            if st == 0:
                size = (n + 255) // 256 * 256
                assert off % 256 == 0 and off + size <= (1 << 16)
                for o, s_ in live.values():
                    assert off + size <= o or o + s_ <= off, "overlap"
                live[t] = (off, size)
            else:
                assert st == 5
        s = _stats(lib, h)
        assert s["in_use_bytes"] == sum(v[1] for v in live.values()) and s["live_regions"] == len(live)
    lib.flame_restore_arena_destroy(h)
