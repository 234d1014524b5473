"""ctypes binding of libflame_offload.so (the C ABI in include/flame_offload.h).

This is the binding a maintainer of the reference would write in Rust
(`extern "C"` blocks like src/cuda/ffi.rs:83-94 and
src/activation_offload.rs:99-115); here it is ctypes because the host side of
this build is Python.  There is no fallback: if the library is missing,
``lib()`` raises ImportError.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflame_offload.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_STATE = range(6)


class Handle(C.Structure):
    _fields_ = [("slot", C.c_uint64), ("epoch", C.c_uint64)]


class PoolConfig(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("chunk_bytes", C.c_uint64),
        ("staging_tiles", C.c_uint32), ("codec_flags", C.c_uint32), ("host_budget_bytes", C.c_uint64),
        ("host_alloc_flags", C.c_uint32), ("codec_max_ctas", C.c_int32), ("numa_node", C.c_int32),
        ("tile_chunks", C.c_uint32), ("d2h_piece_bytes", C.c_uint64), ("h2d_piece_bytes", C.c_uint64),
        ("deferred_inflight_bytes", C.c_uint64), ("collect_timing", C.c_uint32), ("reserved0", C.c_uint32),
    ]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "pushes", "pulls", "bytes_logical_out", "bytes_logical_in", "bytes_link_out", "bytes_link_in",
        "chunks_out", "chunks_in", "codec_launches", "host_chunks_total", "host_chunks_free", "push_rejected_full",
        "pushes_cancelled", "pushes_queued", "offload_span_us", "restore_span_us", "ready_wait_us", "spans_timed", "spans_pending")]


class SlotInfo(C.Structure):
    _fields_ = [("numel", C.c_uint64), ("dtype", C.c_int32), ("compression", C.c_int32),
                ("bytes", C.c_uint64), ("stored_bytes", C.c_uint64), ("chunks", C.c_uint64)]


class ActTensor(C.Structure):
    _fields_ = [("bf16", C.c_void_p), ("codes", C.c_void_p), ("scales", C.c_void_p), ("n", C.c_size_t)]


class WeightJob(C.Structure):
    _fields_ = [("input_fp8", C.c_void_p), ("output_bf16", C.c_void_p), ("scale", C.c_float), ("M", C.c_int32), ("N", C.c_int32),
                ("reserved", C.c_int32)]


class ActLaunchInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("grid", "resident_per_sm", "tiles_per_block", "form")]


class LinkProbe(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("d2h_gbs", "h2d_gbs", "hbm_copy_gbs", "quant_gbs", "dequant_gbs")]


class PolicyTensor(C.Structure):
    _fields_ = [("bytes", C.c_uint64), ("recompute_ms", C.c_double), ("group", C.c_int32), ("allow_lossy", C.c_int32)]


class PolicyInput(C.Structure):
    _fields_ = [("d2h_gbs", C.c_double), ("h2d_gbs", C.c_double), ("fwd_ms", C.c_double), ("bwd_ms", C.c_double),
                ("device_budget_bytes", C.c_uint64), ("lossy_codec", C.c_int32), ("link_utilisation", C.c_double),
                ("interference", C.c_double), ("overhead_cap_ms", C.c_double)]


class PolicyBlock(C.Structure):
    _fields_ = [("saved_bytes", C.c_uint64), ("fwd_ms", C.c_double), ("bwd_ms", C.c_double)]


class PolicyBlockPlan(C.Structure):
    _fields_ = [("est_stall_ms", C.c_double), ("est_recompute_ms", C.c_double), ("resident_bytes", C.c_uint64), ("link_bytes", C.c_uint64),
                ("est_interference_ms", C.c_double)]


_vp, _sz, _i, _u, _f, _d = C.c_void_p, C.c_size_t, C.c_int, C.c_uint, C.c_float, C.c_double

# name -> (restype, argtypes); one entry per declaration in include/flame_offload.h
class ArenaStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("capacity_bytes", "in_use_bytes", "peak_in_use_bytes", "allocs", "releases",
                                          "rejected", "resets", "live_regions")]


SIGNATURES = {
    "flame_offload_last_error": (C.c_char_p, []),
    "flame_cuda_alloc_pinned_host": (_vp, [_sz, _u]),
    "flame_cuda_free_pinned_host": (_i, [_vp]),
    "flame_cuda_memcpy_async": (_i, [_vp, _vp, _sz, _i, _vp]),
    "flame_cuda_host_register": (_i, [_vp, _sz, _u]),
    "flame_cuda_host_unregister": (_i, [_vp]),
    "flame_h2d_async": (_i, [_vp, _vp, C.c_uint64, _vp]),
    "flame_d2h_async": (_i, [_vp, _vp, C.c_uint64, _vp]),
    "flame_d2d_async": (_i, [_vp, _vp, C.c_uint64, _vp]),
    "flame_bf16_to_fp8": (_i, [_vp, _vp, _f, _sz, _vp]),
    "flame_fp8_to_bf16": (_i, [_vp, _vp, _f, _sz, _vp]),
    "flame_fused_dequant_transpose_bf16": (_i, [_vp, _vp, _f, _i, _i, _vp]),
    "flame_fused_dequant_transpose_bf16_multi": (_i, [C.POINTER(WeightJob), _i, _vp]),
    "flame_act_quant_int8_b128": (_i, [_vp, _vp, _vp, _sz, _u, _vp]),
    "flame_act_dequant_int8_b128": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "flame_act_quant_fp8_b128": (_i, [_vp, _vp, _vp, _sz, _u, _vp]),
    "flame_act_dequant_fp8_b128": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "flame_act_quant_b128_multi": (_i, [_i, C.POINTER(ActTensor), _sz, _u, _vp]),
    "flame_act_dequant_b128_multi": (_i, [_i, C.POINTER(ActTensor), _sz, _vp]),
    "flame_act_packed_scales_offset": (_sz, [_sz]),
    "flame_act_packed_bytes": (_sz, [_sz]),
    "flame_act_set_max_ctas": (_i, [_i]),
    "flame_act_set_compress_form": (_i, [_i]),
    "flame_act_last_launch": (None, [C.POINTER(ActLaunchInfo)]),
    "flame_act_query_resident_blocks": (_i, [_i, _u, _i, _i]),
    "flame_act_offload_packed_noalloc": (_i, [_vp, _vp, _sz, _i, _u, _vp]),
    "flame_offload_pool_create": (_vp, [_sz, _sz, _i, C.POINTER(PoolConfig)]),
    "flame_offload_pool_destroy": (None, [_vp]),
    "flame_offload_pool_num_slots": (_sz, [_vp]),
    "flame_offload_pool_slot_bytes": (_sz, [_vp]),
    "flame_offload_pool_host_bytes": (_sz, [_vp]),
    "flame_offload_pool_in_flight": (_sz, [_vp]),
    "flame_offload_pool_compression": (_i, [_vp]),
    "flame_offload_pool_push": (_i, [_vp, _vp, _sz, _i, _vp, C.POINTER(Handle)]),
    "flame_offload_pool_pull_into": (_i, [_vp, Handle, _vp, _sz, _vp, _u]),
    "flame_offload_pool_wait_ready": (_i, [_vp, _sz, _vp]),
    "flame_offload_pool_clear": (_i, [_vp]),
    "flame_offload_pool_discard": (_i, [_vp, Handle]),
    "flame_offload_pool_source_released": (_i, [_vp, Handle]),
    "flame_offload_pool_slot_info": (_i, [_vp, Handle, C.POINTER(SlotInfo)]),
    "flame_offload_pool_synchronize": (_i, [_vp, _d]),
    "flame_offload_pool_read_slot": (_i, [_vp, Handle, _vp, _vp, _d]),
    "flame_offload_pool_stats": (_i, [_vp, C.POINTER(Stats)]),
    "flame_offload_inject_fault": (None, [_i, _i]),
    "flame_offload_pool_pull_packed": (_i, [_vp, Handle, _vp, _vp, _vp, _u]),
    "flame_offload_pool_push_packed": (_i, [_vp, _vp, _vp, _sz, _vp, C.POINTER(Handle)]),
    "flame_act_rmsnorm_quant_b128": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float, _i, _u, _vp]),
    "flame_act_swiglu_quant_b128": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _i, _u, _vp]),
    "flame_offload_pool_prefetch": (_i, [_vp, Handle, _vp, _sz, _vp]),
    "flame_offload_pool_cancel": (_i, [_vp, Handle]),
    "flame_offload_pool_hold": (_i, [_vp, _i]),
    "flame_offload_pool_hold_after": (_i, [_vp, _vp]),
    "flame_restore_arena_create": (_vp, [_vp, _sz, _sz]),
    "flame_restore_arena_destroy": (None, [_vp]),
    "flame_restore_arena_alloc": (_i, [_vp, _sz, C.POINTER(_vp), C.POINTER(C.c_uint64)]),
    "flame_restore_arena_release": (_i, [_vp, C.c_uint64]),
    "flame_restore_arena_reset": (_i, [_vp]),
    "flame_restore_arena_stats": (_i, [_vp, C.POINTER(ArenaStats)]),
    "flame_pinned_pool_create": (_vp, [_u, _sz]),
    "flame_pinned_pool_destroy": (None, [_vp]),
    "flame_pinned_pool_checkout": (_i, [_vp, _sz, C.POINTER(_vp), C.POINTER(_sz)]),
    "flame_pinned_pool_checkin": (_i, [_vp, _vp, _sz]),
    "flame_pinned_pool_stats": (None, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "flame_offload_probe": (_i, [_sz, _i, C.POINTER(LinkProbe)]),
    "flame_offload_policy_plan_blocks": (_i, [C.POINTER(PolicyInput), C.POINTER(PolicyBlock), _sz, _i, C.POINTER(C.c_int32), C.POINTER(PolicyBlockPlan)]),
    "flame_offload_policy_plan": (_i, [C.POINTER(PolicyInput), C.POINTER(PolicyTensor), _sz, C.POINTER(C.c_int32), C.POINTER(_d)]),
}

_LIB = None


def lib() -> C.CDLL:
    """The loaded library with every prototype set.  Raises ImportError if it was not built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C flame_b200/csrc` "
                "(nvcc, sm_100a).  There is no CPU fallback for this path.")
        handle = C.CDLL(LIB_PATH, mode=C.RTLD_LOCAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = header and library out of step
            fn.restype, fn.argtypes = res, args
        _LIB = handle
    return _LIB


def last_error() -> str:
    return (lib().flame_offload_last_error() or b"").decode("utf-8", "replace")
