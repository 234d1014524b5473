"""Bandwidth probe and recompute-vs-offload plan (flame_offload_probe / flame_offload_policy_plan).

Takes the seat of ``CheckpointPolicy::Adaptive`` in the reference
(src/gradient_checkpointing.rs:70-74, 201-232): the decision per saved tensor
is made from measured link and HBM rates instead of a byte counter.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

from . import _lib
from .errors import raise_for_status


class Decision(enum.IntEnum):
    RESIDENT = 0
    OFFLOAD_BF16 = 1
    OFFLOAD_INT8 = 2
    OFFLOAD_FP8 = 3
    RECOMPUTE = 4


@dataclass
class LinkProbe:
    d2h_gbs: float
    h2d_gbs: float
    hbm_copy_gbs: float
    quant_gbs: float
    dequant_gbs: float


def probe(nbytes: int = 256 << 20, reps: int = 5) -> LinkProbe:
    """Measures, on the current CUDA device, pinned copy rates, a device copy and the int8 codec."""
    out = _lib.LinkProbe()
    raise_for_status(_lib.lib().flame_offload_probe(nbytes, reps, C.byref(out)), _lib.last_error())
    return LinkProbe(*(getattr(out, n) for n, _ in _lib.LinkProbe._fields_))


@dataclass
class SavedTensor:
    nbytes: int
    group: int
    recompute_ms: float = -1.0
    allow_lossy: bool = True


def plan(tensors: list[SavedTensor], *, d2h_gbs: float, h2d_gbs: float, fwd_ms: float, bwd_ms: float,
         device_budget_bytes: int = 0, lossy_codec: Decision = Decision.OFFLOAD_INT8,
         link_utilisation: float = 0.9) -> tuple[list[Decision], float]:
    """Returns (decision per tensor, estimated exposed milliseconds per step)."""
    n = len(tensors)
    arr = (_lib.PolicyTensor * max(n, 1))()
    for i, t in enumerate(tensors):
        arr[i] = _lib.PolicyTensor(t.nbytes, t.recompute_ms, t.group, int(t.allow_lossy))
    inp = _lib.PolicyInput(d2h_gbs, h2d_gbs, fwd_ms, bwd_ms, device_budget_bytes, int(lossy_codec), link_utilisation, 0.0, 0.0)
    dec = (C.c_int32 * max(n, 1))()
    est = C.c_double()
    st = _lib.lib().flame_offload_policy_plan(C.byref(inp), arr, n, dec, C.byref(est))
    raise_for_status(st, _lib.last_error())
    return [Decision(dec[i]) for i in range(n)], est.value


@dataclass
class Block:
    saved_bytes: int
    fwd_ms: float
    bwd_ms: float


@dataclass
class BlockPlan:
    decisions: list
    est_stall_ms: float
    est_recompute_ms: float
    resident_bytes: int
    link_bytes: int
    est_interference_ms: float = 0.0


# Extra compute time per unit of copy-engine busy time, measured on a B200 DiT step with copies in 2 MiB pieces.
DEFAULT_INTERFERENCE = 0.1


def plan_blocks(blocks: list[Block], *, d2h_gbs: float, h2d_gbs: float, device_budget_bytes: int = 0,
                offload: Decision = Decision.OFFLOAD_INT8, interference: float = DEFAULT_INTERFERENCE,
                overhead_cap_ms: float = 0.0) -> BlockPlan:
    """Per-block decision for a stack of checkpointed blocks (flame_offload_policy_plan_blocks).

    ``overhead_cap_ms`` = 0: the least estimated step time with at most ``device_budget_bytes`` resident.
    ``overhead_cap_ms`` > 0: the fewest resident bytes whose estimated extra step time stays under the cap."""
    n = len(blocks)
    arr = (_lib.PolicyBlock * max(n, 1))()
    for i, b in enumerate(blocks):
        arr[i] = _lib.PolicyBlock(b.saved_bytes, b.fwd_ms, b.bwd_ms)
    inp = _lib.PolicyInput(d2h_gbs, h2d_gbs, 0.0, 0.0, device_budget_bytes, int(offload), 0.0, interference, overhead_cap_ms)
    dec = (C.c_int32 * max(n, 1))()
    out = _lib.PolicyBlockPlan()
    st = _lib.lib().flame_offload_policy_plan_blocks(C.byref(inp), arr, n, int(offload), dec, C.byref(out))
    raise_for_status(st, _lib.last_error())
    return BlockPlan([Decision(dec[i]) for i in range(n)], out.est_stall_ms, out.est_recompute_ms, out.resident_bytes, out.link_bytes,
                     out.est_interference_ms)
