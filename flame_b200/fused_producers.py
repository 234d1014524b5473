"""RMSNorm and SwiGLU with the compress step built in (the producers of three of a DiT block's five saved tensors).

Inside ``checkpoint_offload`` of a block that goes to a pool in a per-128-block mode, these functions also write
the int8 / FP8 codes and scales of the tensor the block will save (the norm's output, the gate+up input of SwiGLU)
and remember them; the pack hook then hands that compressed form to the pool (``push_packed``) and no compress
launch ever reads the BF16 tensor again.  Outside such a block they are the plain producers.

The kernels follow src/cuda/fused_rms_norm.cu:26-80 (RMSNorm) and the SwiGLU of Op::FusedSwiGLU
(src/autograd.rs:326-331); the codes equal what flame_act_quant_*_b128 gives for the same BF16 tensor.
"""
from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Optional, Tuple

from . import _lib
from .errors import CudaError, InvalidInput

_STATE = threading.local()
# (data_ptr, numel) -> (tensor version, codes, scales, the tensor itself).  The tensor is held until it is taken or
# the block ends, so that no other tensor can be given its address in between and be mistaken for it.
_READY: dict = {}


def emitting() -> int:
    """0, or the codec (2 = int8, 3 = FP8 per 128) the producers should emit right now."""
    return getattr(_STATE, "codec", 0)


@contextmanager
def emit_codes(codec: int):
    prev = emitting()
    _STATE.codec = int(codec)
    try:
        yield
    finally:
        _STATE.codec = prev
        if not prev:
            _READY.clear()      # what no pack hook took is dropped with the block


def take(t) -> Optional[Tuple[object, object]]:
    """(codes, scales) a producer wrote for exactly this tensor (same memory, same version), once."""
    rec = _READY.pop((t.data_ptr(), t.numel()), None)
    if rec is None or rec[0] != t._version:
        return None
    return rec[1], rec[2]


def _stream(t) -> int:
    import torch

    return torch.cuda.current_stream(t.device).cuda_stream


def rmsnorm(x, weight, eps: float):
    """(y, rstd): y = bf16((x * rstd) * weight) over the last dimension, rstd [rows] float32."""
    import torch

    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous() or not weight.is_contiguous():
        raise InvalidInput("fused rmsnorm: contiguous BF16 input and weight")
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    codec = emitting()
    codes = scales = None
    if codec:
        codes = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        scales = torch.empty(x.numel() // 128, dtype=torch.float32, device=x.device)
    rc = _lib.lib().flame_act_rmsnorm_quant_b128(x.data_ptr(), weight.data_ptr(), y.data_ptr(),
                                                 codes.data_ptr() if codec else None, scales.data_ptr() if codec else None,
                                                 rstd.data_ptr(), rows, cols, float(eps), codec, 0, _stream(x))
    if rc != 0:
        raise CudaError(f"flame_act_rmsnorm_quant_b128 failed ({rc}): {_lib.last_error()}")
    if codec:
        _READY[(y.data_ptr(), y.numel())] = (y._version, codes, scales, y)
    return y, rstd


def swiglu(gate_up):
    """h = bf16(silu(gate) * up) for gate_up [..., 2*hidden] (gate columns, then up columns)."""
    import torch

    if gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous():
        raise InvalidInput("fused swiglu: contiguous BF16 input")
    hidden = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * hidden)
    h = torch.empty(gate_up.shape[:-1] + (hidden,), dtype=torch.bfloat16, device=gate_up.device)
    codec = emitting()
    codes = scales = None
    if codec:
        codes = torch.empty(gate_up.numel(), dtype=torch.uint8, device=gate_up.device)
        scales = torch.empty(gate_up.numel() // 128, dtype=torch.float32, device=gate_up.device)
    rc = _lib.lib().flame_act_swiglu_quant_b128(gate_up.data_ptr(), h.data_ptr(), codes.data_ptr() if codec else None,
                                                scales.data_ptr() if codec else None, rows, hidden, codec, 0, _stream(gate_up))
    if rc != 0:
        raise CudaError(f"flame_act_swiglu_quant_b128 failed ({rc}): {_lib.last_error()}")
    if codec:
        _READY[(gate_up.data_ptr(), gate_up.numel())] = (gate_up._version, codes, scales, gate_up)
    return h
