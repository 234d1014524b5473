"""FP8 weights expanded on the device: the three host functions of the reference's inference path that sit on the
weight-side reuse of the offload pool (src/ops/fused_inference.rs:86-175), with their names, argument meaning and
errors, over torch tensors.

``fp8_data`` is a uint8 tensor of E4M3 codes on the GPU, ``scale`` the tensor's dequantisation scale.  All three run
on the current stream of the output's device and allocate nothing except where the reference does
(``dequant_fp8_to_bf16`` returns a new tensor).  ``dequant_fp8_transpose_many`` is new: every weight of a block in one
launch.
"""
from __future__ import annotations

from typing import Iterable, Sequence, Tuple

from . import _lib
from .errors import CudaError, InvalidInput, InvalidShape


def _check_codes(fp8_data, what: str):
    import torch

    if fp8_data.dtype != torch.uint8 or not fp8_data.is_cuda or not fp8_data.is_contiguous():
        raise InvalidInput(f"{what}: fp8_data must be a contiguous uint8 tensor on the GPU")


def _check_output(output, device, what: str):
    import torch

    if output.dtype != torch.bfloat16 or not output.is_contiguous() or output.device != device:
        raise InvalidInput(f"{what}: output must be a contiguous BF16 tensor on the device of fp8_data")


def _stream(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


def dequant_fp8_to_bf16(fp8_data, scale: float, shape: Sequence[int]):
    """FP8 E4M3 bytes -> a new BF16 tensor of `shape` (src/ops/fused_inference.rs:89-113)."""
    import torch

    _check_codes(fp8_data, "dequant_fp8_to_bf16")
    out = torch.empty(tuple(shape), dtype=torch.bfloat16, device=fp8_data.device)
    if out.numel() > fp8_data.numel():
        raise InvalidShape(f"dequant_fp8_to_bf16: shape {tuple(shape)} has {out.numel()} elements, fp8_data holds {fp8_data.numel()}")
    ret = _lib.lib().flame_fp8_to_bf16(fp8_data.data_ptr(), out.data_ptr(), float(scale), out.numel(), _stream(out.device))
    if ret != 0:
        raise CudaError(f"fp8_to_bf16 CUDA error: {ret}")
    return out


def dequant_fp8_to_bf16_into(fp8_data, scale: float, output) -> None:
    """FP8 E4M3 bytes -> an existing BF16 tensor, no allocation (src/ops/fused_inference.rs:117-138)."""
    _check_codes(fp8_data, "dequant_fp8_to_bf16_into")
    _check_output(output, fp8_data.device, "dequant_fp8_to_bf16_into")
    if output.numel() > fp8_data.numel():
        raise InvalidShape(f"dequant_fp8_to_bf16_into: output has {output.numel()} elements, fp8_data holds {fp8_data.numel()}")
    ret = _lib.lib().flame_fp8_to_bf16(fp8_data.data_ptr(), output.data_ptr(), float(scale), output.numel(), _stream(output.device))
    if ret != 0:
        raise CudaError(f"fp8_to_bf16_into CUDA error: {ret}")


def dequant_fp8_transpose_into(fp8_data, scale: float, output, m: int, n: int) -> None:
    """[M, N] row-major FP8 bytes -> [N, M] row-major BF16 in `output`, one launch, no allocation
    (src/ops/fused_inference.rs:150-185): `m` rows (out_features) and `n` columns (in_features) of the FP8 input."""
    _check_codes(fp8_data, "dequant_fp8_transpose_into")
    _check_output(output, fp8_data.device, "dequant_fp8_transpose_into")
    expected = m * n
    if output.numel() != expected:
        raise InvalidShape(f"dequant_fp8_transpose_into: output has {output.numel()} elements, expected {expected} (N={n} x M={m})")
    if fp8_data.numel() < expected:
        raise InvalidShape(f"dequant_fp8_transpose_into: fp8_data holds {fp8_data.numel()} bytes, expected {expected}")
    ret = _lib.lib().flame_fused_dequant_transpose_bf16(fp8_data.data_ptr(), output.data_ptr(), float(scale), int(m), int(n),
                                                        _stream(output.device))
    if ret != 0:
        raise CudaError(f"flame_fused_dequant_transpose_bf16 CUDA error: {ret}")


def dequant_fp8_transpose_many(jobs: Iterable[Tuple[object, float, object, int, int]]) -> None:
    """`dequant_fp8_transpose_into` for several weights in one launch: jobs of (fp8_data, scale, output, m, n), all on one
    device.  No counterpart in the reference, which loops over the weights."""
    table, device = [], None
    for fp8_data, scale, output, m, n in jobs:
        _check_codes(fp8_data, "dequant_fp8_transpose_many")
        _check_output(output, fp8_data.device, "dequant_fp8_transpose_many")
        if device is None:
            device = output.device
        elif output.device != device:
            raise InvalidInput("dequant_fp8_transpose_many: all weights must be on one device")
        if output.numel() != m * n or fp8_data.numel() < m * n:
            raise InvalidShape(f"dequant_fp8_transpose_many: output has {output.numel()} elements and fp8_data {fp8_data.numel()} bytes, "
                               f"expected {m * n} (N={n} x M={m})")
        table.append(_lib.WeightJob(fp8_data.data_ptr(), output.data_ptr(), float(scale), int(m), int(n), 0))
    if not table:
        return
    ret = _lib.lib().flame_fused_dequant_transpose_bf16_multi((_lib.WeightJob * len(table))(*table), len(table), _stream(device))
    if ret != 0:
        raise CudaError(f"flame_fused_dequant_transpose_bf16 CUDA error: {ret}")
