"""Helpers for the GPU tests: raw C-ABI calls on torch-owned device memory."""
import numpy as np
import torch

from flame_b200 import _lib


def to_dev(bits: np.ndarray, device, offset_elems: int = 0) -> torch.Tensor:
    """uint16 BF16 bit patterns -> torch.bfloat16 tensor; optional element offset to break alignment."""
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16))
    if offset_elems:
        base = torch.empty(t.numel() + offset_elems, dtype=torch.int16, device=device)
        base[offset_elems:] = t.to(device)
        return base[offset_elems:].view(torch.bfloat16)
    return t.to(device).view(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def quant(codec: str, x: torch.Tensor, flags: int = 0, code_offset: int = 0, scale_offset: int = 0):
    """Runs flame_act_quant_{int8,fp8}_b128; returns (codes uint8 tensor, scales float32 tensor)."""
    n = x.numel()
    codes_base = torch.full((n + code_offset + 64,), 0xAB, dtype=torch.uint8, device=x.device)
    scales_base = torch.full(((n + 127) // 128 + scale_offset + 16,), -7.0, dtype=torch.float32, device=x.device)
    codes = codes_base[code_offset:code_offset + n]
    scales = scales_base[scale_offset:scale_offset + (n + 127) // 128]
    fn = getattr(_lib.lib(), f"flame_act_quant_{codec}_b128")
    rc = fn(x.data_ptr() if n else None, codes.data_ptr() if n else None, scales.data_ptr() if n else None, n, flags,
            stream_ptr(x.device))
    assert rc == 0, rc
    torch.cuda.synchronize(x.device)
    # canaries: nothing outside [0, n) may be written
    assert bool((codes_base[:code_offset] == 0xAB).all()) and bool((codes_base[code_offset + n:] == 0xAB).all())
    assert bool((scales_base[:scale_offset] == -7.0).all()) and bool((scales_base[scale_offset + scales.numel():] == -7.0).all())
    return codes, scales


def dequant(codec: str, codes: torch.Tensor, scales: torch.Tensor, n: int, out_offset: int = 0) -> torch.Tensor:
    base = torch.full((n + out_offset + 64,), 0x7F7F, dtype=torch.int16, device=codes.device)
    out = base[out_offset:out_offset + n]
    fn = getattr(_lib.lib(), f"flame_act_dequant_{codec}_b128")
    rc = fn(codes.data_ptr() if n else None, scales.data_ptr() if n else None, out.data_ptr() if n else None, n,
            stream_ptr(codes.device))
    assert rc == 0, rc
    torch.cuda.synchronize(codes.device)
    assert bool((base[:out_offset] == 0x7F7F).all()) and bool((base[out_offset + n:] == 0x7F7F).all())
    return out.view(torch.bfloat16)
