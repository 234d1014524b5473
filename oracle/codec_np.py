"""numpy restatement of the codec arithmetic (test infrastructure only).

Written independently of ``codec_oracle.c`` so that the two can check each
other.  All arithmetic is IEEE binary32 (numpy float32 ops are single, separately
rounded operations).  Reference lines restated:

* FP8 E4M3 encoder, src/cuda/fp8_quant.cu:19-57 -> :func:`fp8_encode_ref`
* FP8 E4M3 decoder, src/cuda/fp8_dequant.cu:20-36 -> :func:`fp8_decode`
* int8 formula, src/sage_attention.rs:524-541 -> :func:`quant_int8_b128`
* fixed-scale calls, src/activation_offload.rs:543-561 -> :func:`bf16_to_fp8`
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(F32)


def f32_to_bf16(x) -> np.ndarray:
    b = np.asarray(x, F32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b.astype(np.uint64) + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, np.uint16(0x7FFF), r)


def fp8_encode_ref(y) -> np.ndarray:
    """Round-half-up mantissa, >= 248 -> 0x7F, sub-normals by (int)(v*512+0.5) clamped to 7."""
    y = np.asarray(y, F32)
    b = y.view(np.uint32)
    a = b & 0x7FFFFFFF
    t = ((a.astype(np.uint64) + 0x80000) >> 20).astype(np.int64) - 960
    c = np.where(t >= 120, 0x7F, t)
    v = a.view(F32)
    with np.errstate(all="ignore"):
        w = (v * F32(512.0) + F32(0.5)).astype(F32)
    small = a < 0x3C800000
    sub = np.minimum(np.floor(np.where(small, w, 0)).astype(np.int64), 7)
    c = np.where(small, sub, c)
    s = np.where(y < 0, 0x80, 0)
    nan = a > 0x7F800000   # the reference's arithmetic ends at 0x30 for NaN (see codec_oracle.c, form A)
    return np.where(nan, 0x30, s | c).astype(np.uint8)


def fp8_decode(c) -> np.ndarray:
    c = np.asarray(c, np.uint8).astype(np.int32)
    e, m = (c >> 3) & 0xF, c & 7
    mag = np.where(e == 0, np.ldexp(m / 8.0, -6), np.ldexp(1.0 + m / 8.0, e - 7)).astype(F32)
    return np.where((c >> 7) == 1, -mag, mag).astype(F32)


def _fp8_code_of(x, inv) -> np.ndarray:
    """Block codecs: enc(x*inv); a zero element stays zero when inv is infinite; a NaN result saturates with x's sign bit."""
    x = np.asarray(x, F32)
    with np.errstate(all="ignore"):
        y = np.where(x == 0, x, (x * inv).astype(F32)).astype(F32)
    c = fp8_encode_ref(np.where(np.isnan(y), F32(0), y))
    nan_code = ((x.view(np.uint32) >> 24) & 0x80 | 0x7F).astype(np.uint8)
    return np.where(np.isnan(y), nan_code, c).astype(np.uint8)


def _blocks(x: np.ndarray) -> np.ndarray:
    n = x.size
    pad = (-n) % 128
    return np.concatenate([x, np.zeros(pad, F32)]).reshape(-1, 128)


def _absmax(xb: np.ndarray) -> np.ndarray:
    return np.fmax.reduce(np.abs(xb), axis=1, initial=F32(0)).astype(F32)  # fmax ignores NaN


def quant_int8_b128(bits, mul_inv: bool = False):
    x = bf16_to_f32(np.asarray(bits).reshape(-1))
    n = x.size
    xb = _blocks(x)
    amax = _absmax(xb)
    scale = (amax / F32(127.0)).astype(F32)
    with np.errstate(all="ignore"):
        if mul_inv:
            q = (xb * (F32(1.0) / scale)[:, None]).astype(F32)
        else:
            q = (xb / scale[:, None]).astype(F32)
        r = np.rint(q)
    r = np.where(np.isnan(r), 0, np.clip(r, -127, 127))
    r = np.where((amax == 0)[:, None], 0, r)
    return r.astype(np.int8).reshape(-1)[:n], scale


def dequant_int8_b128(codes, scales):
    codes = np.asarray(codes, np.int8).reshape(-1)
    s = np.repeat(np.asarray(scales, F32), 128)[: codes.size]
    return f32_to_bf16(codes.astype(F32) * s)


def quant_fp8_b128(bits):
    x = bf16_to_f32(np.asarray(bits).reshape(-1))
    n = x.size
    xb = _blocks(x)
    amax = _absmax(xb)
    scale = (amax / F32(448.0)).astype(F32)
    with np.errstate(all="ignore"):
        inv = (F32(1.0) / scale).astype(F32)
    c = _fp8_code_of(xb, inv[:, None])
    c = np.where((amax == 0)[:, None], 0, c).astype(np.uint8)
    return c.reshape(-1)[:n], scale


def dequant_fp8_b128(codes, scales):
    codes = np.asarray(codes, np.uint8).reshape(-1)
    s = np.repeat(np.asarray(scales, F32), 128)[: codes.size]
    with np.errstate(all="ignore"):
        return f32_to_bf16(fp8_decode(codes) * s)


def bf16_to_fp8(bits, inv_scale):
    """src/cuda/fp8_quant.cu:69-70: the code of the plain product."""
    with np.errstate(all="ignore"):
        return fp8_encode_ref((bf16_to_f32(bits) * F32(inv_scale)).astype(F32))


def fp8_to_bf16(codes, scale):
    with np.errstate(all="ignore"):
        return f32_to_bf16(fp8_decode(codes) * F32(scale))
