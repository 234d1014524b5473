"""ctypes binding of ``oracle/codec_oracle.c`` (test infrastructure only).

``load()`` builds ``liboracle.so`` with gcc when it is missing or older than
its source.  ``load_ref_encoder()`` returns the reference project's own FP8
encoder body (src/cuda/fp8_quant.cu:19-57) compiled from its source by
``oracle/Makefile`` into ``oracle/_ref``, or ``None`` when that file was not
built (the reference checkout is not present on every machine).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

INT8_MUL_INV = 1
FP8_OCP = 1
CODEC_NONE, CODEC_INT8, CODEC_FP8 = 0, 2, 3


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "codec_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return so


def load() -> C.CDLL:
    global _LIB
    if _LIB is None:
        lib = C.CDLL(build())
        vp, sz, u, i, f = C.c_void_p, C.c_size_t, C.c_uint, C.c_int, C.c_float
        sigs = {
            "oracle_bf16_to_f32": (f, [C.c_uint16]),
            "oracle_f32_to_bf16": (C.c_uint16, [f]),
            "oracle_fp8_e4m3_encode_ref": (C.c_uint8, [f]),
            "oracle_fp8_e4m3_encode_bits": (C.c_uint8, [f]),
            "oracle_fp8_e4m3_encode_ocp": (C.c_uint8, [f]),
            "oracle_fp8_e4m3_decode": (f, [C.c_uint8]),
            "oracle_bf16_to_fp8": (None, [vp, vp, f, sz]),
            "oracle_fp8_to_bf16": (None, [vp, vp, f, sz]),
            "oracle_quant_int8_b128": (None, [vp, vp, vp, sz, u]),
            "oracle_dequant_int8_b128": (None, [vp, vp, vp, sz]),
            "oracle_quant_fp8_b128": (None, [vp, vp, vp, sz, u]),
            "oracle_dequant_fp8_b128": (None, [vp, vp, vp, sz]),
            "oracle_packed_scales_offset": (sz, [sz]),
            "oracle_packed_bytes": (sz, [sz]),
            "oracle_pack": (None, [vp, vp, sz, i, u]),
            "oracle_unpack": (None, [vp, vp, sz, i]),
            "oracle_roundtrip_mt": (i, [vp, vp, vp, sz, i, u, i, i]),
            "oracle_fp8_encode_sweep": (C.c_uint64, [vp, C.c_uint64, C.c_uint64, C.c_uint64, vp]),
            "oracle_fp8_encode_many": (None, [vp, vp, sz, i]),
            "oracle_fp8_weight_decode": (f, [C.c_uint8]),
            "oracle_fp8_dequant_transpose": (None, [vp, vp, f, i, i]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _LIB = lib
    return _LIB


def fp8_encode_many(y, form: int = 1) -> np.ndarray:
    """form 0 = frexpf control flow, 1 = integer restatement, 2 = OCP RNE/saturating."""
    y = np.ascontiguousarray(y, np.float32).reshape(-1)
    out = np.empty(y.size, np.uint8)
    load().oracle_fp8_encode_many(_p(y), _p(out), y.size, form)
    return out


def fp8_encode_sweep(other_fn, lo: int, hi: int, stride: int):
    """Count binary32 patterns in [lo,hi) step `stride` where form B != other_fn. Returns (bad, first_bad)."""
    first = C.c_uint32(0)
    bad = load().oracle_fp8_encode_sweep(C.cast(other_fn, C.c_void_p), lo, hi, stride, C.cast(C.pointer(first), C.c_void_p))
    return int(bad), int(first.value)


def load_ref_decoder():
    """The reference's FP8 decode arithmetic (src/cuda/fp8_dequant.cu:21-34) compiled from its source, or None."""
    so = os.path.join(_HERE, "_ref", "libfp8dec_ref.so")
    if not os.path.exists(so):
        return None
    lib = C.CDLL(so)
    fn = lib.fp8_e4m3_decode_ref
    fn.restype, fn.argtypes = C.c_float, [C.c_ubyte]
    return fn


def load_ref_encoder():
    """f32_to_fp8_e4m3 compiled from the reference's own source, or None."""
    so = os.path.join(_HERE, "_ref", "libfp8enc_ref.so")
    if not os.path.exists(so):
        return None
    lib = C.CDLL(so)
    fn = lib.f32_to_fp8_e4m3
    fn.restype, fn.argtypes = C.c_ubyte, [C.c_float]
    return fn


_REF_CUDA = None


def load_ref_cuda():
    """The reference's own CUDA files of this path (src/cuda/fp8_quant.cu, fp8_dequant.cu, pinned_host.cu)
    compiled unmodified by ``make -C oracle refcuda``, or None when that library was not built.

    Its symbols carry the same names as the shipped library's legacy entry points, so it is opened
    RTLD_LOCAL and used only through the handle returned here (GPU tests, and the bench's reference-kernel
    timing)."""
    global _REF_CUDA
    so = os.path.join(_HERE, "_ref", "libflame_ref_cuda.so")
    if not os.path.exists(so):
        return None
    if _REF_CUDA is None:
        lib = C.CDLL(so, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        vp, sz, u, i, f = C.c_void_p, C.c_size_t, C.c_uint, C.c_int, C.c_float
        lib.flame_bf16_to_fp8.restype, lib.flame_bf16_to_fp8.argtypes = i, [vp, vp, f, sz, vp]
        lib.flame_fp8_to_bf16.restype, lib.flame_fp8_to_bf16.argtypes = i, [vp, vp, f, sz, vp]
        lib.flame_cuda_alloc_pinned_host.restype, lib.flame_cuda_alloc_pinned_host.argtypes = vp, [sz, u]
        lib.flame_cuda_free_pinned_host.restype, lib.flame_cuda_free_pinned_host.argtypes = i, [vp]
        lib.flame_cuda_memcpy_async.restype, lib.flame_cuda_memcpy_async.argtypes = i, [vp, vp, sz, i, vp]
        if hasattr(lib, "flame_fused_dequant_transpose_bf16"):   # src/cuda/fused_dequant_transpose.cu, built into the same library
            lib.flame_fused_dequant_transpose_bf16.restype, lib.flame_fused_dequant_transpose_bf16.argtypes = i, [vp, vp, f, i, i, vp]
        if hasattr(lib, "flame_fused_rms_norm_bf16"):      # src/cuda/fused_rms_norm.cu, built into the same library
            lib.flame_fused_rms_norm_bf16.restype, lib.flame_fused_rms_norm_bf16.argtypes = i, [vp, vp, vp, i, i, f, vp]
        _REF_CUDA = lib
    return _REF_CUDA


_REF_SAGE = None


def load_ref_sage():
    """The reference's own int8 quantisation kernel (sage_quantize_tensor, src/sage_attention.rs:510-543) compiled by
    ``make -C oracle refsage`` behind a small launcher, or None.  ``sage_quantize_ref(in_f32, out_s8, scales, rows,
    row_size, stream)`` with row_size 128 quantises per 128-element block."""
    global _REF_SAGE
    so = os.path.join(_HERE, "_ref", "libsage_quant_ref.so")
    if not os.path.exists(so):
        return None
    if _REF_SAGE is None:
        lib = C.CDLL(so, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        lib.sage_quantize_ref.restype = C.c_int
        lib.sage_quantize_ref.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        _REF_SAGE = lib
    return _REF_SAGE


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _u16(x) -> np.ndarray:
    a = np.ascontiguousarray(x)
    assert a.dtype == np.uint16, "BF16 tensors are passed as uint16 bit patterns"
    return a.reshape(-1)


def nblocks(n: int) -> int:
    return (n + 127) // 128


def quant_int8_b128(x_bits, flags: int = 0):
    x = _u16(x_bits)
    codes = np.empty(x.size, np.int8)
    scales = np.empty(nblocks(x.size), np.float32)
    load().oracle_quant_int8_b128(_p(x), _p(codes), _p(scales), x.size, flags)
    return codes, scales


def dequant_int8_b128(codes, scales):
    codes = np.ascontiguousarray(codes, np.int8).reshape(-1)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.empty(codes.size, np.uint16)
    load().oracle_dequant_int8_b128(_p(codes), _p(scales), _p(out), codes.size)
    return out


def quant_fp8_b128(x_bits, flags: int = 0):
    x = _u16(x_bits)
    codes = np.empty(x.size, np.uint8)
    scales = np.empty(nblocks(x.size), np.float32)
    load().oracle_quant_fp8_b128(_p(x), _p(codes), _p(scales), x.size, flags)
    return codes, scales


def dequant_fp8_b128(codes, scales):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.empty(codes.size, np.uint16)
    load().oracle_dequant_fp8_b128(_p(codes), _p(scales), _p(out), codes.size)
    return out


def bf16_to_fp8(x_bits, inv_scale: float):
    x = _u16(x_bits)
    out = np.empty(x.size, np.uint8)
    load().oracle_bf16_to_fp8(_p(x), _p(out), np.float32(inv_scale), x.size)
    return out


def fp8_to_bf16(codes, scale: float):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    out = np.empty(codes.size, np.uint16)
    load().oracle_fp8_to_bf16(_p(codes), _p(out), np.float32(scale), codes.size)
    return out


def fp8_dequant_transpose(codes, scale: float, m: int, n: int):
    """[m, n] FP8 weight codes -> [n, m] BF16 bits with the decoder of src/cuda/fused_dequant_transpose.cu."""
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    assert codes.size == m * n
    out = np.empty(m * n, np.uint16)
    load().oracle_fp8_dequant_transpose(_p(codes), _p(out), np.float32(scale), m, n)
    return out.reshape(n, m)


def packed_bytes(n: int) -> int:
    return load().oracle_packed_bytes(n)


def packed_scales_offset(n: int) -> int:
    return load().oracle_packed_scales_offset(n)


def roundtrip_mt(x_bits, codec: int, threads: int, flags: int = 0, do_unpack: bool = True):
    """Quantise+pack then unpack+dequantise on `threads` host threads; returns (packed, out)."""
    x = _u16(x_bits)
    nbytes = 2 * x.size if codec == CODEC_NONE else packed_bytes(x.size)
    packed = np.empty(nbytes, np.uint8)
    out = np.empty(x.size, np.uint16)
    rc = load().oracle_roundtrip_mt(_p(x), _p(packed), _p(out), x.size, codec, flags, threads, int(do_unpack))
    if rc != 0:
        raise MemoryError("oracle_roundtrip_mt failed")
    return packed, out
