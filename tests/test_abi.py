"""The C-ABI library loads and exports every symbol the header declares; host-only entry points work (CPU only)."""
import ctypes as C
import os
import re

import pytest

from flame_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flame_offload.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flame_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_symbols():
    names = _declared_symbols()
    for legacy in ("flame_cuda_alloc_pinned_host", "flame_cuda_free_pinned_host", "flame_cuda_memcpy_async",
                   "flame_cuda_host_register", "flame_cuda_host_unregister", "flame_bf16_to_fp8", "flame_fp8_to_bf16",
                   "flame_h2d_async", "flame_d2h_async", "flame_d2d_async"):
        assert legacy in names


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    _lib.lib()  # sets every prototype; raises if one is absent


def test_struct_sizes_match_the_header():
    assert C.sizeof(_lib.Handle) == 16
    assert C.sizeof(_lib.PoolConfig) == 80
    assert C.sizeof(_lib.Stats) == 19 * 8
    assert C.sizeof(_lib.SlotInfo) == 40
    assert C.sizeof(_lib.PolicyTensor) == 24
    assert C.sizeof(_lib.PolicyInput) == 72
    assert C.sizeof(_lib.WeightJob) == 32


def test_packed_size_helpers():
    lib = _lib.lib()
    assert lib.flame_act_packed_bytes(12582912) == 12976128
    assert lib.flame_act_packed_scales_offset(1000) == 1024
    assert lib.flame_act_packed_bytes(1000) == 1024 + 32


def test_constructor_argument_errors_need_no_gpu():
    """num_slots == 0 / max_bytes == 0 are rejected before any CUDA call (src/activation_offload.rs:371-380)."""
    lib = _lib.lib()
    assert not lib.flame_offload_pool_create(0, 1024, 0, None)
    assert "num_slots must be > 0" in _lib.last_error()
    assert not lib.flame_offload_pool_create(2, 0, 0, None)
    assert "max_bytes must be > 0" in _lib.last_error()
    assert not lib.flame_offload_pool_create(2, 1024, 9, None)
    assert "unknown compression" in _lib.last_error()


def test_status_copy_entry_points_reject_null_without_cuda():
    lib = _lib.lib()
    assert lib.flame_h2d_async(None, None, 16, None) == _lib.ERR_INVALID
    assert lib.flame_d2h_async(1, 1, 0, None) == _lib.ERR_INVALID
    assert lib.flame_bf16_to_fp8(None, None, 1.0, 0, None) == 0  # n == 0 returns at once, as the reference does


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.lib()


def _cc(*args):
    import subprocess
    return subprocess.run(list(args), capture_output=True, text=True)


def test_header_is_valid_c99_and_cxx():
    """The boundary is a C header: it must compile on its own as pedantic C99 and as C++."""
    hdr = os.path.join(ROOT, "include", "flame_offload.h")
    r = _cc("gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c", hdr)
    assert r.returncode == 0, r.stderr
    r = _cc("g++", "-std=c++11", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c++", hdr)
    assert r.returncode == 0, r.stderr


def build_c_caller(out_path: str):
    """Compiles tests/helpers/abi_roundtrip.c (a caller in plain C) against the header and both libraries."""
    from oracle import capi
    capi.build()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return _cc("gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", os.path.join(ROOT, "tests", "helpers", "abi_roundtrip.c"),
               "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
               "-L", os.path.join(ROOT, "flame_b200"), "-lflame_offload", "-L", os.path.join(ROOT, "oracle"), "-loracle",
               "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm", "-o", out_path)


def test_plain_c_caller_compiles_and_links(tmp_path):
    r = build_c_caller(str(tmp_path / "abi_roundtrip"))
    assert r.returncode == 0, r.stderr
