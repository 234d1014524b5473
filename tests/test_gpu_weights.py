"""flame_fused_dequant_transpose_bf16 (FP8 weights -> BF16 with the transpose built in) against the oracle, the
committed fixture and, where it was built, the reference's own kernel on the same device buffers.  Bit exact."""
import os
import sys

import numpy as np
import pytest
import torch

from flame_b200 import _lib
from oracle import capi

pytestmark = pytest.mark.gpu
SCALES = [1.0, 0.0123, 3.0e-5, 1.0e30, 1.0e-30, -2.5, 0.0]


def _run(lib, codes: np.ndarray, scale: float, m: int, n: int, dev, in_offset: int = 0, out_offset: int = 0) -> np.ndarray:
    base = torch.zeros(m * n + in_offset + 32, dtype=torch.uint8, device=dev)
    base[in_offset:in_offset + m * n] = torch.from_numpy(np.ascontiguousarray(codes).reshape(-1)).to(dev)
    obase = torch.full((m * n + out_offset + 64,), 0x7F7F, dtype=torch.int16, device=dev)
    out = obase[out_offset:out_offset + m * n]
    rc = lib.flame_fused_dequant_transpose_bf16(base.data_ptr() + in_offset, out.data_ptr(), float(scale), m, n,
                                               torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize(dev)
    assert bool((obase[:out_offset] == 0x7F7F).all()) and bool((obase[out_offset + m * n:] == 0x7F7F).all())   # nothing outside
    return out.cpu().numpy().view(np.uint16).reshape(n, m)


@pytest.mark.parametrize("m,n", [(16, 16), (8, 8), (8, 4), (32, 32), (24, 40), (40, 36), (64, 128), (72, 104), (72, 100), (200, 96), (1024, 3072)])
def test_fast_kernel_equals_the_oracle(cuda_device, m, n):
    lib = _lib.lib()
    rng = np.random.default_rng(m * 1000 + n)
    codes = rng.integers(0, 256, size=(m, n), dtype=np.uint8)
    codes.reshape(-1)[:256] = np.arange(256, dtype=np.uint8)[: min(256, m * n)]     # every code, NaN codes included
    for sc in SCALES[:4] + [-2.5]:
        assert np.array_equal(_run(lib, codes, sc, m, n, cuda_device), capi.fp8_dequant_transpose(codes, sc, m, n)), (m, n, sc)


@pytest.mark.parametrize("m,n,io,oo", [(7, 5, 0, 0), (33, 17, 0, 0), (40, 36, 1, 0), (40, 36, 0, 1), (30, 64, 0, 0), (64, 30, 0, 0), (1, 1, 3, 3),
                                         (65, 129, 0, 0), (200, 63, 5, 1), (1, 300, 0, 0), (300, 1, 0, 3), (131, 197, 2, 0)])
def test_odd_shapes_and_pointers_take_the_fallback_kernel(cuda_device, m, n, io, oo):
    lib = _lib.lib()
    codes = np.random.default_rng(m + n + io).integers(0, 256, size=(m, n), dtype=np.uint8)
    for sc in (1.0, 0.37):
        assert np.array_equal(_run(lib, codes, sc, m, n, cuda_device, io, oo), capi.fp8_dequant_transpose(codes, sc, m, n))


def test_several_weights_in_one_launch(cuda_device):
    """The multi entry point gives every job the bytes of a call of its own: fast and odd shapes mixed, empty jobs skipped,
    more jobs than one launch's table holds, nothing written outside the outputs."""
    import ctypes as C
    lib = _lib.lib()
    rng = np.random.default_rng(11)
    shapes = [(64, 128), (7, 5), (72, 104), (0, 16), (200, 96), (8, 8)] + [(16 + 8 * k, 24 + 8 * (k % 5)) for k in range(18)] + [(1024, 3072)]
    dev, ins, outs, jobs, want = cuda_device, [], [], [], []
    for k, (m, n) in enumerate(shapes):
        codes = rng.integers(0, 256, size=(m, n), dtype=np.uint8)
        sc = SCALES[k % 4]
        src = torch.from_numpy(codes.reshape(-1).copy()).to(dev) if m * n else torch.zeros(8, dtype=torch.uint8, device=dev)
        dst = torch.full((m * n + 64,), 0x7F7F, dtype=torch.int16, device=dev)
        ins.append(src); outs.append(dst)
        jobs.append(_lib.WeightJob(src.data_ptr(), dst.data_ptr(), float(sc), m, n, 0))
        want.append(capi.fp8_dequant_transpose(codes, sc, m, n) if m * n else None)
    arr = (_lib.WeightJob * len(jobs))(*jobs)
    assert lib.flame_fused_dequant_transpose_bf16_multi(arr, len(jobs), torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize(dev)
    for (m, n), dst, w in zip(shapes, outs, want):
        got = dst.cpu().numpy().view(np.uint16)
        assert (got[m * n:] == 0x7F7F).all(), (m, n)
        if w is not None:
            assert np.array_equal(got[:m * n].reshape(n, m), w), (m, n)
    assert lib.flame_fused_dequant_transpose_bf16_multi(None, 0, None) == 0
    assert lib.flame_fused_dequant_transpose_bf16_multi(None, 2, None) == 1
    bad = (_lib.WeightJob * 1)(_lib.WeightJob(None, None, 1.0, 8, 8, 0))
    assert lib.flame_fused_dequant_transpose_bf16_multi(bad, 1, None) == 1
    neg = (_lib.WeightJob * 1)(_lib.WeightJob(ins[0].data_ptr(), outs[0].data_ptr(), 1.0, -8, 8, 0))
    assert lib.flame_fused_dequant_transpose_bf16_multi(neg, 1, None) == 1


def test_empty_and_bad_arguments(cuda_device):
    lib = _lib.lib()
    assert lib.flame_fused_dequant_transpose_bf16(None, None, 1.0, 0, 16, None) == 0
    assert lib.flame_fused_dequant_transpose_bf16(None, None, 1.0, 16, 16, None) == 1          # cudaErrorInvalidValue


def test_committed_fixture_of_the_reference_kernel(cuda_device, golden_dir):
    path = os.path.join(golden_dir, "fp8_weight_reference_kernel_sm100.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated yet")
    z = np.load(path)
    sys.path.insert(0, golden_dir)
    from make_reference_kernel_golden import weight_inputs

    lib = _lib.lib()
    for name, (codes, m, n) in weight_inputs().items():
        for k, sc in enumerate(z["scales"]):
            assert np.array_equal(_run(lib, codes, sc, m, n, cuda_device), z[name][k]), (name, float(sc))


def test_equals_the_reference_kernel_on_this_gpu(cuda_device):
    ref = capi.load_ref_cuda()
    if ref is None or not hasattr(ref, "flame_fused_dequant_transpose_bf16"):
        pytest.skip("oracle/_ref/libflame_ref_cuda.so was not built with the weight kernel")
    lib = _lib.lib()
    rng = np.random.default_rng(9)
    for m, n in ((16, 16), (96, 160), (3072, 1024), (37, 53)):
        codes = rng.integers(0, 256, size=(m, n), dtype=np.uint8)
        codes.reshape(-1)[:256] = np.arange(256, dtype=np.uint8)
        c = torch.from_numpy(codes).to(cuda_device)
        for sc in SCALES:
            want = torch.empty(m * n, dtype=torch.int16, device=cuda_device)
            assert ref.flame_fused_dequant_transpose_bf16(c.data_ptr(), want.data_ptr(), float(sc), m, n, None) == 0
            torch.cuda.synchronize()
            got = _run(lib, codes, sc, m, n, cuda_device)
            assert np.array_equal(got, want.cpu().numpy().view(np.uint16).reshape(n, m)), (m, n, sc)


def test_host_functions_of_the_inference_path(cuda_device):
    """dequant_fp8_to_bf16 / _into / dequant_fp8_transpose_into / _many (src/ops/fused_inference.rs:86-185) over torch
    tensors: the oracle's bytes, the reference's shape error, nothing allocated by the `_into` forms."""
    from flame_b200 import InvalidInput, InvalidShape, fused_inference as fi

    rng = np.random.default_rng(3)
    m, n, scale = 72, 104, 0.37
    codes = rng.integers(0, 256, size=(m, n), dtype=np.uint8)
    dev_codes = torch.from_numpy(codes).to(cuda_device)
    want_t = capi.fp8_dequant_transpose(codes, scale, m, n)
    want = capi.fp8_to_bf16(codes.reshape(-1), scale).reshape(m, n)                 # the element-wise decoder, src/cuda/fp8_dequant.cu
    out_t = torch.empty(n, m, dtype=torch.bfloat16, device=cuda_device)
    fi.dequant_fp8_transpose_into(dev_codes, scale, out_t, m, n)
    plain = fi.dequant_fp8_to_bf16(dev_codes, scale, (m, n))
    into = torch.empty(m, n, dtype=torch.bfloat16, device=cuda_device)
    torch.cuda.synchronize(cuda_device)
    before = torch.cuda.memory_allocated(cuda_device)
    fi.dequant_fp8_to_bf16_into(dev_codes, scale, into)
    fi.dequant_fp8_transpose_into(dev_codes, scale, out_t, m, n)
    assert torch.cuda.memory_allocated(cuda_device) == before
    torch.cuda.synchronize(cuda_device)
    assert np.array_equal(out_t.view(torch.int16).cpu().numpy().view(np.uint16), want_t)
    assert np.array_equal(plain.view(torch.int16).cpu().numpy().view(np.uint16), want)
    assert torch.equal(plain.view(torch.int16), into.view(torch.int16))
    outs = [torch.empty(n, m, dtype=torch.bfloat16, device=cuda_device) for _ in range(3)]
    fi.dequant_fp8_transpose_many([(dev_codes, scale, o, m, n) for o in outs])
    fi.dequant_fp8_transpose_many([])
    torch.cuda.synchronize(cuda_device)
    for o in outs:
        assert torch.equal(o.view(torch.int16), out_t.view(torch.int16))
    with pytest.raises(InvalidShape, match=r"expected %d \(N=%d x M=%d\)" % (m * n, n, m)):
        fi.dequant_fp8_transpose_into(dev_codes, scale, torch.empty(n, m + 1, dtype=torch.bfloat16, device=cuda_device), m, n)
    with pytest.raises(InvalidInput):
        fi.dequant_fp8_transpose_into(dev_codes.to(torch.int32), scale, out_t, m, n)
    with pytest.raises(InvalidInput):
        fi.dequant_fp8_to_bf16_into(dev_codes, scale, torch.empty(m, n, dtype=torch.float32, device=cuda_device))
