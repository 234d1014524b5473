"""The entry point that allocates nothing: flame_act_offload_packed_noalloc.

It exists for callers that must spill an activation at a moment when they cannot
allocate (an out-of-memory handler, or a step loop whose memory plan is fixed and
where cudaMalloc/cudaFree would stall the device or fail).  Its device staging is
an array built into the library, shared by all calls and never cleared between
them, so this test makes two calls in a row (the second one smaller, with other
data) and checks each against the ordinary quantise entry point: same codes, same
scales, zero padding in between.  Collected last on purpose: if it fails, a run
that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from flame_b200 import _lib, synthetic

pytestmark = pytest.mark.gpu

INT8, FP8 = 2, 3
MAX_ELEMS = 8 << 20


def _reference_packed(lib, x: torch.Tensor, codec: int, flags: int) -> np.ndarray:
    """Packed bytes built from the existing entry point's separate codes and scales."""
    n = x.numel()
    codes = torch.empty(n, dtype=torch.uint8, device=x.device)
    scales = torch.empty((n + 127) // 128, dtype=torch.float32, device=x.device)
    fn = lib.flame_act_quant_int8_b128 if codec == INT8 else lib.flame_act_quant_fp8_b128
    assert fn(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, flags, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    so = lib.flame_act_packed_scales_offset(n)
    packed = np.zeros(lib.flame_act_packed_bytes(n), np.uint8)
    packed[:n] = codes.cpu().numpy()
    packed[so:] = scales.cpu().numpy().view(np.uint8)
    return packed


@pytest.mark.parametrize("codec", [INT8, FP8])
def test_two_calls_in_a_row_match_the_allocating_entry_point(cuda_device, codec):
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    host = torch.empty(lib.flame_act_packed_bytes(MAX_ELEMS), dtype=torch.uint8).pin_memory()
    # second call is smaller and ragged: stale bytes of the first call lie behind it in the shared array
    for n, seed in ((3 * 8192 * 40 + 77, 11), (8192 * 7 + 1001, 12)):
        bits = synthetic.normal_with_outliers(n, seed=seed)
        x = torch.from_numpy(bits.view(np.int16)).to(cuda_device).view(torch.bfloat16)
        host.fill_(0xEE)
        rc = lib.flame_act_offload_packed_noalloc(x.data_ptr(), host.data_ptr(), n, codec, 0, stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        nbytes = lib.flame_act_packed_bytes(n)
        got = host.numpy()[:nbytes]
        want = _reference_packed(lib, x, codec, 0)
        assert np.array_equal(got, want)                     # bit exact, padding included
        assert bool((host.numpy()[nbytes:nbytes + 4096] == 0xEE).all())  # nothing written past the result


def test_after_a_warm_up_call_no_device_memory_is_taken(cuda_device):
    """The array, and the kernels, take their device memory when they are first used on a device (CUDA loads a
    library's modules lazily), not when the library is opened: that is what the warm-up call at start-up is for.
    After it, a call changes nothing in what the device has free: aligned input (the tiled kernel) and an input
    that starts one element off a 32-byte boundary (the element-wise kernel), both codecs."""
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    n = 8192 * 5 + 300
    base = torch.randn(n + 1, device=cuda_device).to(torch.bfloat16)
    out = torch.empty(lib.flame_act_packed_bytes(n), dtype=torch.uint8, device=cuda_device)
    inputs = [base[:n], base[1:]]
    for codec in (INT8, FP8):                                   # the warm-up: one call per codec and kernel kind
        for x in inputs:
            assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), n, codec, 0, stream) == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(cuda_device)
    for codec in (INT8, FP8):
        for x in inputs:
            assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), n, codec, 0, stream) == 0
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), _reference_packed(lib, x, codec, 0))
    free1, _ = torch.cuda.mem_get_info(cuda_device)
    # out.cpu() and the reference entry point go through torch's caching allocator, which may grow; a second pass
    # with everything cached must leave the free figure where it is
    for codec in (INT8, FP8):
        for x in inputs:
            assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), n, codec, 0, stream) == 0
    torch.cuda.synchronize()
    free2, _ = torch.cuda.mem_get_info(cuda_device)
    assert free2 == free1, (free0, free1, free2)


def test_device_output_and_largest_size(cuda_device):
    lib = _lib.lib()
    n = MAX_ELEMS
    x = torch.randn(n, device=cuda_device).to(torch.bfloat16)
    out = torch.empty(lib.flame_act_packed_bytes(n), dtype=torch.uint8, device=cuda_device)
    assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), n, INT8, 0, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), _reference_packed(lib, x, INT8, 0))


def test_sizes_beyond_the_built_in_scratch_are_refused(cuda_device):
    lib = _lib.lib()
    x = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)
    out = torch.zeros(64, dtype=torch.uint8, device=cuda_device)
    assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), MAX_ELEMS + 1, INT8, 0, None) == 1
    assert "exceed the built-in scratch" in _lib.last_error()
    assert lib.flame_act_offload_packed_noalloc(x.data_ptr(), out.data_ptr(), 16, 7, 0, None) == 1
    assert lib.flame_act_offload_packed_noalloc(None, None, 0, INT8, 0, None) == 0
    assert not out.any()
