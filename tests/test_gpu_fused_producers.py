"""RMSNorm / SwiGLU with the compress step built in, push_packed, and the checkpoint path that uses them."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from flame_b200 import ActivationOffloadPool, InvalidOperation, OffloadCompression, Unsupported, _lib, fused_producers
from flame_b200 import checkpoint as ckpt
from oracle import capi
from tests import gpu_util as G

pytestmark = pytest.mark.gpu
INT8, FP8 = 2, 3
# BF16 keeps 8 significant bits: two correctly rounded results of slightly different fp32 values differ by one unit
# in the last place, 2^-8 relative at most (2^-7 across a binade edge).
ONE_ULP = 2.0 ** -7


def _oracle(codec, bits):
    return (capi.quant_int8_b128 if codec == INT8 else capi.quant_fp8_b128)(bits)


@pytest.mark.parametrize("rows,cols", [(37, 3072), (5, 128), (64, 1024), (3, 16384)])
@pytest.mark.parametrize("codec", [0, INT8, FP8])
def test_rmsnorm_with_codes(cuda_device, rows, cols, codec):
    g = torch.Generator(device=cuda_device).manual_seed(rows * cols)
    x = (torch.randn(rows, cols, device=cuda_device, generator=g) * 3).to(torch.bfloat16)
    x[0, :7] = 40.0                                     # an outlier block
    w = (1 + 0.1 * torch.randn(cols, device=cuda_device, generator=g)).to(torch.bfloat16)
    with fused_producers.emit_codes(codec):
        y, rstd = fused_producers.rmsnorm(x, w, 1e-6)
        got = fused_producers.take(y)
    torch.cuda.synchronize()
    xf = x.float()
    want_rstd = torch.rsqrt(xf.pow(2).mean(-1) + 1e-6)
    want = (xf * want_rstd[:, None] * w.float()).to(torch.bfloat16)
    assert torch.allclose(rstd, want_rstd, rtol=1e-5, atol=0)
    assert torch.allclose(y.float(), want.float(), rtol=ONE_ULP, atol=1e-30)
    assert (y != want).float().mean() < 0.02            # and almost all elements are identical
    if codec == 0:
        assert got is None
        return
    codes, scales = got
    wc, ws = _oracle(codec, G.bits_of(y).reshape(-1))   # the codes must be those of the BF16 tensor that was written
    assert np.array_equal(codes.cpu().numpy(), wc.view(np.uint8))
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    assert fused_producers.take(y) is None              # handed out once


@pytest.mark.parametrize("rows,cols", [(64, 3072), (9, 128), (17, 4096)])
def test_rmsnorm_against_the_reference_kernel_on_this_gpu(cuda_device, rows, cols):
    """src/cuda/fused_rms_norm.cu compiled unmodified: the same formula with another summation order, so the two BF16
    outputs may differ by one unit in the last place where the fp32 values straddle a rounding boundary."""
    ref = capi.load_ref_cuda()
    if ref is None or not hasattr(ref, "flame_fused_rms_norm_bf16"):
        pytest.skip("oracle/_ref/libflame_ref_cuda.so with the RMSNorm kernel was not built")
    g = torch.Generator(device=cuda_device).manual_seed(cols)
    x = (torch.randn(rows, cols, device=cuda_device, generator=g) * 2).to(torch.bfloat16)
    w = (1 + 0.2 * torch.randn(cols, device=cuda_device, generator=g)).to(torch.bfloat16)
    y, _ = fused_producers.rmsnorm(x, w, 1e-6)
    theirs = torch.empty_like(x)
    assert ref.flame_fused_rms_norm_bf16(x.data_ptr(), w.data_ptr(), theirs.data_ptr(), rows, cols, 1e-6, G.stream_ptr(cuda_device)) == 0
    torch.cuda.synchronize()
    assert torch.allclose(y.float(), theirs.float(), rtol=ONE_ULP, atol=1e-30)
    assert (y != theirs).float().mean() < 0.02


@pytest.mark.parametrize("rows,hidden", [(33, 9216), (7, 128), (129, 512)])
@pytest.mark.parametrize("codec", [0, INT8, FP8])
def test_swiglu_with_codes(cuda_device, rows, hidden, codec):
    g = torch.Generator(device=cuda_device).manual_seed(rows + hidden)
    gu = (torch.randn(rows, 2 * hidden, device=cuda_device, generator=g) * 2).to(torch.bfloat16)
    gu[0, :3] = -30.0
    gu[0, hidden:hidden + 3] = 55.0
    with fused_producers.emit_codes(codec):
        h = fused_producers.swiglu(gu)
        got = fused_producers.take(gu)
    torch.cuda.synchronize()
    gf, uf = gu.float().chunk(2, dim=-1)
    want = (F.silu(gf) * uf).to(torch.bfloat16)
    assert torch.allclose(h.float(), want.float(), rtol=ONE_ULP, atol=1e-12)
    assert (h != want).float().mean() < 0.02
    if codec == 0:
        assert got is None
        return
    codes, scales = got
    wc, ws = _oracle(codec, G.bits_of(gu).reshape(-1))
    assert np.array_equal(codes.cpu().numpy(), wc.view(np.uint8))
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), ws.view(np.uint32))


def test_shapes_the_kernels_refuse(cuda_device):
    lib = _lib.lib()
    x = torch.zeros(4, 200, dtype=torch.bfloat16, device=cuda_device)
    w = torch.ones(200, dtype=torch.bfloat16, device=cuda_device)
    y = torch.empty_like(x)
    assert lib.flame_act_rmsnorm_quant_b128(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, None, None, 4, 200, 1e-6, 0, 0, None) == 1
    assert "cols % 128" in _lib.last_error()
    assert lib.flame_act_rmsnorm_quant_b128(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, None, None, 4, 128, 1e-6, INT8, 0, None) == 1  # codes missing
    assert lib.flame_act_swiglu_quant_b128(x.data_ptr(), y.data_ptr(), None, None, 4, 100, 0, 0, None) == 1
    assert lib.flame_act_rmsnorm_quant_b128(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, None, None, 0, 128, 1e-6, 0, 0, None) == 0   # nothing to do


@pytest.mark.parametrize("mode,codec", [(OffloadCompression.INT8_B128, INT8), (OffloadCompression.FP8_B128, FP8)])
def test_push_packed_round_trip(cuda_device, mode, codec):
    n = 300000 + 128 * 3
    bits = np.random.default_rng(1).integers(0, 1 << 16, n, dtype=np.uint16)
    bits[(bits & 0x7F80) == 0x7F80] = 0x3F80
    x = G.to_dev(bits, cuda_device)
    codes, scales = G.quant("int8" if codec == INT8 else "fp8", x)
    wc, ws = _oracle(codec, bits)
    want = (capi.dequant_int8_b128 if codec == INT8 else capi.dequant_fp8_b128)(wc, ws)
    for deferred in (0, 1 << 20):
        pool = ActivationOffloadPool(cuda_device, 2, 2 * n, mode, chunk_bytes=64 << 10, deferred_inflight_bytes=deferred)
        h = pool.push_packed(codes, scales, (n,))
        rc, rs = pool.read_slot(h)
        assert np.array_equal(rc, wc.view(np.uint8)) and np.array_equal(rs.view(np.uint32), ws.view(np.uint32))
        st = pool.stats()
        assert st["codec_launches"] == 0 and st["bytes_link_out"] == n + 4 * ((n + 127) // 128)
        out = pool.pull(h)
        torch.cuda.synchronize()
        assert np.array_equal(G.bits_of(out), want) and pool.stats()["codec_launches"] > 0      # only the restore launched
        # and the compressed form itself back, from a tensor the pool compressed on its own
        launches = pool.stats()["codec_launches"]
        h = pool.push(x)
        c2, s2 = torch.zeros_like(codes), torch.zeros_like(scales)
        pool.pull_packed(h, c2, s2)
        torch.cuda.synchronize()
        assert np.array_equal(c2.cpu().numpy(), wc.view(np.uint8)) and np.array_equal(s2.cpu().numpy().view(np.uint32), ws.view(np.uint32))
        assert pool.stats()["codec_launches"] == launches + (n + (1 << 15) * 8 - 1) // ((1 << 15) * 8) and pool.in_flight() == 0
        if deferred:                                    # cancelled before it went out: dequantised on the device
            pool.hold_offloads(True)
            h = pool.push_packed(codes, scales, (n,))
            back = pool.cancel(h)
            torch.cuda.synchronize()
            assert back is not None and np.array_equal(G.bits_of(back), want) and pool.in_flight() == 0
        pool.close()
    plain = ActivationOffloadPool(cuda_device, 2, 2 * n, OffloadCompression.NONE)
    with pytest.raises(Unsupported):
        plain.push_packed(codes, scales, (n,))
    with pytest.raises(Unsupported):
        plain.pull_packed(plain.push(x), codes, scales)
    plain.close()


def test_checkpointed_dit_block_pushes_producer_codes(cuda_device):
    """One DiT block (seven saved tensors, six of them 28 MB, so the allocator hands freed addresses out again within
    the block).  Uncompressed offload reproduces the resident gradients; with the fused producers the two norm
    outputs and gate+up reach an int8 pool already compressed (no compress launch for them)."""
    from flame_b200 import dit_workload as W

    torch.manual_seed(0)
    blk = W.DiTBlock().to(cuda_device, torch.bfloat16)
    x = torch.randn(1, W.TOKENS, W.HIDDEN, device=cuda_device, dtype=torch.bfloat16)
    cos, sin = W.rope_tables(cuda_device)

    def grads(offload):
        for p in blk.parameters():
            p.grad = None
        xin = x.clone().requires_grad_(True)
        y = ckpt.checkpoint_offload([xin, cos, sin], blk) if offload else blk(xin, cos, sin)
        y.float().pow(2).mean().backward()
        torch.cuda.synchronize()
        return [xin.grad.clone()] + [p.grad.clone() for p in blk.parameters()]

    def rel(a, b):
        return float((a.float() - b.float()).norm() / a.float().norm().clamp_min(1e-30))

    saved = ckpt.saved_bytes_of(blk, [x.detach().requires_grad_(True), cos, sin])
    assert saved == 12 * W.TOKENS * W.HIDDEN * 2
    try:
        for fused in (False, True):
            W.FUSED_PRODUCERS = fused
            want = grads(False)
            pool = ActivationOffloadPool(cuda_device, 16, saved, OffloadCompression.NONE)
            ckpt.set_activation_offload_pool(pool)
            for _ in range(3):      # the attention backward is not bit-reproducible run to run; everything else is
                got = grads(True)
                assert max(rel(a, b) for a, b in zip(want, got)) < 5e-3, [rel(a, b) for a, b in zip(want, got)]
            assert pool.stats()["pushes"] == 3 * 7
            ckpt.clear_activation_offload_pool()
            pool.close()
        launches = {}
        for fused in (False, True):
            W.FUSED_PRODUCERS = fused
            want = grads(False)
            pool = ActivationOffloadPool(cuda_device, 16, saved, OffloadCompression.INT8_B128)
            ckpt.set_activation_offload_pool(pool)
            got = grads(True)
            st = pool.stats()
            assert st["pushes"] == 7 and st["pulls"] == 7
            # quantised activations: the large gradients stay close
            for i in (0, 5, 6):     # input, gate_up.weight, down.weight
                assert rel(want[i], got[i]) < 0.05, (i, rel(want[i], got[i]))
            launches[fused] = st["codec_launches"]
            ckpt.clear_activation_offload_pool()
            pool.close()
        assert launches[True] < launches[False]            # three of the seven tensors needed no compress launch
    finally:
        W.FUSED_PRODUCERS = False
        ckpt.clear_activation_offload_pool()
