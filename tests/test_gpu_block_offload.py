"""Block weights streamed through the pool: non-consuming restores and the BlockOffloader interface."""
import numpy as np
import pytest
import torch

from flame_b200 import ActivationOffloadPool, BlockOffloader, InvalidInput, InvalidOperation, OffloadCompression, Unsupported
from oracle import capi

from tests import gpu_util as G

pytestmark = pytest.mark.gpu


def _blocks(device, n_blocks=4, d=256, seed=0, with_f32=True):
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for b in range(n_blocks):
        blk = {
            "attn.qkv.weight": torch.randn(3 * d, d, generator=g).mul(0.05).to(torch.bfloat16),
            "attn.out.weight": torch.randn(d, d, generator=g).mul(0.05).to(torch.bfloat16),
            "mlp.up.weight": torch.randn(4 * d + 8 * b, d, generator=g).mul(0.05).to(torch.bfloat16),   # ragged across blocks
            "norm.weight": torch.ones(d + 1, dtype=torch.bfloat16),                                      # odd size
        }
        if with_f32:
            blk["norm.bias_f32"] = torch.randn(d, generator=g)
        out.append(blk)
    return out


def test_keep_flag_restores_the_same_handle_again(cuda_device):
    pool = ActivationOffloadPool(cuda_device, 2, 1 << 20, OffloadCompression.INT8_B128)
    bits = np.random.default_rng(0).integers(0, 1 << 16, 5000, dtype=np.uint16)
    bits[(bits & 0x7F80) == 0x7F80] = 0x3F80
    x = G.to_dev(bits, cuda_device)
    h = pool.push(x)
    want = capi.dequant_int8_b128(*capi.quant_int8_b128(bits))
    for _ in range(3):
        dst = torch.zeros(5000, dtype=torch.bfloat16, device=cuda_device)
        pool.pull_into(h, dst, keep=True)
        torch.cuda.synchronize()
        assert np.array_equal(G.bits_of(dst), want)
        assert pool.in_flight() == 1
    dst = torch.zeros(5000, dtype=torch.bfloat16, device=cuda_device)
    pool.pull_into(h, dst)                      # a consuming pull ends it
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(dst), want) and pool.in_flight() == 0
    with pytest.raises(InvalidOperation):
        pool.pull_into(h, dst, keep=True)
    # a kept slot that is discarded while a restore may still read it: the next offload into its chunks is ordered behind
    h1 = pool.push(x)
    big = torch.zeros(5000, dtype=torch.bfloat16, device=cuda_device)
    pool.pull_into(h1, big, keep=True, defer_wait=True)
    pool.discard(h1)
    y = G.to_dev(np.full(5000, 0x4000, np.uint16), cuda_device)
    h2 = pool.push(y)
    pool.wait_ready(h1.slot)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(big), want)
    out = pool.pull(h2)
    torch.cuda.synchronize()
    assert np.array_equal(G.bits_of(out), np.full(5000, 0x4000, np.uint16))
    pool.close()


@pytest.mark.parametrize("mode", [OffloadCompression.NONE, OffloadCompression.INT8_B128, OffloadCompression.FP8_B128])
def test_blocks_stream_in_both_directions(cuda_device, mode):
    blocks = _blocks(cuda_device, with_f32=(mode == OffloadCompression.NONE))
    off = BlockOffloader(cuda_device, blocks, mode, chunk_bytes=64 << 10)     # several chunks per weight
    assert off.block_count() == 4 and off.pinned_bytes() > 0

    def expect(t):
        if mode == OffloadCompression.NONE or t.dtype != torch.bfloat16:
            return t
        bits = t.contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)
        q, d = (capi.quant_int8_b128, capi.dequant_int8_b128) if mode == OffloadCompression.INT8_B128 else (capi.quant_fp8_b128, capi.dequant_fp8_b128)
        return torch.from_numpy(d(*q(bits)).view(np.int16)).view(torch.bfloat16).view(t.shape)

    order = [0, 1, 2, 3, 3, 2, 1, 0, 2]            # forward, backward, a jump
    off.prefetch_block(order[0])
    for i, idx in enumerate(order):
        w = off.await_block(idx)
        if i + 1 < len(order):
            off.prefetch_block(order[i + 1])      # overlaps the use of block idx below
        acc = [v.float().sum() for v in w.values()]   # some compute that reads the slot
        torch.cuda.synchronize()
        for name, t in blocks[idx].items():
            got = w[name].cpu()
            assert got.shape == t.shape and got.dtype == t.dtype
            assert torch.equal(got.view(torch.int16) if t.dtype == torch.bfloat16 else got, expect(t).view(torch.int16) if t.dtype == torch.bfloat16 else t), (idx, name)
        del acc
    st = off.stats()
    groups = 2 if mode == OffloadCompression.NONE else 1      # BF16 and F32 groups per block
    # seven loads: the repeated 3 and the 2 after it are still held by one of the two device slots
    assert st["pulls"] == 7 * groups and st["pushes"] == 4 * groups
    off.evict_block()
    w = off.ensure_block(1)
    torch.cuda.synchronize()
    assert torch.equal(w["attn.out.weight"].cpu().view(torch.int16), expect(blocks[1]["attn.out.weight"]).view(torch.int16))
    off.close()


def test_block_offloader_argument_errors(cuda_device):
    with pytest.raises(InvalidInput):
        BlockOffloader(cuda_device, [])
    with pytest.raises(Unsupported):
        BlockOffloader(cuda_device, [{"w": torch.zeros(4, dtype=torch.float16)}])
    with pytest.raises(Unsupported):
        BlockOffloader(cuda_device, [{"w": torch.zeros(4)}], OffloadCompression.INT8_B128)
    off = BlockOffloader(cuda_device, _blocks(cuda_device, 2), gpu_slots=1)
    off.await_block(0)
    with pytest.raises(InvalidOperation):
        off.prefetch_block(1)                     # the only slot holds the active block
    w = off.await_block(1)                        # awaiting replaces it
    torch.cuda.synchronize()
    assert w["norm.weight"].shape == (257,)
    with pytest.raises(InvalidInput):
        off.await_block(5)
    off.close()


def test_fp8_weight_bytes_stream_as_they_are_and_expand_on_the_device(cuda_device):
    """FP8 E4M3 weights with one scale per tensor (src/ops/fused_inference.rs:86-175): one byte per element over the
    link, BF16 after await_block, transposed where the caller asks for it."""
    rng = np.random.default_rng(4)
    d = 128
    scale_qkv, scale_out = 0.0123, 0.5
    blocks = []
    for b in range(3):
        codes_qkv = rng.integers(0, 0x78, size=(3 * d, d), dtype=np.uint8) | (rng.integers(0, 2, size=(3 * d, d), dtype=np.uint8) << 7)
        codes_out = rng.integers(0, 256, size=(d, d + 8 * b), dtype=np.uint8)
        blocks.append({"attn.qkv.weight": torch.from_numpy(codes_qkv), "attn.out.weight": torch.from_numpy(codes_out),
                       "norm.weight": torch.ones(d, dtype=torch.bfloat16) * (b + 1)})
    with pytest.raises(Unsupported):
        BlockOffloader(cuda_device, blocks, OffloadCompression.NONE)                      # uint8 without a description
    with pytest.raises(Unsupported):
        BlockOffloader(cuda_device, blocks, OffloadCompression.INT8_B128, fp8_weights={"attn.qkv.weight": (1.0, True), "attn.out.weight": (1.0, False)})
    off = BlockOffloader(cuda_device, blocks, OffloadCompression.NONE, chunk_bytes=64 << 10,
                         fp8_weights={"attn.qkv.weight": (scale_qkv, True), "attn.out.weight": (scale_out, False)})
    try:
        st0 = off.stats()
        for idx in (0, 1, 2, 1, 0):
            off.prefetch_block(idx)
            w = off.await_block(idx)
            torch.cuda.synchronize()
            cq, co = blocks[idx]["attn.qkv.weight"].numpy(), blocks[idx]["attn.out.weight"].numpy()
            assert w["attn.qkv.weight"].shape == (d, 3 * d) and w["attn.qkv.weight"].dtype == torch.bfloat16
            assert np.array_equal(G.bits_of(w["attn.qkv.weight"]).reshape(d, 3 * d), capi.fp8_dequant_transpose(cq, scale_qkv, 3 * d, d))
            assert w["attn.out.weight"].shape == co.shape
            assert np.array_equal(G.bits_of(w["attn.out.weight"]).reshape(-1), capi.fp8_to_bf16(co.reshape(-1), scale_out))
            assert torch.equal(w["norm.weight"].cpu(), blocks[idx]["norm.weight"])
        # one byte per FP8 element crossed the link (plus the BF16 norm weight and padding to 256 bytes); with two
        # device slots block 1 is still on the device when it is asked for again, so four loads: 0, 1, 2, 0
        per_block = [3 * d * d + d * (d + 8 * b) for b in range(3)]
        moved = off.stats()["bytes_link_in"] - st0["bytes_link_in"]
        assert sum(per_block[i] for i in (0, 1, 2, 0)) <= moved < sum(per_block[i] for i in (0, 1, 2, 0)) + 4 * 4096
    finally:
        off.close()
