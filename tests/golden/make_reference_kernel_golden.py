"""Writes fp8_reference_kernel_sm100.npz and int8_reference_sage_sm100.npz: what the reference's own kernels return
on a B200.

Needs a GPU and oracle/_ref/libflame_ref_cuda.so (the reference's src/cuda/fp8_quant.cu, fp8_dequant.cu and
pinned_host.cu compiled unmodified by `make -C oracle refcuda`).  For every BF16 bit pattern, NaN and infinity
included, and a list of inverse scales (ordinary, extreme, zero, infinite, NaN, negative) it stores the byte
flame_bf16_to_fp8 of the reference wrote; for every FP8 code and a list of scales the BF16 bits its
flame_fp8_to_bf16 wrote.  The CPU tests hold the oracle to these vectors.

The second file holds the output of the reference's int8 quantisation kernel (sage_quantize_tensor,
src/sage_attention.rs:510-543, built by `make -C oracle refsage`) run with row_size = 128, i.e. as a per-128-block
quantiser, on the inputs of `int8_inputs()` below (every BF16 bit pattern in order and shuffled, and N(0,1) data with
outliers), given to it as fp32.

The third file holds per-128-block FP8: the reference has no such mode, but its rule for one scale
(src/activation_offload.rs:543-561: scale = absmax/448, inv_scale = 1/scale, both fp32) applied to each block with its
own flame_bf16_to_fp8 kernel, one launch per block, defines the bytes.  Inputs: every finite BF16 value shuffled into
blocks, and N(0,1) data with outliers.

The fourth file holds what the reference's FP8 weight kernel (flame_fused_dequant_transpose_bf16,
src/cuda/fused_dequant_transpose.cu) wrote for a [16,16] matrix of all 256 codes at several scales and for a seeded
random [40,36] matrix.

    python tests/golden/make_reference_kernel_golden.py OUT_FP8.npz [OUT_INT8.npz [OUT_FP8_BLOCKS.npz [OUT_WEIGHTS.npz]]]
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import capi  # noqa: E402

F32 = np.float32
SCALES = [F32(8.0) / F32(448.0), F32(1.0), F32(0.37) / F32(448.0), F32(3.0e-5), F32(1.0e30), F32(1.0e-30)]
INV_SCALES = np.array([F32(1.0) / s for s in SCALES] + [0.0, np.inf, np.nan, -2.0, -np.inf], F32)
DEC_SCALES = np.array(SCALES + [0.0, np.inf, -1.5], F32)


def int8_inputs():
    """name -> uint16 BF16 bit patterns, each a multiple of 256 long (the reference kernel needs whole thread blocks)."""
    from flame_b200 import synthetic

    every = np.arange(1 << 16, dtype=np.uint16)
    rng = np.random.Generator(np.random.PCG64(7))
    return {"every_pattern_in_order": every, "every_pattern_shuffled": rng.permutation(every),
            "normal_with_outliers": synthetic.normal_with_outliers(1 << 16, seed=0)}


def write_int8(out_path: str) -> None:
    sage = capi.load_ref_sage()
    assert sage is not None, "build oracle/_ref/libsage_quant_ref.so first (make -C oracle refsage)"
    dev = torch.device("cuda", 0)
    out = {}
    for name, bits in int8_inputs().items():
        x = torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16).float().contiguous()
        codes = torch.empty(bits.size, dtype=torch.int8, device=dev)
        scales = torch.empty(bits.size // 128, dtype=torch.float32, device=dev)
        assert sage.sage_quantize_ref(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), bits.size // 128, 128, None) == 0
        torch.cuda.synchronize()
        out[name + "_codes"] = codes.cpu().numpy()
        out[name + "_scales"] = scales.cpu().numpy()
    np.savez_compressed(out_path, device=np.array(torch.cuda.get_device_name(0)), **out)
    print("wrote", out_path, sorted(out))


def main(out_path: str) -> None:
    ref = capi.load_ref_cuda()
    assert ref is not None, "build oracle/_ref/libflame_ref_cuda.so first (make -C oracle refcuda)"
    dev = torch.device("cuda", 0)
    bits = np.arange(1 << 16, dtype=np.uint16)
    x = torch.from_numpy(bits.view(np.int16)).to(dev)
    codes = np.empty((INV_SCALES.size, bits.size), np.uint8)
    for k, inv in enumerate(INV_SCALES):
        out = torch.empty(bits.size, dtype=torch.uint8, device=dev)
        assert ref.flame_bf16_to_fp8(x.data_ptr(), out.data_ptr(), float(inv), bits.size, None) == 0
        torch.cuda.synchronize()
        codes[k] = out.cpu().numpy()
    all_codes = torch.arange(256, dtype=torch.int16, device=dev).to(torch.uint8)
    decoded = np.empty((DEC_SCALES.size, 256), np.uint16)
    for k, sc in enumerate(DEC_SCALES):
        out = torch.empty(256, dtype=torch.int16, device=dev)
        assert ref.flame_fp8_to_bf16(all_codes.data_ptr(), out.data_ptr(), float(sc), 256, None) == 0
        torch.cuda.synchronize()
        decoded[k] = out.cpu().numpy().view(np.uint16)
    np.savez_compressed(out_path, inv_scales=INV_SCALES, codes=codes, dec_scales=DEC_SCALES, decoded_bf16_bits=decoded,
                        device=np.array(torch.cuda.get_device_name(0)))
    print("wrote", out_path, codes.shape, decoded.shape, torch.cuda.get_device_name(0))


def fp8_block_inputs():
    from flame_b200 import synthetic

    rng = np.random.Generator(np.random.PCG64(11))
    return {"every_finite_value_shuffled": rng.permutation(synthetic.edge_values()),
            "normal_with_outliers": synthetic.normal_with_outliers(1 << 16, seed=0)}


def write_fp8_blocks(out_path: str) -> None:
    ref = capi.load_ref_cuda()
    assert ref is not None, "build oracle/_ref/libflame_ref_cuda.so first (make -C oracle refcuda)"
    from flame_b200 import synthetic

    dev = torch.device("cuda", 0)
    out = {}
    for name, bits in fp8_block_inputs().items():
        assert bits.size % 128 == 0
        x = torch.from_numpy(bits.view(np.int16)).to(dev)
        codes = torch.zeros(bits.size, dtype=torch.uint8, device=dev)
        absmax = np.abs(synthetic.bf16_bits_to_f32(bits)).reshape(-1, 128).max(axis=1).astype(F32)
        scales = absmax / F32(448.0)
        inv = F32(1.0) / scales
        for b in range(bits.size // 128):
            assert ref.flame_bf16_to_fp8(x.data_ptr() + 256 * b, codes.data_ptr() + 128 * b, float(inv[b]), 128, None) == 0
        torch.cuda.synchronize()
        out[name + "_codes"] = codes.cpu().numpy()
        out[name + "_scales"] = scales
    np.savez_compressed(out_path, device=np.array(torch.cuda.get_device_name(0)), **out)
    print("wrote", out_path, sorted(out))


WEIGHT_SCALES = np.array([1.0, 0.0123, 3.0e-5, 1.0e30, 1.0e-30, -2.5, 0.0], F32)


def weight_inputs():
    rng = np.random.Generator(np.random.PCG64(5))
    return {"all_codes_16x16": (np.arange(256, dtype=np.uint8), 16, 16),
            "random_40x36": (rng.integers(0, 256, size=40 * 36, dtype=np.uint8), 40, 36)}


def write_weights(out_path: str) -> None:
    ref = capi.load_ref_cuda()
    assert ref is not None and hasattr(ref, "flame_fused_dequant_transpose_bf16"), "rebuild oracle/_ref (make -C oracle refcuda)"
    dev = torch.device("cuda", 0)
    out = {"scales": WEIGHT_SCALES}
    for name, (codes, m, n) in weight_inputs().items():
        c = torch.from_numpy(codes).to(dev)
        got = np.empty((WEIGHT_SCALES.size, n, m), np.uint16)
        for k, sc in enumerate(WEIGHT_SCALES):
            o = torch.empty(n * m, dtype=torch.int16, device=dev)
            assert ref.flame_fused_dequant_transpose_bf16(c.data_ptr(), o.data_ptr(), float(sc), m, n, None) == 0
            torch.cuda.synchronize()
            got[k] = o.cpu().numpy().view(np.uint16).reshape(n, m)
        out[name] = got
    np.savez_compressed(out_path, device=np.array(torch.cuda.get_device_name(0)), **out)
    print("wrote", out_path, sorted(out))


if __name__ == "__main__":
    main(sys.argv[1])
    if len(sys.argv) > 2:
        write_int8(sys.argv[2])
    if len(sys.argv) > 3:
        write_fp8_blocks(sys.argv[3])
    if len(sys.argv) > 4:
        write_weights(sys.argv[4])
