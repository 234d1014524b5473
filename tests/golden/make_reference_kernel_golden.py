"""Writes fp8_reference_kernel_sm100.npz: what the reference's own FP8 kernels return on a B200.

Needs a GPU and oracle/_ref/libflame_ref_cuda.so (the reference's src/cuda/fp8_quant.cu, fp8_dequant.cu and
pinned_host.cu compiled unmodified by `make -C oracle refcuda`).  For every BF16 bit pattern, NaN and infinity
included, and a list of inverse scales (ordinary, extreme, zero, infinite, NaN, negative) it stores the byte
flame_bf16_to_fp8 of the reference wrote; for every FP8 code and a list of scales the BF16 bits its
flame_fp8_to_bf16 wrote.  The CPU tests hold the oracle to these vectors.

    python tests/golden/make_reference_kernel_golden.py OUT.npz
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


if __name__ == "__main__":
    main(sys.argv[1])
