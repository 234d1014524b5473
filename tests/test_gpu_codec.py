"""Parity of the CUDA codec kernels with the CPU oracle, through the C ABI.  Bit exact."""
import os

import numpy as np
import pytest
import torch

from flame_b200 import _lib, synthetic
from oracle import capi
from tests import gpu_util as G

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 8, 9, 127, 128, 129, 1000, 8191, 8192, 8193, 3 * 8192 + 77, (1 << 20) + 13]


def _check_int8(x_bits, dev, flags=0, **offs):
    x = G.to_dev(x_bits, dev, offs.pop("in_offset", 0))
    codes, scales = G.quant("int8", x, flags, **offs)
    want_c, want_s = capi.quant_int8_b128(x_bits, flags & 1)
    assert np.array_equal(codes.cpu().numpy().view(np.int8), want_c)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    out = G.dequant("int8", codes, scales, x.numel())
    assert np.array_equal(G.bits_of(out), capi.dequant_int8_b128(want_c, want_s))
    return codes, scales, out


def _check_fp8(x_bits, dev, flags=0, **offs):
    x = G.to_dev(x_bits, dev, offs.pop("in_offset", 0))
    codes, scales = G.quant("fp8", x, flags, **offs)
    want_c, want_s = capi.quant_fp8_b128(x_bits, flags & 1)
    assert np.array_equal(codes.cpu().numpy(), want_c)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    out = G.dequant("fp8", codes, scales, x.numel())
    assert np.array_equal(G.bits_of(out), capi.dequant_fp8_b128(want_c, want_s))
    return codes, scales, out


@pytest.mark.parametrize("n", SIZES)
def test_int8_sizes(cuda_device, n):
    _check_int8(synthetic.normal_with_outliers(n, seed=n), cuda_device)


@pytest.mark.parametrize("n", SIZES)
def test_fp8_sizes(cuda_device, n):
    _check_fp8(synthetic.normal_with_outliers(n, seed=n + 1), cuda_device)


@pytest.mark.parametrize("n", [8192, 8193, 5 * 8192 + 4000, (1 << 22) + 8192 * 3 + 9])
def test_staged_store_path_gives_the_same_bytes(cuda_device, n):
    """FLAME_ACT_STAGED_STORES: each warp's shared-memory slice drained by bulk asynchronous copies."""
    bits = synthetic.normal_with_outliers(n, seed=n + 2)
    _check_int8(bits, cuda_device, flags=2)
    _check_int8(bits, cuda_device, flags=3)
    _check_fp8(bits, cuda_device, flags=2)
    _check_fp8(bits, cuda_device, flags=3)


@pytest.mark.parametrize("form", [0, 1, 2])
def test_every_kernel_form_gives_the_same_bytes(cuda_device, form):
    """The three forms of the compress kernel (plain, software-pipelined, plain with four resident blocks), with
    direct and with staged stores, against the oracle: full tiles, a ragged last tile, many rounds per block."""
    lib = _lib.lib()
    lib.flame_act_set_compress_form(form)
    try:
        info = _lib.ActLaunchInfo()
        for n in (8192, 3 * 8192 + 77, (1 << 20) + 13, (1 << 24) + 8192 * 5 + 1):
            bits = synthetic.normal_with_outliers(n, seed=n + form)
            for flags in (0, 2):
                _check_int8(bits, cuda_device, flags=flags)
                lib.flame_act_last_launch(info)            # the dequantise launch of the check ran last
                _check_fp8(bits, cuda_device, flags=flags)
        x = G.to_dev(synthetic.normal(1 << 20, seed=3), cuda_device)
        G.quant("fp8", x, 2)
        lib.flame_act_last_launch(info)
        assert info.form == form + 4
    finally:
        lib.flame_act_set_compress_form(-1)


_OCCUPANCY_SCRIPT = r"""
import sys, json
import numpy as np, torch
sys.path.insert(0, {root!r})
from flame_b200 import _lib
lib = _lib.lib()
torch.cuda.set_device(0)
n = 1 << 24
x = torch.randn(n, device="cuda").to(torch.bfloat16)
codes = torch.empty(n, dtype=torch.uint8, device="cuda")
scales = torch.empty(n // 128, dtype=torch.float32, device="cuda")
info = _lib.ActLaunchInfo()
out = {{}}
for codec in {order!r}:
    fn = getattr(lib, "flame_act_quant_%s_b128" % codec)
    assert fn(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, 0, None) == 0
    lib.flame_act_last_launch(info)
    cid = 2 if codec == "int8" else 3
    out[codec] = dict(used=info.resident_per_sm, fresh=lib.flame_act_query_resident_blocks(cid, 0, -1, 1), grid=info.grid, form=info.form)
torch.cuda.synchronize()
print(json.dumps(out))
"""


@pytest.mark.parametrize("order", [("fp8", "int8"), ("int8", "fp8")])
def test_each_kernel_is_sized_by_its_own_occupancy(cuda_device, order):
    """The grid of a launch comes from the occupancy of the kernel that is launched, whichever kernel ran first in
    the process (the kernels are instantiations of one template and differ in registers per thread)."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _OCCUPANCY_SCRIPT.format(root=root, order=order)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = json.loads(r.stdout.strip().splitlines()[-1])
    for codec in order:
        assert got[codec]["used"] == got[codec]["fresh"] > 0, got
    # the two default kernels differ in registers per thread, so a shared answer would show here
    lib = _lib.lib()
    assert got["int8"]["fresh"] == lib.flame_act_query_resident_blocks(2, 0, -1, 1)
    assert got["fp8"]["fresh"] == lib.flame_act_query_resident_blocks(3, 0, -1, 1)


_BACK_TO_BACK_SCRIPT = r"""
import sys, hashlib
import numpy as np, torch
sys.path.insert(0, {root!r})
from flame_b200 import _lib, synthetic
lib = _lib.lib()
torch.cuda.set_device(0)
n = (1 << 23) + 128 * 3
h = hashlib.sha256()
xs = [torch.from_numpy(synthetic.normal_with_outliers(n, seed).view(np.int16)).cuda().view(torch.bfloat16) for seed in (1, 2, 3)]
codes = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in xs]
scales = [torch.empty((n + 127) // 128, dtype=torch.float32, device="cuda") for _ in xs]
outs = [torch.empty_like(x) for x in xs]
for codec in ("int8", "fp8"):
    q, d = getattr(lib, "flame_act_quant_%s_b128" % codec), getattr(lib, "flame_act_dequant_%s_b128" % codec)
    for rep in range(3):                       # kernels directly behind one another in one stream, each reading what the last wrote
        for x, c, s, o in zip(xs, codes, scales, outs):
            assert q(x.data_ptr(), c.data_ptr(), s.data_ptr(), n, 0, None) == 0
            assert d(c.data_ptr(), s.data_ptr(), o.data_ptr(), n, None) == 0
            assert q(o.data_ptr(), c.data_ptr(), s.data_ptr(), n, 0, None) == 0      # codes of the restored tensor
    torch.cuda.synchronize()
    for t in codes + scales + outs:
        h.update(t.view(torch.uint8).cpu().numpy().tobytes())
print(h.hexdigest())
"""


def test_kernels_behind_one_another_give_the_same_bytes_with_and_without_the_launch_attribute(cuda_device):
    """The fast kernels are launched with programmatic stream serialisation and wait inside the kernel for their
    predecessors.  A chain in which every kernel reads what the one before it wrote gives the same bytes as the same
    chain with plain launches (FLAME_ACT_PDL=0)."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    digests = []
    for pdl in ("1", "0"):
        env = dict(os.environ, FLAME_ACT_PDL=pdl)
        r = subprocess.run([sys.executable, "-c", _BACK_TO_BACK_SCRIPT.format(root=root)], capture_output=True, text=True, timeout=600, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1]


def test_empty_input_is_a_no_op(cuda_device):
    lib = _lib.lib()
    assert lib.flame_act_quant_int8_b128(None, None, None, 0, 0, None) == 0
    assert lib.flame_act_dequant_fp8_b128(None, None, None, 0, None) == 0
    assert lib.flame_act_quant_fp8_b128(None, None, None, 5, 0, None) == 1  # cudaErrorInvalidValue


@pytest.mark.parametrize("n", [129, 8192 + 9, 50001])
def test_unaligned_pointers_take_the_generic_kernels(cuda_device, n):
    bits = synthetic.normal(n, seed=7)
    _check_int8(bits, cuda_device, in_offset=1, code_offset=3, scale_offset=1)
    _check_fp8(bits, cuda_device, in_offset=3, code_offset=1, scale_offset=3)
    # dequantise into an odd destination
    x = G.to_dev(bits, cuda_device)
    codes, scales = G.quant("int8", x, code_offset=5)
    out = G.dequant("int8", codes, scales, n, out_offset=1)
    wc, ws = capi.quant_int8_b128(bits)
    assert np.array_equal(G.bits_of(out), capi.dequant_int8_b128(wc, ws))


def test_random_sizes_alignments_and_magnitudes(cuda_device):
    """Seeded fuzz: ragged sizes, odd pointer offsets, block magnitudes spread over the whole BF16 range."""
    rng = np.random.default_rng(12345)
    for trial in range(40):
        n = int(rng.choice([rng.integers(1, 300), rng.integers(300, 20000), rng.integers(20000, 400000)]))
        bits = synthetic.normal_with_outliers(n, seed=500 + trial)
        # scale every 128-block by a random power of two between 2^-60 and 2^60, flip some blocks to zero
        expo = rng.integers(-60, 61, size=(n + 127) // 128)
        f = synthetic.bf16_bits_to_f32(bits) * np.repeat(np.exp2(expo.astype(np.float64)), 128)[:n].astype(np.float32)
        f[np.repeat(rng.random((n + 127) // 128) < 0.05, 128)[:n]] = 0.0
        bits = synthetic.f32_to_bf16_bits(f.astype(np.float32))
        offs = dict(in_offset=int(rng.integers(0, 3)) * int(rng.integers(0, 2)), code_offset=int(rng.integers(0, 4)) * int(rng.integers(0, 2)),
                    scale_offset=int(rng.integers(0, 2)))
        _check_int8(bits, cuda_device, **dict(offs))
        _check_fp8(bits, cuda_device, **dict(offs))


def test_every_finite_bf16_value(cuda_device):
    """All 65,280 finite BF16 patterns, in blocks that mix magnitudes and in blocks of similar magnitude."""
    vals = synthetic.edge_values()
    rng = np.random.default_rng(0)
    for bits in (vals, rng.permutation(vals), np.sort(vals.view(np.int16)).view(np.uint16)):
        _check_int8(bits, cuda_device)
        _check_int8(bits, cuda_device, flags=1)  # MUL_INV form
        _check_fp8(bits, cuda_device)


def test_scale_edge_blocks(cuda_device):
    """Zero blocks, -0.0, one-hot blocks, sub-normal magnitudes, huge magnitudes, all-ones scale significands."""
    x = np.zeros(128 * 12, np.uint16)
    x[128 + 5] = 0x8000                                     # block 1: only a -0.0
    x[256 + 17] = 0x3F80                                    # block 2: one-hot 1.0
    x[384:512] = 0x0001                                     # block 3: smallest BF16 sub-normal
    x[512:640] = np.arange(128, dtype=np.uint16) + 0x0001   # block 4: sub-normal ramp
    x[640:768] = 0x7F7F                                     # block 5: BF16 max
    x[768:896] = (np.arange(128) % 2 * 0x8000 + 0x7F00).astype(np.uint16)  # block 6: huge, mixed sign
    x[896:1024] = synthetic.normal(128, 1)
    x[896] = 0x42FE                                         # 127.0 -> scale 1.0 exactly
    x[1024:1152] = synthetic.normal(128, 2)
    x[1152:1280] = (synthetic.normal(128, 3) & 0x807F) | 0x0080  # tiny normals
    _check_int8(x, cuda_device)
    _check_int8(x, cuda_device, flags=1)
    _check_fp8(x, cuda_device)


def test_sparse_activations_with_signed_zeros(cuda_device):
    """ReLU-like data: half the elements are exact zeros, some of them -0.0, a few tiny values among them."""
    rng = np.random.default_rng(3)
    bits = synthetic.normal(200000 + 5, seed=8)
    zero = rng.random(bits.size) < 0.5
    bits[zero] = np.where(rng.random(int(zero.sum())) < 0.3, 0x8000, 0x0000).astype(np.uint16)
    tiny = rng.choice(bits.size, 300, replace=False)
    bits[tiny] = (0x2000 | (rng.integers(0, 2, 300) << 15) | rng.integers(0, 128, 300)).astype(np.uint16)  # ~1e-19
    _check_fp8(bits, cuda_device)
    _check_int8(bits, cuda_device)
    lib = _lib.lib()
    x = G.to_dev(bits, cuda_device)
    codes = torch.empty(bits.size, dtype=torch.uint8, device=cuda_device)
    assert lib.flame_bf16_to_fp8(x.data_ptr(), codes.data_ptr(), 56.0, bits.size, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(codes.cpu().numpy(), capi.bf16_to_fp8(bits, 56.0))


def test_nan_elements_do_not_poison_a_block(cuda_device):
    x = synthetic.normal(512, 4)
    x[3] = 0x7FC0
    x[200] = 0xFFC1
    _check_int8(x, cuda_device)
    _check_fp8(x, cuda_device)


def test_ocp_encoder_flag(cuda_device):
    bits = synthetic.student_t3_times2(100000 + 3, 5)
    _check_fp8(bits, cuda_device, flags=1)
    _check_fp8(synthetic.edge_values(), cuda_device, flags=1)


@pytest.mark.parametrize("codec,name", [(2, "int8"), (3, "fp8")])
def test_multi_tensor_launch_equals_single_launches(cuda_device, codec, name):
    """One launch over many tensors of ragged sizes (more than one table's worth) gives the same bytes."""
    import ctypes as C

    lib = _lib.lib()
    sizes = [8192 * 3, 1, 129, 8192 * 2 + 77, 16384 * 5, 16384 * 2 + 15, 100000, 8191] * 7  # 56 tensors
    xs, codes, scales, outs = [], [], [], []
    for i, n in enumerate(sizes):
        xs.append(G.to_dev(synthetic.normal_with_outliers(n, seed=1000 + i), cuda_device))
        codes.append(torch.full((n,), 0xAB, dtype=torch.uint8, device=cuda_device))
        scales.append(torch.full(((n + 127) // 128,), -7.0, dtype=torch.float32, device=cuda_device))
        outs.append(torch.zeros(n, dtype=torch.bfloat16, device=cuda_device))
    arr = (_lib.ActTensor * len(sizes))(*[_lib.ActTensor(x.data_ptr(), c.data_ptr(), s.data_ptr(), n)
                                           for x, c, s, n in zip(xs, codes, scales, sizes)])
    assert lib.flame_act_quant_b128_multi(codec, arr, len(sizes), 0, G.stream_ptr(cuda_device)) == 0
    arr2 = (_lib.ActTensor * len(sizes))(*[_lib.ActTensor(o.data_ptr(), c.data_ptr(), s.data_ptr(), n)
                                            for o, c, s, n in zip(outs, codes, scales, sizes)])
    assert lib.flame_act_dequant_b128_multi(codec, arr2, len(sizes), G.stream_ptr(cuda_device)) == 0
    torch.cuda.synchronize()
    for x, c, s, o, n in zip(xs, codes, scales, outs, sizes):
        c1, s1 = G.quant(name, x)
        assert torch.equal(c, c1) and torch.equal(s, s1)
        assert torch.equal(o.view(torch.int16), G.dequant(name, c1, s1, n).view(torch.int16))
    assert lib.flame_act_quant_b128_multi(codec, None, 0, 0, None) == 0
    assert lib.flame_act_quant_b128_multi(9, arr, 1, 0, None) == 1


def test_block_codec_goldens(cuda_device, golden_dir):
    from tests.golden.make_golden import BLOCK_CASES

    g = np.load(os.path.join(golden_dir, "block_codec_cases.npz"))
    for name, (gen, n, seed) in BLOCK_CASES.items():
        bits = getattr(synthetic, gen)(n, seed)
        codes, scales, out = _check_int8(bits, cuda_device)
        assert np.array_equal(codes.cpu().numpy().view(np.int8), g[f"{name}.int8_codes"])
        assert np.array_equal(G.bits_of(out), g[f"{name}.int8_out"])
        codes, scales, out = _check_fp8(bits, cuda_device)
        assert np.array_equal(codes.cpu().numpy(), g[f"{name}.fp8_codes"])
        assert np.array_equal(scales.cpu().numpy(), g[f"{name}.fp8_scales"])
        assert np.array_equal(G.bits_of(out), g[f"{name}.fp8_out"])


def test_config1_full_tensor_int8(cuda_device):
    """[1,4096,3072] BF16, N(0,1) with 0.1 % +-U(20,60) outliers, seed 0: codes, scales and values bit exact;
    every dequantised value within absmax/127 of its source."""
    bits = synthetic.normal_with_outliers(4096 * 3072, 0)
    codes, scales, out = _check_int8(bits, cuda_device)
    xf = G.to_dev(bits, cuda_device).float()
    err = (out.float() - xf).abs().view(-1, 128).amax(dim=1)
    assert bool((err <= scales).all())


def test_config3_mixed_activations_fp8(cuda_device):
    """GELU outputs, 2*t(3) attention outputs and a SwiGLU hidden state [1,4608,9216]."""
    _check_fp8(synthetic.gelu_of_normal(4608 * 3072, 0), cuda_device)
    _check_fp8(synthetic.student_t3_times2(4608 * 3072, 0), cuda_device)
    _check_fp8(synthetic.swiglu_hidden(4608 * 9216, 0), cuda_device)
    _check_int8(synthetic.student_t3_times2(4608 * 3072, 1), cuda_device)


# ---- element-wise FP8 with a caller-supplied scale (the reference's two entry points) --------

@pytest.mark.parametrize("n", [1, 5, 8, 1000, 65536 + 3])
@pytest.mark.parametrize("offset", [0, 1])
def test_flame_bf16_to_fp8_and_back(cuda_device, n, offset):
    lib = _lib.lib()
    bits = synthetic.normal_with_outliers(n, seed=n)
    x = G.to_dev(bits, cuda_device, offset)
    scale = np.float32(8.0) / np.float32(448.0)      # the reference pool's fixed scale
    inv = np.float32(1.0) / scale
    codes = torch.empty(n + offset, dtype=torch.uint8, device=cuda_device)[offset:]
    assert lib.flame_bf16_to_fp8(x.data_ptr(), codes.data_ptr(), float(inv), n, G.stream_ptr(cuda_device)) == 0
    out = torch.empty(n + offset, dtype=torch.bfloat16, device=cuda_device)[offset:]
    assert lib.flame_fp8_to_bf16(codes.data_ptr(), out.data_ptr(), float(scale), n, G.stream_ptr(cuda_device)) == 0
    torch.cuda.synchronize()
    want = capi.bf16_to_fp8(bits, inv)
    assert np.array_equal(codes.cpu().numpy(), want)
    assert np.array_equal(G.bits_of(out), capi.fp8_to_bf16(want, scale))


def test_elementwise_encoder_against_reference_golden(cuda_device, golden_dir):
    """The codes the reference's own encoder gave for every finite BF16 value (committed fixture)."""
    lib = _lib.lib()
    g = np.load(os.path.join(golden_dir, "fp8_reference_encoder.npz"))
    bits = synthetic.edge_values()
    x = G.to_dev(bits, cuda_device)
    for k, inv in enumerate(g["inv_scales"]):
        codes = torch.empty(bits.size, dtype=torch.uint8, device=cuda_device)
        assert lib.flame_bf16_to_fp8(x.data_ptr(), codes.data_ptr(), float(inv), bits.size, None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(codes.cpu().numpy(), g[f"codes_{k}"])
    # bytes the reference's own kernels wrote on a B200, every BF16 pattern x eleven inverse scales
    k100 = np.load(os.path.join(golden_dir, "fp8_reference_kernel_sm100.npz"))
    every = G.to_dev(np.arange(1 << 16, dtype=np.uint16), cuda_device)
    for k, inv in enumerate(k100["inv_scales"]):
        codes = torch.empty(1 << 16, dtype=torch.uint8, device=cuda_device)
        assert lib.flame_bf16_to_fp8(every.data_ptr(), codes.data_ptr(), float(inv), 1 << 16, None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(codes.cpu().numpy(), k100["codes"][k]), float(inv)
    dec = np.load(os.path.join(golden_dir, "fp8_reference_decoder.npy"))
    all_codes = torch.arange(256, dtype=torch.int16, device=cuda_device).to(torch.uint8)
    out = torch.empty(256, dtype=torch.bfloat16, device=cuda_device)
    assert lib.flame_fp8_to_bf16(all_codes.data_ptr(), out.data_ptr(), 1.0, 256, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy().view(np.uint32), dec.view(np.uint32))  # every decoded value is a BF16


def test_legacy_entry_points_equal_the_reference_kernels_on_this_gpu(cuda_device):
    """flame_bf16_to_fp8 / flame_fp8_to_bf16 against the reference's own src/cuda/fp8_quant.cu and
    fp8_dequant.cu, compiled unmodified and run on the same device buffers: every BF16 bit pattern
    (NaN and infinity included) at several scales, and every code at several scales."""
    ref = capi.load_ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/libflame_ref_cuda.so was not built (reference checkout absent at build time)")
    lib = _lib.lib()
    bits = np.arange(1 << 16, dtype=np.uint16)
    x = G.to_dev(bits, cuda_device)
    sp = G.stream_ptr(cuda_device)
    scales = [np.float32(8.0) / np.float32(448.0), np.float32(1.0), np.float32(0.37) / np.float32(448.0),
              np.float32(3.0e-5), np.float32(1.0e30), np.float32(1.0e-30)]
    invs = [np.float32(1.0) / sc for sc in scales] + [np.float32(v) for v in (0.0, np.inf, np.nan, -2.0, -np.inf)]
    for inv in invs:
        mine = torch.empty(bits.size, dtype=torch.uint8, device=cuda_device)
        theirs = torch.empty_like(mine)
        assert lib.flame_bf16_to_fp8(x.data_ptr(), mine.data_ptr(), float(inv), bits.size, sp) == 0
        assert ref.flame_bf16_to_fp8(x.data_ptr(), theirs.data_ptr(), float(inv), bits.size, sp) == 0
        torch.cuda.synchronize()
        a, b = mine.cpu().numpy(), theirs.cpu().numpy()
        assert np.array_equal(a, b), (float(inv), bits[a != b][:8], a[a != b][:8], b[a != b][:8])
        assert np.array_equal(a, capi.bf16_to_fp8(bits, inv)), float(inv)       # and the CPU oracle says the same
        # an unaligned copy of the same values takes this library's scalar kernel
        xu = G.to_dev(bits, cuda_device, 1)
        mu = torch.empty(bits.size + 1, dtype=torch.uint8, device=cuda_device)[1:]
        assert lib.flame_bf16_to_fp8(xu.data_ptr(), mu.data_ptr(), float(inv), bits.size, sp) == 0
        torch.cuda.synchronize()
        assert np.array_equal(mu.cpu().numpy(), b), float(inv)
    all_codes = torch.arange(256, dtype=torch.int16, device=cuda_device).to(torch.uint8)
    for scale in scales + [np.float32(0.0)]:
        mine = torch.empty(256, dtype=torch.bfloat16, device=cuda_device)
        theirs = torch.empty_like(mine)
        assert lib.flame_fp8_to_bf16(all_codes.data_ptr(), mine.data_ptr(), float(scale), 256, sp) == 0
        assert ref.flame_fp8_to_bf16(all_codes.data_ptr(), theirs.data_ptr(), float(scale), 256, sp) == 0
        torch.cuda.synchronize()
        assert np.array_equal(G.bits_of(mine), G.bits_of(theirs)), float(scale)
    # a tensor of the pool's size class, through both libraries: same bytes out, same BF16 back
    vals = synthetic.normal_with_outliers(1 << 22, seed=3)
    xv = G.to_dev(vals, cuda_device)
    inv = np.float32(448.0) / np.float32(8.0)
    c1 = torch.empty(vals.size, dtype=torch.uint8, device=cuda_device); c2 = torch.empty_like(c1)
    assert lib.flame_bf16_to_fp8(xv.data_ptr(), c1.data_ptr(), float(inv), vals.size, sp) == 0
    assert ref.flame_bf16_to_fp8(xv.data_ptr(), c2.data_ptr(), float(inv), vals.size, sp) == 0
    o1 = torch.empty(vals.size, dtype=torch.bfloat16, device=cuda_device); o2 = torch.empty_like(o1)
    assert lib.flame_fp8_to_bf16(c1.data_ptr(), o1.data_ptr(), float(1 / inv), vals.size, sp) == 0
    assert ref.flame_fp8_to_bf16(c2.data_ptr(), o2.data_ptr(), float(1 / inv), vals.size, sp) == 0
    torch.cuda.synchronize()
    assert torch.equal(c1, c2) and torch.equal(o1.view(torch.int16), o2.view(torch.int16))


def test_int8_block_codec_equals_the_reference_int8_kernel_on_this_gpu(cuda_device):
    """The reference has no per-128-block offload codec, but it has an int8 quantiser with this very formula:
    sage_quantize_tensor (src/sage_attention.rs:510-543; scale = max|x|/127 per row, __float2int_rn(x/scale)).
    Compiled unmodified and run with row_size = 128 on the same values, it must give the codes and scales of
    flame_act_quant_int8_b128."""
    sage = capi.load_ref_sage()
    if sage is None:
        pytest.skip("oracle/_ref/libsage_quant_ref.so was not built (reference checkout absent at build time)")
    rng = np.random.Generator(np.random.PCG64(11))
    every = np.arange(1 << 16, dtype=np.uint16)
    cases = {"every pattern": every, "shuffled": rng.permutation(every),
             "normal": synthetic.normal_with_outliers(1 << 20, seed=5),
             "zeros and signed zeros": np.where(rng.random(1 << 12) < 0.5, 0, 0x8000).astype(np.uint16),
             "tiny": (rng.integers(0, 0x0100, 1 << 12)).astype(np.uint16),            # sub-normal BF16 values
             "huge": (0x7F00 + rng.integers(0, 0x80, 1 << 12)).astype(np.uint16)}    # up to the largest finite value
    for name, bits in cases.items():
        x = G.to_dev(bits, cuda_device)
        codes, scales = G.quant("int8", x)
        xf = x.float().contiguous()
        rc = torch.empty(bits.size, dtype=torch.int8, device=cuda_device)
        rs = torch.empty(bits.size // 128, dtype=torch.float32, device=cuda_device)
        assert sage.sage_quantize_ref(xf.data_ptr(), rc.data_ptr(), rs.data_ptr(), bits.size // 128, 128, G.stream_ptr(cuda_device)) == 0
        torch.cuda.synchronize()
        a, b = codes.cpu().numpy().view(np.int8), rc.cpu().numpy()
        sa, sb = scales.cpu().numpy(), rs.cpu().numpy()
        bad = np.nonzero(a != b)[0]
        assert bad.size == 0, (name, bad[:8], a[bad[:8]], b[bad[:8]], bits[bad[:8]])
        assert np.array_equal(sa.view(np.uint32), sb.view(np.uint32)), name


def test_fp8_block_codec_equals_the_reference_kernel_called_block_by_block(cuda_device):
    """The reference has no per-block FP8 mode.  What it has is flame_bf16_to_fp8(x, inv_scale) and the rule of its
    pool (src/activation_offload.rs:543-561): scale = absmax / 448, inv_scale = 1 / scale, both in fp32.  Calling the
    reference's own kernel once per 128-element block with that block's inv_scale must give the bytes of
    flame_act_quant_fp8_b128, and the scales must be absmax / 448."""
    ref = capi.load_ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/libflame_ref_cuda.so was not built (reference checkout absent at build time)")
    rng = np.random.Generator(np.random.PCG64(13))
    finite = synthetic.edge_values()
    cases = {"normal": synthetic.normal_with_outliers(128 * 300, seed=9),
             "every finite value, shuffled": rng.permutation(np.resize(finite, (finite.size + 127) // 128 * 128)),
             "tiny": rng.integers(0x0500, 0x0C00, 128 * 40).astype(np.uint16)}      # 1e-36 .. 1e-31: 1/scale still finite
    sp = G.stream_ptr(cuda_device)
    for name, bits in cases.items():
        x = G.to_dev(bits, cuda_device)
        codes, scales = G.quant("fp8", x)
        absmax = x.float().abs().view(-1, 128).amax(dim=1)
        want_scales = absmax.cpu().numpy() / np.float32(448.0)           # IEEE fp32 division, as the pool does it (torch would multiply by 1/448)
        assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_scales.view(np.uint32)), name
        theirs = torch.zeros(bits.size, dtype=torch.uint8, device=cuda_device)
        with np.errstate(all="ignore"):
            invs = (np.float32(1.0) / want_scales).astype(np.float32)
        for b in range(bits.size // 128):
            if not np.isfinite(invs[b]):
                continue                                                 # an all-zero block, or a scale whose reciprocal overflows
            assert ref.flame_bf16_to_fp8(x.data_ptr() + 256 * b, theirs.data_ptr() + 128 * b, float(invs[b]), 128, sp) == 0
        torch.cuda.synchronize()
        a, r = codes.cpu().numpy().reshape(-1, 128), theirs.cpu().numpy().reshape(-1, 128)
        ok = np.isfinite(invs)
        bad = np.nonzero((a[ok] != r[ok]).any(axis=1))[0]
        assert bad.size == 0, (name, bad[:5])
        assert ok.sum() >= 0.9 * ok.size, name


# ---- size-independent properties at benchmark sizes -------------------------------------------

def test_large_tensor_properties(cuda_device):
    """512 MiB of BF16: round trip within one step per block, max |code| == 127 in every non-zero block,
    and chunk invariance: quantising two halves separately gives the same codes as one launch."""
    n = 1 << 28
    g = torch.Generator(device=cuda_device).manual_seed(0)
    x = torch.randn(n, device=cuda_device, dtype=torch.float32, generator=g).to(torch.bfloat16)
    codes, scales = G.quant("int8", x)
    out = G.dequant("int8", codes, scales, n)
    blk_err = (out.float() - x.float()).abs().view(-1, 128).amax(dim=1)
    assert bool((blk_err <= scales).all())
    assert bool((codes.view(torch.int8).abs().view(-1, 128).amax(dim=1) == 127).all())
    half = n // 2
    c0, s0 = G.quant("int8", x[:half])
    c1, s1 = G.quant("int8", x[half:])
    assert torch.equal(codes[:half], c0) and torch.equal(codes[half:], c1)
    assert torch.equal(scales[: half // 128], s0) and torch.equal(scales[half // 128:], s1)
    # spot check against the oracle on a slice that straddles tile boundaries
    lo, hi = 8192 * 1000 - 300, 8192 * 1000 + 128 * 200
    lo -= lo % 128
    want_c, want_s = capi.quant_int8_b128(G.bits_of(x[lo:hi]))
    assert np.array_equal(codes[lo:hi].cpu().numpy().view(np.int8), want_c)
    assert np.array_equal(scales[lo // 128: hi // 128].cpu().numpy(), want_s)


def _randn_bf16_bits(n: int, device, seed: int) -> torch.Tensor:
    """n BF16 values N(0,1) as an int16 tensor, made in pieces so that no fp32 copy of the whole exists."""
    x = torch.empty(n, dtype=torch.bfloat16, device=device)
    g = torch.Generator(device=device).manual_seed(seed)
    piece = 1 << 27
    for lo in range(0, n, piece):
        hi = min(n, lo + piece)
        x[lo:hi] = torch.randn(hi - lo, device=device, dtype=torch.float32, generator=g).to(torch.bfloat16)
    return x


@pytest.mark.parametrize("codec", ["int8", "fp8"])
def test_more_than_2_to_the_32_elements_in_one_call(cuda_device, codec):
    """2^32 + 128 * 1000 + 37 elements: element, block and tile indices beyond 32 bits.  The first tiles, the blocks on
    both sides of element 2^32 and the ragged tail against the oracle; the whole tensor against the same tensor
    compressed in two calls; the round trip within the codec's step per block, piece by piece."""
    n = (1 << 32) + 128 * 1000 + 37
    free, _ = torch.cuda.mem_get_info(cuda_device)
    if free < (40 << 30):
        pytest.skip("needs 40 GB of free device memory")
    x = _randn_bf16_bits(n, cuda_device, 5)
    codes, scales = G.quant(codec, x)
    q_oracle = capi.quant_int8_b128 if codec == "int8" else capi.quant_fp8_b128
    d_oracle = capi.dequant_int8_b128 if codec == "int8" else capi.dequant_fp8_b128
    windows = [(0, 128 * 200), ((1 << 32) - 128 * 150, (1 << 32) + 128 * 150), ((1 << 31) - 128 * 64, (1 << 31) + 128 * 64), (n - 37 - 128 * 90, n)]
    for lo, hi in windows:
        wc, ws = q_oracle(G.bits_of(x[lo:hi]))
        assert np.array_equal(codes[lo:hi].cpu().numpy(), wc.view(np.uint8)), (lo, hi)
        assert np.array_equal(scales[lo // 128: (hi + 127) // 128].cpu().numpy().view(np.uint32), ws.view(np.uint32)), (lo, hi)
    cut = (1 << 31) + 128 * 3
    c0, s0 = G.quant(codec, x[:cut])
    assert torch.equal(codes[:cut], c0) and torch.equal(scales[: cut // 128], s0)
    del c0, s0
    c1, s1 = G.quant(codec, x[cut:])
    assert torch.equal(codes[cut:], c1) and torch.equal(scales[cut // 128:], s1)
    del c1, s1
    out = G.dequant(codec, codes, scales, n)
    for lo, hi in windows:
        want = d_oracle(codes[lo:hi].cpu().numpy().view(np.int8 if codec == "int8" else np.uint8), scales[lo // 128: (hi + 127) // 128].cpu().numpy())
        assert np.array_equal(G.bits_of(out[lo:hi]), want), (lo, hi)
    # size-independent property over the whole tensor: |x - restored| stays within one int8 step (scale) per block, and within
    # the FP8 format's worst relative step of the block maximum (the reference's encoder sends [248, 448] to one code: 0.53)
    full = n - n % 128
    piece = 1 << 27
    for lo in range(0, full, piece):
        hi = min(full, lo + piece)
        err = (out[lo:hi].float() - x[lo:hi].float()).abs().view(-1, 128).amax(dim=1)
        sc = scales[lo // 128: hi // 128]
        bound = sc if codec == "int8" else sc * 448.0 * 0.53
        assert bool((err <= bound).all()), lo


@pytest.mark.parametrize("codec", ["int8", "fp8"])
def test_codec_launches_replay_from_a_cuda_graph(cuda_device, codec):
    """The codec entry points are plain launches on the caller's stream: compress + dequantise captured once in a CUDA
    graph and replayed on new contents of the same buffers give the oracle's bytes for the new contents."""
    lib = _lib.lib()
    n = (1 << 21) + 128 * 5          # full tiles and a ragged one
    rng_bits = [synthetic.normal_with_outliers(n, seed) for seed in (21, 22)]
    x = G.to_dev(rng_bits[0], cuda_device)
    codes = torch.empty(n, dtype=torch.uint8, device=cuda_device)
    scales = torch.empty(n // 128, dtype=torch.float32, device=cuda_device)
    out = torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
    quant = getattr(lib, f"flame_act_quant_{codec}_b128")
    dequant = getattr(lib, f"flame_act_dequant_{codec}_b128")
    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):     # first use outside the capture: module loading and the occupancy query happen here
        assert quant(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, 0, side.cuda_stream) == 0
        assert dequant(codes.data_ptr(), scales.data_ptr(), out.data_ptr(), n, side.cuda_stream) == 0
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sp = torch.cuda.current_stream(cuda_device).cuda_stream
        assert quant(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), n, 0, sp) == 0
        assert dequant(codes.data_ptr(), scales.data_ptr(), out.data_ptr(), n, sp) == 0
    q_oracle = capi.quant_int8_b128 if codec == "int8" else capi.quant_fp8_b128
    d_oracle = capi.dequant_int8_b128 if codec == "int8" else capi.dequant_fp8_b128
    for bits in (rng_bits[1], rng_bits[0]):
        x.copy_(G.to_dev(bits, cuda_device))
        codes.zero_(); scales.zero_(); out.zero_()
        torch.cuda.synchronize(cuda_device)
        graph.replay()
        torch.cuda.synchronize(cuda_device)
        wc, ws = q_oracle(bits)
        assert np.array_equal(codes.cpu().numpy(), wc.view(np.uint8))
        assert np.array_equal(scales.cpu().numpy().view(np.uint32), ws.view(np.uint32))
        assert np.array_equal(G.bits_of(out), d_oracle(wc, ws))
