"""The oracle against the reference's own arithmetic, the golden vectors and itself (CPU only)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from flame_b200 import synthetic
from oracle import capi, codec_np


def _golden(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


# ---- FP8 encoder / decoder pinned to the reference ------------------------------------------

def test_encoder_matches_reference_golden(golden_dir):
    """Codes the reference's encoder produced for every finite BF16 value at three scales."""
    g = _golden(golden_dir, "fp8_reference_encoder.npz")
    x = synthetic.bf16_bits_to_f32(synthetic.edge_values())
    for k, inv in enumerate(g["inv_scales"]):
        with np.errstate(all="ignore"):
            y = (x * np.float32(inv)).astype(np.float32)
        want = g[f"codes_{k}"]
        assert np.array_equal(capi.fp8_encode_many(y, 0), want), "frexpf-form oracle"
        assert np.array_equal(capi.fp8_encode_many(y, 1), want), "integer-form oracle"
        assert np.array_equal(codec_np.fp8_encode_ref(y), want), "numpy restatement"
        # and through the element-wise entry point
        assert np.array_equal(capi.bf16_to_fp8(synthetic.edge_values(), inv), want)


def test_oracle_equals_the_reference_kernels_run_on_a_b200(golden_dir):
    """fp8_reference_kernel_sm100.npz: bytes written by the reference's own flame_bf16_to_fp8 / flame_fp8_to_bf16,
    compiled unmodified and run on a B200, for every BF16 pattern (NaN, infinity) and every code, at ordinary,
    extreme, zero, infinite, NaN and negative scales."""
    g = _golden(golden_dir, "fp8_reference_kernel_sm100.npz")
    bits = np.arange(1 << 16, dtype=np.uint16)
    for k, inv in enumerate(g["inv_scales"]):
        want = g["codes"][k]
        assert np.array_equal(capi.bf16_to_fp8(bits, inv), want), float(inv)
        assert np.array_equal(codec_np.bf16_to_fp8(bits, inv), want), float(inv)
    codes = np.arange(256, dtype=np.uint8)
    for k, sc in enumerate(g["dec_scales"]):
        want = g["decoded_bf16_bits"][k]
        nan = (want & 0x7FFF) > 0x7F80                       # 0 * inf: a NaN, whose payload bits are not compared
        got = capi.fp8_to_bf16(codes, sc)
        assert np.array_equal(got[~nan], want[~nan]) and np.all((got[nan] & 0x7FFF) > 0x7F80), float(sc)
        got = codec_np.fp8_to_bf16(codes, sc)
        assert np.array_equal(got[~nan], want[~nan]) and np.all((got[nan] & 0x7FFF) > 0x7F80), float(sc)


def test_int8_block_oracle_equals_the_reference_int8_kernel_run_on_a_b200(golden_dir):
    """int8_reference_sage_sm100.npz: codes and scales written by the reference's own int8 quantisation kernel
    (sage_quantize_tensor, src/sage_attention.rs:510-543) run on a B200 with row_size = 128, on every BF16 bit
    pattern (in order and shuffled; NaN and infinity included) and on N(0,1) data with outliers."""
    src = open(os.path.join(golden_dir, "make_reference_kernel_golden.py")).read()
    # the generator's input recipe, restated here because that script needs torch and a GPU to import
    every = np.arange(1 << 16, dtype=np.uint16)
    inputs = {"every_pattern_in_order": every,
              "every_pattern_shuffled": np.random.Generator(np.random.PCG64(7)).permutation(every),
              "normal_with_outliers": synthetic.normal_with_outliers(1 << 16, seed=0)}
    assert "PCG64(7)" in src and "normal_with_outliers(1 << 16, seed=0)" in src      # the recipe above is the script's
    g = _golden(golden_dir, "int8_reference_sage_sm100.npz")
    for name, bits in inputs.items():
        for impl in (capi.quant_int8_b128, codec_np.quant_int8_b128):
            codes, scales = impl(bits)
            assert np.array_equal(np.asarray(codes).view(np.int8), g[name + "_codes"]), (name, impl.__module__)
            assert np.array_equal(np.asarray(scales, np.float32).view(np.uint32), g[name + "_scales"].view(np.uint32)), (name, impl.__module__)


def test_decoder_matches_reference_golden(golden_dir):
    want = _golden(golden_dir, "fp8_reference_decoder.npy")
    lib = capi.load()
    got = np.array([lib.oracle_fp8_e4m3_decode(c) for c in range(256)], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(codec_np.fp8_decode(np.arange(256, dtype=np.uint8)).view(np.uint32), want.view(np.uint32))
    assert want[0x7F] == 480.0 and want[0xFF] == -480.0          # the reference's own read-back of its saturation code
    assert want[0x80] == 0.0 and np.signbit(want[0x80])           # -0.0


def test_encoder_quirks_known_answers():
    """Known answers worked out from src/cuda/fp8_quant.cu:19-57."""
    lib = capi.load()
    enc = lib.oracle_fp8_e4m3_encode_bits
    assert enc(448.0) == 0x7F and enc(1e9) == 0x7F and enc(float("inf")) == 0x7F
    assert enc(248.0) == 0x7F          # rounds up into exponent 15
    assert enc(240.0) == 0x77          # largest value that survives
    assert enc(1.0625) == 0x39         # tie rounds UP (half-even would give 0x38)
    assert enc(17.0) == 0x59
    assert enc(-0.0) == 0x00           # sign taken from `val < 0`
    assert enc(-1e-9) == 0x80          # negative that rounds to zero keeps its sign
    assert enc(2.0 ** -6 - 2.0 ** -12) == 0x07  # sub-normal arm clamps at 7


def test_integer_form_equals_frexp_form_dense_sweep():
    lib = capi.load()
    bad, first = capi.fp8_encode_sweep(lib.oracle_fp8_e4m3_encode_ref, 0, 1 << 32, 257)
    assert bad == 0, hex(first)


def test_integer_form_equals_compiled_reference_dense_sweep():
    ref = capi.load_ref_encoder()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine (reference checkout absent); golden vectors cover it")
    bad, first = capi.fp8_encode_sweep(ref, 0, 1 << 32, 257)
    assert bad == 0, hex(first)
    dec = capi.load_ref_decoder()
    lib = capi.load()
    for c in range(256):
        assert np.float32(dec(c)).view(np.uint32) == np.float32(lib.oracle_fp8_e4m3_decode(c)).view(np.uint32)


def test_ocp_encoder_matches_ml_dtypes():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(0)
    y = np.concatenate([rng.standard_normal(200000).astype(np.float32) * 100,
                        rng.standard_normal(50000).astype(np.float32) * 0.01,
                        np.float32([0, -0.0, 448, -448, 464, 1e9, -1e9, 2 ** -9, 2 ** -10, 3 * 2 ** -10])])
    want = np.clip(y, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(capi.fp8_encode_many(y, 2), want)


# ---- block codecs: two restatements agree, goldens hold, bounds hold ------------------------

CASES = [("normal_with_outliers", 12582912 // 64, 0), ("normal", 1, 1), ("normal", 127, 2), ("normal", 128, 3),
         ("normal", 129, 4), ("gelu_of_normal", 40000, 5), ("student_t3_times2", 30001, 6), ("swiglu_hidden", 65536 + 5, 7)]


@pytest.mark.parametrize("gen,n,seed", CASES)
def test_c_and_numpy_restatements_agree(gen, n, seed):
    x = getattr(synthetic, gen)(n, seed)
    c8, s8 = capi.quant_int8_b128(x)
    n8, ns8 = codec_np.quant_int8_b128(x)
    assert np.array_equal(c8, n8) and np.array_equal(s8.view(np.uint32), ns8.view(np.uint32))
    m8, _ = capi.quant_int8_b128(x, capi.INT8_MUL_INV)
    assert np.array_equal(m8, codec_np.quant_int8_b128(x, mul_inv=True)[0])
    assert np.array_equal(capi.dequant_int8_b128(c8, s8), codec_np.dequant_int8_b128(c8, s8))
    cf, sf = capi.quant_fp8_b128(x)
    nf, nsf = codec_np.quant_fp8_b128(x)
    assert np.array_equal(cf, nf) and np.array_equal(sf.view(np.uint32), nsf.view(np.uint32))
    assert np.array_equal(capi.dequant_fp8_b128(cf, sf), codec_np.dequant_fp8_b128(cf, sf))


def test_block_codec_goldens(golden_dir):
    from tests.golden.make_golden import BLOCK_CASES

    g = _golden(golden_dir, "block_codec_cases.npz")
    for name, (gen, n, seed) in BLOCK_CASES.items():
        x = getattr(synthetic, gen)(n, seed)
        c8, s8 = capi.quant_int8_b128(x)
        assert np.array_equal(c8, g[f"{name}.int8_codes"]) and np.array_equal(s8, g[f"{name}.int8_scales"])
        assert np.array_equal(capi.dequant_int8_b128(c8, s8), g[f"{name}.int8_out"])
        cf, sf = capi.quant_fp8_b128(x)
        assert np.array_equal(cf, g[f"{name}.fp8_codes"]) and np.array_equal(sf, g[f"{name}.fp8_scales"])
        assert np.array_equal(capi.dequant_fp8_b128(cf, sf), g[f"{name}.fp8_out"])


def test_int8_error_bound_config1_distribution():
    """|dequant - x| <= absmax/127 per block (quantisation half-step + BF16 output rounding)."""
    x = synthetic.normal_with_outliers(1 << 20, 0)
    codes, scales = capi.quant_int8_b128(x)
    out = synthetic.bf16_bits_to_f32(capi.dequant_int8_b128(codes, scales))
    xf = synthetic.bf16_bits_to_f32(x)
    err = np.abs(out - xf).reshape(-1, 128).max(axis=1)
    assert np.all(err <= scales)            # scale == absmax/127
    assert np.abs(codes.astype(np.int32)).max() <= 127
    assert np.array_equal(np.abs(codes.astype(np.int32)).reshape(-1, 128).max(axis=1) == 127, scales > 0)


def test_zero_and_nonfinite_blocks_are_defined():
    x = np.zeros(256, np.uint16)
    x[130] = 0x8000  # -0.0
    c, s = capi.quant_int8_b128(x)
    assert not c.any() and not s.any()
    c, s = capi.quant_fp8_b128(x)
    assert not c.any() and not s.any()
    x[5] = 0x7FC0  # NaN does not become the absmax and encodes as 0 (int8) / sign|0x7F (fp8)
    x[6] = 0x3F80
    c, s = capi.quant_int8_b128(x)
    assert c[5] == 0 and c[6] == 127 and s[0] == np.float32(1.0) / np.float32(127.0)
    c, s = capi.quant_fp8_b128(x)
    assert c[5] == 0x7F and s[0] == np.float32(1.0) / np.float32(448.0)


def test_packed_layout():
    for n in (1, 128, 255, 256, 257, 8192, 12582912):
        so = capi.packed_scales_offset(n)
        assert so % 256 == 0 and so >= n and so - n < 256
        assert capi.packed_bytes(n) == so + 4 * ((n + 127) // 128)
    assert capi.packed_bytes(12582912) == 12976128
    x = synthetic.normal(1000, 9)
    packed, out = capi.roundtrip_mt(x, capi.CODEC_INT8, threads=3)
    codes, scales = capi.quant_int8_b128(x)
    assert np.array_equal(packed[:1000].view(np.int8), codes)
    assert not packed[1000:1024].any()
    assert np.array_equal(packed[1024:].view(np.float32), scales)
    assert np.array_equal(out, capi.dequant_int8_b128(codes, scales))


@pytest.mark.parametrize("codec", [capi.CODEC_NONE, capi.CODEC_INT8, capi.CODEC_FP8])
def test_threaded_roundtrip_equals_single_thread(codec):
    x = synthetic.normal_with_outliers(300000 + 17, 3)
    p1, o1 = capi.roundtrip_mt(x, codec, threads=1)
    p8, o8 = capi.roundtrip_mt(x, codec, threads=8)
    assert np.array_equal(p1, p8) and np.array_equal(o1, o8)
    if codec == capi.CODEC_NONE:
        assert np.array_equal(o1, x)  # uncompressed round trip is bit exact


def test_int8_kernel_quotient_shortcut_is_exact(tmp_path):
    """The reciprocal+residual quotient the int8 kernel uses equals IEEE division (host replay)."""
    src = os.path.join(os.path.dirname(__file__), "helpers", "markstein_check.c")
    exe = str(tmp_path / "markstein_check")
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-o", exe, src, "-lm"], check=True)
    r = subprocess.run([exe, "1500"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    checked, bad = map(int, r.stdout.split())
    assert checked > 10_000_000 and bad == 0


def test_fp8_hardware_path_differs_from_the_reference_only_at_codes_00_and_08(tmp_path):
    """The FP8 compress kernel converts on the conversion hardware and encodes again, exactly, only elements whose
    code came out as 0x00 or 0x08.  Host model of that path against the oracle: every binary32 magnitude in
    [2^-20, 2^-5) and a sparse sweep over all others."""
    here = os.path.dirname(__file__)
    exe = str(tmp_path / "fp8_fast_path_check")
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-o", exe, os.path.join(here, "helpers", "fp8_fast_path_check.c"),
                    os.path.join(os.path.dirname(here), "oracle", "codec_oracle.c"), "-lm", "-lpthread"], check=True)
    r = subprocess.run([exe, "257"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    checked, unexpected, at_08, at_00 = map(int, r.stdout.split())
    assert checked > 130_000_000 and unexpected == 0
    assert at_08 >= 1 << 20 and at_00 == 1      # [7.5, 8) * 2^-9, and the float just under 2^-10


def test_restatements_agree_on_random_magnitude_spread():
    """C and numpy restatements on blocks whose magnitudes span the BF16 range (seeded)."""
    rng = np.random.default_rng(7)
    for trial in range(10):
        n = int(rng.integers(1, 50000))
        bits = synthetic.normal_with_outliers(n, seed=900 + trial)
        expo = rng.integers(-100, 101, size=(n + 127) // 128)
        with np.errstate(all="ignore"):
            f = synthetic.bf16_bits_to_f32(bits).astype(np.float64) * np.repeat(np.exp2(expo.astype(np.float64)), 128)[:n]
        bits = synthetic.f32_to_bf16_bits(np.clip(f, -3e38, 3e38).astype(np.float32))
        c8, s8 = capi.quant_int8_b128(bits)
        n8, ns8 = codec_np.quant_int8_b128(bits)
        assert np.array_equal(c8, n8) and np.array_equal(s8.view(np.uint32), ns8.view(np.uint32))
        cf, sf = capi.quant_fp8_b128(bits)
        nf, nsf = codec_np.quant_fp8_b128(bits)
        assert np.array_equal(cf, nf) and np.array_equal(sf.view(np.uint32), nsf.view(np.uint32))
        assert np.array_equal(capi.dequant_fp8_b128(cf, sf), codec_np.dequant_fp8_b128(cf, sf))
        assert np.array_equal(capi.dequant_int8_b128(c8, s8), codec_np.dequant_int8_b128(c8, s8))


def test_fp8_weight_decoder_restatement(oracle):
    """src/cuda/fused_dequant_transpose.cu:37-72: every code, and the transposed layout."""
    vals = np.array([oracle.load().oracle_fp8_weight_decode(c) for c in range(256)], np.float32)
    assert vals[0] == 0 and np.signbit(vals[0x80]) and vals[0x80] == 0
    assert vals[0x01] == 2.0 ** -9 and vals[0x07] == 7 * 2.0 ** -9 and vals[0x08] == 2.0 ** -6
    assert vals[0x38] == 1.0 and vals[0x77] == 240.0 and vals[0x78] == 256.0 and vals[0xF8] == -256.0
    assert np.isnan(vals[0x79:0x80]).all() and np.isnan(vals[0xF9:]).all() and np.isfinite(vals[:0x79]).all()
    codes = np.arange(6, dtype=np.uint8).reshape(2, 3) + 0x38
    out = oracle.fp8_dequant_transpose(codes, 2.0, 2, 3)
    want = synthetic_f32_to_bf16(np.array([[1.0, 1.375], [1.125, 1.5], [1.25, 1.625]], np.float32) * 2.0)
    assert out.shape == (3, 2) and np.array_equal(out, want)


def synthetic_f32_to_bf16(x):
    from flame_b200 import synthetic

    return synthetic.f32_to_bf16_bits(x.reshape(-1)).reshape(x.shape)


def test_oracle_reproduces_the_reference_weight_kernel_fixture(oracle, golden_dir):
    """What the reference's flame_fused_dequant_transpose_bf16 wrote on a B200 (tests/golden/make_reference_kernel_golden.py)."""
    import os

    path = os.path.join(golden_dir, "fp8_weight_reference_kernel_sm100.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated yet")
    z = np.load(path)
    sys.path.insert(0, golden_dir)
    from make_reference_kernel_golden import weight_inputs

    for name, (codes, m, n) in weight_inputs().items():
        for k, sc in enumerate(z["scales"]):
            assert np.array_equal(oracle.fp8_dequant_transpose(codes, sc, m, n), z[name][k]), (name, float(sc))


def test_oracle_reproduces_the_block_by_block_reference_fp8_fixture(oracle, golden_dir):
    """Per-128-block FP8 pinned to the reference's own kernel run once per block with that block's 1/(absmax/448)."""
    import os

    path = os.path.join(golden_dir, "fp8_b128_reference_kernel_sm100.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated yet")
    z = np.load(path)
    sys.path.insert(0, golden_dir)
    from make_reference_kernel_golden import fp8_block_inputs

    for name, bits in fp8_block_inputs().items():
        codes, scales = oracle.quant_fp8_b128(bits)
        assert np.array_equal(codes, z[name + "_codes"]), name
        assert np.array_equal(scales.view(np.uint32), z[name + "_scales"].view(np.uint32)), name
