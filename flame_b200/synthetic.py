"""Seeded synthetic activations (numpy PCG64), shared by the tests, the smoke check and the benchmark.

They stand in for real DiT activations: the reference and its benchmark
specification use no dataset for this path.  Every generator returns BF16 bit
patterns as a uint16 array (round-to-nearest-even from float32), so the CPU
checker and the GPU see exactly the same bits.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def normal_with_outliers(numel: int, seed: int = 0, outlier_frac: float = 1e-3) -> np.ndarray:
    """N(0,1) with `outlier_frac` of the entries replaced by +-U(20,60)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal(numel, dtype=np.float32)
    k = int(round(numel * outlier_frac))
    if k:
        idx = rng.choice(numel, size=k, replace=False)
        mag = rng.uniform(20.0, 60.0, size=k).astype(np.float32)
        sign = np.where(rng.integers(0, 2, size=k) == 0, np.float32(-1), np.float32(1))
        x[idx] = mag * sign
    return f32_to_bf16_bits(x)


def normal(numel: int, seed: int = 0) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    return f32_to_bf16_bits(rng.standard_normal(numel, dtype=np.float32))


def gelu_of_normal(numel: int, seed: int = 0) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal(numel, dtype=np.float32).astype(np.float64)
    # tanh form of GELU
    y = 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    return f32_to_bf16_bits(y.astype(np.float32))


def student_t3_times2(numel: int, seed: int = 0) -> np.ndarray:
    """Heavy-tailed attention-output stand-in: 2 * Student-t(nu=3)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return f32_to_bf16_bits((2.0 * rng.standard_t(3.0, size=numel)).astype(np.float32))


def swiglu_hidden(numel: int, seed: int = 0) -> np.ndarray:
    """silu(g) * u with g, u ~ N(0,1)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    g = rng.standard_normal(numel, dtype=np.float32).astype(np.float64)
    u = rng.standard_normal(numel, dtype=np.float32).astype(np.float64)
    return f32_to_bf16_bits((g / (1.0 + np.exp(-g)) * u).astype(np.float32))


def edge_values() -> np.ndarray:
    """Every BF16 bit pattern that is finite, in order (65,280 values)."""
    bits = np.arange(1 << 16, dtype=np.uint32)
    finite = ((bits >> 7) & 0xFF) != 0xFF
    return bits[finite].astype(np.uint16)
