"""Seeded synthetic inputs with the shapes and value distributions of the SDXL UNet projections,
and comparison helpers shared by the tests, the smoke test and the benchmark."""
from __future__ import annotations

import numpy as np


def make_activations(seed: int, m: int, k: int, outliers: bool = True) -> np.ndarray:
    """X ~ N(0,1) in FP32, 1% of the channels (a fixed index set drawn from the seed) scaled by 20,
    rounded to FP16. Returns float16 [m, k]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    if outliers and k >= 100:
        channels = rng.choice(k, size=max(1, k // 100), replace=False)
        x[:, channels] *= 20.0
    return x.astype(np.float16)


def make_weight(seed: int, n: int, k: int) -> np.ndarray:
    """W ~ N(0, 1/K) rounded to FP16, [n, k]."""
    rng = np.random.default_rng(seed + 1000003)
    return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(np.float32(k))).astype(np.float16)


def make_bias(seed: int, n: int) -> np.ndarray:
    """b ~ N(0, 0.01) (standard deviation 0.1) rounded to FP16."""
    rng = np.random.default_rng(seed + 2000003)
    return (rng.standard_normal(n, dtype=np.float32) * np.float32(0.1)).astype(np.float16)


def max_rel(actual: np.ndarray, expected: np.ndarray, floor_fraction: float = 1e-3) -> float:
    """max |a-b| / max(|b|, floor_fraction * max|b|): relative error with a floor that avoids
    blow-up near 0. The floor is 1e-3 of the largest output for exact-arithmetic comparisons and
    1e-2 for tensor-core floating-point paths (see the tolerances in test_gpu_parity.py)."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    floor = floor_fraction * float(np.max(np.abs(expected))) if expected.size else 0.0
    denominator = np.maximum(np.abs(expected), max(floor, 1e-30))
    return float(np.max(np.abs(actual - expected) / denominator)) if expected.size else 0.0


def max_abs_over_max(actual: np.ndarray, expected: np.ndarray) -> float:
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    scale = float(np.max(np.abs(expected))) if expected.size else 1.0
    return float(np.max(np.abs(actual - expected))) / max(scale, 1e-30) if expected.size else 0.0


def rms_rel(actual: np.ndarray, expected: np.ndarray) -> float:
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    return float(np.sqrt(np.mean((actual - expected) ** 2)) / max(np.sqrt(np.mean(expected ** 2)), 1e-30))


def f16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in FP16 representable steps between two uint16 bit patterns (finite values)."""
    def ordered(bits):
        bits = bits.astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits & 0x7FFF)
    return np.abs(ordered(np.asarray(a_bits)) - ordered(np.asarray(b_bits)))


def reference_dense(oracle, x_f16: np.ndarray, w_f16: np.ndarray, bias_f16, activation: int) -> np.ndarray:
    """What the reference's CPU build computes for a dense projection, in FP32 throughout:
    linear_2d (bias-initialised FP32 accumulator, products added in index order), then the FP32
    activation (silu_in_place / gelu / geglu of src/unet.cpp). No FP16 rounding anywhere."""
    from scipy.special import erf
    bias = None if bias_f16 is None else bias_f16.astype(np.float32)
    y = oracle.linear_f32(x_f16.astype(np.float32), w_f16.astype(np.float32), bias)
    if activation == 0:
        return y
    if activation == 4:
        return oracle.geglu_f32(y)
    if activation == 1:
        return (y / (np.float32(1.0) + np.exp(-y))).astype(np.float32)
    if activation == 2:
        return (np.float32(0.5) * y * (np.float32(1.0) + erf(y * np.float32(0.7071067811865475)))).astype(np.float32)
    return (y / (np.float32(1.0) + np.exp(np.float32(-1.702) * y))).astype(np.float32)
