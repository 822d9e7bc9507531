"""Pins the CPU oracle: (1) the reference's own known-answer tests for the projection path
(tests/cuda/cuda_ops_test.cu of the reference, cited per test) replayed through the oracle,
(2) the oracle's dense path against the unmodified reference `linear_2d`/`geglu` compiled from
the reference sources (oracle/_ref, skipped where that library was not built), and
(3) committed golden vectors generated from the reference (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_dense.npz")


def f16(values):
    return np.asarray(values, np.float32).astype(np.float16)


def bits(values):
    return f16(values).view(np.uint16)


def close(actual, expected, tolerance):
    return np.max(np.abs(np.asarray(actual, np.float64) - np.asarray(expected, np.float64))) <= tolerance


LINEAR_INPUT = f16([[1, 2], [3, 4]])
LINEAR_WEIGHT = f16([[1, 0], [0, 1], [1, 1]])
LINEAR_BIAS = f16([0.5, 0.5, 0.5])
LINEAR_EXPECTED = np.array([[1.5, 2.5, 3.5], [3.5, 4.5, 7.5]], np.float32)


def dense_f16(x, w, bias, activation):
    """FP16 Linear as Ops::linear runs it: GEMM result rounded to FP16, then the epilogue."""
    y = O.f2h(O.linear_f32(x.astype(np.float32), w.astype(np.float32), None))
    return O.h2f(O.epilogue_f16(y, None if bias is None else bias.view(np.uint16), activation))


def test_fp16_linear_known_answers():
    # cuda_ops_test.cu:187-199 — 2x2 . 3x2 + bias, tolerance 0.03
    out = dense_f16(LINEAR_INPUT, LINEAR_WEIGHT, LINEAR_BIAS, O.ACT_NONE)
    assert close(out, LINEAR_EXPECTED, 0.03)
    assert np.array_equal(out, LINEAR_EXPECTED)


def test_fused_activation_equals_unfused():
    # cuda_ops_test.cu:201-222 — linear_activation(SiLU / GEGLU) vs separate kernels, tolerance 0.03
    linear = dense_f16(LINEAR_INPUT, LINEAR_WEIGHT, LINEAR_BIAS, O.ACT_NONE)
    separate_silu = (linear / (1.0 + np.exp(-linear))).astype(np.float16).astype(np.float32)
    fused_silu = dense_f16(LINEAR_INPUT, LINEAR_WEIGHT, LINEAR_BIAS, O.ACT_SILU)
    assert close(fused_silu, separate_silu, 0.03)
    geglu_weight = f16([[1, 0], [0, 1], [0.5, 0], [0, 0.5]])
    geglu_bias = f16([0.1, 0.2, 0.3, 0.4])
    projected = dense_f16(LINEAR_INPUT, geglu_weight, geglu_bias, O.ACT_NONE)
    separate = O.geglu_f32(projected).astype(np.float16).astype(np.float32)
    fused = dense_f16(LINEAR_INPUT, geglu_weight, geglu_bias, O.ACT_GEGLU)
    assert fused.shape == (2, 2)
    assert close(fused, separate, 0.03)


@pytest.mark.parametrize("fmt,tolerance", [(O.E4M3, 0.20), (O.E5M2, 0.35)])
def test_fp8_linear_known_answers(fmt, tolerance):
    # cuda_ops_test.cu:224-246 — the weight goes through quantize_e4m3 / quantize_e5m2 (tensor-wide
    # scale), the input through the native path's activation quantiser.
    wq, w_scale = O.fp8_quantize_activation(LINEAR_WEIGHT, fmt)
    result = O.fp8_native_linear(LINEAR_INPUT, wq, fmt, np.array([w_scale], np.float32),
                                 LINEAR_BIAS.view(np.uint16), O.ACT_NONE)
    assert close(O.h2f(result["out"]), LINEAR_EXPECTED, tolerance)


def test_fp8_aligned_identity():
    # cuda_ops_test.cu:248-267 — 16x16 identity weight, inputs ((r + c) % 7 - 3) / 8, tolerance 0.08
    rows = np.arange(16)
    x = (((rows[:, None] + rows[None, :]) % 7) - 3).astype(np.float32) * 0.125
    wq, w_scale = O.fp8_quantize_activation(f16(np.eye(16)), O.E4M3)
    result = O.fp8_native_linear(f16(x), wq, O.E4M3, np.array([w_scale], np.float32))
    assert close(O.h2f(result["out"]), x, 0.08)


INT8_INPUT = f16([[0.25, -0.5, 0.75, 1.0], [-1.0, 0.5, 0.0, 0.25]])


def test_int8_convrot_identity_weight():
    # cuda_ops_test.cu:269-307 — identity weight quantised on the fly with ConvRot g = 4:
    # the rotation cancels, output == input within 0.04.
    wq, w_scales = O.int8_quantize_rows(np.eye(4, dtype=np.float32), 4)
    assert wq.dtype == np.int8 and w_scales.shape == (4,)
    result = O.int8_convrot_linear(INT8_INPUT, wq, w_scales, 4)
    assert close(O.h2f(result["out"]), INT8_INPUT.astype(np.float32), 0.04)


def test_int8_prequantized_hadamard():
    # cuda_ops_test.cu:309-348 — prequantised +-127 regular-Hadamard rows, weight_scale 0.5 / 127,
    # comfy_quant {convrot, group 4}: the stored weight is the rotated identity.
    wq = np.array([[127, 127, 127, -127], [127, 127, -127, 127], [127, -127, 127, 127],
                   [-127, 127, 127, 127]], np.int8)
    scales = np.full(4, 0.5 / 127.0, np.float32)
    result = O.int8_convrot_linear(INT8_INPUT, wq, scales, 4)
    assert close(O.h2f(result["out"]), INT8_INPUT.astype(np.float32), 0.04)


def test_hadamard_rows_match_the_stored_weight_pattern():
    # The H4 used by the reference (int8_convrot.cu:138-141): rows of the rotated identity / 2.
    rotated = O.hadamard_rows(np.eye(4, dtype=np.float32), 4) * 0.5
    expected = np.array([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], np.float32) * 0.5
    assert np.array_equal(rotated, expected.T)
    for group in (16, 64, 256):
        x = np.random.default_rng(group).standard_normal((3, group)).astype(np.float32)
        once = O.hadamard_rows(x, group) / np.sqrt(group)
        # H / sqrt(g) is orthogonal: norms are preserved
        assert np.allclose(np.linalg.norm(once, axis=1), np.linalg.norm(x, axis=1), rtol=1e-5)


@pytest.mark.parametrize("fmt", [O.E4M3, O.E5M2])
@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("k_major", [False, True])
def test_fp8_weight_pack_pattern(fmt, per_channel, k_major):
    # cuda_ops_test.cu:676-681, 697-701 — weight pattern ((i % 29) - 14) / 32 survives packing
    # (either layout) within 0.04 after dequantisation.
    rows, columns = 128, 32
    index = np.arange(rows * columns)
    w = (((index % 29) - 14) * 0.03125).astype(np.float32).reshape(rows, columns)
    q, scales = O.fp8_quantize_weight(w, fmt, per_channel, k_major)
    logical = O.fp8_decode(q, fmt)
    if k_major:
        assert q.shape == (columns, rows)
        logical = logical.T
    logical = logical * (scales[:, None] if per_channel else scales[0])
    tolerance = 0.04 if fmt == O.E4M3 else 0.07     # the reference test pins E4M3 only
    assert close(logical, w, tolerance)


def test_valid_convrot_group_size():
    # int8_convrot.cu:489-496
    assert [g for g in range(0, 300) if O.valid_convrot_group_size(g)] == [4, 16, 64, 256]


def test_zero_rows_get_unit_scale():
    # int8_convrot.cu:199, 304-305; fp8_kernels.cu:36 — amax == 0 -> scale 1
    q, s = O.int8_quantize_rows(np.zeros((2, 8), np.float32), 4)
    assert np.all(q == 0) and np.all(s == 1.0)
    q8, s8 = O.fp8_quantize_activation(np.zeros((2, 8), np.float16), O.E4M3)
    assert np.all(q8 == 0) and s8 == 1.0


def test_int8_saturation_and_rounding():
    x = np.array([[127.0, -127.0, 63.5, 0.5, 1.5, 2.5, -0.5, -1.5]], np.float32)
    q, s = O.int8_quantize_rows(x, 0)
    assert s[0] == 1.0
    assert q.tolist() == [[127, -127, 64, 0, 2, 2, 0, -2]]      # round half to even


needs_ref = pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (reference tree absent)")


@needs_ref
def test_dense_oracle_is_bit_equal_to_reference_linear_2d():
    rng = np.random.default_rng(7)
    x = rng.standard_normal((24, 640)).astype(np.float32)
    w = (rng.standard_normal((80, 640)) / 25).astype(np.float16)
    bias = (rng.standard_normal(80) * 0.1).astype(np.float16)
    reference = O.ref_linear_2d(x, w, bias)
    restated = O.linear_f32(x, w.astype(np.float32), bias.astype(np.float32))
    assert np.array_equal(reference.view(np.uint32), restated.view(np.uint32))
    assert np.array_equal(O.ref_geglu(reference).view(np.uint32), O.geglu_f32(restated).view(np.uint32))


@needs_ref
@pytest.mark.parametrize("fmt", [O.E4M3, O.E5M2])
def test_fp8_decode_matches_reference_tensor_reader(fmt):
    # The reference CPU path decodes FP8 weights per element (src/unet.cpp:91-142).
    rng = np.random.default_rng(9)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    finite = np.array([b for b in range(256) if np.isfinite(O.fp8_decode(np.array([b], np.uint8), fmt)[0])], np.uint8)
    wq = rng.choice(finite, size=(32, 64)).astype(np.uint8)
    reference = O.ref_linear_2d(x, wq, None, fp8_fmt=fmt)
    restated = O.linear_f32(x, O.fp8_decode(wq, fmt))
    assert np.array_equal(reference.view(np.uint32), restated.view(np.uint32))


def test_committed_golden_vectors_from_the_reference():
    data = np.load(GOLDEN)
    x, w, bias = data["x"], data["w"], data["bias"]
    restated = O.linear_f32(x.astype(np.float32), w.astype(np.float32), bias.astype(np.float32))
    assert np.array_equal(restated.view(np.uint32), data["linear_2d"].view(np.uint32))
    assert np.array_equal(O.geglu_f32(restated).view(np.uint32), data["geglu"].view(np.uint32))
    for fmt, name in ((O.E4M3, "e4m3"), (O.E5M2, "e5m2")):
        restated8 = O.linear_f32(data["x8"].astype(np.float32), O.fp8_decode(data[f"w_{name}"], fmt))
        assert np.array_equal(restated8.view(np.uint32), data[f"linear_2d_{name}"].view(np.uint32))
