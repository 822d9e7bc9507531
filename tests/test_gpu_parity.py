"""GPU parity tests: every CUDA path is called through the C ABI (ctypes front end) and compared
with the CPU oracle on the same seeded inputs.

Bars (stated here, used below):
  * INT8 ConvRot: quantised activations, per-row scales, INT32 accumulators and the FP16
    projection (dequant, and dequant + bias) are BIT-EXACT against the oracle.
  * Activations (SiLU / GELU / QuickGELU / GEGLU) go through expf and 1 + erf(x / sqrt 2), whose
    CUDA evaluation differs from glibc's in the last FP32 bits; for strongly negative gates the
    reference's `1.0f + erff(...)` cancels, so its own value there is only accurate to about 1e-5
    relative while the outputs are tiny. Bar: every output at least 1 % of the largest one is
    within 1 FP16 ulp, at least 90 % of all outputs are bit-equal, and
    max |a-b| / max(|b|, 1e-3 max|b|) <= 2e-3.
  * FP8: quantised activations and the tensor-wide scale are bit-exact; the FP16 output is within
    FP8_TOL = 1e-2 max-rel of the oracle's order-free FP64-accumulated result.
  * FP16: within FP16_TOL = 2e-3 max-rel of the reference's CPU build (FP32 linear_2d + FP32
    activation, no FP16 rounding anywhere); the CUDA path rounds the projection to FP16 before the
    bias / activation like the reference's CUDA operators do, which is what the bound measures.
  For the two floating-point tensor-core paths max-rel is |a-b| / max(|b|, 1e-2 max|b|): the
  tensor cores add each group of products into the FP32 accumulator with truncation, an absolute
  error of about 1e-5 of the largest partial sum that grows with K and that no kernel running on
  these units can avoid, so outputs much smaller than 1 % of the largest one carry no relative
  guarantee. max|a-b| / max|b| <= 1e-3 is asserted as well. Measured on B200: FP8 1e-3..2.2e-2 and
  FP16 6e-4..1e-2 with the stricter 1e-3 floor, 2e-4..2e-3 and 1e-4..1e-3 with the 1e-2 floor.
"""
import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle as O

pytestmark = pytest.mark.gpu

FP8_TOL = 1e-2      # max_rel, floor 1e-2 * max
FP8_ABS_TOL = 1e-3  # max|a-b| / max|b|
FP16_TOL = 2e-3     # max_rel, floor 1e-2 * max, vs the FP32-sequential CPU reference
FLOAT_FLOOR = 1e-2
ACT_TOL = 2e-3      # INT8 activations vs the oracle, floor 1e-3 * max


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def int8_weight(pkg, n, k, g, seed):
    w = H.make_weight(seed, n, k)
    wq, ws = O.int8_quantize_rows(w.astype(np.float32), g)
    weight = pkg.Weight(dev(wq), pkg.ScalarType.Int8, n, k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                        pkg.FP8StorageLayout.RowMajorNK, g)
    return weight, wq, ws


# ------------------------------------------------------------------------------------------------
# activation quantisers
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,k,g", [
    (2, 4, 4), (2, 4, 0), (1, 16, 16), (37, 640, 0), (37, 640, 64), (37, 640, 16), (37, 640, 4),
    (300, 2560, 256), (154, 2048, 256), (2, 2816, 256), (2, 320, 0), (2, 320, 64), (513, 1280, 256),
    (64, 5120, 256), (3, 12, 4), (5, 8192, 256),
])
def test_int8_activation_quantiser_is_bit_exact(gpu, m, k, g):
    pkg, ctx, ops = gpu
    x = H.make_activations(m * 7 + k + g, m, k)
    xq, scales = ops.quantize_int8(dev(x), g)
    ctx.check()
    want_q, want_s = O.int8_quantize_rows(x.astype(np.float32), g)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(xq.cpu().numpy(), want_q)


def test_int8_quantiser_edge_values(gpu):
    pkg, ctx, ops = gpu
    x = np.zeros((6, 256), np.float16)
    x[1, :] = 65504.0                      # largest FP16: rotated sums stay finite in FP32
    x[2, 3] = np.float16(6e-8)             # FP16 subnormal
    x[3, ::2] = -1.0
    x[4, 7] = np.inf                       # non-finite values are ignored by the row maximum
    x[4, 9] = 2.0
    x[5, 0] = 0.5
    x[5, 1] = 1.5
    x[5, 2] = 2.5                          # ties round to even
    x[5, 3] = 127.0
    for g in (0, 4, 256):
        xq, scales = ops.quantize_int8(dev(x), g)
        ctx.check()
        want_q, want_s = O.int8_quantize_rows(x.astype(np.float32), g)
        finite_rows = [0, 1, 2, 3, 5] if g else [0, 1, 2, 3, 4, 5]
        assert np.array_equal(scales.cpu().numpy().view(np.uint32)[finite_rows], want_s.view(np.uint32)[finite_rows])
        assert np.array_equal(xq.cpu().numpy()[finite_rows], want_q[finite_rows])


def test_int8_quantiser_ties_after_rotation(gpu):
    """These activations hold five values whose rotated, scaled product rounds to an exact x.5 in FP32 although
    the exact product does not: the cast must round the FP32 product (ties to even), not the exact one — a
    multiply fused with the rounding step gives the neighbouring integer there."""
    pkg, ctx, ops = gpu
    x = H.make_activations(12544, 2048, 1280)
    xq, scales = ops.quantize_int8(dev(x), 256)
    ctx.check()
    want_q, want_s = O.int8_quantize_rows(x.astype(np.float32), 256)
    rotated = O.hadamard_rows(x.astype(np.float32), 256)
    scaled = (rotated * np.float32(0.0625)) * (np.float32(1.0) / want_s)[:, None]
    assert int(np.sum(np.abs(scaled - np.trunc(scaled)) == 0.5)) >= 5          # the ties are there
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(xq.cpu().numpy(), want_q)


def test_int8_quantiser_non_finite_values_in_rotated_rows(gpu):
    """A NaN or an infinity poisons its own group of 256 (NaN -> 0, +-inf -> +-127 / -128 after the rotation, as the
    reference's cast gives them); the row's scale comes from its finite values and the other groups are exact."""
    pkg, ctx, ops = gpu
    x = H.make_activations(91, 6, 1280)
    x[1, 300] = np.inf
    x[2, 700] = np.nan
    x[3, 5] = -np.inf
    x[3, 1279] = np.nan
    x[4, 256] = np.float16(65504.0)
    xq, scales = ops.quantize_int8(dev(x), 256)
    ctx.check()
    with np.errstate(invalid="ignore", over="ignore"):
        want_q, want_s = O.int8_quantize_rows(x.astype(np.float32), 256)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(xq.cpu().numpy(), want_q)


def test_int8_quantiser_accepts_fp32_input(gpu):
    pkg, ctx, ops = gpu
    x = np.random.default_rng(5).standard_normal((33, 1280)).astype(np.float32)
    xq, scales = ops.quantize_int8(dev(x), 256)
    want_q, want_s = O.int8_quantize_rows(x, 256)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(xq.cpu().numpy(), want_q)


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("shape", [(2, 2), (154, 2048), (2048, 1280), (3, 5), (1, 8)])
def test_fp8_activation_quantiser_is_bit_exact(gpu, fmt, shape):
    pkg, ctx, ops = gpu
    x = H.make_activations(11 + fmt, *shape)
    quantised = ops.quantize_fp8(dev(x), pkg.ScalarType(fmt))
    ctx.check()
    want_q, want_scale = O.fp8_quantize_activation(x, fmt)
    assert quantised.scale_mode == pkg.FP8ScaleMode.TensorWide and quantised.has_dequant_scale()
    assert np.array_equal(quantised.scales.cpu().numpy().view(np.uint32),
                          np.array([want_scale], np.float32).view(np.uint32))
    assert np.array_equal(quantised.data.cpu().numpy(), want_q)


def test_fp8_quantiser_repeated_calls_and_zero_input(gpu):
    # The amax scratch words alternate between two sets; many calls in a row must not leak state.
    pkg, ctx, ops = gpu
    for step in range(7):
        x = H.make_activations(100 + step, 64, 320, outliers=False) * np.float16(0.5 + step)
        quantised = ops.quantize_e4m3(dev(x))
        want_q, want_scale = O.fp8_quantize_activation(x, 0)
        assert quantised.scales.item() == want_scale
        assert np.array_equal(quantised.data.cpu().numpy(), want_q)
    zero = ops.quantize_e5m2(dev(np.zeros((4, 16), np.float16)))
    assert zero.scales.item() == 1.0 and int(zero.data.max()) == 0


# ------------------------------------------------------------------------------------------------
# INT8 ConvRot Linear
# ------------------------------------------------------------------------------------------------
INT8_CASES = [
    # m, n, k, g, activation, bias, tile_n (0 = library choice), label
    (128, 128, 128, 0, 0, False, 128),
    (256, 256, 640, 0, 0, False, 128),
    (2048, 1280, 1280, 256, 0, False, 0),
    (1000, 640, 640, 64, 0, True, 160),
    (1000, 640, 640, 0, 0, True, 0),
    (154, 1280, 2048, 256, 0, False, 0),
    (154, 640, 2048, 256, 0, False, 0),
    (2, 1280, 320, 0, 1, True, 0),          # time_embedding.linear_1 + SiLU, K = 320
    (2, 1280, 2816, 256, 1, True, 0),       # add_embedding.linear_1 + SiLU, K = 2816
    (2, 320, 1280, 256, 0, True, 0),        # resnet time_emb_proj, N = 320
    (2, 1280, 1280, 256, 0, True, 0),
    (512, 5120, 640, 0, 4, True, 0),        # ff.net.0.proj + GEGLU
    (512, 5120, 640, 64, 4, True, 96),
    (300, 10240, 1280, 256, 4, True, 0),
    (512, 640, 2560, 256, 0, True, 0),      # ff.net.2
    (300, 640, 640, 0, 2, True, 16),        # GELU
    (300, 640, 640, 0, 3, True, 256),       # QuickGELU
    (129, 72, 48, 16, 0, True, 0),          # ragged everything (N not a multiple of 16)
    # the text encoders' projections (src/cuda/text_encoder.cpp:71-105): M = 2 x 77 tokens
    (154, 768, 768, 256, 0, True, 0),       # CLIP-L self_attn q/k/v/out_proj
    (154, 3072, 768, 256, 3, True, 0),      # CLIP-L mlp.fc1 + QuickGELU
    (154, 768, 3072, 256, 0, True, 0),      # CLIP-L mlp.fc2
    (154, 5120, 1280, 256, 2, True, 0),     # OpenCLIP bigG mlp.fc1 + GELU
    (154, 1280, 5120, 256, 0, True, 0),     # OpenCLIP bigG mlp.fc2
]


@pytest.mark.parametrize("m,n,k,g,activation,bias,tile_n", INT8_CASES)
def test_int8_linear_matches_oracle(gpu, m, n, k, g, activation, bias, tile_n):
    pkg, ctx, ops = gpu
    seed = m + 3 * n + 5 * k + g + activation
    x = H.make_activations(seed, m, k)
    weight, wq, ws = int8_weight(pkg, n, k, g, seed)
    b = H.make_bias(seed, n) if (bias or activation) else None
    acc = torch.full((m, n), -7, dtype=torch.int32, device="cuda")
    ctx.set_tile_n(tile_n)
    try:
        if activation:
            y = ops.linear_activation(dev(x), weight, dev(b), activation, acc_out=acc)
        else:
            y = ops.linear(dev(x), weight, dev(b) if b is not None else None, acc_out=acc)
        ctx.check()
    finally:
        ctx.set_tile_n(0)
    ref = O.int8_convrot_linear(x, wq, ws, g, b.view(np.uint16) if b is not None else None, activation)
    assert np.array_equal(acc.cpu().numpy(), ref["acc"]), "INT32 accumulators must be bit-exact"
    got = y.cpu().numpy().view(np.uint16)
    if activation == 0:
        assert np.array_equal(got, ref["out"]), "dequantised FP16 output must be bit-exact"
    else:
        want = O.h2f(ref["out"])
        exact = float(np.mean(got == ref["out"]))
        assert exact >= 0.90, exact
        large = np.abs(want) >= 1e-2 * np.max(np.abs(want))
        assert int(H.f16_ulp_distance(got, ref["out"])[large].max(initial=0)) <= 1
        assert H.max_rel(O.h2f(got), want) <= ACT_TOL
    # against the float Linear on the unquantised operands: quantisation error only
    dense = O.linear_f32(x.astype(np.float32), H.make_weight(seed, n, k).astype(np.float32), None)
    if activation == 0 and b is None:
        assert H.rms_rel(O.h2f(got), dense) < 0.05


def test_int8_linear_full_size_config(gpu):
    """The 640-dim layer set at full size: [8192,640]x[640,640], bit-exact accumulators."""
    pkg, ctx, ops = gpu
    x = H.make_activations(640, 8192, 640)
    weight, wq, ws = int8_weight(pkg, 640, 640, 0, 640)
    acc = torch.empty((8192, 640), dtype=torch.int32, device="cuda")
    y = ops.linear(dev(x), weight, None, acc_out=acc)
    ctx.check()
    ref = O.int8_convrot_linear(x, wq, ws, 0)
    assert np.array_equal(acc.cpu().numpy(), ref["acc"])
    assert np.array_equal(y.cpu().numpy().view(np.uint16), ref["out"])


def test_int8_prequantised_activations_are_reused(gpu):
    pkg, ctx, ops = gpu
    x = H.make_activations(77, 300, 1280)
    weight, wq, ws = int8_weight(pkg, 1280, 1280, 256, 77)
    xq, xs = ops.quantize_int8(dev(x), 256)
    y_shared = ops.linear(None, weight, None, xq=xq, xq_scales=xs)
    y_direct = ops.linear(dev(x), weight, None)
    ctx.check()
    assert torch.equal(y_shared, y_direct)


def test_int8_stats_count_tensor_core_calls(gpu):
    pkg, ctx, ops = gpu
    before = ctx.int8_execution_stats()
    weight, _, _ = int8_weight(pkg, 128, 128, 0, 1)
    ops.linear(dev(H.make_activations(1, 16, 128)), weight, None)
    small, _, _ = int8_weight(pkg, 4, 4, 4, 2)
    ops.linear(dev(H.make_activations(2, 2, 4)), small, None)
    after = ctx.int8_execution_stats()
    assert after["linear_calls"] == before["linear_calls"] + 2
    assert after["tensor_core_calls"] == before["tensor_core_calls"] + 1
    assert after["tensor_core_plan_misses"] == 0 and after["tensor_core_execution_failures"] == 0


# ------------------------------------------------------------------------------------------------
# FP8 and FP16 Linear
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("per_channel", [True, False])
@pytest.mark.parametrize("m,n,k,activation", [
    (256, 1280, 1280, 0), (154, 1280, 2048, 0), (300, 2560, 1280, 4), (2, 1280, 2816, 1), (2048, 1280, 5120, 0),
])
def test_fp8_linear_matches_oracle(gpu, fmt, per_channel, m, n, k, activation):
    pkg, ctx, ops = gpu
    x = H.make_activations(20 + fmt, m, k, outliers=False)
    w = H.make_weight(21, n, k)
    wq, ws = O.fp8_quantize_weight(w.astype(np.float32), fmt, per_channel)
    weight = pkg.Weight(dev(wq), pkg.ScalarType(fmt), n, k, dev(ws),
                        pkg.FP8ScaleMode.PerOutputChannel if per_channel else pkg.FP8ScaleMode.TensorWide)
    b = H.make_bias(22, n)
    y = ops.linear_activation(dev(x), weight, dev(b), activation) if activation else ops.linear(dev(x), weight, dev(b))
    ctx.check()
    ref = O.fp8_native_linear(x, wq, fmt, ws, b.view(np.uint16), activation)
    got = y.cpu().numpy().astype(np.float32)
    want = O.h2f(ref["out"])
    assert H.max_rel(got, want, FLOAT_FLOOR) <= FP8_TOL
    assert H.max_abs_over_max(got, want) <= FP8_ABS_TOL


@pytest.mark.parametrize("m,n,k", [(256, 5120, 640), (300, 640, 640), (2, 1280, 320), (154, 1280, 2048), (130, 72, 40),
                                   (2048, 1280, 5120)])
def test_fp16_projection_matches_reference_cpu_arithmetic(gpu, m, n, k):
    """FP16 weights, no bias: against the reference CPU build (linear_2d, FP32 throughout)."""
    pkg, ctx, ops = gpu
    x = H.make_activations(30, m, k)
    w = H.make_weight(31, n, k)
    y = ops.linear(dev(x), ops.fp16_weight(dev(w)), None)
    ctx.check()
    want = H.reference_dense(O, x, w, None, 0)
    got = y.cpu().numpy().astype(np.float32)
    assert H.max_rel(got, want, FLOAT_FLOOR) <= FP16_TOL
    assert H.max_abs_over_max(got, want) <= 1e-3


@pytest.mark.parametrize("m,n,k,activation", [
    (256, 5120, 640, 4), (300, 640, 640, 0), (2, 1280, 320, 1), (154, 1280, 2048, 0), (130, 72, 40, 0), (64, 256, 640, 2),
])
def test_fp16_linear_with_bias_and_activation(gpu, m, n, k, activation):
    """FP16 weights with bias / activation. The CUDA operators of the reference round the projection
    to FP16 before the bias or activation kernel runs; with that rounding sequence modelled the
    result is within 2 FP16 ulps (4 behind an activation; the FP32 sums differ in their last bits,
    which can move either rounding by one step). Against the all-FP32 CPU build the same two roundings bound the error
    by 2^-11 (|projection| + |output|)."""
    pkg, ctx, ops = gpu
    x = H.make_activations(30, m, k)
    w = H.make_weight(31, n, k)
    b = H.make_bias(32, n)
    weight = ops.fp16_weight(dev(w))
    y = ops.linear_activation(dev(x), weight, dev(b), activation) if activation else ops.linear(dev(x), weight, dev(b))
    ctx.check()
    got_bits = y.cpu().numpy().view(np.uint16)
    got = O.h2f(got_bits)
    projection = O.linear_f32(x.astype(np.float32), w.astype(np.float32), None)
    modelled_bits = O.epilogue_f16(O.f2h(projection), b.view(np.uint16), activation)
    modelled = O.h2f(modelled_bits)
    large = np.abs(modelled) >= FLOAT_FLOOR * np.max(np.abs(modelled))
    worst_ulp = int(H.f16_ulp_distance(got_bits, modelled_bits)[large].max(initial=0))
    # an activation turns a one-step change of its FP16 input into up to ~2 steps of its output
    assert worst_ulp <= (2 if activation == 0 else 4), worst_ulp
    assert H.max_abs_over_max(got, modelled) <= 2e-3, H.max_abs_over_max(got, modelled)
    if activation == 0:
        want = H.reference_dense(O, x, w, b, 0)
        bound = 2.0 ** -11 * (np.abs(projection) + np.abs(want)) * 1.02 + 2e-5 * np.max(np.abs(projection))
        assert np.all(np.abs(got - want) <= bound)


# ------------------------------------------------------------------------------------------------
# the reference's own known-answer cases through the CUDA path (tests/cuda/cuda_ops_test.cu)
# ------------------------------------------------------------------------------------------------
def test_reference_known_answers_on_gpu(gpu):
    pkg, ctx, ops = gpu
    f16 = lambda v: np.asarray(v, np.float32).astype(np.float16)  # noqa: E731
    x = dev(f16([[1, 2], [3, 4]]))
    w = f16([[1, 0], [0, 1], [1, 1]])
    bias = dev(f16([0.5, 0.5, 0.5]))
    expected = np.array([[1.5, 2.5, 3.5], [3.5, 4.5, 7.5]], np.float32)
    linear = ops.linear(x, ops.fp16_weight(dev(w)), bias)                        # :187-199, tol 0.03
    assert np.max(np.abs(linear.cpu().numpy().astype(np.float32) - expected)) <= 0.03
    fused = ops.linear_activation(x, ops.fp16_weight(dev(w)), bias, pkg.ACT_SILU)  # :201-210
    separate = torch.nn.functional.silu(linear.float()).half()
    assert torch.max(torch.abs(fused.float() - separate.float())).item() <= 0.03
    for quantise, tolerance in ((ops.quantize_e4m3, 0.20), (ops.quantize_e5m2, 0.35)):   # :224-246
        out = ops.linear(x, quantise(dev(w)), bias)
        assert np.max(np.abs(out.cpu().numpy().astype(np.float32) - expected)) <= tolerance
    # :269-307 — identity weight, ConvRot group 4, on-the-fly quantisation
    options = pkg.INT8WeightLoadOptions(enable_convrot=True, convrot_group_size=4, strict=True)
    identity = ops.upload_or_quantize_int8_weight(dev(np.eye(4, dtype=np.float32)), None, options)
    assert identity.type == pkg.ScalarType.Int8 and identity.convrot_group_size == 4
    assert identity.dequant_scale_count() == 4
    int8_input = f16([[0.25, -0.5, 0.75, 1.0], [-1.0, 0.5, 0.0, 0.25]])
    out = ops.linear(dev(int8_input), identity, None)
    assert np.max(np.abs(out.cpu().numpy().astype(np.float32) - int8_input.astype(np.float32))) <= 0.04
    # :309-348 — prequantised +-127 Hadamard rows, weight_scale 0.5/127 shaped [4,1], group 4
    hadamard = np.array([[127, 127, 127, -127], [127, 127, -127, 127], [127, -127, 127, 127],
                         [-127, 127, 127, 127]], np.int8)
    metadata = pkg.QuantizationMetadata(weight_scale=dev(np.full((4, 1), 0.5 / 127.0, np.float32)),
                                        convrot=True, per_row=True, convrot_group_size=4)
    options = pkg.INT8WeightLoadOptions(require_prequantized=True, quantize_floating_weights=False,
                                        enable_convrot=True, convrot_group_size=4, strict=True)
    direct = ops.upload_or_quantize_int8_weight(dev(hadamard), metadata, options)
    out = ops.linear(dev(int8_input), direct, None)
    ctx.check()
    assert np.max(np.abs(out.cpu().numpy().astype(np.float32) - int8_input.astype(np.float32))) <= 0.04


# ------------------------------------------------------------------------------------------------
# load-time packers
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("g", [0, 64, 256])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_int8_weight_packer_is_bit_exact(gpu, g, dtype):
    pkg, ctx, ops = gpu
    w = H.make_weight(9, 320, 1280).astype(dtype)
    options = pkg.INT8WeightLoadOptions(enable_convrot=g != 0, convrot_group_size=g if g else 256)
    packed = ops.upload_or_quantize_int8_weight(dev(w), None, options)
    ctx.check()
    want_q, want_s = O.int8_quantize_rows(w.astype(np.float32), g)
    assert packed.convrot_group_size == g
    assert np.array_equal(packed.scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(packed.data.cpu().numpy(), want_q)


def test_int8_default_group_rule(gpu):
    # int8_convrot.cu:520 — rotation only when K is a multiple of the group size (256 by default)
    pkg, ctx, ops = gpu
    options = pkg.INT8WeightLoadOptions()
    assert ops.upload_or_quantize_int8_weight(dev(H.make_weight(1, 64, 640)), None, options).convrot_group_size == 0
    assert ops.upload_or_quantize_int8_weight(dev(H.make_weight(1, 64, 2560)), None, options).convrot_group_size == 256


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("mode", ["tensor", "channel"])
@pytest.mark.parametrize("k_major", [False, True])
def test_fp8_weight_packer_is_bit_exact(gpu, fmt, mode, k_major):
    pkg, ctx, ops = gpu
    rows, columns = 128, 32
    index = np.arange(rows * columns)
    w = (((index % 29) - 14) * 0.03125).astype(np.float32).reshape(rows, columns)   # cuda_ops_test.cu:676-681
    options = pkg.FP8WeightLoadOptions(
        format=pkg.ScalarType(fmt),
        scale_mode=pkg.FP8ScaleMode.PerOutputChannel if mode == "channel" else pkg.FP8ScaleMode.TensorWide,
        layout=pkg.FP8StorageLayout.KMajorKN if k_major else pkg.FP8StorageLayout.RowMajorNK)
    packed = ops.upload_fp8_weight(dev(w), options)
    ctx.check()
    want_q, want_s = O.fp8_quantize_weight(w, fmt, mode == "channel", k_major)
    assert np.array_equal(packed.scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(packed.data.cpu().numpy(), want_q)
    # a K-major weight runs through the small-shape kernel and gives the same Linear
    x = H.make_activations(3, 8, columns, outliers=False)
    y = ops.linear(dev(x), packed, None)
    row_major = ops.upload_fp8_weight(dev(w), pkg.FP8WeightLoadOptions(format=options.format, scale_mode=options.scale_mode))
    y_row = ops.linear(dev(x), row_major, None)
    ctx.check()
    assert H.max_rel(y.float().cpu().numpy(), y_row.float().cpu().numpy(), FLOAT_FLOOR) <= FP8_TOL


def test_native_fp8_checkpoint_is_kept_verbatim(gpu):
    pkg, ctx, ops = gpu
    w = torch.from_numpy(H.make_weight(4, 64, 128).astype(np.float32)).cuda().to(torch.float8_e4m3fn)
    packed = ops.upload_fp8_weight(w, pkg.FP8WeightLoadOptions(format=pkg.ScalarType.Float8E4M3))
    assert torch.equal(packed.data, w.view(torch.uint8)) and float(packed.scales[0]) == 1.0


# ------------------------------------------------------------------------------------------------
# grouped launch
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pair_mode", [0, 1, -1])
def test_grouped_launch_equals_single_calls(gpu, pair_mode):
    """pair_mode 1 / -1 run the 256-row tiles of the plan on CTA pairs (cta_group::2); the single
    calls they are compared with are made with pair_mode 0, on single CTAs, so the two kernel flavours
    must agree bit for bit (outputs the fixture allocates start as NaN, so nothing may stay unwritten)."""
    pkg, ctx, ops = gpu
    ctx.set_pair_mode(pair_mode)
    x1 = dev(H.make_activations(1, 300, 640))
    x2 = dev(H.make_activations(2, 154, 2048))
    x3 = dev(H.make_activations(3, 2, 1280))
    wq, _, _ = int8_weight(pkg, 640, 640, 0, 10)
    wk, _, _ = int8_weight(pkg, 640, 640, 0, 11)
    wff, _, _ = int8_weight(pkg, 5120, 640, 0, 12)
    wkv, _, _ = int8_weight(pkg, 640, 2048, 256, 13)
    wemb, _, _ = int8_weight(pkg, 320, 1280, 256, 14)
    bias_ff = dev(H.make_bias(12, 5120))
    bias_emb = dev(H.make_bias(14, 320))
    w8q, w8s = O.fp8_quantize_weight(H.make_weight(15, 640, 640).astype(np.float32), 0, True)
    w8 = pkg.Weight(dev(w8q), pkg.ScalarType.Float8E4M3, 640, 640, dev(w8s), pkg.FP8ScaleMode.PerOutputChannel)
    w16 = ops.fp16_weight(dev(H.make_weight(16, 640, 640)))
    calls = [
        pkg.LinearCall(x1, wq), pkg.LinearCall(x1, wk),                       # share one quantised x1
        pkg.LinearCall(x1, wff, bias_ff, pkg.ACT_GEGLU),
        pkg.LinearCall(x2, wkv), pkg.LinearCall(x3, wemb, bias_emb),
        pkg.LinearCall(x1, w8), pkg.LinearCall(x1, w16),
    ]
    plan = ops.plan(calls)
    # INT8 quantisers (one launch for the unrotated rows, one for the rotated ones), FP8 amax + cast,
    # and one GEMM launch per kernel flavour in use (single CTA, CTA pair)
    assert 2 + 2 + 1 <= plan.launches <= 2 + 2 + 2
    grouped = [y.clone() for y in plan.run()]
    grouped_again = [y.clone() for y in plan.run()]
    ctx.check()
    one_shot = ops.linear_grouped([pkg.LinearCall(x1, wq), pkg.LinearCall(x3, wemb, bias_emb)])
    ctx.set_pair_mode(0)
    for call, y, y2 in zip(calls, grouped, grouped_again):
        single = ops.linear_activation(call.x, call.weight, call.bias, call.activation) if call.activation \
            else ops.linear(call.x, call.weight, call.bias)
        assert torch.equal(y, single)
        assert torch.equal(y2, single)
    plan.close()
    assert torch.equal(one_shot[0], grouped[0]) and torch.equal(one_shot[1], grouped[4])


@pytest.mark.parametrize("m,n,k,activation", [(300, 640, 640, 0), (2048, 1280, 1280, 0), (1024, 5120, 640, 4), (513, 256, 2560, 1)])
def test_cta_pair_flavour_equals_single_cta_for_single_calls(gpu, m, n, k, activation):
    """One projection per call (its problem record travels in the kernel parameters) on CTA pairs
    (cta_group::2) against the same call on single CTAs: bit-identical, nothing left unwritten."""
    pkg, ctx, ops = gpu
    x = dev(H.make_activations(61, m, k))
    weight, _, _ = int8_weight(pkg, n, k, 0, 62)
    bias = dev(H.make_bias(63, n))
    outputs = []
    for mode in (0, 1):
        ctx.set_pair_mode(mode)
        y = ops.linear_activation(x, weight, bias, activation) if activation else ops.linear(x, weight, bias)
        ctx.check()
        outputs.append(y.clone())
    ctx.set_pair_mode(0)
    assert not torch.isnan(outputs[1]).any()
    assert torch.equal(outputs[0], outputs[1])


def test_empty_input_is_a_no_op(gpu):
    pkg, ctx, ops = gpu
    weight, _, _ = int8_weight(pkg, 64, 64, 0, 1)
    y = ops.linear(torch.empty((0, 64), dtype=torch.float16, device="cuda"), weight, None)
    ctx.check()
    assert tuple(y.shape) == (0, 64)


# ------------------------------------------------------------------------------------------------
# error behaviour (the reference throws CudaError; here: status codes -> CudaError)
# ------------------------------------------------------------------------------------------------
def test_invalid_arguments_raise_cuda_error(gpu):
    pkg, ctx, ops = gpu
    weight, _, _ = int8_weight(pkg, 64, 64, 0, 1)
    x = dev(H.make_activations(1, 4, 64))
    with pytest.raises(pkg.CudaError):
        ops.linear(dev(H.make_activations(1, 4, 32)), weight, None)                 # feature mismatch
    with pytest.raises(pkg.CudaError):
        ops.linear(x, weight, dev(H.make_bias(1, 32)))                               # bias mismatch
    with pytest.raises(pkg.CudaError):
        ops.linear(x.float(), weight, None)                                           # FP32 activations
    bad_group = pkg.Weight(weight.data, weight.type, 64, 64, weight.scales, weight.scale_mode, weight.layout, 48)
    with pytest.raises(pkg.CudaError, match="ConvRot"):
        ops.linear(x, bad_group, None)
    bad_scales = pkg.Weight(weight.data, weight.type, 64, 64, weight.scales[:32].contiguous(), weight.scale_mode)
    with pytest.raises(pkg.CudaError, match="scale"):
        ops.linear(x, bad_scales, None)
    no_scales = pkg.Weight(weight.data, weight.type, 64, 64, None, pkg.FP8ScaleMode.None_)
    with pytest.raises(pkg.CudaError):
        ops.linear(x, no_scales, None)
    odd = pkg.Weight(dev(np.zeros((3, 64), np.float16)), pkg.ScalarType.Float16, 3, 64)
    with pytest.raises(pkg.CudaError, match="GEGLU"):
        ops.linear_activation(x, odd, dev(np.zeros(3, np.float16)), pkg.ACT_GEGLU)
    ctx.check()      # nothing was launched, the context is still healthy
    y = ops.linear(x, weight, None)
    ctx.check()
    assert tuple(y.shape) == (4, 64)


def test_workspace_too_small_is_reported(pkg):
    context = pkg.Context(0, workspace_bytes=4096)
    ops = pkg.Ops(context)
    weight, _, _ = int8_weight(pkg, 64, 640, 0, 1)
    with pytest.raises(pkg.CudaError) as error:
        ops.linear(dev(H.make_activations(1, 512, 640)), weight, None)
    assert error.value.status == 5
    context.close()


def test_bounded_wait_reports_timeout_and_context_survives(gpu):
    """Failure detection without a GPU fault: a wait that nothing satisfies runs out after a short
    limit, the kernel returns, the host reads the status, and the context keeps working."""
    pkg, ctx, ops = gpu
    ctx.selftest_bounded_wait(2_000_000)          # about a millisecond
    with pytest.raises(pkg.CudaError) as error:
        ctx.check()
    assert error.value.status == 3
    ctx.check()
    weight, wq, ws = int8_weight(pkg, 128, 128, 0, 3)
    x = H.make_activations(3, 128, 128)
    y = ops.linear(dev(x), weight, None)
    ctx.check()
    assert np.array_equal(y.cpu().numpy().view(np.uint16), O.int8_convrot_linear(x, wq, ws, 0)["out"])


# ------------------------------------------------------------------------------------------------
# cross-attention K/V projections computed once per generation
# ------------------------------------------------------------------------------------------------
def test_cross_attention_kv_cache_matches_per_call_projections(gpu):
    """The text-encoder hidden states [2*77, 2048] feed attn2.to_k / to_v of every block; the cache
    runs all of them as one grouped launch (one shared quantisation per rotation setting) and must
    return what the per-call operator returns, bit for bit, also after a refresh with a new prompt."""
    pkg, ctx, ops = gpu
    hidden = dev(H.make_activations(31, 154, 2048))
    projections = []
    for index, (n, group) in enumerate([(640, 256), (640, 256), (1280, 256), (1280, 256), (1280, 0)]):
        weight, _, _ = int8_weight(pkg, n, 2048, group, 40 + index)
        projections.append((f"block{index // 2}.attn2.{'to_k' if index % 2 == 0 else 'to_v'}", weight, None))
    cache = pkg.CrossAttentionKVCache(ops, hidden, projections)
    # one rotated and one unrotated quantisation of the hidden states, one GEMM launch
    assert cache.launches == 3
    for name, weight, bias in projections:
        assert torch.equal(cache[name], ops.linear(hidden, weight, bias))
    hidden.copy_(dev(H.make_activations(32, 154, 2048)))
    cache.refresh()
    ctx.check()
    for name, weight, bias in projections:
        assert torch.equal(cache[name], ops.linear(hidden, weight, bias))
    cache.close()


# ------------------------------------------------------------------------------------------------
# prequantised checkpoint -> device -> Linear
# ------------------------------------------------------------------------------------------------
def test_prequantised_int8_checkpoint_loads_and_runs(gpu, tmp_path):
    """A checkpoint in the reference's prequantised layout (weight I8 + weight_scale + comfy_quant)
    written and read by packed_formats goes through the prequantised branch of
    upload_or_quantize_int8_weight and computes what the oracle computes from the same bytes."""
    pkg, ctx, ops = gpu
    pf = pkg.packed_formats
    n, k, group = 320, 1280, 256
    wq, ws = O.int8_quantize_rows(H.make_weight(51, n, k).astype(np.float32), group)
    path = str(tmp_path / "unet_int8.safetensors")
    pf.write_int8_checkpoint(path, {"unet.mid.attn1.to_out.0": pf.Int8LinearRecord(wq, ws.reshape(n, 1), True, True, group)})
    record = pf.read_int8_checkpoint(path)["unet.mid.attn1.to_out.0"]
    metadata = pkg.QuantizationMetadata(weight_scale=dev(record.weight_scale), convrot=record.convrot,
                                        per_row=record.per_row, convrot_group_size=record.convrot_group_size)
    weight = ops.upload_or_quantize_int8_weight(dev(record.weight), metadata,
                                                pkg.INT8WeightLoadOptions(require_prequantized=True))
    assert weight.convrot_group_size == group
    x = H.make_activations(51, 77, k)
    bias = H.make_bias(51, n)
    y = ops.linear(dev(x), weight, dev(bias))
    ctx.check()
    want = O.int8_convrot_linear(x, wq, ws, group, bias.view(np.uint16), 0)["out"]
    assert np.array_equal(y.cpu().numpy().view(np.uint16), want)


# ------------------------------------------------------------------------------------------------
# sharding images over ranks does not change any image's result
# ------------------------------------------------------------------------------------------------
def test_per_image_results_do_not_depend_on_the_shard(gpu):
    """Ranks take whole images (rows of M). With per-token INT8 activation scales and per-row
    accumulation, the rows a rank computes for its images are bit-identical to the same rows of the
    full batch, so an 8-GPU job equals the 1-GPU job image by image. (FP8 activations use one
    tensor-wide scale, so there the shards agree within the FP8 tolerance only.)"""
    pkg, ctx, ops = gpu
    tokens, images = 256, 4
    x = H.make_activations(77, tokens * images, 1280)
    weight, _, _ = int8_weight(pkg, 2560, 1280, 256, 77)
    bias = dev(H.make_bias(77, 2560))
    full = ops.linear_activation(dev(x), weight, bias, pkg.ACT_GEGLU)
    for image in range(images):
        rows = slice(image * tokens, (image + 1) * tokens)
        shard = ops.linear_activation(dev(x[rows]), weight, bias, pkg.ACT_GEGLU)
        assert torch.equal(shard, full[rows])
    wq8, ws8 = O.fp8_quantize_weight(H.make_weight(78, 640, 1280).astype(np.float32), O.E4M3, True)
    weight8 = pkg.Weight(dev(wq8), pkg.ScalarType.Float8E4M3, 640, 1280, dev(ws8), pkg.FP8ScaleMode.PerOutputChannel)
    x8 = H.make_activations(78, tokens * images, 1280, outliers=False)
    full8 = ops.linear(dev(x8), weight8).float().cpu().numpy()
    half8 = ops.linear(dev(x8[: tokens * 2]), weight8).float().cpu().numpy()
    ctx.check()
    assert H.max_rel(half8, full8[: tokens * 2], 1e-2) <= 2e-2
