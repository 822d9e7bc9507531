"""LayerNorm (Ops::layer_norm of the reference, src/cuda/ops_kernels.cu:185-256) alone and fused with
the INT8 / FP8 activation quantisers.

Bars:
  * oracle (CPU, column-order FP32 sums, correctly rounded 1/sqrt) against the FP64 formula: every
    FP16 output within 1 ulp, at least 99.5 % bit-equal.
  * CUDA FP16 output against the oracle and against the reference's own device kernel (both of its
    builds): at least 99 % of the outputs bit-equal and every output within one FP16 step of the
    larger of |y| and |beta|, i.e. |a - b| <= 2^-10 max(|b|, |beta|). The order of the FP32 additions
    and rsqrtf's 2-ulp error (the device function the reference calls too) move the statistics in
    their last bits, which flips a rounding now and then; where the normalised term and beta cancel
    the result is small and the same absolute difference is several of ITS steps, hence the bound
    in terms of the addends.
  * Fused quantised outputs against quantising THIS library's FP16 LayerNorm result with the
    stand-alone quantisers: bit-exact (scales and bytes), INT8 with and without rotation and both
    FP8 formats -- the fusion changes where the bytes go, not the arithmetic.
"""
import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle as O


def make_case(seed, rows, width):
    rng = np.random.default_rng(seed)
    x = (H.make_activations(seed, rows, width).astype(np.float32) * 2.5 + 0.75).astype(np.float16)
    gamma = (1.0 + 0.2 * rng.standard_normal(width)).astype(np.float16)
    beta = (0.1 * rng.standard_normal(width)).astype(np.float16)
    return x, gamma, beta


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


@pytest.mark.parametrize("rows,width", [(5, 8), (37, 640), (16, 1280), (3, 2048), (4, 100)])
def test_oracle_layer_norm_matches_the_fp64_formula(rows, width):
    x, gamma, beta = make_case(7, rows, width)
    got = O.layer_norm_f16(x.view(np.uint16), gamma.view(np.uint16), beta.view(np.uint16), 1e-5)
    xf = x.astype(np.float64)
    mean = xf.mean(axis=1, keepdims=True)
    variance = xf.var(axis=1, keepdims=True)
    want = ((xf - mean) / np.sqrt(variance + 1e-5) * gamma.astype(np.float64) + beta.astype(np.float64)).astype(np.float16)
    distance = H.f16_ulp_distance(got, want.view(np.uint16))
    assert int(distance.max()) <= 1
    assert float(np.mean(distance == 0)) >= 0.995 or rows * width < 2000


def test_oracle_layer_norm_constant_rows_give_beta():
    # variance 0: inverse = 1 / sqrt(epsilon), centred values are exactly 0, the output is beta
    x = np.full((3, 64), 2.5, np.float16)
    gamma = np.full(64, 1.5, np.float16)
    beta = np.linspace(-1, 1, 64).astype(np.float16)
    got = O.layer_norm_f16(x.view(np.uint16), gamma.view(np.uint16), beta.view(np.uint16), 1e-5)
    assert np.array_equal(got, np.broadcast_to(beta.view(np.uint16), (3, 64)))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,width", [(1, 8), (37, 640), (513, 1280), (9, 2048), (4096, 640), (77, 768), (2, 320), (20011, 640), (7001, 2048)])
def test_layer_norm_f16_matches_oracle_and_reference_device_code(gpu, rows, width):
    pkg, ctx, ops = gpu
    x, gamma, beta = make_case(11, rows, width)
    y = ops.layer_norm(dev(x), dev(gamma), dev(beta), 1e-5)
    ctx.check()
    got = y.cpu().numpy().view(np.uint16)
    want = O.layer_norm_f16(x.view(np.uint16), gamma.view(np.uint16), beta.view(np.uint16), 1e-5)

    def close(actual_bits, expected_bits):
        actual, expected = O.h2f(actual_bits).astype(np.float64), O.h2f(expected_bits).astype(np.float64)
        bound = 2.0 ** -10 * np.maximum(np.abs(expected), np.abs(beta.astype(np.float64))[None, :]) + 1e-7
        assert np.all(np.abs(actual - expected) <= bound), float(np.max(np.abs(actual - expected) / bound))
        assert float(np.mean(actual_bits == expected_bits)) >= 0.99 or rows * width < 2000

    close(got, want)
    if O.RefCuda.available(ieee=True):
        for ieee in (True, False):
            close(got, O.RefCuda(ieee=ieee).layer_norm(x.view(np.uint16), gamma.view(np.uint16), beta.view(np.uint16), 1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("rows,width", [(37, 640), (513, 1280), (2048, 640), (3, 2048), (20011, 640), (9001, 1280), (131073 + 5, 64)])
def test_layer_norm_fp8_equals_layer_norm_then_quantiser(gpu, fmt, rows, width):
    # 20011 / 9001 rows: several rows per warp (the warps' rings wrap around, the cast launch walks backwards);
    # 131078 rows: more than the scratch for the rows' statistics holds, the cast launch reduces the rows again
    pkg, ctx, ops = gpu
    x, gamma, beta = make_case(12 + fmt, rows, width)
    consumer = pkg.Weight(torch.zeros((16, width), dtype=torch.uint8, device="cuda"), pkg.ScalarType(fmt), 16, width,
                          torch.ones(1, device="cuda"), pkg.FP8ScaleMode.TensorWide)
    xd, gd, bd = dev(x), dev(gamma), dev(beta)
    for _ in range(3):                                  # the scratch words clear themselves between calls
        xq, scales = ops.layer_norm_quantized(xd, gd, bd, consumer, 1e-5)
    ctx.check()
    normalised = ops.layer_norm(xd, gd, bd, 1e-5)
    want = ops.quantize_fp8(normalised, pkg.ScalarType(fmt))
    ctx.check()
    assert scales.item() == want.scales.item()
    assert torch.equal(xq, want.data)
    # and the stand-alone quantiser still works after the fused one used the same scratch words
    again = ops.quantize_fp8(normalised, pkg.ScalarType(fmt))
    assert torch.equal(again.data, want.data)


@pytest.mark.gpu
@pytest.mark.parametrize("group", [0, 4, 64, 256])
@pytest.mark.parametrize("rows,width", [(37, 640), (513, 1280), (300, 2560), (5, 256), (4, 100)])
def test_layer_norm_int8_equals_layer_norm_then_quantiser(gpu, group, rows, width):
    pkg, ctx, ops = gpu
    if group and width % group:
        pytest.skip("group does not divide the width")
    x, gamma, beta = make_case(14, rows, width)
    consumer = pkg.Weight(torch.zeros((16, width), dtype=torch.int8, device="cuda"), pkg.ScalarType.Int8, 16, width,
                          torch.ones(16, device="cuda"), pkg.FP8ScaleMode.PerOutputChannel,
                          pkg.FP8StorageLayout.RowMajorNK, group)
    xd, gd, bd = dev(x), dev(gamma), dev(beta)
    xq, scales = ops.layer_norm_quantized(xd, gd, bd, consumer, 1e-5)
    ctx.check()
    if width <= 2048 and width % 8 == 0:
        normalised = ops.layer_norm(xd, gd, bd, 1e-5)
        want_q, want_scales = ops.quantize_int8(normalised, group)
        ctx.check()
        assert torch.equal(scales, want_scales)
        assert torch.equal(xq, want_q)
    # against the oracle end to end: LayerNorm (oracle) -> rotate + quantise (oracle); the statistics
    # may differ in their last bits, so a small share of the bytes may sit one step away
    normalised_bits = O.layer_norm_f16(x.view(np.uint16), gamma.view(np.uint16), beta.view(np.uint16), 1e-5)
    oracle_q, oracle_scales = O.int8_quantize_rows(O.h2f(normalised_bits), group)
    got_q = xq.cpu().numpy().astype(np.int32)
    assert int(np.abs(got_q - oracle_q.astype(np.int32)).max()) <= 1
    assert float(np.mean(got_q == oracle_q)) >= 0.99 or rows * width < 2000
    assert np.allclose(scales.cpu().numpy(), oracle_scales, rtol=2e-3)


@pytest.mark.gpu
def test_layer_norm_feeds_a_projection_like_the_unfused_chain(gpu):
    """norm -> projection through xq / xq_scales equals projection(layer_norm(x)) bit for bit."""
    pkg, ctx, ops = gpu
    rows, width, n = 300, 1280, 640
    x, gamma, beta = make_case(15, rows, width)
    w = H.make_weight(16, n, width)
    bias = dev(H.make_bias(17, n))
    xd, gd, bd = dev(x), dev(gamma), dev(beta)
    normalised = ops.layer_norm(xd, gd, bd)
    wq8, ws8 = O.fp8_quantize_weight(w.astype(np.float32), 0, True)
    fp8 = pkg.Weight(dev(wq8), pkg.ScalarType.Float8E4M3, n, width, dev(ws8), pkg.FP8ScaleMode.PerOutputChannel)
    wq, ws = O.int8_quantize_rows(w.astype(np.float32), 256)
    int8 = pkg.Weight(dev(wq), pkg.ScalarType.Int8, n, width, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                      pkg.FP8StorageLayout.RowMajorNK, 256)
    for weight in (fp8, int8):
        want = ops.linear(normalised, weight, bias)
        xq, scales = ops.layer_norm_quantized(xd, gd, bd, weight)
        got = ops.linear(None, weight, bias, xq=xq, xq_scales=scales)
        ctx.check()
        assert torch.equal(got, want)


@pytest.mark.gpu
def test_layer_norm_argument_errors(gpu):
    pkg, ctx, ops = gpu
    x, gamma, beta = make_case(18, 4, 100)                 # width not a multiple of 8
    with pytest.raises(pkg.CudaError, match="multiple of 8"):
        ops.layer_norm(dev(x), dev(gamma), dev(beta))
    with pytest.raises(pkg.CudaError, match="width mismatch"):
        ops.layer_norm(dev(x), dev(gamma[:50]), dev(beta))
    wide = torch.zeros((2, 4096), dtype=torch.float16, device="cuda")
    with pytest.raises(pkg.CudaError, match="at most 2048"):
        ops.layer_norm(wide, torch.ones(4096, dtype=torch.float16, device="cuda"),
                       torch.zeros(4096, dtype=torch.float16, device="cuda"))
    empty = torch.zeros((0, 640), dtype=torch.float16, device="cuda")
    assert ops.layer_norm(empty, dev(make_case(1, 1, 640)[1]), dev(make_case(1, 1, 640)[2])).shape == (0, 640)
    ctx.check()
