"""GPU tests of the residual epilogue, of small groups carried in the kernel parameters, of
stream-ordered grouped calls, of stream capture, and of contexts sharing one GPU."""
import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def int8_weight(pkg, n, k, g, seed):
    wq, ws = O.int8_quantize_rows(H.make_weight(seed, n, k).astype(np.float32), g)
    return pkg.Weight(dev(wq), pkg.ScalarType.Int8, n, k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                      pkg.FP8StorageLayout.RowMajorNK, g), wq, ws


def fp8_weight(pkg, n, k, seed, fmt=0, per_channel=True):
    wq, ws = O.fp8_quantize_weight(H.make_weight(seed, n, k).astype(np.float32), fmt, per_channel)
    kind = pkg.ScalarType.Float8E4M3 if fmt == 0 else pkg.ScalarType.Float8E5M2
    mode = pkg.FP8ScaleMode.PerOutputChannel if per_channel else pkg.FP8ScaleMode.TensorWide
    return pkg.Weight(dev(wq), kind, n, k, dev(ws), mode)


def half_add(a_bits, b_bits):
    """__hadd on FP16 bit patterns: one rounding of the exact sum (float32 holds it exactly)."""
    return (a_bits.view(np.float16).astype(np.float32) + b_bits.view(np.float16).astype(np.float32)).astype(np.float16).view(np.uint16)


# ------------------------------------------------------------------------------------------------
# residual add in the epilogue (Ops::add_in_place after to_out / ff.net.2 / proj_out)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k,g,with_bias", [
    (300, 640, 640, 0, True), (513, 1280, 5120, 256, True), (154, 640, 2560, 256, False), (130, 72, 40, 4, True),
    (2048, 1280, 1280, 256, True),
])
def test_int8_residual_epilogue_is_bit_exact(gpu, m, n, k, g, with_bias):
    pkg, ctx, ops = gpu
    x = H.make_activations(21, m, k)
    weight, wq, ws = int8_weight(pkg, n, k, g, 21)
    bias = H.make_bias(21, n) if with_bias else None
    residual = H.make_activations(22, m, n, outliers=False)
    y = ops.linear(dev(x), weight, dev(bias) if with_bias else None, residual=dev(residual))
    ctx.check()
    want = O.int8_convrot_linear(x, wq, ws, g, bias.view(np.uint16) if with_bias else None, 0)["out"]
    want = half_add(want, residual.view(np.uint16))
    assert np.array_equal(y.cpu().numpy().view(np.uint16), want)
    # in place: the hidden state is both the residual and the output
    hidden = dev(residual).clone()
    out = ops.linear(dev(x), weight, dev(bias) if with_bias else None, residual=hidden, out=hidden)
    ctx.check()
    assert out.data_ptr() == hidden.data_ptr()
    assert np.array_equal(hidden.cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("kind", ["e4m3", "e5m2", "f16"])
def test_residual_epilogue_equals_unfused_add(gpu, kind):
    pkg, ctx, ops = gpu
    m, n, k = 1000, 1280, 1280
    x = dev(H.make_activations(23, m, k, outliers=False))
    bias = dev(H.make_bias(23, n))
    residual = dev(H.make_activations(24, m, n, outliers=False))
    weight = ops.fp16_weight(dev(H.make_weight(23, n, k))) if kind == "f16" else fp8_weight(pkg, n, k, 23, 0 if kind == "e4m3" else 1)
    fused = ops.linear(x, weight, bias, residual=residual)
    unfused = ops.linear(x, weight, bias) + residual          # FP16 add = __hadd
    ctx.check()
    assert torch.equal(fused, unfused)


def test_residual_requires_no_activation(gpu):
    pkg, ctx, ops = gpu
    weight, _, _ = int8_weight(pkg, 64, 64, 0, 1)
    x = dev(H.make_activations(1, 4, 64))
    call = pkg.LinearCall(x, weight, dev(H.make_bias(1, 64)), pkg.ACT_SILU, residual=torch.zeros((4, 64), dtype=torch.float16, device="cuda"))
    with pytest.raises(pkg.CudaError, match="un-activated"):
        ops.linear_grouped([call])


# ------------------------------------------------------------------------------------------------
# small groups in the kernel parameters, larger ones through stream-ordered tables
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["int8", "int8_rot", "e4m3", "f16"])
@pytest.mark.parametrize("m", [300, 2048])
def test_attention_projection_group_equals_single_calls(gpu, kind, m):
    """to_q / to_k / to_v of one input as one grouped call (no table, one quantisation)."""
    pkg, ctx, ops = gpu
    c = 1280 if kind == "int8_rot" else 640
    x = dev(H.make_activations(31, m, c))
    if kind.startswith("int8"):
        weights = [int8_weight(pkg, c, c, 256 if kind == "int8_rot" else 0, 31 + i)[0] for i in range(3)]
    elif kind == "e4m3":
        weights = [fp8_weight(pkg, c, c, 31 + i) for i in range(3)]
    else:
        weights = [ops.fp16_weight(dev(H.make_weight(31 + i, c, c))) for i in range(3)]
    stats_before = ctx.int8_execution_stats()["linear_calls"]
    grouped = ops.linear_grouped([pkg.LinearCall(x, w) for w in weights])
    ctx.check()
    for w, y in zip(weights, grouped):
        assert torch.equal(y, ops.linear(x, w))
    if kind.startswith("int8"):
        assert ctx.int8_execution_stats()["linear_calls"] == stats_before + 6


def test_group_of_four_with_mixed_shapes(gpu):
    pkg, ctx, ops = gpu
    x = dev(H.make_activations(35, 700, 640))
    weights = [int8_weight(pkg, n, 640, 0, 35 + i)[0] for i, n in enumerate((640, 320, 5120, 72))]
    biases = [None, dev(H.make_bias(36, 320)), dev(H.make_bias(37, 5120)), None]
    activations = [0, pkg.ACT_SILU, pkg.ACT_GEGLU, 0]
    calls = [pkg.LinearCall(x, w, b, a) for w, b, a in zip(weights, biases, activations)]
    grouped = ops.linear_grouped(calls)
    ctx.check()
    for call, y in zip(calls, grouped):
        single = ops.linear_activation(call.x, call.weight, call.bias, call.activation) if call.activation else ops.linear(call.x, call.weight, call.bias)
        assert torch.equal(y, single)


def test_large_one_shot_group_is_stream_ordered(gpu):
    """More than four projections (or several distinct inputs): tables travel through the staging
    buffer; two such calls back to back, no synchronisation in between, then compared."""
    pkg, ctx, ops = gpu
    xs = [dev(H.make_activations(40 + i, 200 + 50 * i, 640)) for i in range(3)]
    weights = [int8_weight(pkg, 640, 640, 64, 40 + i)[0] for i in range(6)]
    first = [pkg.LinearCall(xs[i % 3], weights[i]) for i in range(6)]
    second = [pkg.LinearCall(xs[(i + 1) % 3], weights[i]) for i in range(6)]
    out_first = ops.linear_grouped(first)
    out_second = ops.linear_grouped(second)
    ctx.check()
    for call, y in zip(first + second, out_first + out_second):
        assert torch.equal(y, ops.linear(call.x, call.weight))


def test_plan_runs_only_on_its_context(gpu, pkg):
    _, ctx, ops = gpu
    weight, _, _ = int8_weight(pkg, 64, 64, 0, 1)
    plan = ops.plan([pkg.LinearCall(dev(H.make_activations(1, 8, 64)), weight)])
    other = pkg.Context(0, workspace_bytes=1 << 20)
    status = plan._lib.sdxlq_group_plan_run(other.handle, plan._handle)
    assert status == 1 and b"another context" in plan._lib.sdxlq_last_error(other.handle)
    other.close()
    plan.run()
    ctx.check()
    plan.close()


# ------------------------------------------------------------------------------------------------
# stream capture: single calls and small groups record into a CUDA graph and replay
# ------------------------------------------------------------------------------------------------
def test_calls_can_be_captured_and_replayed(gpu):
    pkg, ctx, ops = gpu
    m, c = 512, 640
    x = dev(H.make_activations(50, m, c))
    w8 = [fp8_weight(pkg, c, c, 50 + i) for i in range(3)]
    wi, _, _ = int8_weight(pkg, c, c, 64, 53)
    bias = dev(H.make_bias(54, c))
    static_x = x.clone()
    # eager results for two different inputs
    def eager(inp):
        q, k, v = ops.linear_grouped([pkg.LinearCall(inp, w) for w in w8])
        o = ops.linear(q, wi, bias, residual=inp)          # an odd number of FP8 quantisations per replay
        p = ops.linear(o, w8[0])
        return [t.clone() for t in (q, k, v, o, p)]
    want_a = eager(x)
    x_b = dev(H.make_activations(51, m, c))
    want_b = eager(x_b)
    ctx.check()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ctx.set_stream(side)
        eager(static_x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        ctx.set_stream(torch.cuda.current_stream())
        q, k, v = ops.linear_grouped([pkg.LinearCall(static_x, w) for w in w8])
        o = ops.linear(q, wi, bias, residual=static_x)
        p = ops.linear(o, w8[0])
    ctx.set_stream(torch.cuda.current_stream())
    for inp, want in ((x, want_a), (x_b, want_b), (x, want_a)):
        static_x.copy_(inp)
        graph.replay()
        torch.cuda.synchronize()
        for got, expected in zip((q, k, v, o, p), want):
            assert torch.equal(got, expected)
    # a grouped call that needs device tables refuses to be captured, and says what to do instead
    big = [pkg.LinearCall(static_x, w8[i % 3]) for i in range(6)]
    graph2 = torch.cuda.CUDAGraph()
    with pytest.raises(pkg.CudaError, match="build a plan"):
        with torch.cuda.graph(graph2):
            ctx.set_stream(torch.cuda.current_stream())
            ops.linear_grouped(big)
    ctx.set_stream(torch.cuda.current_stream())
    torch.cuda.synchronize()
    ctx.check()


@pytest.mark.parametrize("kind", ["e4m3", "int8"])
def test_dependent_launches_do_not_change_a_block(gpu, pkg, monkeypatch, kind):
    """Every kernel of the path is launched as a programmatic dependent of the one before it (it may be scheduled
    while that one still runs and waits before it touches memory). A chain shaped like a transformer block
    (LayerNorm -> q/k/v -> out + residual -> LayerNorm -> GEGLU -> ff.net.2 + residual, the quantisers in
    between reusing the same scratch) must give the same bits with the attribute, without it, and in a replayed
    graph, repeat after repeat."""
    _, ctx, ops = gpu
    m, c = 4096, 640
    if kind == "e4m3":
        make = lambda n, k, seed: fp8_weight(pkg, n, k, seed)
        group = 0
    else:
        make = lambda n, k, seed: int8_weight(pkg, n, k, 64, seed)[0]
        group = 64
    w_qkv = [make(c, c, 70 + i) for i in range(3)]
    w_out, w_ff0, w_ff2 = make(c, c, 73), make(2 * 4 * c, c, 74), make(c, 4 * c, 75)
    bias_out, bias_ff0, bias_ff2 = dev(H.make_bias(76, c)), dev(H.make_bias(77, 8 * c)), dev(H.make_bias(78, c))
    gamma = dev((1.0 + 0.1 * np.random.default_rng(79).standard_normal(c)).astype(np.float16))
    beta = dev((0.1 * np.random.default_rng(80).standard_normal(c)).astype(np.float16))
    x0 = dev(H.make_activations(81, m, c))

    def block(operator, hidden):
        xq, scales = operator.layer_norm_quantized(hidden, gamma, beta, w_qkv[0], 1e-5)
        q, k, v = operator.linear_grouped([pkg.LinearCall(hidden, w, xq=xq, xq_scales=scales) for w in w_qkv])
        mixed = (q.float() * 0.5 + k.float() * 0.25 + v.float() * 0.25).half()       # stands in for the attention
        hidden = operator.linear(mixed, w_out, bias_out, residual=hidden)
        xq, scales = operator.layer_norm_quantized(hidden, gamma, beta, w_ff0, 1e-5)
        gated = operator.linear_activation(hidden, w_ff0, bias_ff0, pkg.ACT_GEGLU, xq=xq, xq_scales=scales)
        return operator.linear(gated, w_ff2, bias_ff2, residual=hidden)

    def run(operator, repeats):
        hidden = x0
        for _ in range(repeats):
            hidden = block(operator, hidden)
        return hidden

    monkeypatch.setenv("SDXLQ_EARLY_LAUNCH", "0")
    plain_context = pkg.Context(0, workspace_bytes=64 << 20)
    monkeypatch.delenv("SDXLQ_EARLY_LAUNCH")
    plain = pkg.Ops(plain_context)
    want = run(plain, 4).clone()
    plain_context.check()
    got = run(ops, 4)
    ctx.check()
    assert torch.isfinite(want.float()).all()
    assert torch.equal(got, want)
    # replayed graph on the session's context
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ctx.set_stream(side)
        run(ops, 1)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        ctx.set_stream(torch.cuda.current_stream())
        held = run(ops, 4)
    ctx.set_stream(torch.cuda.current_stream())
    for _ in range(5):
        held.zero_()
        graph.replay()
    torch.cuda.synchronize()
    ctx.check()
    assert torch.equal(held, want)
    plain_context.close()


# ------------------------------------------------------------------------------------------------
# several contexts on one GPU
# ------------------------------------------------------------------------------------------------
def test_contexts_with_different_tile_geometries_share_a_gpu(gpu, pkg):
    """Context A runs a projection with 256-column tiles (4 x 48 KB stages), context B a narrow one
    (small stages), the allocation-free entry point another, then A runs its wide tiles again: the
    shared-memory opt-in of the kernel is per device, not per context."""
    import ctypes
    _, ctx_a, ops_a = gpu
    ctx_b = pkg.Context(0, workspace_bytes=64 << 20)
    ops_b = pkg.Ops(ctx_b, poison_outputs=True)
    x_wide = dev(H.make_activations(60, 1024, 640))
    wide, wq, ws = int8_weight(pkg, 5120, 640, 0, 60)
    bias = dev(H.make_bias(60, 5120))
    x_narrow = dev(H.make_activations(61, 40, 64))
    narrow, nq, ns = int8_weight(pkg, 16, 64, 0, 61)
    want_wide = ops_a.linear_activation(x_wide, wide, bias, pkg.ACT_GEGLU)
    want_narrow = O.int8_convrot_linear(H.make_activations(61, 40, 64), nq, ns, 0)["out"]
    for _ in range(2):
        got_narrow = ops_b.linear(x_narrow, narrow)
        ctx_b.check()
        assert np.array_equal(got_narrow.cpu().numpy().view(np.uint16), want_narrow)
        call = pkg.LinearCall(x_narrow, narrow)
        desc = ops_a._desc(call)
        message = ctypes.create_string_buffer(256)
        status = pkg.load_library().sdxlq_linear_static(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                                        ctypes.byref(desc), message, 256)
        assert status == 0, message.value
        torch.cuda.synchronize()
        assert np.array_equal(call.y.cpu().numpy().view(np.uint16), want_narrow)
        again = ops_a.linear_activation(x_wide, wide, bias, pkg.ACT_GEGLU)
        ctx_a.check()
        assert torch.equal(again, want_wide)
    ctx_b.close()


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("m,n,k,activation", [(300, 2560, 640, 4), (256, 640, 640, 0), (37, 72, 40, 0)])
def test_output_maximum_hand_over_to_the_fp8_quantiser(gpu, fmt, m, n, k, activation):
    """y_amax: the producing projection leaves max |y| (FP32 bits) in a device word; x_amax: the consuming
    FP8 projection skips its maximum pass, reads the word and clears it. Bit-identical to the plain calls;
    the last shape runs on the small-shape kernel (row pitch not a multiple of 16 bytes)."""
    pkg, ctx, ops = gpu
    x = dev(H.make_activations(81, m, k, outliers=False))
    first = H.make_weight(82, n, k)
    n_mid = n // 2 if activation == 4 else n
    second = H.make_weight(83, 320, n_mid)
    weights = []
    for w in (first, second):
        wq, ws = O.fp8_quantize_weight(w.astype(np.float32), fmt, True)
        weights.append(pkg.Weight(dev(wq), pkg.ScalarType(fmt), w.shape[0], w.shape[1], dev(ws), pkg.FP8ScaleMode.PerOutputChannel))
    bias = dev(H.make_bias(84, n))
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain_mid = ops.linear_activation(x, weights[0], bias, activation) if activation else ops.linear(x, weights[0], bias)
    plain_out = ops.linear(plain_mid, weights[1], None)
    for _ in range(2):                                   # twice: the word must be back at zero after each use
        mid = ops.linear_activation(x, weights[0], bias, activation, y_amax=word) if activation \
            else ops.linear(x, weights[0], bias, y_amax=word)
        ctx.check()
        assert torch.equal(mid, plain_mid)
        want_bits = plain_mid.float().abs().max().view(torch.int32)
        assert int(word.item()) == int(want_bits.item())
        out = ops.linear(mid, weights[1], None, x_amax=word)
        ctx.check()
        assert int(word.item()) == 0
        assert torch.equal(out, plain_out)
