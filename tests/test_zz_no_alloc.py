"""The allocation-free entry point `sdxlq_linear_static`.

It serves hosts that may not allocate device memory when they need a projection (all GPU memory
already owned by the host's pool, allocator lock held by the caller, audited allocation-free
steady state): the quantised activations live in an array inside the library image instead of a
context workspace. The test calls it through the C ABI twice in a row, with different inputs and
weights, and requires the outputs to be bit-identical to `sdxlq_linear` on a regular context (same
kernels, same arithmetic, only the scratch differs). Collected last so that a run that stops at the
first failure has already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def static_linear(pkg, ops, call):
    """Builds the C descriptor like Ops.linear does and runs it through sdxlq_linear_static."""
    lib = pkg.load_library()
    desc = ops._desc(call)
    message = ctypes.create_string_buffer(256)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = lib.sdxlq_linear_static(torch.cuda.current_device(), stream, ctypes.byref(desc), message, len(message))
    return status, message.value.decode(), call.y


def int8_weight(pkg, n, k, group, seed):
    wq, ws = O.int8_quantize_rows(H.make_weight(seed, n, k).astype(np.float32), group)
    return pkg.Weight(dev(wq), pkg.ScalarType.Int8, n, k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                      pkg.FP8StorageLayout.RowMajorNK, group), wq, ws


def test_static_linear_matches_context_linear_twice_in_a_row(gpu):
    pkg, ctx, ops = gpu
    # first call: INT8 ConvRot, rotated input, bias; second call right after it: a different,
    # larger INT8 projection with the GEGLU epilogue, so stale scratch from call one would show.
    cases = [(300, 1280, 1280, 256, pkg.ACT_NONE, 41), (1024, 2560, 640, 64, pkg.ACT_GEGLU, 42)]
    for m, n, k, group, activation, seed in cases:
        x = H.make_activations(seed, m, k)
        weight, wq, ws = int8_weight(pkg, n, k, group, seed)
        bias = H.make_bias(seed, n)
        status, message, y_static = static_linear(pkg, ops, pkg.LinearCall(dev(x), weight, dev(bias), activation))
        assert status == 0, message
        if activation:
            y_context = ops.linear_activation(dev(x), weight, dev(bias), activation)
        else:
            y_context = ops.linear(dev(x), weight, dev(bias))
        ctx.check()
        assert torch.equal(y_static, y_context)          # same kernels: bit-identical
        if activation == pkg.ACT_NONE:                     # and both equal the oracle bit for bit
            want = O.int8_convrot_linear(x, wq, ws, group, bias.view(np.uint16), 0)["out"]
            assert np.array_equal(y_static.cpu().numpy().view(np.uint16), want)


def test_static_linear_fp8_and_fp16_paths(gpu):
    pkg, ctx, ops = gpu
    x = H.make_activations(7, 154, 2048, outliers=False)
    wq, ws = O.fp8_quantize_weight(H.make_weight(7, 640, 2048).astype(np.float32), 0, True)
    weight8 = pkg.Weight(dev(wq), pkg.ScalarType.Float8E4M3, 640, 2048, dev(ws), pkg.FP8ScaleMode.PerOutputChannel)
    for repeat in range(2):                                 # the FP8 amax words alternate per call
        status, message, y_static = static_linear(pkg, ops, pkg.LinearCall(dev(x), weight8))
        assert status == 0, message
        assert torch.equal(y_static, ops.linear(dev(x), weight8))
    weight16 = ops.fp16_weight(dev(H.make_weight(8, 640, 2048)))
    status, message, y_static = static_linear(pkg, ops, pkg.LinearCall(dev(x), weight16))
    assert status == 0, message
    assert torch.equal(y_static, ops.linear(dev(x), weight16))
    ctx.check()


def test_static_linear_rejects_what_does_not_fit(gpu):
    pkg, ctx, ops = gpu
    # [8192, 2560] INT8 activations need 21 MB of scratch: more than the 16 MiB array.
    weight, _, _ = int8_weight(pkg, 64, 2560, 256, 3)
    x = torch.zeros((8192, 2560), dtype=torch.float16, device="cuda")
    status, message, _ = static_linear(pkg, ops, pkg.LinearCall(x, weight))
    assert status == 5
    assert "scratch" in message and "16777216" in message
    # invalid arguments are reported, not executed
    lib = pkg.load_library()
    assert lib.sdxlq_linear_static(torch.cuda.current_device(), None, None, None, 0) == 1
    assert lib.sdxlq_linear_static(99, None, None, None, 0) == 1
    # a projection that fits still works afterwards
    small, wq, ws = int8_weight(pkg, 64, 2560, 256, 4)
    xs = H.make_activations(4, 128, 2560)
    status, message, y = static_linear(pkg, ops, pkg.LinearCall(dev(xs), small))
    assert status == 0, message
    assert np.array_equal(y.cpu().numpy().view(np.uint16), O.int8_convrot_linear(xs, wq, ws, 256)["out"])


def test_static_linear_leaves_device_memory_untouched(gpu):
    """cudaMemGetInfo before and after a burst of calls through the static entry point: the free
    figure does not move, i.e. the entry point neither allocates device memory nor grows a pool
    (outputs and inputs are allocated before the first reading; the first call of the process has
    already run in the tests above, so module loading is behind us)."""
    pkg, ctx, ops = gpu
    cases = []
    for seed, (m, n, k, group, activation) in enumerate([(300, 1280, 1280, 256, pkg.ACT_NONE), (1024, 2560, 640, 0, pkg.ACT_GEGLU),
                                                        (154, 640, 2048, 256, pkg.ACT_NONE)]):
        weight, _, _ = int8_weight(pkg, n, k, group, 70 + seed)
        x = dev(H.make_activations(70 + seed, m, k))
        bias = dev(H.make_bias(70 + seed, n))
        y = torch.empty((m, n // 2 if activation == pkg.ACT_GEGLU else n), dtype=torch.float16, device="cuda")
        cases.append(pkg.LinearCall(x, weight, bias, activation, y))
    wq, ws = O.fp8_quantize_weight(H.make_weight(75, 640, 2048).astype(np.float32), 0, True)
    weight8 = pkg.Weight(dev(wq), pkg.ScalarType.Float8E4M3, 640, 2048, dev(ws), pkg.FP8ScaleMode.PerOutputChannel)
    cases.append(pkg.LinearCall(dev(H.make_activations(75, 154, 2048, outliers=False)), weight8, None, pkg.ACT_NONE,
                                torch.empty((154, 640), dtype=torch.float16, device="cuda")))
    for call in cases:                                     # once before the reading
        status, message, _ = static_linear(pkg, ops, call)
        assert status == 0, message
    torch.cuda.synchronize()
    free_before, total = torch.cuda.mem_get_info()
    for _ in range(5):
        for call in cases:
            status, message, _ = static_linear(pkg, ops, call)
            assert status == 0, message
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
