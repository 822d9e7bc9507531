"""Runs the C++20 host side (sdxl-end2end_b200/cpp/sdxlq_ops.hpp, sdxlq_weights.hpp) on the GPU: a
small C++ program (tests/cpp/shim_driver.cpp) is compiled against the header and libsdxlq.so, fed
vectors from this test, and its outputs are compared with the oracle. The program also checks the
precision-profile parser and the eligibility rules on the host."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import helpers as H
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, "sdxl-end2end_b200")


def build_driver(directory) -> str:
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    binary = os.path.join(directory, "shim_driver")
    command = [shutil.which("g++") or "g++", "-std=c++20", "-Wall", "-Wextra", "-O1", "-I", os.path.join(ROOT, "include"),
               "-I", os.path.join(PACKAGE, "cpp"), "-I", os.path.join(cuda, "include"),
               os.path.join(ROOT, "tests", "cpp", "shim_driver.cpp"), "-o", binary, "-L", PACKAGE, "-lsdxlq",
               "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{PACKAGE}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    result = subprocess.run(command, capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    return binary


def test_cxx_driver_compiles(tmp_path, pkg):
    """Host-only: the driver builds against the headers and the library (no GPU needed)."""
    pkg.load_library()
    build_driver(str(tmp_path))


@pytest.mark.gpu
@pytest.mark.parametrize("precision,m,n,k,group,activation,residual", [
    (0, 300, 640, 640, 64, 0, False), (0, 300, 1280, 640, 0, 4, False), (0, 513, 1280, 2560, 256, 0, True),
    (1, 300, 640, 1280, 0, 0, False), (2, 154, 640, 2048, 0, 1, False),
])
def test_cxx_ops_match_the_oracle(tmp_path, pkg, precision, m, n, k, group, activation, residual):
    pkg.load_library()
    binary = build_driver(str(tmp_path))
    x = H.make_activations(90, m, k, outliers=precision != 1)
    w = H.make_weight(90, n, k)
    bias = H.make_bias(90, n)
    n_out = n // 2 if activation == 4 else n
    extra = H.make_activations(91, m, n_out, outliers=False)
    case, result = str(tmp_path / "case.bin"), str(tmp_path / "result.bin")
    with open(case, "wb") as handle:
        handle.write(np.array([m, n, k, group, activation, precision, int(residual)], np.uint64).tobytes())
        for array in (x, w, bias, extra):
            handle.write(np.ascontiguousarray(array).tobytes())
    run = subprocess.run([binary, case, result], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr + run.stdout
    raw = np.fromfile(result, np.uint8)
    y = raw[: m * n_out * 2].view(np.uint16).reshape(m, n_out)
    offset = m * n_out * 2
    bias_bits = bias.view(np.uint16)
    if precision == 0:
        wq, ws = O.int8_quantize_rows(w.astype(np.float32), group)
        want = O.int8_convrot_linear(x, wq, ws, group, bias_bits, activation)["out"]
        if residual:
            want = (want.view(np.float16).astype(np.float32) + extra.astype(np.float32)).astype(np.float16).view(np.uint16)
        if activation == 0:
            assert np.array_equal(y, want)
        else:
            assert H.max_rel(O.h2f(y), O.h2f(want)) <= 2e-3
    elif precision == 1:
        wq, ws = O.fp8_quantize_weight(w.astype(np.float32), 0, True)
        want = O.fp8_native_linear(x, wq, 0, ws, bias_bits, activation)["out"]
        assert H.max_rel(O.h2f(y), O.h2f(want), 1e-2) <= 1e-2
    else:
        want = H.reference_dense(O, x, w, bias, activation)
        assert H.max_rel(O.h2f(y), want, 1e-2) <= 2e-3
    if activation == 0:
        group_bytes = 3 * m * n * 2
        grouped = raw[offset: offset + group_bytes].view(np.uint16).reshape(3, m, n)
        offset += group_bytes
        plain = y if not residual else None
        for part in grouped:                       # three projections of one input: all equal, and equal to linear() - bias
            assert np.array_equal(part, grouped[0])
        if precision == 0 and not residual:
            no_bias = O.int8_convrot_linear(x, wq, ws, group, None, 0)["out"]
            assert np.array_equal(grouped[0], no_bias)
    calls = int(raw[offset: offset + 8].view(np.uint64)[0])
    assert calls == ((1 + (3 if activation == 0 else 0)) if precision == 0 else 0)
