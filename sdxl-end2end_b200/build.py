"""Builds libsdxlq.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBRARY = os.path.join(HERE, "libsdxlq.so")
SOURCES = ["capi.cu", "gemm_umma.cu", "quantize.cu", "quantize_int8_fast.cu", "linear_small.cu", "layer_norm.cu", "harness_norm.cu"]
HEADERS = ["internal.cuh", "ptx.cuh", "quantize.cuh", "fp8_math.cuh", "int8_math.cuh", os.path.join("..", "..", "include", "sdxlq.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC", "-shared",
    "--fmad=true",
]


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def needs_build() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    inputs = [os.path.join(CSRC, s) for s in SOURCES] + [os.path.join(CSRC, h) for h in HEADERS]
    return _newest(inputs) > os.path.getmtime(LIBRARY)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every CUDA source for sm_100a into one shared library. Returns its path."""
    if not force and not needs_build():
        return LIBRARY
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    command = [nvcc, *NVCC_FLAGS]
    if os.environ.get("SDXLQ_BUILD_DIAGNOSTICS"):
        # tuning build: SDXLQ_DIAGNOSTIC_SKIP can switch parts of the GEMM kernel off
        command.append("-DSDXLQ_DIAGNOSTICS")
    if verbose:
        command += ["-Xptxas", "-v"]
    command += ["-o", LIBRARY] + [os.path.join(CSRC, s) for s in SOURCES]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed building libsdxlq.so")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
