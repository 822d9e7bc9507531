"""CPU-side checks of the boundary: the C-ABI library loads and exports every symbol the header
declares, the ctypes structures match the C layout, and the host-side mirror of the reference
interface validates arguments like the reference does (no GPU needed, no compute calls)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sdxlq.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sdxlq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    pkg.build()
    lib = pkg.load_library()
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/sdxlq.h but not exported"
    assert sorted(pkg.api.EXPORTED_SYMBOLS) == names
    assert b"sm_100a" in lib.sdxlq_build_info()


def test_ctypes_structures_match_the_c_layout(pkg, tmp_path):
    source = tmp_path / "layout.c"
    source.write_text(
        '#include "sdxlq.h"\n#include <stdio.h>\n#include <stddef.h>\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(sdxlq_weight),\n'
        "         sizeof(sdxlq_linear_desc),\n"
        "         offsetof(sdxlq_linear_desc, weight), offsetof(sdxlq_linear_desc, bias),\n"
        "         offsetof(sdxlq_linear_desc, y), offsetof(sdxlq_linear_desc, acc_out),\n"
        "         offsetof(sdxlq_weight, convrot_group_size), sizeof(sdxlq_int8_stats),\n"
        "         offsetof(sdxlq_linear_desc, residual), sizeof(sdxlq_layer_norm_desc),\n"
        "         offsetof(sdxlq_layer_norm_desc, epsilon), offsetof(sdxlq_layer_norm_desc, y),\n"
        "         offsetof(sdxlq_layer_norm_desc, xq_scales), sizeof(sdxlq_kernel_times));\n"
        "  return 0;\n}\n")
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(source), "-o", str(binary)], check=True)
    c_sizes = [int(v) for v in subprocess.run([str(binary)], capture_output=True, text=True, check=True).stdout.split()]
    api = pkg.api
    py_sizes = [ctypes.sizeof(api._CWeight), ctypes.sizeof(api._CLinearDesc), api._CLinearDesc.weight.offset,
                api._CLinearDesc.bias.offset, api._CLinearDesc.y.offset, api._CLinearDesc.acc_out.offset,
                api._CWeight.convrot_group_size.offset, ctypes.sizeof(api._CStats),
                api._CLinearDesc.residual.offset, ctypes.sizeof(api._CLayerNormDesc),
                api._CLayerNormDesc.epsilon.offset, api._CLayerNormDesc.y.offset,
                api._CLayerNormDesc.xq_scales.offset, ctypes.sizeof(api._CKernelTimes)]
    assert c_sizes == py_sizes


def test_header_compiles_as_c_and_cxx(tmp_path):
    for compiler, suffix in (("gcc", "c"), ("g++", "cpp")):
        source = tmp_path / f"include_only.{suffix}"
        source.write_text('#include "sdxlq.h"\nint main(void) { return SDXLQ_OK; }\n')
        subprocess.run([compiler, "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(source),
                        "-o", str(tmp_path / f"a_{suffix}")], check=True)


def test_cxx_shim_compiles_against_the_header(tmp_path):
    """The C++20 shim that mirrors Ops::linear / linear_activation is header-only over the C ABI."""
    shim = os.path.join(ROOT, "sdxl-end2end_b200", "cpp")
    source = tmp_path / "shim.cpp"
    source.write_text(
        '#include "sdxlq_ops.hpp"\n'
        '// instantiates the grouped projection set (no GPU work is launched: no context exists)\n'
        'static void unused(const sdxlq::Ops& ops, const std::vector<sdxlq::Ops::ProjectionSet::Entry>& entries) {\n'
        '    sdxlq::Ops::ProjectionSet set(ops, entries);\n'
        '    set.run();\n'
        '    (void)set.outputs();\n'
        '    (void)set.launches();\n'
        '}\n'
        'int main() { (void)&unused; return sdxlq::valid_convrot_group_size(64) ? 0 : 1; }\n')
    lib_dir = os.path.join(ROOT, "sdxl-end2end_b200")
    subprocess.run(["g++", "-std=c++20", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", shim,
                    str(source), "-L", lib_dir, "-lsdxlq", f"-Wl,-rpath,{lib_dir}", "-o", str(tmp_path / "shim")],
                   check=True)
    assert subprocess.run([str(tmp_path / "shim")]).returncode == 0


def test_enum_values_match_the_reference(pkg):
    # include/sdxl/cuda/tensor.hpp:17-48 and ops.hpp:15 of the reference
    assert [int(v) for v in pkg.ScalarType] == [0, 1, 2, 3, 4, 5]
    assert pkg.ScalarType.Int8 == 2 and pkg.ScalarType.Float16 == 3
    assert [int(v) for v in pkg.FP8ScaleMode] == [0, 1, 2]
    assert [int(v) for v in pkg.FP8StorageLayout] == [0, 1]
    assert [int(v) for v in pkg.LinearActivation] == [0, 1, 2, 3, 4]
    header = open(HEADER).read()
    for name, value in (("SDXLQ_INT8", 2), ("SDXLQ_FP16", 3), ("SDXLQ_ACT_GEGLU", 4),
                        ("SDXLQ_SCALE_PER_OUTPUT_CHANNEL", 2), ("SDXLQ_K_MAJOR_KN", 1)):
        assert re.search(rf"{name}\s*=\s*{value}\b", header), name


def test_valid_convrot_group_size_host_and_library(pkg):
    lib = pkg.load_library()
    for group in range(0, 1100):
        expected = group in (4, 16, 64, 256)
        assert pkg.valid_convrot_group_size(group) == expected
        assert bool(lib.sdxlq_valid_convrot_group_size(group)) == expected


def test_null_context_is_rejected_without_a_gpu(pkg):
    lib = pkg.load_library()
    assert lib.sdxlq_linear(None, None) == 1
    assert lib.sdxlq_context_check(None) == 1
    assert lib.sdxlq_get_stats(None, None) == 1
    assert lib.sdxlq_status_string(3) == b"device wait timed out"
    assert lib.sdxlq_last_error(None) == b""
    assert lib.sdxlq_workspace_bytes(None, 0) == 0


class _FakeContext:
    """Enough of Context for the host-side validation paths that never reach the library."""

    def __init__(self, pkg):
        self._lib = pkg.load_library()
        self.handle = None

    def raise_for(self, status):
        raise AssertionError("validation should have failed before any library call")


def test_weight_loader_validation_mirrors_the_reference(pkg):
    import torch
    ops = pkg.Ops(_FakeContext(pkg))
    options = pkg.INT8WeightLoadOptions()
    with pytest.raises(pkg.CudaError, match="rank 2"):
        ops.upload_or_quantize_int8_weight(torch.zeros(4), None, options)
    with pytest.raises(pkg.CudaError, match="cannot be empty"):
        ops.upload_or_quantize_int8_weight(torch.zeros((0, 4)), None, options)
    with pytest.raises(pkg.CudaError, match="prequantized-only"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 4)), None,
                                           pkg.INT8WeightLoadOptions(require_prequantized=True))
    with pytest.raises(pkg.CudaError, match="disabled"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 4)), None,
                                           pkg.INT8WeightLoadOptions(quantize_floating_weights=False))
    with pytest.raises(pkg.CudaError, match="missing weight_scale"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 4), dtype=torch.int8), None, options)
    metadata = pkg.QuantizationMetadata(weight_scale=torch.ones(4), convrot=True, convrot_group_size=8)
    with pytest.raises(pkg.CudaError, match="incompatible with weight shape"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 16), dtype=torch.int8), metadata, options)
    metadata = pkg.QuantizationMetadata(weight_scale=torch.ones(3), convrot=False)
    with pytest.raises(pkg.CudaError, match="not per-output-row"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 16), dtype=torch.int8), metadata, options)
    with pytest.raises(pkg.CudaError, match="power of four"):
        ops.upload_or_quantize_int8_weight(torch.zeros((4, 16)), None,
                                           pkg.INT8WeightLoadOptions(convrot_group_size=8))
    with pytest.raises(pkg.CudaError, match="float16 input"):
        ops.quantize_fp8(torch.zeros((2, 2)), pkg.ScalarType.Float8E4M3)
    with pytest.raises(pkg.CudaError, match="rank-2"):
        ops.upload_fp8_weight(torch.zeros(4), pkg.FP8WeightLoadOptions(scale_mode=pkg.FP8ScaleMode.PerOutputChannel))


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    monkeypatch.setattr(pkg.api, "_lib", None)
    monkeypatch.setattr(pkg.api._build, "LIBRARY", str(tmp_path / "absent.so"))
    with pytest.raises(pkg.CudaError, match="no CPU fallback"):
        pkg.load_library()


def test_product_does_not_import_the_oracle():
    package = os.path.join(ROOT, "sdxl-end2end_b200")
    for directory, _, files in os.walk(package):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".hpp", ".h", ".cpp")):
                text = open(os.path.join(directory, name), errors="ignore").read()
                assert "oracle" not in text.lower(), f"{name} refers to the oracle"
    assert "oracle" not in open(HEADER).read().lower()
