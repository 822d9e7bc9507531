"""numpy front end of the CPU oracle (oracle/sdxlq_oracle.c) and of the reference-built
checker (oracle/_ref/libsdxl_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU
arms of ``bench.py``; never by the shipped package.

Activation codes follow the reference's ``LinearActivation`` enum
(include/sdxl/cuda/ops.hpp:15): 0 None, 1 SiLU, 2 GELU, 3 QuickGELU, 4 GEGLU.
FP8 format codes: 0 = E4M3FN, 1 = E5M2.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libsdxlq_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libsdxl_ref.so")

ACT_NONE, ACT_SILU, ACT_GELU, ACT_QUICK_GELU, ACT_GEGLU = 0, 1, 2, 3, 4
E4M3, E5M2 = 0, 1

_c_size = ctypes.c_size_t
_p = ctypes.c_void_p


def reference_root() -> str:
    """Where the reference project's sources lie: $SDXL_REFERENCE_ROOT, else a `reference` directory
    beside this repository."""
    return os.environ.get("SDXL_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref_root: str | None = None) -> None:
    """Compile the oracle; also the reference checker when the reference tree is present."""
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
    ref_root = ref_root or reference_root()
    if os.path.isdir(os.path.join(ref_root, "src")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={ref_root}"], check=True, capture_output=True)
        if os.path.isdir(os.path.join(ref_root, "src", "cuda")) and shutil.which("nvcc", path=_nvcc_path()):
            subprocess.run(["make", "-C", _HERE, "refcuda", f"REF={ref_root}"], check=True, capture_output=True)


def _nvcc_path() -> str:
    return os.pathsep.join([os.environ.get("PATH", ""), "/usr/local/cuda/bin"])


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        _lib = ctypes.CDLL(_ORACLE_SO)
        _lib.orc_h2f.restype = ctypes.c_float
        _lib.orc_h2f.argtypes = [ctypes.c_uint16]
        _lib.orc_f2h.restype = ctypes.c_uint16
        _lib.orc_f2h.argtypes = [ctypes.c_float]
        _lib.orc_fp8_decode.restype = ctypes.c_float
        _lib.orc_fp8_decode.argtypes = [ctypes.c_uint8, ctypes.c_int]
        _lib.orc_fp8_encode.restype = ctypes.c_uint8
        _lib.orc_fp8_encode.argtypes = [ctypes.c_float, ctypes.c_int]
        _lib.orc_fp8_quantize_activation.restype = ctypes.c_float
        _lib.orc_valid_convrot_group_size.argtypes = [_c_size]
    return _lib


def _ptr(array: np.ndarray) -> ctypes.c_void_p:
    assert array.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(array.ctypes.data)


def _c(array, dtype) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


def as_f16_bits(x) -> np.ndarray:
    """Any float array -> uint16 bit pattern of its FP16 rounding (through the oracle's rounder)."""
    x = np.asarray(x)
    if x.dtype == np.uint16:
        return np.ascontiguousarray(x)
    if x.dtype == np.float16:
        return np.ascontiguousarray(x).view(np.uint16)
    return f2h(x)


def h2f(bits: np.ndarray) -> np.ndarray:
    bits = _c(bits, np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().orc_h2f_array(_ptr(bits), _ptr(out), _c_size(bits.size))
    return out


def f2h(values: np.ndarray) -> np.ndarray:
    values = _c(values, np.float32)
    out = np.empty(values.shape, np.uint16)
    lib().orc_f2h_array(_ptr(values), _ptr(out), _c_size(values.size))
    return out


def fp8_decode(bits: np.ndarray, fmt: int) -> np.ndarray:
    bits = _c(bits, np.uint8)
    out = np.empty(bits.shape, np.float32)
    lib().orc_fp8_decode_array(_ptr(bits), _ptr(out), _c_size(bits.size), ctypes.c_int(fmt))
    return out


def fp8_encode(values: np.ndarray, fmt: int) -> np.ndarray:
    values = _c(values, np.float32)
    out = np.empty(values.shape, np.uint8)
    lib().orc_fp8_encode_array(_ptr(values), _ptr(out), _c_size(values.size), ctypes.c_int(fmt))
    return out


def valid_convrot_group_size(group_size: int) -> bool:
    return bool(lib().orc_valid_convrot_group_size(_c_size(group_size)))


def hadamard_rows(x: np.ndarray, group_size: int) -> np.ndarray:
    x = _c(x, np.float32)
    rows, columns = x.shape
    out = np.empty_like(x)
    lib().orc_hadamard_rows(_ptr(x), _ptr(out), _c_size(rows), _c_size(columns), _c_size(group_size))
    return out


def int8_quantize_rows(x: np.ndarray, group_size: int):
    """x: [rows, columns] float32 values (FP16 inputs widened first). -> (int8 [rows,cols], f32 [rows])."""
    x = _c(x, np.float32)
    rows, columns = x.shape
    if group_size:
        assert valid_convrot_group_size(group_size) and columns % group_size == 0
    q = np.empty((rows, columns), np.int8)
    scales = np.empty((rows,), np.float32)
    lib().orc_int8_quantize_rows(_ptr(x), _c_size(rows), _c_size(columns), _c_size(group_size),
                                 _ptr(q), _ptr(scales))
    return q, scales


def int8_gemm_i32(xq: np.ndarray, wq: np.ndarray) -> np.ndarray:
    xq = _c(xq, np.int8)
    wq = _c(wq, np.int8)
    m, k = xq.shape
    n, k2 = wq.shape
    assert k == k2
    acc = np.empty((m, n), np.int32)
    lib().orc_int8_gemm_i32(_ptr(xq), _ptr(wq), _ptr(acc), _c_size(m), _c_size(n), _c_size(k))
    return acc


def int8_dequant_f16(acc: np.ndarray, a_scales: np.ndarray, w_scales: np.ndarray) -> np.ndarray:
    acc = _c(acc, np.int32)
    a_scales = _c(a_scales, np.float32)
    w_scales = _c(w_scales, np.float32)
    m, n = acc.shape
    out = np.empty((m, n), np.uint16)
    lib().orc_int8_dequant_f16(_ptr(acc), _ptr(a_scales), _ptr(w_scales), _c_size(m), _c_size(n), _ptr(out))
    return out


def epilogue_f16(y_bits: np.ndarray, bias_bits: np.ndarray | None, activation: int) -> np.ndarray:
    """Applies what Ops::linear / Ops::linear_activation run after the GEMM
    (src/cuda/ops_blas.cpp:259, 296, 384, 388-397 of the reference) to an FP16 result."""
    y = np.array(_c(y_bits, np.uint16))
    rows, width = y.shape
    if bias_bits is None:
        assert activation == ACT_NONE
        return y
    bias = _c(bias_bits, np.uint16)
    assert bias.shape == (width,)
    if activation == ACT_NONE:
        lib().orc_bias_add_f16(_ptr(y), _ptr(bias), _c_size(rows), _c_size(width))
        return y
    if activation == ACT_GEGLU:
        assert width % 2 == 0
        out = np.empty((rows, width // 2), np.uint16)
        lib().orc_bias_geglu_f16(_ptr(y), _ptr(bias), _ptr(out), _c_size(rows), _c_size(width // 2))
        return out
    lib().orc_bias_activation_f16(_ptr(y), _ptr(bias), _c_size(rows), _c_size(width), ctypes.c_int(activation))
    return y


def int8_convrot_linear(x_bits: np.ndarray, wq: np.ndarray, w_scales: np.ndarray, group_size: int,
                        bias_bits: np.ndarray | None = None, activation: int = ACT_NONE) -> dict:
    """The whole INT8 Linear as the reference runs it (int8_convrot_linear,
    src/cuda/int8_convrot.cu:579-751, then the epilogue of Ops::linear[_activation])."""
    x = h2f(as_f16_bits(x_bits))
    xq, a_scales = int8_quantize_rows(x, group_size)
    acc = int8_gemm_i32(xq, wq)
    y = int8_dequant_f16(acc, a_scales, w_scales)
    out = epilogue_f16(y, bias_bits, activation)
    return {"xq": xq, "a_scales": a_scales, "acc": acc, "y": y, "out": out}


def fp8_quantize_activation(x_bits: np.ndarray, fmt: int):
    x_bits = as_f16_bits(x_bits)
    q = np.empty(x_bits.shape, np.uint8)
    scale = lib().orc_fp8_quantize_activation(_ptr(x_bits), _c_size(x_bits.size), ctypes.c_int(fmt), _ptr(q))
    return q, np.float32(scale)


def fp8_quantize_weight(w: np.ndarray, fmt: int, per_channel: bool, k_major: bool = False):
    w = _c(w, np.float32)
    rows, columns = w.shape
    count = rows if per_channel else 1
    q = np.empty((columns, rows) if k_major else (rows, columns), np.uint8)
    scales = np.empty((count,), np.float32)
    lib().orc_fp8_quantize_weight(_ptr(w), _c_size(rows), _c_size(columns), ctypes.c_int(fmt),
                                  _c_size(count), ctypes.c_int(int(k_major)), _ptr(q), _ptr(scales))
    return q, scales


def fp8_linear(xq: np.ndarray, x_fmt: int, x_scale: float, wq: np.ndarray, w_fmt: int,
               w_scales: np.ndarray, bias_bits: np.ndarray | None = None,
               activation: int = ACT_NONE) -> dict:
    xq = _c(xq, np.uint8)
    wq = _c(wq, np.uint8)
    w_scales = _c(w_scales, np.float32)
    m, k = xq.shape
    n, k2 = wq.shape
    assert k == k2 and w_scales.size in (1, n)
    y = np.empty((m, n), np.uint16)
    acc = np.empty((m, n), np.float32)
    lib().orc_fp8_linear_f16(_ptr(xq), ctypes.c_int(x_fmt), ctypes.c_float(x_scale), _ptr(wq),
                             ctypes.c_int(w_fmt), _ptr(w_scales), _c_size(w_scales.size),
                             _c_size(m), _c_size(n), _c_size(k), _ptr(y), _ptr(acc))
    return {"acc": acc, "y": y, "out": epilogue_f16(y, bias_bits, activation)}


def fp8_native_linear(x_bits: np.ndarray, wq: np.ndarray, w_fmt: int, w_scales: np.ndarray,
                      bias_bits: np.ndarray | None = None, activation: int = ACT_NONE) -> dict:
    """native_fp8_linear (src/cuda/ops_blas.cpp:153-225): activations are quantised to the
    weight's FP8 format with a tensor-wide dynamic scale, then the FP8 x FP8 Linear."""
    x_bits = as_f16_bits(x_bits)
    xq, x_scale = fp8_quantize_activation(x_bits, w_fmt)
    result = fp8_linear(xq, w_fmt, float(x_scale), wq, w_fmt, w_scales, bias_bits, activation)
    result.update({"xq": xq, "x_scale": x_scale})
    return result


def linear_f32(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    m, k = x.shape
    n, k2 = w.shape
    assert k == k2
    out = np.empty((m, n), np.float32)
    b = _c(bias, np.float32) if bias is not None else None
    lib().orc_linear_f32(_ptr(x), _ptr(w), _ptr(b) if b is not None else None,
                         _c_size(m), _c_size(n), _c_size(k), _ptr(out))
    return out


def geglu_f32(y: np.ndarray) -> np.ndarray:
    y = _c(y, np.float32)
    rows, width2 = y.shape
    out = np.empty((rows, width2 // 2), np.float32)
    lib().orc_geglu_f32(_ptr(y), _c_size(rows), _c_size(width2 // 2), _ptr(out))
    return out


def layer_norm_f16(x_bits: np.ndarray, gamma_bits: np.ndarray, beta_bits: np.ndarray,
                   epsilon: float = 1e-5) -> np.ndarray:
    """layer_norm_kernel (src/cuda/ops_kernels.cu:185-221) on FP16 bits [rows, width] -> FP16 bits."""
    x_bits = _c(x_bits, np.uint16)
    rows, width = x_bits.shape
    out = np.empty((rows, width), np.uint16)
    lib().orc_layer_norm_f16(_ptr(x_bits), _ptr(_c(gamma_bits, np.uint16)), _ptr(_c(beta_bits, np.uint16)),
                             _c_size(rows), _c_size(width), ctypes.c_float(epsilon), _ptr(out))
    return out


def threads() -> int:
    return int(lib().orc_threads())


# ---------------------------------------------------------------------------------------
# The reference's own CPU Linear, when oracle/_ref was built (see oracle/Makefile).
# ---------------------------------------------------------------------------------------

_ref = None
_DTYPE_CODE = {np.dtype(np.float16): 0, np.dtype(np.float32): 1}


def ref_available() -> bool:
    return os.path.exists(_REF_SO)


def ref_lib() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_SO)
        _ref.ref_gelu.restype = ctypes.c_float
        _ref.ref_gelu.argtypes = [ctypes.c_float]
        _ref.ref_hardware_threads.restype = ctypes.c_uint
    return _ref


def _weight_code(w: np.ndarray, fp8_fmt: int | None) -> int:
    if fp8_fmt is not None:
        assert w.dtype == np.uint8
        return 2 + fp8_fmt
    return _DTYPE_CODE[w.dtype]


def ref_linear_2d(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None = None,
                  fp8_fmt: int | None = None) -> np.ndarray:
    """Reference linear_2d (src/unet.cpp:202-225). w: float16/float32 array, or uint8 FP8 bytes
    with fp8_fmt given; bias float16/float32."""
    x = _c(x, np.float32)
    w = np.ascontiguousarray(w)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    b = np.ascontiguousarray(bias) if bias is not None else None
    rc = ref_lib().ref_linear_2d(_ptr(x), ctypes.c_uint64(m), ctypes.c_uint64(k), _ptr(w),
                                 ctypes.c_int(_weight_code(w, fp8_fmt)), ctypes.c_uint64(n),
                                 _ptr(b) if b is not None else None,
                                 ctypes.c_int(_DTYPE_CODE[b.dtype] if b is not None else 1), _ptr(out))
    if rc != 0:
        raise RuntimeError("reference linear_2d threw")
    return out


def ref_geglu(y: np.ndarray) -> np.ndarray:
    y = _c(y, np.float32)
    rows, width2 = y.shape
    out = np.empty((rows, width2 // 2), np.float32)
    if ref_lib().ref_geglu(_ptr(y), ctypes.c_uint64(rows), ctypes.c_uint64(width2), _ptr(out)) != 0:
        raise RuntimeError("reference geglu threw")
    return out


def ref_linear_threaded(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None = None,
                        threads: int = 0) -> np.ndarray:
    """Reference threaded AVX2 linear (src/text_encoder.cpp:266-310)."""
    x = _c(x, np.float32)
    w = np.ascontiguousarray(w)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    b = np.ascontiguousarray(bias) if bias is not None else None
    rc = ref_lib().ref_linear_threaded(_ptr(x), ctypes.c_uint64(m), ctypes.c_uint64(k), _ptr(w),
                                       ctypes.c_int(_DTYPE_CODE[w.dtype]), ctypes.c_uint64(n),
                                       _ptr(b) if b is not None else None,
                                       ctypes.c_int(_DTYPE_CODE[b.dtype] if b is not None else 1),
                                       ctypes.c_uint64(threads), _ptr(out))
    if rc != 0:
        raise RuntimeError("reference threaded linear threw")
    return out


def ref_safetensors_probe(path: str, key: str, capacity: int = 64):
    """(dtype value of the reference's DType enum, shape, byte count, leading bytes) of one tensor
    as the reference's own safetensors parser sees it; raises when that parser rejects the file."""
    library = ref_lib()
    dtype, rank = ctypes.c_int(), ctypes.c_int()
    shape = (ctypes.c_uint64 * 4)()
    size = ctypes.c_uint64()
    data = (ctypes.c_ubyte * capacity)()
    status = library.ref_safetensors_probe(path.encode(), key.encode(), ctypes.byref(dtype), ctypes.byref(rank), shape,
                                           ctypes.byref(size), data, ctypes.c_uint64(capacity))
    if status != 0:
        raise RuntimeError(f"the reference safetensors parser rejected {path}:{key} (status {status})")
    count = min(int(size.value), capacity)
    return int(dtype.value), [int(shape[d]) for d in range(rank.value)], int(size.value), bytes(data[:count])


def ref_hardware_threads() -> int:
    return int(ref_lib().ref_hardware_threads())


# ---------------------------------------------------------------------------------------
# The reference's parameter graph, CPU UNet executor and sigma schedule (oracle/_ref).
# ---------------------------------------------------------------------------------------
class RefUNet:
    """sdxl::SDXLModel + sdxl::SDXLUNet of the reference (src/sdxl.cpp:84-238, src/unet.cpp:699-807)
    behind the checker library. `config` = (channels[3], heads[3], transformer_depth[3],
    cross_attention_dim, time_embed_dim, addition_time_embed_dim, addition_input_dim,
    layers_per_block, norm_groups) or None for SDXL Base 1.0."""

    def __init__(self, config=None):
        library = ref_lib()
        library.ref_unet_create.restype = ctypes.c_void_p
        library.ref_unet_create.argtypes = [ctypes.c_void_p]
        library.ref_unet_destroy.argtypes = [ctypes.c_void_p]
        library.ref_unet_parameter_count.restype = ctypes.c_uint64
        library.ref_unet_parameter_count.argtypes = [ctypes.c_void_p]
        library.ref_unet_parameter.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint64,
                                               ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint64)]
        library.ref_unet_bind_f32.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_uint64]
        library.ref_unet_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64,
                                             ctypes.c_uint64, ctypes.c_float, ctypes.c_void_p, ctypes.c_uint64,
                                             ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_char_p, ctypes.c_uint64]
        self._library = library
        packed = None
        if config is not None:
            flat = [int(v) for group in config for v in (group if isinstance(group, (tuple, list)) else (group,))]
            assert len(flat) == 15
            packed = (ctypes.c_uint64 * 15)(*flat)
        self._handle = library.ref_unet_create(packed)
        if not self._handle:
            raise RuntimeError("the reference rejected the UNet configuration")
        self._bound = {}

    def close(self):
        if self._handle:
            self._library.ref_unet_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def parameters(self) -> dict:
        """name (without the `unet.` prefix) -> expected shape, for every UNet parameter of the graph."""
        out = {}
        name = ctypes.create_string_buffer(256)
        rank = ctypes.c_int()
        shape = (ctypes.c_uint64 * 4)()
        for index in range(int(self._library.ref_unet_parameter_count(self._handle))):
            status = self._library.ref_unet_parameter(self._handle, index, name, 256, ctypes.byref(rank), shape)
            if status != 0:
                raise RuntimeError(f"ref_unet_parameter({index}) failed with {status}")
            out[name.value.decode()[len("unet."):]] = tuple(int(shape[d]) for d in range(rank.value))
        return out

    def bind(self, parameters: dict) -> None:
        """Binds FP32 arrays by name (without prefix); the arrays are kept alive by this object."""
        for name, values in parameters.items():
            array = np.ascontiguousarray(values, dtype=np.float32)
            status = self._library.ref_unet_bind_f32(self._handle, f"unet.{name}".encode(), _ptr(array), array.size)
            if status != 0:
                raise RuntimeError(f"binding {name} failed with {status}")
            self._bound[name] = array

    def forward(self, latents, timestep, context, pooled, time_ids) -> np.ndarray:
        latents = _c(latents, np.float32)
        context = _c(context, np.float32)
        pooled = _c(pooled, np.float32)
        time_ids = _c(time_ids, np.float32)
        batch, _, height, width = latents.shape
        out = np.empty_like(latents)
        error = ctypes.create_string_buffer(512)
        status = self._library.ref_unet_forward(self._handle, _ptr(latents), batch, height, width, float(timestep),
                                                _ptr(context), context.shape[1], _ptr(pooled), pooled.shape[1],
                                                _ptr(time_ids), _ptr(out), error, 512)
        if status != 0:
            raise RuntimeError(f"reference SDXLUNet::forward threw: {error.value.decode()}")
        return out


def ref_normal_sigma_schedule(steps: int):
    """(timesteps[steps], sigmas[steps + 1]) of SigmaSchedule(steps, Normal), src/scheduler.cpp:601-668."""
    timesteps = np.empty(steps, np.float32)
    sigmas = np.empty(steps + 1, np.float32)
    status = ref_lib().ref_normal_sigma_schedule(ctypes.c_uint64(steps), _ptr(timesteps), _ptr(sigmas))
    if status != 0:
        raise RuntimeError("the reference sigma schedule threw")
    return timesteps, sigmas


class RefCuda:
    """The reference's own CUDA Ops class compiled for sm_100 (oracle/_ref/libsdxl_ref_cuda*.so; recipe in
    the Makefile, entry points in ref_harness_cuda.cpp). `ieee=True` picks the build without the
    reference's --use_fast_math switch. Needs a GPU; a checker and a comparator, never shipped."""

    WEIGHT_CODE = {"e4m3": 0, "e5m2": 1, "f16": 2}

    def __init__(self, ieee: bool = False):
        name = "libsdxl_ref_cuda_ieee.so" if ieee else "libsdxl_ref_cuda.so"
        path = os.path.join(_HERE, "_ref", name)
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self._lib = ctypes.CDLL(path)
        self._error = ctypes.create_string_buffer(512)

    @staticmethod
    def available(ieee: bool = False) -> bool:
        name = "libsdxl_ref_cuda_ieee.so" if ieee else "libsdxl_ref_cuda.so"
        return os.path.exists(os.path.join(_HERE, "_ref", name))

    def _check(self, status: int, what: str) -> None:
        if status != 0:
            raise RuntimeError(f"reference {what} threw: {self._error.value.decode(errors='replace')}")

    def quantize_fp8(self, x_bits: np.ndarray, fmt: int):
        """quantize_tensor_fp8 (src/cuda/fp8_kernels.cu:157-190) -> (fp8 bytes, dequantisation scale)."""
        x_bits = _c(x_bits, np.uint16)
        rows, columns = x_bits.shape
        q = np.empty((rows, columns), np.uint8)
        scale = np.zeros(1, np.float32)
        self._check(self._lib.refcuda_quantize_fp8(_ptr(x_bits), ctypes.c_uint64(rows), ctypes.c_uint64(columns),
                                                   ctypes.c_int(fmt), _ptr(q), _ptr(scale), self._error,
                                                   ctypes.c_uint64(len(self._error))), "quantize_tensor_fp8")
        return q, float(scale[0])

    def fp8_weight_only_linear(self, x_bits: np.ndarray, wq: np.ndarray, fmt: int, scales: np.ndarray,
                               k_major: bool = False) -> np.ndarray:
        """fp8_weight_only_linear (src/cuda/fp8_kernels.cu:192-245) -> FP16 bits [m, n]. wq is [n, k], or
        [k, n] with k_major."""
        x_bits = _c(x_bits, np.uint16)
        wq = _c(wq, np.uint8)
        scales = _c(scales, np.float32).reshape(-1)
        m, k = x_bits.shape
        n = wq.shape[1] if k_major else wq.shape[0]
        y = np.empty((m, n), np.uint16)
        self._check(self._lib.refcuda_fp8_weight_only_linear(
            _ptr(x_bits), ctypes.c_uint64(m), ctypes.c_uint64(k), _ptr(wq), ctypes.c_uint64(n), ctypes.c_int(fmt),
            _ptr(scales), ctypes.c_uint64(scales.size), ctypes.c_int(1 if k_major else 0), _ptr(y), self._error,
            ctypes.c_uint64(len(self._error))), "fp8_weight_only_linear")
        return y

    def ops_linear(self, x_bits: np.ndarray, w: np.ndarray, kind: str, scales: np.ndarray | None = None,
                   bias_bits: np.ndarray | None = None, activation: int = ACT_NONE,
                   fp32_accumulation: bool = False) -> np.ndarray:
        """Ops::linear / Ops::linear_activation (src/cuda/ops_blas.cpp:244-397) -> FP16 bits. `kind` is
        "f16" (w holds FP16 bits), "e4m3" or "e5m2" (w holds FP8 bytes, `scales` 1 or n values)."""
        x_bits = _c(x_bits, np.uint16)
        m, k = x_bits.shape
        n = w.shape[0]
        w = _c(w.view(np.uint16) if kind == "f16" else w, np.uint16 if kind == "f16" else np.uint8)
        scales = _c(scales if scales is not None else np.ones(1), np.float32).reshape(-1)
        columns = n // 2 if activation == ACT_GEGLU else n
        y = np.empty((m, columns), np.uint16)
        bias = None if bias_bits is None else _c(bias_bits, np.uint16)
        self._check(self._lib.refcuda_ops_linear(
            _ptr(x_bits), ctypes.c_uint64(m), ctypes.c_uint64(k), _ptr(w), ctypes.c_uint64(n),
            ctypes.c_int(self.WEIGHT_CODE[kind]), _ptr(scales), ctypes.c_uint64(scales.size),
            _ptr(bias) if bias is not None else None, ctypes.c_int(activation),
            ctypes.c_int(1 if fp32_accumulation else 0), _ptr(y), ctypes.c_uint64(columns), self._error,
            ctypes.c_uint64(len(self._error))), "Ops::linear")
        return y

    def time_linear(self, m: int, k: int, n: int, kind: str, activation: int = ACT_NONE, has_bias: bool = True,
                    fp32_accumulation: bool = False, warmup: int = 3, iterations: int = 10) -> float:
        """Milliseconds per Ops::linear_activation call with device-resident operands, timed with CUDA
        events on the reference's stream."""
        ms = ctypes.c_float(0.0)
        self._check(self._lib.refcuda_time_linear(
            ctypes.c_uint64(m), ctypes.c_uint64(k), ctypes.c_uint64(n), ctypes.c_int(self.WEIGHT_CODE[kind]),
            ctypes.c_int(activation), ctypes.c_int(1 if has_bias else 0), ctypes.c_int(1 if fp32_accumulation else 0),
            ctypes.c_int(warmup), ctypes.c_int(iterations), ctypes.byref(ms), self._error,
            ctypes.c_uint64(len(self._error))), "Ops::linear timing")
        return float(ms.value)

    def layer_norm(self, x_bits: np.ndarray, gamma_bits: np.ndarray, beta_bits: np.ndarray,
                   epsilon: float = 1e-5) -> np.ndarray:
        """Ops::layer_norm (src/cuda/ops_kernels.cu:1425-1470) -> FP16 bits."""
        x_bits = _c(x_bits, np.uint16)
        rows, width = x_bits.shape
        y = np.empty((rows, width), np.uint16)
        self._check(self._lib.refcuda_layer_norm(
            _ptr(x_bits), ctypes.c_uint64(rows), ctypes.c_uint64(width), _ptr(_c(gamma_bits, np.uint16)),
            _ptr(_c(beta_bits, np.uint16)), ctypes.c_float(epsilon), _ptr(y), self._error,
            ctypes.c_uint64(len(self._error))), "Ops::layer_norm")
        return y

    def shutdown(self) -> None:
        self._lib.refcuda_shutdown()
