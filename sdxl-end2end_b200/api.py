"""ctypes binding of include/sdxlq.h plus the host-side mirror of the reference interface."""
from __future__ import annotations

import ctypes
import enum
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import build as _build

# --------------------------------------------------------------------------------------------
# Enumerations: numeric values of the reference enums (tensor.hpp:17-48, ops.hpp:15).
# --------------------------------------------------------------------------------------------


class ScalarType(enum.IntEnum):
    Float8E4M3 = 0
    Float8E5M2 = 1
    Int8 = 2
    Float16 = 3
    Float32 = 4
    Int32 = 5


class FP8ScaleMode(enum.IntEnum):
    None_ = 0
    TensorWide = 1
    PerOutputChannel = 2


class FP8StorageLayout(enum.IntEnum):
    RowMajorNK = 0
    KMajorKN = 1


class LinearActivation(enum.IntEnum):
    None_ = 0
    SiLU = 1
    GELU = 2
    QuickGELU = 3
    GEGLU = 4


ACT_NONE, ACT_SILU, ACT_GELU, ACT_QUICK_GELU, ACT_GEGLU = 0, 1, 2, 3, 4

STATUS_OK, STATUS_INVALID, STATUS_UNSUPPORTED, STATUS_TIMEOUT, STATUS_CUDA, STATUS_WORKSPACE = range(6)


class CudaError(RuntimeError):
    """The reference's sdxl::cuda::CudaError (include/sdxl/cuda/runtime.hpp:18-21)."""

    def __init__(self, message: str, status: int = STATUS_INVALID):
        super().__init__(message)
        self.status = status


# --------------------------------------------------------------------------------------------
# C structures
# --------------------------------------------------------------------------------------------


class _CWeight(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("layout", ctypes.c_int32),
        ("n", ctypes.c_uint64),
        ("k", ctypes.c_uint64),
        ("scales", ctypes.c_void_p),
        ("scale_count", ctypes.c_uint64),
        ("scale_mode", ctypes.c_int32),
        ("convrot_group_size", ctypes.c_uint32),
    ]


class _CLinearDesc(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p),
        ("m", ctypes.c_uint64),
        ("weight", _CWeight),
        ("bias", ctypes.c_void_p),
        ("activation", ctypes.c_int32),
        ("reserved0", ctypes.c_int32),
        ("y", ctypes.c_void_p),
        ("xq", ctypes.c_void_p),
        ("xq_scales", ctypes.c_void_p),
        ("acc_out", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("y_amax", ctypes.c_void_p),
        ("x_amax", ctypes.c_void_p),
    ]


class _CStats(ctypes.Structure):
    _fields_ = [
        ("linear_calls", ctypes.c_uint64),
        ("tensor_core_calls", ctypes.c_uint64),
        ("dp4a_fallback_calls", ctypes.c_uint64),
        ("tensor_core_plan_misses", ctypes.c_uint64),
        ("tensor_core_execution_failures", ctypes.c_uint64),
    ]


class _CLayerNormDesc(ctypes.Structure):
    """sdxlq_layer_norm_desc."""
    _fields_ = [
        ("x", ctypes.c_void_p), ("rows", ctypes.c_uint64), ("width", ctypes.c_uint64),
        ("gamma", ctypes.c_void_p), ("beta", ctypes.c_void_p), ("epsilon", ctypes.c_float),
        ("out_dtype", ctypes.c_int32), ("convrot_group_size", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("y", ctypes.c_void_p), ("xq", ctypes.c_void_p), ("xq_scales", ctypes.c_void_p),
    ]


class _CGroupNormDesc(ctypes.Structure):
    """sdxlq_group_norm_desc."""
    _fields_ = [
        ("x", ctypes.c_void_p), ("channel_bias", ctypes.c_void_p), ("gamma", ctypes.c_void_p), ("beta", ctypes.c_void_p),
        ("y", ctypes.c_void_p), ("batch", ctypes.c_uint64), ("rows", ctypes.c_uint64), ("channels", ctypes.c_uint64),
        ("groups", ctypes.c_uint32), ("silu", ctypes.c_int32), ("epsilon", ctypes.c_float), ("reserved", ctypes.c_uint32),
    ]


class _CKernelTimes(ctypes.Structure):
    _fields_ = [("milliseconds", ctypes.c_double * 6), ("launches", ctypes.c_uint64 * 6)]


KERNEL_CLASSES = ("quant_int8", "quant_fp8", "gemm", "small", "layer_norm", "harness")

EXPORTED_SYMBOLS = [
    "sdxlq_context_create", "sdxlq_context_destroy", "sdxlq_context_set_stream", "sdxlq_context_check",
    "sdxlq_last_error", "sdxlq_status_string", "sdxlq_get_stats", "sdxlq_linear", "sdxlq_linear_grouped",
    "sdxlq_group_plan_create", "sdxlq_group_plan_run", "sdxlq_group_plan_destroy",
    "sdxlq_group_plan_launches", "sdxlq_quantize_act_int8", "sdxlq_quantize_act_fp8",
    "sdxlq_pack_weight_int8", "sdxlq_pack_weight_fp8", "sdxlq_valid_convrot_group_size",
    "sdxlq_workspace_bytes", "sdxlq_build_info", "sdxlq_context_set_tile_n",
    "sdxlq_selftest_bounded_wait", "sdxlq_profile_enable", "sdxlq_profile_read", "sdxlq_linear_static",
    "sdxlq_context_set_pair_mode", "sdxlq_layer_norm", "sdxlq_group_norm_nhwc", "sdxlq_harness_bias_residual_add",
]

_lib: Optional[ctypes.CDLL] = None


def library_path() -> str:
    return _build.LIBRARY


def load_library() -> ctypes.CDLL:
    """Loads libsdxlq.so; fails loudly when it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("SDXLQ_LIBRARY") or library_path()
    if not os.path.exists(path):
        raise CudaError(f"{path} is missing: build it first (build() of this package, or "
                        "__graft_entry__.build()); there is no CPU fallback", STATUS_CUDA)
    lib = ctypes.CDLL(path)
    vp, i32, u32, u64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t
    lib.sdxlq_context_create.argtypes = [ctypes.c_int, vp, sz, ctypes.POINTER(vp)]
    lib.sdxlq_context_destroy.argtypes = [vp]
    lib.sdxlq_context_destroy.restype = None
    lib.sdxlq_context_set_stream.argtypes = [vp, vp]
    lib.sdxlq_context_check.argtypes = [vp]
    lib.sdxlq_last_error.argtypes = [vp]
    lib.sdxlq_last_error.restype = ctypes.c_char_p
    lib.sdxlq_status_string.argtypes = [ctypes.c_int]
    lib.sdxlq_status_string.restype = ctypes.c_char_p
    lib.sdxlq_get_stats.argtypes = [vp, ctypes.POINTER(_CStats)]
    lib.sdxlq_linear.argtypes = [vp, ctypes.POINTER(_CLinearDesc)]
    lib.sdxlq_linear_grouped.argtypes = [vp, ctypes.POINTER(_CLinearDesc), sz]
    lib.sdxlq_group_plan_create.argtypes = [vp, ctypes.POINTER(_CLinearDesc), sz, ctypes.POINTER(vp)]
    lib.sdxlq_group_plan_run.argtypes = [vp, vp]
    lib.sdxlq_group_plan_destroy.argtypes = [vp]
    lib.sdxlq_group_plan_destroy.restype = None
    lib.sdxlq_group_plan_launches.argtypes = [vp]
    lib.sdxlq_quantize_act_int8.argtypes = [vp, vp, i32, u64, u64, u32, vp, vp]
    lib.sdxlq_quantize_act_fp8.argtypes = [vp, vp, u64, i32, vp, vp]
    lib.sdxlq_pack_weight_int8.argtypes = [vp, vp, i32, u64, u64, u32, vp, vp]
    lib.sdxlq_pack_weight_fp8.argtypes = [vp, vp, i32, u64, u64, i32, i32, i32, vp, vp]
    lib.sdxlq_valid_convrot_group_size.argtypes = [sz]
    lib.sdxlq_workspace_bytes.argtypes = [ctypes.POINTER(_CLinearDesc), sz]
    lib.sdxlq_workspace_bytes.restype = sz
    lib.sdxlq_build_info.restype = ctypes.c_char_p
    lib.sdxlq_context_set_tile_n.argtypes = [vp, ctypes.c_int]
    lib.sdxlq_selftest_bounded_wait.argtypes = [vp, ctypes.c_longlong]
    lib.sdxlq_context_set_pair_mode.argtypes = [vp, ctypes.c_int]
    lib.sdxlq_profile_enable.argtypes = [vp, ctypes.c_int]
    lib.sdxlq_profile_read.argtypes = [vp, ctypes.POINTER(_CKernelTimes)]
    lib.sdxlq_linear_static.argtypes = [ctypes.c_int, vp, ctypes.POINTER(_CLinearDesc), ctypes.c_char_p, sz]
    lib.sdxlq_layer_norm.argtypes = [vp, ctypes.POINTER(_CLayerNormDesc)]
    lib.sdxlq_group_norm_nhwc.argtypes = [vp, ctypes.POINTER(_CGroupNormDesc)]
    lib.sdxlq_harness_bias_residual_add.argtypes = [vp, vp, vp, vp, vp, u64, u64]
    _lib = lib
    return lib


def valid_convrot_group_size(group_size: int) -> bool:
    """valid_convrot_group_size (src/cuda/int8_convrot.cu:489-496): power of four in 4..256."""
    if group_size < 4 or group_size > 256:
        return False
    while group_size > 1:
        if group_size % 4:
            return False
        group_size //= 4
    return True


# --------------------------------------------------------------------------------------------
# Host-side mirror of the reference types
# --------------------------------------------------------------------------------------------

_TORCH_FP8 = {ScalarType.Float8E4M3: torch.float8_e4m3fn, ScalarType.Float8E5M2: torch.float8_e5m2}


@dataclass
class Weight:
    """A packed projection weight: what the reference keeps on a weight ``cuda::Tensor``
    (data, ScalarType, [N,K], dequant scale pointer/count/mode, FP8 layout, ConvRot group)."""

    data: torch.Tensor                     # int8 / uint8 (FP8 bytes) / float16, logical [N, K]
    type: ScalarType
    n: int
    k: int
    scales: Optional[torch.Tensor] = None  # float32 [N] or [1]
    scale_mode: FP8ScaleMode = FP8ScaleMode.None_
    layout: FP8StorageLayout = FP8StorageLayout.RowMajorNK
    convrot_group_size: int = 0

    def has_dequant_scale(self) -> bool:
        return self.scales is not None

    def dequant_scale_count(self) -> int:
        return 0 if self.scales is None else int(self.scales.numel())

    def uses_convrot(self) -> bool:
        return self.convrot_group_size != 0

    def c_struct(self) -> _CWeight:
        return _CWeight(
            self.data.data_ptr(), int(self.type), int(self.layout), self.n, self.k,
            self.scales.data_ptr() if self.scales is not None else None,
            self.dequant_scale_count(), int(self.scale_mode), self.convrot_group_size)


@dataclass
class QuantizationMetadata:
    """sdxl::QuantizationMetadata (include/sdxl/model.hpp:17-23) for a prequantised weight."""

    weight_scale: Optional[torch.Tensor] = None
    input_scale: Optional[torch.Tensor] = None
    convrot: bool = False
    per_row: bool = False
    convrot_group_size: int = 0


@dataclass
class INT8WeightLoadOptions:
    """sdxl::cuda::INT8WeightLoadOptions (include/sdxl/cuda/weights.hpp:54-66)."""

    quantize_floating_weights: bool = True
    require_prequantized: bool = False
    strict: bool = False
    require_tensor_cores: bool = False
    enable_convrot: bool = True
    convrot_group_size: int = 256


@dataclass
class FP8WeightLoadOptions:
    """The fields of sdxl::cuda::FP8WeightLoadOptions (weights.hpp:45-51) that select kernels."""

    format: ScalarType = ScalarType.Float8E4M3
    scale_mode: FP8ScaleMode = FP8ScaleMode.TensorWide
    preserve_native_fp8: bool = True
    layout: FP8StorageLayout = FP8StorageLayout.RowMajorNK


@dataclass
class LinearCall:
    """One projection of a grouped launch."""

    x: Optional[torch.Tensor]
    weight: Weight
    bias: Optional[torch.Tensor] = None
    activation: int = ACT_NONE
    y: Optional[torch.Tensor] = None
    xq: Optional[torch.Tensor] = None
    xq_scales: Optional[torch.Tensor] = None
    acc_out: Optional[torch.Tensor] = None
    residual: Optional[torch.Tensor] = None
    y_amax: Optional[torch.Tensor] = None      # one int32 device word: receives max |y| (FP32 bits)
    x_amax: Optional[torch.Tensor] = None      # the word a producer filled for x (FP8 weights)
    keep: list = field(default_factory=list)


class Context:
    """Owns an ``sdxlq_context``: device, stream and scratch workspace (the part of the
    reference ``Runtime`` the operator needs, include/sdxl/cuda/runtime.hpp:120-163)."""

    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None,
                 workspace_bytes: int = 0):
        self._lib = load_library()
        self._handle = ctypes.c_void_p()
        self.device = device
        self.stream = stream
        stream_ptr = ctypes.c_void_p(stream.cuda_stream) if stream is not None else \
            ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        status = self._lib.sdxlq_context_create(device, stream_ptr, workspace_bytes, ctypes.byref(self._handle))
        if status != STATUS_OK:
            raise CudaError(f"sdxlq_context_create failed: {self._lib.sdxlq_status_string(status).decode()}", status)

    def close(self) -> None:
        if getattr(self, "_handle", None) and self._handle.value:
            self._lib.sdxlq_context_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self) -> ctypes.c_void_p:
        return self._handle

    def raise_for(self, status: int) -> None:
        if status != STATUS_OK:
            raise CudaError(self._lib.sdxlq_last_error(self._handle).decode(), status)

    def set_stream(self, stream: torch.cuda.Stream) -> None:
        self.stream = stream
        self.raise_for(self._lib.sdxlq_context_set_stream(self._handle, ctypes.c_void_p(stream.cuda_stream)))

    def check(self) -> None:
        """Synchronises and raises CudaError on a device-side timeout or CUDA error."""
        self.raise_for(self._lib.sdxlq_context_check(self._handle))

    def set_tile_n(self, tile_n: int) -> None:
        self.raise_for(self._lib.sdxlq_context_set_tile_n(self._handle, tile_n))

    def set_pair_mode(self, mode: int) -> None:
        """-1 automatic, 0 never use CTA pairs, 1 for every projection with more than 128 rows."""
        self.raise_for(self._lib.sdxlq_context_set_pair_mode(self._handle, mode))

    def int8_execution_stats(self) -> dict:
        stats = _CStats()
        self.raise_for(self._lib.sdxlq_get_stats(self._handle, ctypes.byref(stats)))
        return {name: int(getattr(stats, name)) for name, _ in _CStats._fields_}

    def profile(self, enabled: bool) -> None:
        """Turns per-kernel CUDA-event timing on or off."""
        self.raise_for(self._lib.sdxlq_profile_enable(self._handle, int(enabled)))

    def kernel_times(self) -> dict:
        """{class: (milliseconds, launches)} since the last read; synchronises the stream."""
        times = _CKernelTimes()
        self.raise_for(self._lib.sdxlq_profile_read(self._handle, ctypes.byref(times)))
        return {name: (float(times.milliseconds[i]), int(times.launches[i])) for i, name in enumerate(KERNEL_CLASSES)}

    def selftest_bounded_wait(self, limit_cycles: int) -> None:
        self.raise_for(self._lib.sdxlq_selftest_bounded_wait(self._handle, limit_cycles))


def _ptr(tensor: Optional[torch.Tensor]):
    return None if tensor is None else tensor.data_ptr()


class Ops:
    """The projection operators of sdxl::cuda::Ops (include/sdxl/cuda/ops.hpp:17-30)."""

    def __init__(self, context: Context, poison_outputs: bool = False):
        self.ctx = context
        self._lib = context._lib
        # Tests set this: outputs this class allocates start as NaN, so that an element a kernel
        # failed to write cannot pass for a result left in recycled memory.
        self.poison_outputs = poison_outputs

    # -- descriptor ---------------------------------------------------------------------------
    def _desc(self, call: LinearCall) -> _CLinearDesc:
        weight = call.weight
        x = call.x
        if x is not None:
            if x.dtype != torch.float16 or x.dim() < 2:
                kind = "INT8" if weight.type == ScalarType.Int8 else "FP8 UNet" if weight.type in _TORCH_FP8 else "CUDA"
                raise CudaError(f"{kind} linear requires FP16 model activations and a rank-2 weight")
            if not x.is_contiguous():
                raise CudaError("CUDA linear expects contiguous activations")
            if x.shape[-1] != weight.k:
                raise CudaError("CUDA linear feature mismatch")
            m = x.numel() // weight.k
            lead = tuple(x.shape[:-1])
        else:
            if call.xq is None:
                raise CudaError("linear: no input")
            m = call.xq.numel() // weight.k
            lead = tuple(call.xq.shape[:-1])
        if call.bias is not None:
            if call.bias.dtype != torch.float16 or call.bias.dim() != 1 or call.bias.shape[0] != weight.n:
                raise CudaError("CUDA linear bias mismatch")
        n_out = weight.n // 2 if call.activation == ACT_GEGLU else weight.n
        if call.y is None:
            device = (x if x is not None else call.xq).device
            call.y = torch.empty(lead + (n_out,), dtype=torch.float16, device=device)
            if self.poison_outputs:
                call.y.fill_(float("nan"))
        if call.residual is not None:
            if call.residual.dtype != torch.float16 or not call.residual.is_contiguous() or \
                    call.residual.numel() != m * n_out:
                raise CudaError("CUDA add requires matching FP16 tensors")
        return _CLinearDesc(_ptr(x), m, weight.c_struct(), _ptr(call.bias), int(call.activation), 0,
                            _ptr(call.y), _ptr(call.xq), _ptr(call.xq_scales), _ptr(call.acc_out),
                            _ptr(call.residual), _ptr(call.y_amax), _ptr(call.x_amax))

    # -- Ops::linear / Ops::linear_activation ----------------------------------------------------
    def linear(self, input: torch.Tensor, weight: Weight, bias: Optional[torch.Tensor] = None, *,
               xq: Optional[torch.Tensor] = None, xq_scales: Optional[torch.Tensor] = None,
               acc_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               residual: Optional[torch.Tensor] = None, y_amax: Optional[torch.Tensor] = None,
               x_amax: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`residual` folds the Ops::add_in_place that follows the projection in the reference's
        transformer block (src/cuda/unet.cpp:118, 132, 147) into the epilogue; pass out=residual to
        update the hidden state in place."""
        call = LinearCall(input, weight, bias, ACT_NONE, out, xq, xq_scales, acc_out, residual, y_amax, x_amax)
        desc = self._desc(call)
        self.ctx.raise_for(self._lib.sdxlq_linear(self.ctx.handle, ctypes.byref(desc)))
        return call.y

    def linear_activation(self, input: torch.Tensor, weight: Weight, bias: torch.Tensor,
                          activation: int, *, xq: Optional[torch.Tensor] = None,
                          xq_scales: Optional[torch.Tensor] = None,
                          acc_out: Optional[torch.Tensor] = None,
                          out: Optional[torch.Tensor] = None, y_amax: Optional[torch.Tensor] = None,
                          x_amax: Optional[torch.Tensor] = None) -> torch.Tensor:
        call = LinearCall(input, weight, bias, int(activation), out, xq, xq_scales, acc_out, None, y_amax, x_amax)
        desc = self._desc(call)
        self.ctx.raise_for(self._lib.sdxlq_linear(self.ctx.handle, ctypes.byref(desc)))
        return call.y

    # -- grouped launches --------------------------------------------------------------------------
    def _desc_array(self, calls: Sequence[LinearCall]):
        array = (_CLinearDesc * len(calls))()
        for i, call in enumerate(calls):
            array[i] = self._desc(call)
        return array

    def linear_grouped(self, calls: Sequence[LinearCall]) -> list:
        array = self._desc_array(calls)
        self.ctx.raise_for(self._lib.sdxlq_linear_grouped(self.ctx.handle, array, len(calls)))
        return [call.y for call in calls]

    def plan(self, calls: Sequence[LinearCall]) -> "GroupPlan":
        return GroupPlan(self, calls)

    def workspace_bytes(self, calls: Sequence[LinearCall]) -> int:
        array = self._desc_array(calls)
        return int(self._lib.sdxlq_workspace_bytes(array, len(calls)))

    # -- Ops::layer_norm, alone or fused with the next projection's quantiser -------------------------
    def _layer_norm_check(self, input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> tuple:
        if input.dtype != torch.float16 or weight.dtype != torch.float16 or bias.dtype != torch.float16 or \
                input.dim() < 1 or weight.dim() != 1 or bias.dim() != 1:
            raise CudaError("CUDA layer_norm expects an FP16 input with rank-1 FP16 weight and bias")
        width = int(input.shape[-1])
        if weight.shape[0] != width or bias.shape[0] != width:
            raise CudaError("CUDA layer_norm width mismatch")
        if width == 0:
            raise CudaError("layer_norm requires a non-empty last dimension")
        if not input.is_contiguous():
            raise CudaError("CUDA layer_norm expects a contiguous input")
        return input.numel() // width, width

    def layer_norm(self, input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                   epsilon: float = 1.0e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Ops::layer_norm (include/sdxl/cuda/ops.hpp:39-42): FP16 in, FP16 out."""
        rows, width = self._layer_norm_check(input, weight, bias)
        y = out if out is not None else torch.empty_like(input)
        desc = _CLayerNormDesc(input.data_ptr(), rows, width, weight.data_ptr(), bias.data_ptr(), epsilon,
                               int(ScalarType.Float16), 0, 0, y.data_ptr(), None, None)
        self.ctx.raise_for(self._lib.sdxlq_layer_norm(self.ctx.handle, ctypes.byref(desc)))
        return y

    def layer_norm_quantized(self, input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                             consumer: Weight, epsilon: float = 1.0e-5):
        """LayerNorm fused with the activation quantiser of the projection(s) that read the result:
        returns (xq, xq_scales) in the form `consumer` (an INT8 or FP8 projection weight) wants, to be
        passed as linear(None, consumer, ..., xq=xq, xq_scales=xq_scales). Equal to quantising
        layer_norm(input) with quantize_int8 / quantize_fp8, without the FP16 tensor in between."""
        rows, width = self._layer_norm_check(input, weight, bias)
        if consumer.k != width:
            raise CudaError("CUDA linear feature mismatch")
        if consumer.type == ScalarType.Int8:
            xq = torch.empty(input.shape, dtype=torch.int8, device=input.device)
            scales = torch.empty(rows, dtype=torch.float32, device=input.device)
            group = consumer.convrot_group_size
        elif consumer.type in _TORCH_FP8:
            xq = torch.empty(input.shape, dtype=torch.uint8, device=input.device)
            scales = torch.empty(1, dtype=torch.float32, device=input.device)
            group = 0
        else:
            raise CudaError("layer_norm_quantized wants an INT8 or FP8 projection weight")
        desc = _CLayerNormDesc(input.data_ptr(), rows, width, weight.data_ptr(), bias.data_ptr(), epsilon,
                               int(consumer.type), group, 0, None, xq.data_ptr(), scales.data_ptr())
        self.ctx.raise_for(self._lib.sdxlq_layer_norm(self.ctx.handle, ctypes.byref(desc)))
        return xq, scales

    # -- harness scaffolding: GroupNorm (+ SiLU) on channels-last activations -------------------------------
    def group_norm_nhwc(self, input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, groups: int,
                        epsilon: float = 1.0e-5, silu: bool = False,
                        channel_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Ops::group_norm_nchw / group_norm_silu_nchw (include/sdxl/cuda/ops.hpp:43-52) for a logical
        [B, C, H, W] FP16 tensor held channels-last (NHWC memory); the result has the same shape and
        memory format. `channel_bias` [B, C] is added first with FP16 rounding (add_spatial_bias)."""
        if input.dtype != torch.float16 or input.dim() != 4 or weight.dtype != torch.float16 or bias.dtype != torch.float16:
            raise CudaError("CUDA group_norm expects an FP16 NCHW tensor")
        batch, channels, height, width = (int(v) for v in input.shape)
        if weight.dim() != 1 or bias.dim() != 1 or weight.shape[0] != channels or bias.shape[0] != channels:
            raise CudaError("CUDA group_norm weight / bias mismatch")
        if groups <= 0 or channels % groups != 0:
            raise CudaError("CUDA group_norm channels must be divisible by groups")
        if not input.is_contiguous(memory_format=torch.channels_last):
            raise CudaError("group_norm_nhwc expects a channels-last tensor")
        if channel_bias is not None and (channel_bias.dtype != torch.float16 or tuple(channel_bias.shape) != (batch, channels)
                                         or not channel_bias.is_contiguous()):
            raise CudaError("CUDA spatial bias must have shape [batch, channels]")
        out = torch.empty_like(input, memory_format=torch.channels_last)
        desc = _CGroupNormDesc(input.data_ptr(), _ptr(channel_bias), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
                               batch, height * width, channels, groups, int(silu), epsilon, 0)
        self.ctx.raise_for(self._lib.sdxlq_group_norm_nhwc(self.ctx.handle, ctypes.byref(desc)))
        return out

    def bias_residual_add_nhwc(self, input: torch.Tensor, bias: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """half(half(input + bias[c]) + residual) for channels-last [B, C, H, W] FP16 tensors: a convolution's
        bias add and Ops::add with the resnet's residual (src/cuda/unet.cpp:92) in one pass."""
        if input.dtype != torch.float16 or residual.dtype != torch.float16 or bias.dtype != torch.float16 or \
                input.shape != residual.shape or input.dim() != 4 or bias.shape != (input.shape[1],):
            raise CudaError("CUDA add requires matching FP16 tensors")
        if not (input.is_contiguous(memory_format=torch.channels_last) and residual.is_contiguous(memory_format=torch.channels_last)):
            raise CudaError("bias_residual_add_nhwc expects channels-last tensors")
        batch, channels, height, width = (int(v) for v in input.shape)
        out = torch.empty_like(input, memory_format=torch.channels_last)
        self.ctx.raise_for(self._lib.sdxlq_harness_bias_residual_add(
            self.ctx.handle, input.data_ptr(), bias.data_ptr(), residual.data_ptr(), out.data_ptr(),
            batch * height * width, channels))
        return out

    # -- Ops::quantize_fp8 / quantize_e4m3 / quantize_e5m2 ------------------------------------------
    def quantize_fp8(self, input: torch.Tensor, fp8_type: ScalarType) -> Weight:
        """quantize_tensor_fp8 (src/cuda/fp8_kernels.cu:157-190). Returns the FP8 tensor with its
        tensor-wide dequantisation scale attached, like the reference (a rank-2 result can be
        used as a weight, as the reference's operator test does)."""
        if input.dtype != torch.float16 or fp8_type not in _TORCH_FP8:
            raise CudaError("FP8 activation quantization requires float16 input and an FP8 destination")
        source = input.contiguous()
        q = torch.empty(source.shape, dtype=torch.uint8, device=source.device)
        scale = torch.empty(1, dtype=torch.float32, device=source.device)
        self.ctx.raise_for(self._lib.sdxlq_quantize_act_fp8(
            self.ctx.handle, source.data_ptr(), source.numel(), int(fp8_type), q.data_ptr(), scale.data_ptr()))
        n = source.shape[0] if source.dim() == 2 else source.numel() // source.shape[-1]
        return Weight(q, ScalarType(fp8_type), n, source.shape[-1], scale, FP8ScaleMode.TensorWide)

    def quantize_e4m3(self, input: torch.Tensor) -> Weight:
        return self.quantize_fp8(input, ScalarType.Float8E4M3)

    def quantize_e5m2(self, input: torch.Tensor) -> Weight:
        return self.quantize_fp8(input, ScalarType.Float8E5M2)

    # -- activation quantiser of int8_convrot_linear -----------------------------------------------
    def quantize_int8(self, input: torch.Tensor, convrot_group_size: int):
        """The H1+H2 step of int8_convrot_linear (src/cuda/int8_convrot.cu:602-628) on its own:
        returns (xq int8 [M,K], scales float32 [M])."""
        if input.dtype not in (torch.float16, torch.float32) or input.dim() < 2:
            raise CudaError("native INT8 linear received incompatible tensors")
        source = input.contiguous()
        k = source.shape[-1]
        m = source.numel() // k
        xq = torch.empty(source.shape, dtype=torch.int8, device=source.device)
        scales = torch.empty(m, dtype=torch.float32, device=source.device)
        dtype = ScalarType.Float16 if source.dtype == torch.float16 else ScalarType.Float32
        self.ctx.raise_for(self._lib.sdxlq_quantize_act_int8(
            self.ctx.handle, source.data_ptr(), int(dtype), m, k, convrot_group_size, xq.data_ptr(),
            scales.data_ptr()))
        return xq, scales

    # -- load-time packers ------------------------------------------------------------------------
    def upload_or_quantize_int8_weight(self, source: torch.Tensor,
                                       metadata: Optional[QuantizationMetadata],
                                       options: INT8WeightLoadOptions) -> Weight:
        """upload_or_quantize_int8_weight (src/cuda/int8_convrot.cu:498-577) for a weight that is
        already on the device: same option/metadata rules, same error messages."""
        if source.dim() != 2:
            raise CudaError("native INT8 weight must be rank 2")
        rows, columns = int(source.shape[0]), int(source.shape[1])
        if rows == 0 or columns == 0:
            raise CudaError("native INT8 weight cannot be empty")
        prequantized = source.dtype == torch.int8
        if options.require_prequantized and not prequantized:
            raise CudaError("INT8 prequantized-only profile received a floating-point linear weight")
        if not prequantized and not options.quantize_floating_weights:
            raise CudaError("on-the-fly INT8 quantization is disabled")
        use_convrot = options.enable_convrot and options.convrot_group_size > 0 and \
            columns % options.convrot_group_size == 0
        group = options.convrot_group_size if use_convrot else 0
        if prequantized:
            if metadata is None or metadata.weight_scale is None:
                raise CudaError("prequantized INT8 weight is missing weight_scale")
            use_convrot = metadata.convrot
            group = metadata.convrot_group_size if use_convrot else 0
            if use_convrot and (not valid_convrot_group_size(group) or columns % group != 0):
                raise CudaError("prequantized ConvRot metadata is incompatible with weight shape")
            if metadata.weight_scale.numel() != rows:
                raise CudaError("prequantized INT8 weight_scale is not per-output-row")
        elif use_convrot and not valid_convrot_group_size(group):
            raise CudaError("INT8 ConvRot group size must be a power of four between 4 and 256")
        if not prequantized and source.dtype not in (torch.float16, torch.float32):
            source = source.to(torch.float32)
        source = source.contiguous()
        weight = torch.empty((rows, columns), dtype=torch.int8, device=source.device)
        if prequantized:
            scales = metadata.weight_scale.to(device=source.device, dtype=torch.float32).reshape(rows).contiguous()
            dtype = ScalarType.Int8
        else:
            scales = torch.empty(rows, dtype=torch.float32, device=source.device)
            dtype = ScalarType.Float16 if source.dtype == torch.float16 else ScalarType.Float32
        self.ctx.raise_for(self._lib.sdxlq_pack_weight_int8(
            self.ctx.handle, source.data_ptr(), int(dtype), rows, columns, group, weight.data_ptr(),
            scales.data_ptr()))
        return Weight(weight, ScalarType.Int8, rows, columns, scales, FP8ScaleMode.PerOutputChannel,
                      FP8StorageLayout.RowMajorNK, group if use_convrot else 0)

    def upload_fp8_weight(self, source: torch.Tensor, options: FP8WeightLoadOptions) -> Weight:
        """The FP8 branch of WeightStore::upload_tensor (src/cuda/weights.cu:301-415)."""
        if options.format not in _TORCH_FP8:
            raise CudaError("CUDA weight upload target must be FP8, float16, or float32")
        if options.scale_mode == FP8ScaleMode.PerOutputChannel and source.dim() != 2:
            raise CudaError("per-output-channel FP8 scaling requires a rank-2 matrix")
        if source.dim() != 2:
            raise CudaError("FP8 linear weights are rank 2")
        rows, columns = int(source.shape[0]), int(source.shape[1])
        if source.dtype == _TORCH_FP8[options.format] and options.preserve_native_fp8:
            src_dtype = options.format
            source = source.contiguous().view(torch.uint8)
        elif source.dtype == torch.float16:
            src_dtype = ScalarType.Float16
        else:
            source = source.to(torch.float32)
            src_dtype = ScalarType.Float32
        source = source.contiguous()
        count = rows if options.scale_mode == FP8ScaleMode.PerOutputChannel else 1
        shape = (columns, rows) if options.layout == FP8StorageLayout.KMajorKN else (rows, columns)
        packed = torch.empty(shape, dtype=torch.uint8, device=source.device)
        scales = torch.empty(count, dtype=torch.float32, device=source.device)
        self.ctx.raise_for(self._lib.sdxlq_pack_weight_fp8(
            self.ctx.handle, source.data_ptr(), int(src_dtype), rows, columns, int(options.format),
            int(options.scale_mode), int(options.layout), packed.data_ptr(), scales.data_ptr()))
        return Weight(packed, ScalarType(options.format), rows, columns, scales, options.scale_mode, options.layout)

    @staticmethod
    def fp16_weight(source: torch.Tensor) -> Weight:
        source = source.to(torch.float16).contiguous()
        return Weight(source, ScalarType.Float16, int(source.shape[0]), int(source.shape[1]))


class GroupPlan:
    """Build-once / run-many grouped launch (sdxlq_group_plan_*)."""

    def __init__(self, ops: Ops, calls: Sequence[LinearCall]):
        self.ops = ops
        self.calls = list(calls)       # keeps every tensor alive for the plan's lifetime
        self._lib = ops._lib
        self._handle = ctypes.c_void_p()
        array = ops._desc_array(self.calls)
        ops.ctx.raise_for(self._lib.sdxlq_group_plan_create(ops.ctx.handle, array, len(self.calls),
                                                            ctypes.byref(self._handle)))

    @property
    def launches(self) -> int:
        return int(self._lib.sdxlq_group_plan_launches(self._handle))

    def run(self) -> list:
        self.ops.ctx.raise_for(self._lib.sdxlq_group_plan_run(self.ops.ctx.handle, self._handle))
        return [call.y for call in self.calls]

    def close(self) -> None:
        if self._handle.value:
            self._lib.sdxlq_group_plan_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CrossAttentionKVCache:
    """Every cross-attention to_k / to_v projection of the UNet computed once per generation.

    `attn2.to_k` and `attn2.to_v` of every transformer block project the text encoder's hidden
    states (UNet::transformer_block, src/cuda/unet.cpp:120-127), which do not change between
    denoising steps; the reference recomputes all 140 of them in each of its steps. This cache runs
    them as ONE grouped launch (one quantisation of the hidden states shared by every projection
    with the same rotation, one GEMM launch) and hands the results out by name for all steps.
    """

    def __init__(self, ops: Ops, encoder_hidden_states: torch.Tensor, projections: Sequence[tuple]):
        """projections: (name, Weight, bias or None) per to_k / to_v weight."""
        self.names = [name for name, _, _ in projections]
        if len(set(self.names)) != len(self.names):
            raise CudaError("cross-attention cache: duplicate projection name")
        calls = [LinearCall(encoder_hidden_states, weight, bias) for _, weight, bias in projections]
        self._plan = ops.plan(calls)
        self._outputs = dict(zip(self.names, self._plan.run()))

    @property
    def launches(self) -> int:
        return self._plan.launches

    def refresh(self) -> None:
        """Recomputes every projection (new prompt written into the same hidden-state buffer)."""
        self._plan.run()

    def __getitem__(self, name: str) -> torch.Tensor:
        return self._outputs[name]

    def close(self) -> None:
        self._plan.close()
