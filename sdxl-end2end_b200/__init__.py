"""B200 (sm_100a) quantized-Linear operator for the SDXL UNet projection path.

Python front end over the C ABI in ``include/sdxlq.h`` (``libsdxlq.so``). It mirrors the
reference's operator interface for this path — ``Ops.linear`` / ``Ops.linear_activation`` /
``Ops.quantize_fp8`` (include/sdxl/cuda/ops.hpp:15-30 of the reference),
``upload_or_quantize_int8_weight`` (src/cuda/int8_convrot.hpp:11-16), the FP8 weight upload of
``WeightStore::upload_tensor`` (src/cuda/weights.cu:301-415) and the packed-weight + scale
metadata of ``cuda::Tensor`` (include/sdxl/cuda/tensor.hpp:123-157) — with the same names,
argument meaning and error behaviour (``CudaError`` where the reference throws it).

PyTorch is used only to own device memory and streams. There is no CPU fallback: importing
works anywhere, but creating a ``Context`` requires the compiled library and an sm_100 GPU.
"""
from __future__ import annotations

from .api import (  # noqa: F401
    ACT_GEGLU, ACT_GELU, ACT_NONE, ACT_QUICK_GELU, ACT_SILU,
    CrossAttentionKVCache, CudaError, Context, FP8WeightLoadOptions, GroupPlan, INT8WeightLoadOptions, LinearActivation,
    LinearCall, Ops, QuantizationMetadata, ScalarType, FP8ScaleMode, FP8StorageLayout, Weight,
    library_path, load_library, valid_convrot_group_size,
)
from .build import build  # noqa: F401
from . import packed_formats  # noqa: F401
from . import unet_harness  # noqa: F401
from .unet_harness import EulerDenoiser, UNetConfig, UNetHarness  # noqa: F401
