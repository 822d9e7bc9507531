"""The reference's two on-disk packed-weight formats for this path, read and written byte for byte.

1. FP8 sidecar cache (``<checkpoint>.sdxlfp8``; WeightStore::write_fp8_cache / load_fp8_cache,
   src/cuda/weights.cu:513-668 of the reference). Native-endian binary:

       char[8]  magic "SDXLF8C3"
       string   cache key                      (u32 length + bytes)
       u32      entry count                    (1 .. 100000)
       per entry, sorted by name:
         string name                           (must begin with "unet.")
         u8     ScalarType                     (0 Float8E4M3, 1 Float8E5M2)
         u8     FP8ScaleMode                   (1 TensorWide, 2 PerOutputChannel)
         u8     rank                           (1 .. 4)
         u8     FP8StorageLayout               (0 RowMajorNK, 1 KMajorKN)
         u64    shape[rank]
         u64    data bytes                     (= product of the shape)
         u64    scale count                    (shape[0] for PerOutputChannel, else 1)
         bytes  data
         f32    scales[scale count]

   A reader that finds anything unexpected reports a miss (the reference returns ``false`` and
   re-quantises); strings longer than 16 MiB and truncated strings raise, as the reference throws.

2. Prequantised INT8 ConvRot checkpoints (INT8_CONVROT.md:139-161, bind_quantization_metadata in
   src/sdxl.cpp:654-715): a safetensors file in which every quantised Linear is the triple

       <prefix>.weight        I8  [out_features, in_features]
       <prefix>.weight_scale  F32 [out_features, 1] or [out_features]
       <prefix>.comfy_quant   U8  JSON bytes, e.g. {"convrot":true,"convrot_groupsize":256,"per_row":true}

   with the group size accepted under ``convrot_groupsize``, ``convrot_group_size`` or
   ``group_size`` (in that order of precedence), 256 when ConvRot is on and no size is given, and
   ``per_row`` inferred from the scale count when the JSON does not say.

Pure host code (numpy + struct): no GPU, no torch. The arrays it returns go to the device through
``Ops.upload_or_quantize_int8_weight`` / ``Ops.upload_fp8_weight``'s prequantised paths.
"""
from __future__ import annotations

import io
import json
import os
import struct
from dataclasses import dataclass, field
from typing import BinaryIO, Dict, List, Optional, Sequence

import numpy as np

FP8_CACHE_MAGIC = b"SDXLF8C3"
MAX_STRING = 16 * 1024 * 1024
MAX_ENTRIES = 100000

# numeric values of the reference's enums (include/sdxl/cuda/tensor.hpp:17-48)
FLOAT8_E4M3, FLOAT8_E5M2 = 0, 1
SCALE_NONE, SCALE_TENSOR_WIDE, SCALE_PER_OUTPUT_CHANNEL = 0, 1, 2
ROW_MAJOR_NK, K_MAJOR_KN = 0, 1


class PackedFormatError(RuntimeError):
    """What the reference throws as CudaError while reading a cache (bad or truncated string)."""


# ------------------------------------------------------------------------------------------------
# FP8 sidecar cache
# ------------------------------------------------------------------------------------------------
@dataclass
class Fp8CacheEntry:
    name: str
    type: int                       # FLOAT8_E4M3 / FLOAT8_E5M2
    scale_mode: int                 # SCALE_TENSOR_WIDE / SCALE_PER_OUTPUT_CHANNEL
    storage_layout: int             # ROW_MAJOR_NK / K_MAJOR_KN
    shape: Sequence[int]
    data: np.ndarray                # uint8, prod(shape) bytes
    scales: np.ndarray              # float32, 1 or shape[0] values


def _write_string(output: BinaryIO, text: str) -> None:
    raw = text.encode("utf-8")
    output.write(struct.pack("=I", len(raw)))
    output.write(raw)


def _read_exact(source: BinaryIO, count: int) -> Optional[bytes]:
    raw = source.read(count)
    return raw if len(raw) == count else None


def _read_string(source: BinaryIO) -> str:
    header = _read_exact(source, 4)
    if header is None:
        raise PackedFormatError("truncated FP8 cache string")
    (size,) = struct.unpack("=I", header)
    if size > MAX_STRING:
        raise PackedFormatError("invalid FP8 cache string size")
    raw = _read_exact(source, size)
    if raw is None:
        raise PackedFormatError("truncated FP8 cache string")
    return raw.decode("utf-8")


def fp8_cache_bytes(key: str, entries: Sequence[Fp8CacheEntry]) -> bytes:
    """The file image write_fp8_cache produces for these entries (sorted by name, like the reference)."""
    output = io.BytesIO()
    output.write(FP8_CACHE_MAGIC)
    _write_string(output, key)
    ordered = sorted(entries, key=lambda entry: entry.name)
    output.write(struct.pack("=I", len(ordered)))
    for entry in ordered:
        data = np.ascontiguousarray(entry.data, dtype=np.uint8).reshape(-1)
        scales = np.ascontiguousarray(entry.scales, dtype=np.float32).reshape(-1)
        _write_string(output, entry.name)
        output.write(struct.pack("=BBBB", entry.type, entry.scale_mode, len(entry.shape), entry.storage_layout))
        for dimension in entry.shape:
            output.write(struct.pack("=Q", int(dimension)))
        output.write(struct.pack("=QQ", data.size, scales.size))
        output.write(data.tobytes())
        output.write(scales.tobytes())
    return output.getvalue()


def write_fp8_cache(path: str, key: str, entries: Sequence[Fp8CacheEntry]) -> int:
    """Writes the cache through a temporary file and a rename, like the reference. Entries that are
    not FP8 UNet tensors are left out (the reference caches `unet.` FP8 tensors only); nothing is
    written when none remain. Returns the bytes of data and scales written."""
    kept = [entry for entry in entries if entry.name.startswith("unet.") and entry.type in (FLOAT8_E4M3, FLOAT8_E5M2)]
    if not kept:
        return 0
    directory = os.path.dirname(path)
    if directory:
        os.makedirs(directory, exist_ok=True)
    temporary = path + ".tmp"
    with open(temporary, "wb") as output:
        output.write(fp8_cache_bytes(key, kept))
    if os.path.exists(path):
        os.remove(path)
    os.rename(temporary, path)
    return sum(int(np.asarray(e.data).size) + 4 * int(np.asarray(e.scales).size) for e in kept)


def parse_fp8_cache(source: BinaryIO, key: str, expected_layout: int = ROW_MAJOR_NK,
                    expected_shapes: Optional[Dict[str, Sequence[int]]] = None) -> Optional[List[Fp8CacheEntry]]:
    """load_fp8_cache's parsing and checks. Returns None where the reference reports a miss.

    expected_layout   the layout the runtime wants (K-major only for the weight-only FP8 mode,
                      which does not exist on B200).
    expected_shapes   name -> shape of the model's parameters; entries that are unknown or have
                      another shape make the cache a miss. None skips that check.
    """
    if _read_exact(source, 8) != FP8_CACHE_MAGIC:
        return None
    if _read_string(source) != key:
        return None
    header = _read_exact(source, 4)
    if header is None:
        return None
    (count,) = struct.unpack("=I", header)
    if count == 0 or count > MAX_ENTRIES:
        return None
    entries: List[Fp8CacheEntry] = []
    for _ in range(count):
        name = _read_string(source)
        fixed = _read_exact(source, 4)
        if fixed is None:
            return None
        type_, scale_mode, rank, layout = struct.unpack("=BBBB", fixed)
        if type_ not in (FLOAT8_E4M3, FLOAT8_E5M2) or rank == 0 or rank > 4:
            return None
        if layout not in (ROW_MAJOR_NK, K_MAJOR_KN) or layout != expected_layout:
            return None
        raw_shape = _read_exact(source, 8 * rank)
        if raw_shape is None:
            return None
        shape = list(struct.unpack(f"={rank}Q", raw_shape))
        if any(dimension == 0 for dimension in shape):
            return None
        elements = int(np.prod(np.array(shape, dtype=object)))
        sizes = _read_exact(source, 16)
        if sizes is None:
            return None
        data_bytes, scale_count = struct.unpack("=QQ", sizes)
        if data_bytes != elements or scale_count == 0:
            return None
        if not name.startswith("unet."):
            return None
        if expected_shapes is not None and list(expected_shapes.get(name, ())) != shape:
            return None
        if scale_count != (shape[0] if scale_mode == SCALE_PER_OUTPUT_CHANNEL else 1):
            return None
        data = _read_exact(source, data_bytes)
        scales = _read_exact(source, 4 * scale_count)
        if data is None or scales is None:
            return None
        entries.append(Fp8CacheEntry(name, type_, scale_mode, layout, shape,
                                     np.frombuffer(data, dtype=np.uint8).copy(),
                                     np.frombuffer(scales, dtype=np.float32).copy()))
    return entries


def read_fp8_cache(path: str, key: str, expected_layout: int = ROW_MAJOR_NK,
                   expected_shapes: Optional[Dict[str, Sequence[int]]] = None) -> Optional[List[Fp8CacheEntry]]:
    if not os.path.exists(path):
        return None
    with open(path, "rb") as source:
        return parse_fp8_cache(source, key, expected_layout, expected_shapes)


# ------------------------------------------------------------------------------------------------
# Prequantised INT8 ConvRot checkpoints (safetensors)
# ------------------------------------------------------------------------------------------------
_SAFETENSORS_DTYPES = {"I8": np.int8, "U8": np.uint8, "F32": np.float32, "F16": np.float16}
_NUMPY_TO_SAFETENSORS = {np.dtype(v): k for k, v in _SAFETENSORS_DTYPES.items()}


@dataclass
class Int8LinearRecord:
    """One quantised Linear of a checkpoint with its metadata as the reference binds it
    (sdxl::QuantizationMetadata, include/sdxl/model.hpp:17-23)."""
    weight: np.ndarray                         # int8 [out_features, in_features]
    weight_scale: np.ndarray                   # float32 [out_features] or [out_features, 1] as stored
    convrot: bool = False
    per_row: bool = False
    convrot_group_size: int = 0
    raw_config: Dict[str, object] = field(default_factory=dict)


def write_safetensors(path: str, tensors: Dict[str, np.ndarray]) -> None:
    """A minimal safetensors writer: u64 little-endian header length, JSON header, raw data."""
    header: Dict[str, object] = {}
    blobs = []
    offset = 0
    for name in sorted(tensors):
        array = np.ascontiguousarray(tensors[name])
        dtype = _NUMPY_TO_SAFETENSORS.get(array.dtype)
        if dtype is None:
            raise PackedFormatError(f"unsupported dtype {array.dtype} for {name}")
        raw = array.tobytes()
        header[name] = {"dtype": dtype, "shape": list(array.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as output:
        output.write(struct.pack("<Q", len(text)))
        output.write(text)
        for raw in blobs:
            output.write(raw)


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as source:
        raw_length = _read_exact(source, 8)
        if raw_length is None:
            raise PackedFormatError("truncated safetensors header")
        (length,) = struct.unpack("<Q", raw_length)
        text = _read_exact(source, length)
        if text is None:
            raise PackedFormatError("truncated safetensors header")
        header = json.loads(text.decode("utf-8"))
        payload = source.read()
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        dtype = _SAFETENSORS_DTYPES.get(entry["dtype"])
        if dtype is None:
            continue                                   # a dtype this path does not use
        begin, end = entry["data_offsets"]
        if end > len(payload) or begin > end:
            raise PackedFormatError(f"safetensors tensor {name} lies outside the file")
        tensors[name] = np.frombuffer(payload[begin:end], dtype=dtype).reshape(entry["shape"]).copy()
    return tensors


def parse_quantization_config(text: str) -> Dict[str, object]:
    """The fields bind_quantization_metadata reads from a comfy_quant JSON, with its precedence of
    the group-size spellings. Malformed JSON is ignored (empty result), as in the reference."""
    result: Dict[str, object] = {}
    if not text:
        return result
    try:
        parsed = json.loads(text)
    except ValueError:
        return result
    if not isinstance(parsed, dict):
        return result
    if "convrot" in parsed:
        result["convrot"] = bool(parsed["convrot"])
    if "per_row" in parsed:
        result["per_row"] = bool(parsed["per_row"])
    for key in ("convrot_groupsize", "convrot_group_size", "group_size"):
        if key in parsed:
            result["convrot_group_size"] = int(parsed[key])
            break
    return result


def int8_record(weight: np.ndarray, weight_scale: np.ndarray, config_text: str = "") -> Int8LinearRecord:
    """Binds one triple like bind_quantization_metadata (src/sdxl.cpp:654-715)."""
    config = parse_quantization_config(config_text)
    record = Int8LinearRecord(weight=weight, weight_scale=weight_scale, raw_config=config)
    record.convrot = bool(config.get("convrot", False))
    record.per_row = bool(config.get("per_row", False))
    record.convrot_group_size = int(config.get("convrot_group_size", 0))
    if not record.per_row:
        record.per_row = int(np.asarray(weight_scale).size) == int(weight.shape[0])
    if record.convrot and record.convrot_group_size == 0:
        record.convrot_group_size = 256
    return record


def read_int8_checkpoint(path: str) -> Dict[str, Int8LinearRecord]:
    """prefix -> record for every `<prefix>.weight` of dtype I8 that has a `<prefix>.weight_scale`."""
    tensors = read_safetensors(path)
    records: Dict[str, Int8LinearRecord] = {}
    for name, weight in tensors.items():
        if not name.endswith(".weight") or weight.dtype != np.int8 or weight.ndim != 2:
            continue
        prefix = name[: -len("weight")]
        scale = tensors.get(prefix + "weight_scale")
        if scale is None:
            continue
        config = tensors.get(prefix + "comfy_quant")
        text = bytes(config.astype(np.uint8)).decode("utf-8", errors="replace") if config is not None else ""
        records[prefix[:-1]] = int8_record(weight, scale.astype(np.float32), text)
    return records


def write_int8_checkpoint(path: str, linears: Dict[str, Int8LinearRecord], legacy_key: bool = True) -> None:
    """Writes the triple per Linear. `legacy_key` picks the `convrot_groupsize` spelling the
    reference's documentation lists first."""
    tensors: Dict[str, np.ndarray] = {}
    for prefix, record in linears.items():
        config = {"convrot": bool(record.convrot)}
        if record.convrot:
            config["convrot_groupsize" if legacy_key else "convrot_group_size"] = int(record.convrot_group_size)
        config["per_row"] = bool(record.per_row)
        tensors[prefix + ".weight"] = np.ascontiguousarray(record.weight, dtype=np.int8)
        tensors[prefix + ".weight_scale"] = np.ascontiguousarray(record.weight_scale, dtype=np.float32)
        tensors[prefix + ".comfy_quant"] = np.frombuffer(json.dumps(config, separators=(",", ":")).encode("utf-8"), dtype=np.uint8)
    write_safetensors(path, tensors)
