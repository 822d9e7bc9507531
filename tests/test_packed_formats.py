"""The reference's on-disk packed-weight formats for this path (CPU only).

The FP8 sidecar layout is pinned against a file image assembled here field by field from the
reference's writer (WeightStore::write_fp8_cache, src/cuda/weights.cu:617-668) and reader checks
(load_fp8_cache, :513-615); the INT8 prequantised triple against the reference's own safetensors
parser (compiled from its sources under oracle/_ref) and the rules of bind_quantization_metadata
(src/sdxl.cpp:654-715, INT8_CONVROT.md:139-161).
"""
import importlib
import io
import json
import struct

import numpy as np
import pytest

pf = importlib.import_module("sdxl-end2end_b200.packed_formats")


def entries():
    rng = np.random.default_rng(5)
    per_row = pf.Fp8CacheEntry("unet.down.0.to_q.weight", pf.FLOAT8_E4M3, pf.SCALE_PER_OUTPUT_CHANNEL, pf.ROW_MAJOR_NK,
                               [4, 8], rng.integers(0, 255, 32, dtype=np.uint8), rng.random(4, dtype=np.float32))
    tensor_wide = pf.Fp8CacheEntry("unet.add_embedding.linear_1.weight", pf.FLOAT8_E5M2, pf.SCALE_TENSOR_WIDE,
                                   pf.ROW_MAJOR_NK, [2, 16], rng.integers(0, 255, 32, dtype=np.uint8),
                                   np.array([0.125], dtype=np.float32))
    return [per_row, tensor_wide]


def hand_built_image(key, ordered):
    """The byte layout, written out independently of the module under test."""
    image = b"SDXLF8C3" + struct.pack("=I", len(key)) + key.encode()
    image += struct.pack("=I", len(ordered))
    for e in ordered:
        image += struct.pack("=I", len(e.name)) + e.name.encode()
        image += bytes([e.type, e.scale_mode, len(e.shape), e.storage_layout])
        for dimension in e.shape:
            image += struct.pack("=Q", dimension)
        image += struct.pack("=Q", e.data.size) + struct.pack("=Q", e.scales.size)
        image += e.data.tobytes() + e.scales.astype(np.float32).tobytes()
    return image


def test_fp8_cache_image_matches_the_reference_layout():
    both = entries()
    ordered = sorted(both, key=lambda e: e.name)           # the reference sorts by name before writing
    assert pf.fp8_cache_bytes("key-1", both) == hand_built_image("key-1", ordered)


def test_fp8_cache_round_trip_and_shape_check(tmp_path):
    path = str(tmp_path / "model.safetensors.sdxlfp8")
    written = pf.write_fp8_cache(path, "abc", entries())
    assert written == 32 + 16 + 32 + 4
    shapes = {e.name: e.shape for e in entries()}
    loaded = pf.read_fp8_cache(path, "abc", pf.ROW_MAJOR_NK, shapes)
    assert [e.name for e in loaded] == sorted(shapes)
    by_name = {e.name: e for e in loaded}
    for want in entries():
        got = by_name[want.name]
        assert (got.type, got.scale_mode, got.storage_layout, list(got.shape)) == \
               (want.type, want.scale_mode, want.storage_layout, list(want.shape))
        assert np.array_equal(got.data, want.data) and np.array_equal(got.scales, want.scales)
    # a model whose parameter has another shape, or lacks the parameter: miss
    shapes["unet.down.0.to_q.weight"] = [8, 4]
    assert pf.read_fp8_cache(path, "abc", pf.ROW_MAJOR_NK, shapes) is None
    assert pf.read_fp8_cache(path, "abc", pf.ROW_MAJOR_NK, {}) is None
    assert pf.read_fp8_cache(str(tmp_path / "absent"), "abc") is None


def test_fp8_cache_misses_like_the_reference():
    good = pf.fp8_cache_bytes("k", entries())
    parse = lambda image, key="k", layout=pf.ROW_MAJOR_NK: pf.parse_fp8_cache(io.BytesIO(image), key, layout)
    assert len(parse(good)) == 2
    assert parse(good, key="other") is None                              # stale key
    assert parse(b"SDXLF8C2" + good[8:]) is None                         # older magic
    assert parse(good, layout=pf.K_MAJOR_KN) is None                     # layout the runtime does not want
    assert parse(good[:-3]) is None                                      # truncated scales
    zero_entries = b"SDXLF8C3" + struct.pack("=I", 1) + b"k" + struct.pack("=I", 0)
    assert parse(zero_entries) is None
    # wrong scale count for a per-channel entry
    e = entries()[0]
    e.scales = e.scales[:2]
    assert parse(pf.fp8_cache_bytes("k", [e])) is None
    # data bytes that do not match the shape
    e = entries()[1]
    e.shape = [2, 8]
    assert parse(pf.fp8_cache_bytes("k", [e])) is None
    # a name outside the UNet
    e = entries()[1]
    e.name = "text_encoder.layer.weight"
    assert parse(pf.fp8_cache_bytes("k", [e])) is None
    # strings: oversized length and truncation raise, as the reference throws
    with pytest.raises(pf.PackedFormatError):
        parse(b"SDXLF8C3" + struct.pack("=I", 17 * 1024 * 1024))
    with pytest.raises(pf.PackedFormatError):
        parse(b"SDXLF8C3" + struct.pack("=I", 10) + b"abc")


def test_fp8_cache_writer_keeps_unet_fp8_tensors_only(tmp_path):
    path = str(tmp_path / "cache.sdxlfp8")
    other = entries()[1]
    other.name = "vae.decoder.weight"
    assert pf.write_fp8_cache(path, "k", [other]) == 0
    assert pf.read_fp8_cache(path, "k") is None                          # nothing was written
    assert pf.write_fp8_cache(path, "k", entries() + [other]) == 84
    assert len(pf.read_fp8_cache(path, "k")) == 2


def test_quantization_config_rules():
    parse = pf.parse_quantization_config
    assert parse('{"convrot":true,"convrot_groupsize":256,"per_row":true}') == \
        {"convrot": True, "per_row": True, "convrot_group_size": 256}
    assert parse('{"convrot":true,"convrot_group_size":64}')["convrot_group_size"] == 64
    assert parse('{"convrot":true,"group_size":16}')["convrot_group_size"] == 16
    # precedence: legacy spelling first, then the explicit one, then the generic one
    assert parse('{"group_size":4,"convrot_group_size":16,"convrot_groupsize":64}')["convrot_group_size"] == 64
    assert parse('{"group_size":4,"convrot_group_size":16}')["convrot_group_size"] == 16
    assert parse("not json") == {} and parse("") == {} and parse("[1,2]") == {}
    weight = np.zeros((8, 256), dtype=np.int8)
    record = pf.int8_record(weight, np.ones((8, 1), dtype=np.float32), '{"convrot":true}')
    assert record.convrot and record.convrot_group_size == 256          # default group size
    assert record.per_row                                                # inferred: one scale per output row
    record = pf.int8_record(weight, np.ones(1, dtype=np.float32), "")
    assert not record.convrot and record.convrot_group_size == 0 and not record.per_row


def test_int8_checkpoint_round_trip_and_reference_parser(tmp_path):
    rng = np.random.default_rng(9)
    linears = {
        "unet.blocks.0.attn1.to_q": pf.Int8LinearRecord(rng.integers(-127, 128, (16, 256), dtype=np.int8),
                                                        rng.random((16, 1), dtype=np.float32), True, True, 256),
        "unet.blocks.0.ff.net.2": pf.Int8LinearRecord(rng.integers(-127, 128, (8, 64), dtype=np.int8),
                                                      rng.random(8, dtype=np.float32), False, True, 0),
    }
    path = str(tmp_path / "int8.safetensors")
    pf.write_int8_checkpoint(path, linears)
    loaded = pf.read_int8_checkpoint(path)
    assert sorted(loaded) == sorted(linears)
    for prefix, want in linears.items():
        got = loaded[prefix]
        assert np.array_equal(got.weight, want.weight) and np.array_equal(got.weight_scale, want.weight_scale)
        assert (got.convrot, got.per_row, got.convrot_group_size) == (want.convrot, want.per_row, want.convrot_group_size)
    # the explicit spelling is read back the same way
    pf.write_int8_checkpoint(path, linears, legacy_key=False)
    assert pf.read_int8_checkpoint(path)["unet.blocks.0.attn1.to_q"].convrot_group_size == 256

    from oracle import oracle as O
    if not O.ref_available():
        pytest.skip("reference-built checker not present")
    # the unmodified reference parser sees the same tensors: DType I8 = 2, F32 = 11, U8 = 1
    dtype, shape, size, head = O.ref_safetensors_probe(path, "unet.blocks.0.attn1.to_q.weight")
    assert (dtype, shape, size) == (2, [16, 256], 16 * 256)
    assert head == linears["unet.blocks.0.attn1.to_q"].weight.tobytes()[:len(head)]
    dtype, shape, size, head = O.ref_safetensors_probe(path, "unet.blocks.0.attn1.to_q.weight_scale")
    assert (dtype, shape, size) == (11, [16, 1], 64)
    assert head == linears["unet.blocks.0.attn1.to_q"].weight_scale.tobytes()
    dtype, shape, size, head = O.ref_safetensors_probe(path, "unet.blocks.0.attn1.to_q.comfy_quant", 128)
    assert dtype == 1 and json.loads(head.decode()) == {"convrot": True, "convrot_group_size": 256, "per_row": True}
