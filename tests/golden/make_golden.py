"""Generates tests/golden/reference_dense.npz and tests/golden/config1_rows.npz by running the UNMODIFIED reference CPU Linear
(`linear_2d` + `geglu`, src/unet.cpp:202-235, 483-493 of the reference, reached through
oracle/_ref/libsdxl_ref.so) on seeded inputs shaped like the GEGLU feed-forward projection
(K = 640, a slice of N = 5120) and on FP8-stored weights. Run from the repository root in a
container that has the reference tree:

    make -C oracle ref && python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as O  # noqa: E402
import helpers as H  # noqa: E402


def main() -> None:
    assert O.ref_available(), "build oracle/_ref first (make -C oracle ref)"
    x = H.make_activations(2024, 16, 640)
    w = H.make_weight(2024, 192, 640)
    bias = H.make_bias(2024, 192)
    linear = O.ref_linear_2d(x.astype(np.float32), w, bias)
    geglu = O.ref_geglu(linear)
    rng = np.random.default_rng(77)
    x8 = H.make_activations(2025, 8, 320, outliers=False)
    out = {"x": x, "w": w, "bias": bias, "linear_2d": linear, "geglu": geglu, "x8": x8}
    for fmt, name in ((O.E4M3, "e4m3"), (O.E5M2, "e5m2")):
        finite = np.array([b for b in range(256)
                           if np.isfinite(O.fp8_decode(np.array([b], np.uint8), fmt)[0])], np.uint8)
        wq = rng.choice(finite, size=(48, 320)).astype(np.uint8)
        out[f"w_{name}"] = wq
        out[f"linear_2d_{name}"] = O.ref_linear_2d(x8.astype(np.float32), wq, None, fp8_fmt=fmt)
    path = os.path.join(ROOT, "tests", "golden", "reference_dense.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")

    # The first benchmark configuration at full size: X [8192, 640] x W [5120, 640] + bias, GEGLU,
    # FP16 weights. 40 rows spread over the 64 row tiles, each a full output row of the reference's
    # linear_2d + geglu (inputs are regenerated from the seed by the test, only rows and results are
    # stored).
    seed = 4242
    x = H.make_activations(seed, 8192, 640)
    w = H.make_weight(seed, 5120, 640)
    bias = H.make_bias(seed, 5120)
    rows = np.unique(np.concatenate([[0, 127, 128, 8191], np.random.default_rng(seed).integers(0, 8192, size=36)]))
    result = O.ref_geglu(O.ref_linear_2d(x[rows].astype(np.float32), w, bias))
    path = os.path.join(ROOT, "tests", "golden", "config1_rows.npz")
    np.savez_compressed(path, seed=np.int64(seed), rows=rows.astype(np.int64), out=result.astype(np.float32))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
