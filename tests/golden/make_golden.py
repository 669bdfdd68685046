#!/usr/bin/env python3
"""Regenerates tests/golden/nsl_kat.json from the NSL source tree.

Usage:  python tests/golden/make_golden.py /path/to/NSL

The NSL sources are Rust, so nothing is executed: the script reads the one JSON
fixture NSL commits for this path and transcribes the known-answer constants
that NSL's own tests assert (each entry records the NSL test file it comes
from).  The output is the only thing the test-suite reads; the NSL tree is not
needed to run the tests.
"""
import json
import os
import sys


def flatten(rows):
    return [v for r in rows for v in r]


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    src = os.path.join(ref, "crates/nsl-codegen/tests/fixtures/bitnet_reference_outputs.json")
    with open(src) as f:
        doc = json.load(f)

    forward = []
    for fx in doc["fixtures"]:
        acts, w = fx["input"]["activations"], fx["input"]["weights"]
        exp = fx["expected"]
        forward.append({
            "name": fx["name"],
            "rows": len(acts), "hidden": len(acts[0]), "out_dim": len(w[0]),
            "x": flatten(acts),                 # [rows, hidden] f32
            "w_kn": flatten(w),                 # [hidden, out_dim] trits (reference orientation)
            "scale": exp["absmax_scale"],       # [rows]
            "q": flatten(exp["quantized_acts"]),  # [rows, hidden] int8, bit-exact target
            "y": flatten(exp["gemm_output"]),   # [rows, out_dim] f32, 1e-6 rel / 1e-7 abs
        })

    kat = {
        "_made_by": "tests/golden/make_golden.py",
        "_source": "crates/nsl-codegen/tests/fixtures/bitnet_reference_outputs.json "
                   "(tolerances: crates/nsl-codegen/tests/bitnet_reference.rs:245-327)",
        "forward": forward,
        # crates/nsl-codegen/tests/bitnet_absmean_quant.rs:12-52
        "absmax_quant": [
            {"x": [0.0] * 8, "scale": 0.0, "q": [0] * 8},
            {"x": [1.5] * 8, "scale": 1.5, "q": [127] * 8},
            {"x": [1.5, -2.5, 0.5, -1.0], "scale": 2.5, "q": [76, -127, 25, -51]},
            {"x": [0.1, 0.2, 10.0, 0.15], "scale": 10.0, "q": [1, 3, 127, 2]},
        ],
        # crates/nsl-codegen/tests/bitnet_gpu_correctness.rs:531-535 (half away, not half even)
        "rounding_row": {"x": [0.5, 2.5, 4.5, 6.5, -0.5, -2.5, 127.0, 1.0],
                         "q": [1, 3, 5, 7, -1, -3, 127, 1]},
        # crates/nsl-codegen/tests/bitnet_packed_repr.rs:13-60
        "pack": {"trits": [-1, 0, 1, 1], "byte": 0x1A, "invalid_bytes": [0xFF, 0xC0]},
        # crates/nsl-codegen/tests/bitnet_loader.rs:82-96
        "loader": {"values": [-2.0, 0.0, 0.2, 1.0, -1.0, 2.0, -0.2, 1.0],
                   "trits": [-1, 0, 0, 1, -1, 1, 0, 1], "scale": 0.925, "scale_tol": 1e-5},
        # crates/nsl-codegen/tests/bitnet_gpu_correctness.rs:571-576 (rows, hidden, out_dim)
        "gpu_random_cases": [[1, 256, 100], [5, 128, 128], [3, 512, 300], [2, 1024, 64]],
        # crates/nsl-runtime/src/awq.rs:426-512 (unit tests)
        "awq": {
            "pack_pairs": [[5, 12], [0, 15]],
            "group": {"values": [0.0, 1.0, 2.0, 3.0], "scale": 0.2, "zero": 0.0},
            "clamp": {"value": 100.0, "scale": 1.0, "zero": 0.0, "q": 15},
            "roundtrip": {"value": 1.5, "scale": 0.2, "zero": 0.0},
            "small_matrix": {"k": 4, "n": 4, "gs": 4, "max_abs_err": 0.15},
            "matmul": {"input": [1, 2, 3, 4, 5, 6, 7, 8], "m": 2, "k": 4, "n": 3, "gs": 4,
                       "weights": [0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0, 1.1, 1.2],
                       "rel": 0.1, "abs": 0.1},
        },
    }
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nsl_kat.json")
    with open(out, "w") as f:
        json.dump(kat, f, separators=(",", ":"))
        f.write("\n")
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
