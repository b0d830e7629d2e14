"""Writes tests/golden/quant_fixture.json from the reference's own golden file
for MLX affine dequantisation (tests/goldens/quant_fixture.json, the cases of
tests/unit/kernels/quant.rs:39-63 dequant_matches_mlx_bit_exactly), with every
float stored as its binary32 bit pattern so that the comparison is bit for bit.

    python tests/golden/make_quant_fixture.py <reference checkout>
"""
import json
import os
import struct
import sys


def bits(values):
    return [struct.unpack("<I", struct.pack("<f", v))[0] for v in values]


def main(reference: str) -> None:
    with open(os.path.join(reference, "tests", "goldens", "quant_fixture.json")) as f:
        src = json.load(f)
    cases = []
    for c in src["cases"]:
        cases.append({
            "name": c["name"], "rows": c["rows"], "cols": c["cols"], "group_size": c["group_size"],
            "bits": c["bits"], "codes": c["codes"], "scales_f32_bits": bits(c["scales"]),
            "biases_f32_bits": bits(c["biases"]), "expected_f32_bits": bits(c["expected"]),
        })
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_fixture.json")
    with open(out, "w") as f:
        json.dump({"source": "tests/goldens/quant_fixture.json", "cases": cases}, f, separators=(",", ":"))
    print(out, len(cases), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
