"""Copies the numbers of the reference's two PyTorch-made op fixtures into one JSON file.

    python tests/golden/make_reference_fixtures.py /path/to/reference

Input: <reference>/testdata/linear_case.json and norm_case.json (the same values as the
.bin files its Zig unit tests read, src/module/linear.zig:110-138, src/module/norm.zig:116-140).
Output: tests/golden/reference_fixtures.json.  The reference's model code itself (Zig) cannot
be compiled here, so these two ops are the only outputs of the reference that the plain
implementation is pinned to; everything else rests on its formulas.
"""
import json
import os
import sys


def main():
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    ref = sys.argv[1]
    out = {}
    for name in ("linear_case", "norm_case"):
        with open(os.path.join(ref, "testdata", name + ".json"), "r", encoding="utf-8") as f:
            out[name] = json.load(f)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(dst, "w", encoding="utf-8") as f:
        json.dump(out, f)
    print("wrote", dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
