"""Regenerates tests/golden/tensor_ops.npz from the reference's own compiled operators.

Run where the reference checkout is mounted (it builds oracle/_ref first):

    python tests/golden/make_golden.py

Every case of tests/cases.py is executed on the compiled reference tensor module
(oracle/_ref/libcamel_tensor_ref.so: the unmodified modules/tensor sources driven through
getTensorOpsMap()); the outputs are stored as "<case>/<index>".  The fixtures let the parity
tests run where the reference checkout does not exist.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from cases import CASES, RefBackend, boundary_cases, run_boundary_case  # noqa: E402


def main():
    oracle.build(ref=True)
    be = RefBackend()
    out = {}
    for name, fn in CASES:
        for i, v in enumerate(fn(be)):
            out[f"{name}/{i}"] = np.asarray(v)
    path = Path(__file__).resolve().parent / "tensor_ops.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {path.stat().st_size / 1e6:.2f} MB")
    # array literals in, host reads and printed text out (tests/cases.py: boundary_cases)
    import json

    boundary = {name: run_boundary_case(oracle.ref(), op, build) for name, op, build in boundary_cases()}
    bpath = Path(__file__).resolve().parent / "boundary.json"
    bpath.write_text(json.dumps(boundary, indent=1) + "\n")
    print(f"wrote {bpath}: {len(boundary)} calls")
    # group \t uri \t signature of getTensorOperatorGroups() (modules/tensor/operators.cpp:196-583)
    table = Path(__file__).resolve().parent / "operator_table.tsv"
    table.write_text("".join("\t".join(row) + "\n" for row in oracle.ref().groups()))
    print(f"wrote {table}")


if __name__ == "__main__":
    main()
