"""Regenerates tests/golden/reference_outputs.npz from the reference's own kernels.

Run in a container that has the reference tree (it is compiled, unmodified, by oracle/Makefile
into oracle/_ref/libck_ref.so):

    python tests/golden/make_golden.py

Inputs are not stored: tests rebuild them from the seeds in tests/cases.py; the file holds only
the reference's outputs for those inputs.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from __graft_entry__ import oracle_loader  # noqa: E402


def main() -> None:
    loader = oracle_loader()
    loader.build()
    ref = loader.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libck_ref.so is not built (reference tree missing?)")
    out = cases.golden_outputs(ref, "")
    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")
    # a second file for the later entry points, so that the first one stays byte for byte what earlier runs wrote
    out = cases.boundary_outputs(ref, "")
    path = os.path.join(HERE, "reference_boundary_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
