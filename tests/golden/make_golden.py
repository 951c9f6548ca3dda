"""Generates tests/golden/hotpath.npz by running the REFERENCE's own CPU kernels (the build in
oracle/_ref, compiled from the reference sources by oracle/Makefile) on seeded inputs.

    python tests/golden/make_golden.py

The fixture pins the oracle restatement (and, on the GPU box where the reference sources do not
exist, the CUDA kernels) to outputs of the reference itself. Cases are small so the file stays
a few hundred KB. Every array is stored as produced; inputs are regenerated from the seeds by
`cases()` so the tests and this script cannot drift apart.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from golden_cases import cases, run_case  # noqa: E402
from harness import CpuBackend, have_ref  # noqa: E402


def main():
    if not have_ref():
        raise SystemExit("oracle/_ref/libplast_ref.so missing: run `make -C oracle` where the reference sources exist")
    ref = CpuBackend("ref")
    out = {}
    for case in cases():
        for key, arr in run_case(ref, case).items():
            out[f"{case['name']}/{key}"] = arr
    path = Path(__file__).resolve().parent / "hotpath.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB, {len(out)} arrays, {len(cases())} cases)")


if __name__ == "__main__":
    main()
