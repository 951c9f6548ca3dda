"""Generates tests/golden/epilogue_pieces.npz by running the REFERENCE's own
matmul_bias_relu_cpu_backward (src/kernels/cpu/fused_ops.c:245-300, compiled into
oracle/_ref/libplast_ref.so by oracle/Makefile) on the seeded cases of tests/epilogue_cases.py.

    python tests/golden/make_golden_epilogue.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import epilogue_cases  # noqa: E402
from harness import CpuBackend, have_ref  # noqa: E402


def main():
    if not have_ref():
        raise SystemExit("oracle/_ref/libplast_ref.so missing: run `make -C oracle` where the reference sources exist")
    ref = CpuBackend("ref")
    out = {}
    for i in range(len(epilogue_cases.CASES)):
        dc_mod, dbias = epilogue_cases.run_reference(ref, i)
        out[f"case{i}/dc_mod"] = dc_mod
        out[f"case{i}/dbias"] = dbias
    path = Path(__file__).resolve().parent / "epilogue_pieces.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()
