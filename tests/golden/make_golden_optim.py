"""Generates tests/golden/optimizers.npz by running the REFERENCE's own sgd_step_cpu,
adam_step_cpu and adamw_step_cpu (compiled into oracle/_ref/libplast_ref.so by oracle/Makefile)
on the seeded runs of tests/optim_cases.py.

    python tests/golden/make_golden_optim.py
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import optim_cases  # noqa: E402
from harness import REF_LIB, have_ref  # noqa: E402
from plast_b200 import CTensor  # noqa: E402
from plast_b200 import optim as O  # noqa: E402


class CArena(C.Structure):
    """include/core/arena.h:26-29"""
    _fields_ = [("current", C.c_void_p), ("device", C.c_int)]


def main():
    if not have_ref():
        raise SystemExit("oracle/_ref/libplast_ref.so missing: run `make -C oracle` where the reference sources exist")
    ref = C.CDLL(str(REF_LIB))
    ref.arena_create.argtypes = [C.c_uint64, C.c_int]
    ref.arena_create.restype = CArena
    out = {}
    for kind, struct in (("sgd", O.SGD), ("adam", O.Adam), ("adamw", O.AdamW)):
        fn = getattr(ref, f"{kind}_step_cpu")
        fn.argtypes = [C.POINTER(struct), C.POINTER(C.POINTER(CTensor)), C.c_int]
        fn.restype = None
        arenas = [ref.arena_create(1 << 20, 0), ref.arena_create(1 << 22, 0)]   # optimizer (meta), data; CPU

        def give_arenas(opt):
            if kind != "sgd":
                opt.optimizer_arena = C.addressof(arenas[0])
                opt.data_arena = C.addressof(arenas[1])

        res, _ = optim_cases.run_through_structs(kind, "cpu", fn, give_arenas)
        out.update(res)
    path = Path(__file__).resolve().parent / "optimizers.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()
