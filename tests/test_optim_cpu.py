"""Optimiser steps on the CPU side: the oracle restatement against the committed outputs of the
reference's own sgd / adam / adamw CPU steps (tests/golden/optimizers.npz, made by
tests/golden/make_golden_optim.py), struct layouts, and the reference build itself when present."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

import optim_cases
from harness import GOLDEN_DIR, ORACLE_LIB, build_oracle
from plast_b200 import optim as O

ROOT = Path(__file__).resolve().parent.parent
REF_INCLUDE = Path(os.environ.get("PLAST_REFERENCE", "/root/reference")) / "include"
GOLDEN = np.load(GOLDEN_DIR / "optimizers.npz")


@pytest.mark.parametrize("kind", ["sgd", "adam", "adamw"])
def test_oracle_matches_reference_golden(kind):
    build_oracle()
    got = optim_cases.run_oracle(kind, C.CDLL(str(ORACLE_LIB)))
    keys = [k for k in GOLDEN.files if k.startswith(kind + "/")]
    assert keys and set(keys) == set(got)
    for k in keys:
        want = GOLDEN[k]
        assert got[k].size == want.size
        want = want.reshape(got[k].shape)                                 # 0-dim parameters come back as [1]
        # The reference build contracts a*b+c into one FMA (gcc -O3, -ffp-contract=fast); the
        # oracle rounds every product, as separate GPU instructions do: a few ulp apart at most.
        np.testing.assert_allclose(got[k], want, rtol=2e-6, atol=5e-7, err_msg=k)     # atol: a difference of operands ~1 can cancel
    # the parameter without a gradient never moves
    p0 = optim_cases.initial_params()[optim_cases.NO_GRAD]
    assert np.array_equal(got[f"{kind}/step{optim_cases.STEPS}/p{optim_cases.NO_GRAD}"], p0)


def test_bias_corrected_step_size_is_evaluated_in_double():
    build_oracle()
    lib = C.CDLL(str(ORACLE_LIB))
    lib.oracle_adam_lr_t.argtypes = [C.c_float, C.c_float, C.c_float, C.c_int]
    lib.oracle_adam_lr_t.restype = C.c_float
    for t in (1, 2, 10, 1000):
        b1, b2, lr = np.float32(0.9), np.float32(0.999), np.float32(1e-3)
        num = np.float32(1.0) - np.float32(np.float32(b2) ** np.float32(t))
        den = np.float32(1.0) - np.float32(np.float32(b1) ** np.float32(t))
        want = np.float32(np.float64(lr) * np.sqrt(np.float64(num)) / np.float64(den))
        got = lib.oracle_adam_lr_t(lr, b1, b2, t)
        assert abs(got - want) <= 2 * np.spacing(want)                    # powf vs numpy's power: 1 ulp each


@pytest.mark.skipif(not REF_INCLUDE.exists(), reason="reference headers not on this machine")
def test_optimizer_struct_layout_matches_reference_headers(tmp_path):
    probe = r'''
#include <stdio.h>
#include <stddef.h>
%s
int main(void) {
  printf("%%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu\n", sizeof(SGD), sizeof(Adam), offsetof(Adam, t),
         offsetof(Adam, m), offsetof(Adam, v), sizeof(AdamW), offsetof(AdamW, weight_decay), offsetof(AdamW, t),
         offsetof(AdamW, m), offsetof(AdamW, v));
  return 0;
}'''
    out = []
    for inc, flags in (('#include "plast_b200_optim.h"', [f"-I{ROOT / 'include'}"]),
                       ('#define PLAST_B200_USE_REFERENCE_TYPES\n#include "plast_b200_optim.h"',
                        [f"-I{ROOT / 'include'}", f"-I{REF_INCLUDE}"])):
        src = tmp_path / "p.c"
        src.write_text(probe % inc)
        subprocess.run(["gcc", "-std=c11", *flags, str(src), "-o", str(tmp_path / "p")], check=True)
        out.append(subprocess.run([str(tmp_path / "p")], check=True, capture_output=True, text=True).stdout.strip())
    assert out[0] == out[1] == "4 56 16 24 32 56 16 20 24 32"
    assert (C.sizeof(O.SGD), C.sizeof(O.Adam), O.Adam.t.offset, O.AdamW.weight_decay.offset) == (4, 56, 16, 16)
