"""Pins the oracle's restatement of the two bandwidth-bound steps of the reference's fused
matmul + bias + leaky-relu backward (oracle_relu_grad_modulate, oracle_bias_grad_reduce) to the
reference: against tests/golden/epilogue_pieces.npz, recorded from matmul_bias_relu_cpu_backward
(src/kernels/cpu/fused_ops.c:105-109, 245-300) by tests/golden/make_golden_epilogue.py, and live
against oracle/_ref where that build is present."""
import ctypes as C

import numpy as np
import pytest

import epilogue_cases
from harness import GOLDEN_DIR, ORACLE_LIB, assert_bit_equal, build_oracle

GOLDEN = np.load(GOLDEN_DIR / "epilogue_pieces.npz")


def oracle_pieces(dout, out, alpha):
    build_oracle()
    lib = C.CDLL(str(ORACLE_LIB))
    f32p = C.POINTER(C.c_float)
    lib.oracle_relu_grad_modulate.argtypes = [f32p, f32p, f32p, C.c_uint64, C.c_float]
    lib.oracle_bias_grad_reduce.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64]
    p = lambda a: a.ctypes.data_as(f32p)
    rows, cols = dout.shape
    mod = np.empty((rows, cols), np.float32)
    lib.oracle_relu_grad_modulate(p(dout), p(out), p(mod), rows * cols, alpha)
    dbias = np.full(cols, -5.0, np.float32)                 # must be overwritten
    lib.oracle_bias_grad_reduce(p(mod), p(dbias), rows * cols, cols)
    return mod, dbias


@pytest.mark.parametrize("i", range(len(epilogue_cases.CASES)))
def test_oracle_matches_the_reference_golden(i):
    dout, out, alpha = epilogue_cases.inputs(i)
    mod, dbias = oracle_pieces(dout, out, alpha)
    # dc_mod came back through a product with the identity matrix: equal values (a -0.0 may have
    # become +0.0 in the sum of zeros)
    assert np.array_equal(mod, GOLDEN[f"case{i}/dc_mod"])
    # same order of additions (rows in order per column): the same bits
    assert_bit_equal(dbias, GOLDEN[f"case{i}/dbias"], "bias gradient")


@pytest.mark.parametrize("i", range(len(epilogue_cases.CASES)))
def test_oracle_matches_the_reference_build_live(ref, i):
    dout, out, alpha = epilogue_cases.inputs(i)
    mod, dbias = oracle_pieces(dout, out, alpha)
    ref_mod, ref_dbias = epilogue_cases.run_reference(ref, i)
    assert np.array_equal(mod, ref_mod)
    assert_bit_equal(dbias, ref_dbias, "bias gradient")
    assert np.array_equal(ref_mod, GOLDEN[f"case{i}/dc_mod"]) and np.array_equal(ref_dbias, GOLDEN[f"case{i}/dbias"])
