"""The backward pieces of the reference's fused GEMM epilogues (relu-gradient modulation and the
bias-gradient column sum) against the oracle restatement of those kernels."""
import ctypes as C

import numpy as np
import pytest

import plast_b200 as pb
from harness import ORACLE_LIB, assert_bit_equal, assert_sum_close, build_oracle, rand_normal

pytestmark = pytest.mark.gpu


def oracle():
    build_oracle()
    lib = C.CDLL(str(ORACLE_LIB))
    f32p = C.POINTER(C.c_float)
    lib.oracle_relu_grad_modulate.argtypes = [f32p, f32p, f32p, C.c_uint64, C.c_float]
    lib.oracle_bias_grad_reduce.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64]
    return lib, (lambda a: a.ctypes.data_as(f32p))


@pytest.mark.parametrize("rows,cols,alpha", [(1, 1, 0.0), (7, 13, 0.0), (1024, 1024, 0.0), (4099, 257, 0.01),
                                              (3, 70001, 0.2), (100000, 8, 0.0)])
def test_modulate_and_bias_grad(rows, cols, alpha):
    lib, p = oracle()
    n = rows * cols
    dout, y = rand_normal(0, (n,)), rand_normal(1, (n,))
    y[::7] = 0.0                                                          # zeros take the slope branch
    want_mod = np.empty(n, np.float32)
    lib.oracle_relu_grad_modulate(p(dout), p(y), p(want_mod), n, alpha)
    want_bias = np.empty(cols, np.float32)
    lib.oracle_bias_grad_reduce(p(want_mod), p(want_bias), n, cols)

    td, ty = pb.Tensor.from_numpy(dout), pb.Tensor.from_numpy(y)
    tmod, tbias, tbias2 = pb.Tensor((n,)), pb.Tensor((cols,)), pb.Tensor((cols,))
    tbias.copy_from(np.full(cols, 123.0, np.float32))                     # must be overwritten, not added to
    tbias2.copy_from(np.full(cols, -7.0, np.float32))
    pb.lib.plast_b200_relu_grad_modulate(td.c.data, ty.c.data, tmod.c.data, n, alpha); pb.check_error()
    assert_bit_equal(tmod.numpy(), want_mod, "relu_grad_modulate")
    pb.lib.plast_b200_bias_grad_reduce(tmod.c.data, tbias.c.data, n, cols); pb.check_error()
    pb.lib.plast_b200_bias_grad_masked(td.c.data, ty.c.data, tbias2.c.data, n, cols, alpha); pb.check_error()
    scale = np.abs(want_mod.reshape(rows, cols)).sum(axis=0)
    assert_sum_close(tbias.numpy(), want_bias, scale, what="bias_grad_reduce")
    assert_sum_close(tbias2.numpy(), want_bias, scale, what="bias_grad_masked")


def test_against_the_outputs_recorded_from_the_reference_backward():
    """tests/golden/epilogue_pieces.npz holds what the reference's matmul_bias_relu_cpu_backward
    produced on these cases (src/kernels/cpu/fused_ops.c:105-109, 288-299)."""
    import epilogue_cases
    from harness import GOLDEN_DIR
    golden = np.load(GOLDEN_DIR / "epilogue_pieces.npz")
    for i, (rows, cols, _) in enumerate(epilogue_cases.CASES):
        dout, out, alpha = epilogue_cases.inputs(i)
        n = rows * cols
        td, ty, tmod, tbias = pb.Tensor.from_numpy(dout), pb.Tensor.from_numpy(out), pb.Tensor((n,)), pb.Tensor((cols,))
        pb.lib.plast_b200_relu_grad_modulate(td.c.data, ty.c.data, tmod.c.data, n, alpha); pb.check_error()
        assert np.array_equal(tmod.numpy().reshape(rows, cols), golden[f"case{i}/dc_mod"])
        pb.lib.plast_b200_bias_grad_masked(td.c.data, ty.c.data, tbias.c.data, n, cols, alpha); pb.check_error()
        scale = np.abs(golden[f"case{i}/dc_mod"]).sum(axis=0)
        assert_sum_close(tbias.numpy(), golden[f"case{i}/dbias"], scale, what=f"case {i} bias gradient")


def test_bad_arguments_are_reported():
    t = pb.Tensor((8,))
    pb.lib.plast_b200_bias_grad_reduce(t.c.data, t.c.data, 8, 3)
    assert pb.lib.plast_b200_last_error() == 2                            # 8 elements are not rows of 3
    pb.lib.plast_b200_bias_grad_reduce(None, t.c.data, 8, 4)
    assert pb.lib.plast_b200_last_error() == 3
    pb.lib.plast_b200_clear_error()
