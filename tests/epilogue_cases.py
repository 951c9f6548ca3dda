"""Cases shared by tests/golden/make_golden_epilogue.py (which records the reference's outputs) and
the tests that replay them: the two bandwidth-bound steps inside the reference's fused
matmul + bias + leaky-relu backward (src/kernels/cpu/fused_ops.c:245-300): the relu-gradient
modulation dc_mod = dout * (out > 0 ? 1 : alpha) (fused_ops.c:105-109) and the bias gradient
dbias[col] = sum over rows of dc_mod (fused_ops.c:288-299).

The reference exposes them only through matmul_bias_relu_cpu_backward(inputs = {a [M,K], b [K,N],
bias [N]}, output [M,N]). With K = N and b the identity matrix, a.grad = dc_mod @ b^T holds dc_mod
itself (every other term of each dot product is an exact zero), and bias.grad is the column sum.
"""
import numpy as np

from harness import rand_normal

# (rows M, cols N, alpha)
CASES = [(1, 1, 0.0), (7, 13, 0.0), (64, 48, 0.01), (257, 33, 0.2), (128, 128, 0.0), (1000, 8, 0.0)]


def inputs(case_index):
    rows, cols, alpha = CASES[case_index]
    dout = rand_normal(400 + case_index, (rows, cols))
    out = rand_normal(500 + case_index, (rows, cols))
    out.reshape(-1)[::7] = 0.0          # exact zeros take the slope branch (x > 0 is false)
    return dout, out, alpha


def run_reference(ref_backend, case_index):
    """matmul_bias_relu_cpu_backward of the reference build on the case; returns (dc_mod, dbias)."""
    import ctypes as C
    from plast_b200 import CTensor, KernelParams, _ptr_array
    rows, cols, alpha = CASES[case_index]
    dout, out, _ = inputs(case_index)
    be = ref_backend
    a = be.tensor(np.zeros((rows, cols), np.float32), requires_grad=True)
    b = be.tensor(np.eye(cols, dtype=np.float32))
    bias = be.tensor(np.zeros((cols,), np.float32), requires_grad=True)
    bias.grad.copy_from(np.full(cols, 123.0, np.float32))     # the reference overwrites, it does not add
    y = be.tensor(out, requires_grad=True)
    y.grad.copy_from(dout)
    fn = be.lib.matmul_bias_relu_cpu_backward
    fn.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
    fn.restype = None
    fn(_ptr_array([a, b, bias]), C.byref(y.c), KernelParams(0, 0, alpha))
    return a.grad.numpy(), bias.grad.numpy()
