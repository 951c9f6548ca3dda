"""Shared test plumbing: the three implementations of plast's kernel entry points behind one
interface, so a parity test reads `cuda.forward("add", ...)` next to `oracle.forward("add", ...)`.

  cuda    libplast_b200.so   <op>_cuda_forward / _backward      device memory (the product)
  oracle  oracle/liboracle.so  oracle_<op>_forward / _backward  host memory (CPU restatement)
  ref     oracle/_ref/libplast_ref.so  <op>_cpu_forward / _backward  host memory (the reference's
          own CPU kernels compiled from its sources; present only where it was built)

All three take the same `Tensor` struct (include/plast_b200.h).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

import plast_b200 as pb
from plast_b200 import CTensor, KernelParams, Tensor, FULL_REDUCE, FLOAT32, INT32  # noqa: F401

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
ORACLE_LIB = ORACLE_DIR / "liboracle.so"
REF_LIB = ORACLE_DIR / "_ref" / "libplast_ref.so"
GOLDEN_DIR = ROOT / "tests" / "golden"

PRIMITIVE_OPS = ["add", "sub", "mul", "div", "abs", "cos", "sin", "tan", "exp", "log", "neg",
                 "leaky_relu", "sum", "mean", "max", "min"]


def build_oracle():
    """Compiles oracle/liboracle.so (and oracle/_ref when the reference sources are present)."""
    if not ORACLE_LIB.exists() or ORACLE_LIB.stat().st_mtime < (ORACLE_DIR / "oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    return ORACLE_LIB


class CpuBackend:
    """oracle or ref: same struct, host pointers."""

    device = "cpu"

    def __init__(self, name: str):
        self.name = name
        if name == "oracle":
            build_oracle()
            self.lib = C.CDLL(str(ORACLE_LIB))
            self._fmt = "oracle_{op}_{dir}"
        elif name == "ref":
            self.lib = C.CDLL(str(REF_LIB))
            self._fmt = "{op}_cpu_{dir}"
        else:
            raise ValueError(name)

    def _fn(self, op, direction):
        fn = getattr(self.lib, self._fmt.format(op=op, dir=direction))
        fn.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
        fn.restype = None
        return fn

    def tensor(self, arr, requires_grad=False):
        return Tensor.from_numpy(np.asarray(arr), device="cpu", requires_grad=requires_grad)

    def empty(self, shape, dtype=FLOAT32, requires_grad=False):
        return Tensor(shape, device="cpu", dtype=dtype, requires_grad=requires_grad)

    def forward(self, op, inputs, out, dim=0, keepdim=0, fval=0.0):
        self._fn(op, "forward")(pb._ptr_array(inputs), C.byref(out.c), KernelParams(dim, keepdim, fval))
        return out

    def backward(self, op, inputs, out, dim=0, keepdim=0, fval=0.0):
        self._fn(op, "backward")(pb._ptr_array(inputs), C.byref(out.c), KernelParams(dim, keepdim, fval))


class CudaBackend:
    name = "cuda"
    device = "cuda"

    def tensor(self, arr, requires_grad=False):
        return Tensor.from_numpy(np.asarray(arr), device="cuda", requires_grad=requires_grad)

    def empty(self, shape, dtype=FLOAT32, requires_grad=False):
        return Tensor(shape, device="cuda", dtype=dtype, requires_grad=requires_grad)

    def forward(self, op, inputs, out, dim=0, keepdim=0, fval=0.0):
        return pb.forward(op, inputs, out, dim, keepdim, fval)

    def backward(self, op, inputs, out, dim=0, keepdim=0, fval=0.0):
        pb.backward(op, inputs, out, dim, keepdim, fval)


def have_ref() -> bool:
    return REF_LIB.exists()


class OracleRecipes:
    """The composite recipes of oracle.c (flat-array signatures)."""

    def __init__(self):
        build_oracle()
        self.lib = C.CDLL(str(ORACLE_LIB))
        f32p, i32p, u64 = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_uint64
        self.lib.oracle_softmax_rows.argtypes = [f32p, f32p, u64, u64]
        self.lib.oracle_log_softmax_rows.argtypes = [f32p, f32p, u64, u64]
        self.lib.oracle_cross_entropy_rows.argtypes = [f32p, i32p, f32p, f32p, u64, u64]
        self.lib.oracle_sigmoid.argtypes = [f32p, f32p, u64]
        self.lib.oracle_sigmoid_mul_add_exp_neg_abs.argtypes = [f32p, f32p, f32p, u64]

    @staticmethod
    def _p(a, t=C.c_float):
        return a.ctypes.data_as(C.POINTER(t))

    def softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.oracle_softmax_rows(self._p(x), self._p(y), x.size // x.shape[-1], x.shape[-1])
        return y

    def log_softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.oracle_log_softmax_rows(self._p(x), self._p(y), x.size // x.shape[-1], x.shape[-1])
        return y

    def cross_entropy(self, x, labels):
        x = np.ascontiguousarray(x, np.float32)
        labels = np.ascontiguousarray(labels, np.int32)
        per_row = np.empty(x.shape[0], np.float32)
        mean = np.zeros(1, np.float32)
        self.lib.oracle_cross_entropy_rows(self._p(x), self._p(labels, C.c_int32), self._p(per_row),
                                           self._p(mean), x.shape[0], x.shape[1])
        return mean, per_row

    def sigmoid(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.oracle_sigmoid(self._p(x), self._p(y), x.size)
        return y

    def chain(self, x, y):
        x = np.ascontiguousarray(x, np.float32)
        y = np.ascontiguousarray(y, np.float32)
        z = np.empty_like(x)
        self.lib.oracle_sigmoid_mul_add_exp_neg_abs(self._p(x), self._p(y), self._p(z), x.size)
        return z


def cpu_recipe_graph(be, mode, X, G=None, labels=None):
    """Forward AND backward of softmax / log_softmax / cross_entropy as the op sequence plast builds
    from primitives (plast/nn/functional.py:77-86, 89-97, 312-333, 391-396), every node run through
    the CPU entry points of `be` in graph order and its backward in reverse order
    (src/core/graph.c:57-65; kernels: src/kernels/cpu/reduce_ops.c:90-262,
    include/kernels/kernel_macros.h:273-325). X is [rows, cols], the axis is 1.
    Returns (forward result, d/dX): G is the upstream gradient of softmax / log_softmax; the
    cross-entropy mean is seeded with 1 (what backward() does, src/core/tensor.c:143-152)."""
    R, Cn = X.shape
    x = be.tensor(X, requires_grad=True)
    m = be.empty((R, 1), requires_grad=True); be.forward("max", [x], m, dim=1, keepdim=1)
    sh = be.empty((R, Cn), requires_grad=True); be.forward("sub", [x, m], sh)
    e = be.empty((R, Cn), requires_grad=True); be.forward("exp", [sh], e)
    s = be.empty((R, 1), requires_grad=True); be.forward("sum", [e], s, dim=1, keepdim=1)

    def head_backward():
        be.backward("sum", [e], s, dim=1, keepdim=1); be.backward("exp", [sh], e)
        be.backward("sub", [x, m], sh); be.backward("max", [x], m, dim=1, keepdim=1)

    if mode == "softmax":
        y = be.empty((R, Cn), requires_grad=True); be.forward("div", [e, s], y)
        y.grad.copy_from(G)
        be.backward("div", [e, s], y)
        head_backward()
        return y.numpy(), x.grad.numpy()
    ls = be.empty((R, 1), requires_grad=True); be.forward("log", [s], ls)
    y = be.empty((R, Cn), requires_grad=True); be.forward("sub", [sh, ls], y)
    if mode == "log_softmax":
        y.grad.copy_from(G)
        be.backward("sub", [sh, ls], y); be.backward("log", [s], ls)
        head_backward()
        return y.numpy(), x.grad.numpy()
    assert mode == "cross_entropy"
    onehot = np.zeros((R, Cn), np.float32); onehot[np.arange(R), labels] = 1.0
    oh = be.tensor(onehot)
    prod = be.empty((R, Cn), requires_grad=True); be.forward("mul", [y, oh], prod)
    rs = be.empty((R,), requires_grad=True); be.forward("sum", [prod], rs, dim=1)
    ng = be.empty((R,), requires_grad=True); be.forward("neg", [rs], ng)
    loss = be.empty((1,), requires_grad=True); be.forward("mean", [ng], loss, dim=FULL_REDUCE)
    loss.grad.copy_from(np.ones(1, np.float32))
    be.backward("mean", [ng], loss, dim=FULL_REDUCE); be.backward("neg", [rs], ng)
    be.backward("sum", [prod], rs, dim=1); be.backward("mul", [y, oh], prod)
    be.backward("sub", [sh, ls], y); be.backward("log", [s], ls)
    head_backward()
    return loss.numpy(), x.grad.numpy()


# ---- comparison helpers ------------------------------------------------------------------------
def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    bad = bits(got) != bits(want)
    if got.dtype.kind == "f":
        bad &= ~(np.isnan(got) & np.isnan(want))  # NaN payload / sign is not part of the contract
    if bad.any():
        i = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements differ bitwise; first at "
                             f"{tuple(i)}: got {got[tuple(i)]!r} want {want[tuple(i)]!r}")


def ulp_distance(a, b) -> np.ndarray:
    """Distance in units in the last place between two float32 arrays (monotone integer map)."""
    def key(x):
        u = bits(x).astype(np.int64)
        return np.where(u & 0x80000000, 0x80000000 - u, u)
    return np.abs(key(a) - key(b))


def assert_ulp(got, want, max_ulp, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    both_nan = np.isnan(got) & np.isnan(want)
    d = np.where(both_nan, 0, ulp_distance(got, want))
    worst = int(d.max()) if d.size else 0
    assert worst <= max_ulp, f"{what}: {worst} ulp > {max_ulp} (at {np.unravel_index(d.argmax(), d.shape)})"


def assert_sum_close(got, want, abs_terms_sum, rel=1e-5, what=""):
    """|got - want| <= rel * sum|terms|: the bound for fp32 accumulations whose order differs
    from the reference's sequential loop (the reference itself is ~1e-7 of sum|x| off fp64)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    bound = rel * np.asarray(abs_terms_sum, np.float64) + 1e-30
    err = np.abs(got - want)
    assert (err <= bound).all(), f"{what}: max err/bound {np.max(err / bound):.3g}"


def rand_uniform(seed, shape, lo=-1.0, hi=1.0):
    return np.random.RandomState(seed).uniform(lo, hi, shape).astype(np.float32)


def rand_normal(seed, shape, std=1.0):
    return (std * np.random.RandomState(seed).randn(*shape)).astype(np.float32)
