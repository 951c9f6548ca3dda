"""GPU parity of the elementwise entry points against the CPU oracle, through the C ABI.

Bounds (from the reference's CPU path being the contract):
  add / sub / mul / div / abs / leaky_relu (incl. relu's -0.0): bit-exact
  neg: equal as values (the reference's AVX body yields +0 for -(+0), its scalar path -0)
  exp / log / sin / cos / tan: <= 2 ulp of the oracle (glibc libm) on the tested ranges
  backward of same-shape operands: same bounds as the forward math they use
"""
import numpy as np
import pytest

import plast_b200 as pb
from harness import (FULL_REDUCE, assert_bit_equal, assert_sum_close, assert_ulp, rand_normal,
                     rand_uniform)

pytestmark = pytest.mark.gpu

BINARY = ["add", "sub", "mul", "div"]
SHAPES_SAME = [(4,), (2, 3), (3, 2, 4), (1025,), (257, 129), (5, 7, 11, 13), (2, 3, 4, 5, 6, 7)]
# (a shape, b shape): the reference's own broadcast cases (tests/test_ops.py:11-15) and the
# layouts of the benchmark configs
BROADCAST = [((4,), (1,)), ((2, 3), (1, 3)), ((3, 1, 4), (1, 2, 1)), ((64, 48), (1, 48)),
             ((64, 48), (64, 1)), ((64, 48), ()), ((), (64, 48)), ((6, 8, 5, 5), (1, 8, 1, 1)),
             ((33, 7), (7,)), ((5, 1, 3), (4, 1)), ((128, 256), (1, 256))]


def bshape(a, b):
    return tuple(np.broadcast_shapes(a, b))


def run_binary(be, op, A, B):
    ta, tb = be.tensor(A), be.tensor(B)
    out = be.empty(bshape(A.shape, B.shape))
    be.forward(op, [ta, tb], out)
    return out.numpy()


@pytest.mark.parametrize("op", BINARY)
@pytest.mark.parametrize("shape", SHAPES_SAME)
def test_binary_same_shape(cuda, oracle, op, shape):
    A = rand_normal(0, shape)
    B = rand_uniform(1, shape, 0.5, 2.0) * np.where(rand_uniform(2, shape) > 0, 1, -1).astype(np.float32)
    assert_bit_equal(run_binary(cuda, op, A, B), run_binary(oracle, op, A, B), f"{op}{shape}")


@pytest.mark.parametrize("op", BINARY)
@pytest.mark.parametrize("sa,sb", BROADCAST)
def test_binary_broadcast(cuda, oracle, op, sa, sb):
    A = rand_normal(0, sa) if sa else np.float32(1.5).reshape(())
    B = rand_uniform(1, sb, 0.5, 2.0) if sb else np.float32(0.75).reshape(())
    assert_bit_equal(run_binary(cuda, op, A, B), run_binary(oracle, op, A, B), f"{op}{sa}{sb}")


def test_binary_unaligned_and_odd_sizes(cuda, oracle):
    # views that start 4 or 8 bytes into an allocation take the float2 / scalar paths
    base = rand_normal(0, (4099,))
    other = rand_normal(1, (4099,))
    for off, n in [(1, 4097), (2, 4096), (3, 1001), (0, 4099), (1, 7), (2, 2)]:
        outs = []
        for be in (cuda, oracle):
            ta, tb = be.tensor(base), be.tensor(other)
            va = ta.view([n], [1]); va.c.data = ta.c.data + 4 * off
            vb = tb.view([n], [1]); vb.c.data = tb.c.data + 4 * off
            out = be.empty((n,))
            be.forward("add", [va, vb], out)
            outs.append(out.numpy())
        assert_bit_equal(outs[0], outs[1], f"offset {off} n {n}")


def test_binary_transposed_and_expanded_views(cuda, oracle):
    A = rand_normal(0, (37, 53))
    B = rand_normal(1, (53, 37))
    row = rand_normal(2, (53,))
    for op in BINARY:
        outs = []
        for be in (cuda, oracle):
            ta, tb = be.tensor(A), be.tensor(B)
            out = be.empty((53, 37))
            be.forward(op, [ta.transpose(0, 1), tb], out)          # strided a, contiguous b
            out2 = be.empty((37, 53))
            tr = be.tensor(row)
            be.forward(op, [ta, tr.view([37, 53], [0, 1])], out2)  # expand view: stride 0, size > 1
            outs.append((out.numpy(), out2.numpy()))
        assert_bit_equal(outs[0][0], outs[1][0], f"{op} transposed")
        assert_bit_equal(outs[0][1], outs[1][1], f"{op} expanded")
    # a transposed operand goes through the shared-memory tile kernel, whatever the extents
    import plast_b200 as pb
    for m, n in [(8, 8), (33, 65), (100, 7), (7, 100), (256, 513)]:
        a, b = rand_normal(3, (m, n)), rand_normal(4, (n, m))
        outs = []
        for be in (cuda, oracle):
            out = be.empty((n, m))
            be.forward("mul", [be.tensor(a).transpose(0, 1), be.tensor(b)], out)
            outs.append(out.numpy())
        if m >= 8 and n >= 8:
            assert pb.last_kernel() == "ew_tiled_transpose"
        assert_bit_equal(outs[0], outs[1], f"tiled {m}x{n}")
    # 3-D: [B, M, N] with the last two axes swapped, plus a broadcast operand
    a, b = rand_normal(5, (5, 40, 24)), rand_normal(6, (1, 24, 1))
    outs = []
    for be in (cuda, oracle):
        out = be.empty((5, 24, 40))
        be.forward("add", [be.tensor(a).transpose(1, 2), be.tensor(b)], out)
        outs.append(out.numpy())
    assert_bit_equal(outs[0], outs[1], "tiled 3-D")


def test_inputs_contiguous_along_two_different_dims(cuda, oracle):
    """out[i, j, k] = a.transpose(0, 2)[i, j, k] op b.transpose(1, 2)[i, j, k]: a is contiguous along
    i, b along j, the output along k. Any stride combination is one code path in the reference
    (include/kernels/kernel_macros.h:213-220); here the input that does not share the first
    3-D tiles turn both dims in one pass when every extent is a multiple of 4; otherwise the input
    that does not share the first transposed dim is gathered through the 2-D tile kernel first."""
    import plast_b200 as pb
    for shape in [(24, 40, 56), (9, 33, 130), (64, 64, 64), (16, 16, 32), (8, 8, 8), (20, 36, 100), (132, 12, 260)]:
        I, J, K = shape
        a, b = rand_normal(7, (K, J, I)), rand_normal(8, (I, K, J))
        small = rand_uniform(9, (1, J, 1), 0.5, 2.0)
        for op in BINARY:
            outs = []
            for be in (cuda, oracle):
                out = be.empty(shape)
                be.forward(op, [be.tensor(a).transpose(0, 2), be.tensor(b).transpose(1, 2)], out)
                outs.append(out.numpy())
            one_pass = all(s % 4 == 0 for s in shape)
            assert pb.last_kernel() == ("ew_tiled_transpose_two_dims" if one_pass else "ew_gather_then_tiled_transpose"), shape
            assert_bit_equal(outs[0], outs[1], f"{op} {shape}: two transposed inputs")
        # three operands through a fused entry point: x transposed one way, scale the other, bias broadcast
        outs = []
        for be, name in ((cuda, "scale_bias_leaky_relu"), (oracle, None)):
            ta, tb, ts = be.tensor(a).transpose(0, 2), be.tensor(b).transpose(1, 2), be.tensor(small)
            out = be.empty(shape)
            if name:
                be.forward(name, [ta, tb, ts], out, fval=0.1)
            else:
                m, u = be.empty(shape), be.empty(shape)
                be.forward("mul", [ta, tb], m); be.forward("add", [m, ts], u); be.forward("leaky_relu", [u], out, fval=0.1)
            outs.append(out.numpy())
        assert_bit_equal(outs[0], outs[1], f"fused epilogue {shape}: two transposed inputs")
    # 4-D: a batch dim outside the three that the tile covers
    a, b = rand_normal(10, (3, 24, 16, 40)), rand_normal(11, (3, 40, 24, 16))
    outs = []
    for be in (cuda, oracle):
        out = be.empty((3, 40, 16, 24))
        be.forward("sub", [be.tensor(a).transpose(1, 3), be.tensor(b).transpose(2, 3)], out)
        outs.append(out.numpy())
    assert pb.last_kernel() == "ew_tiled_transpose_two_dims"
    assert_bit_equal(outs[0], outs[1], "two transposed inputs with a batch dim")


def test_relu_negative_zero_and_config1_forward(cuda, oracle):
    # config 1: C = relu(A + b); s = sum(C, axis=1). relu is leaky_relu(slope 0): x <= 0 -> x * 0
    A, b = rand_uniform(0, (1024, 1024)), rand_uniform(1, (1, 1024))
    res = {}
    for be in (cuda, oracle):
        ta, tb = be.tensor(A), be.tensor(b)
        ab = be.empty((1024, 1024)); be.forward("add", [ta, tb], ab)
        c = be.empty((1024, 1024)); be.forward("leaky_relu", [ab], c, fval=0.0)
        s = be.empty((1024,)); be.forward("sum", [c], s, dim=1)
        res[be.name] = (ab.numpy(), c.numpy(), s.numpy())
    assert_bit_equal(res["cuda"][0], res["oracle"][0], "A+b")
    assert_bit_equal(res["cuda"][1], res["oracle"][1], "relu")
    assert (np.signbit(res["cuda"][1]) & (res["cuda"][1] == 0)).sum() > 500000  # the -0.0 outputs
    assert_sum_close(res["cuda"][2], res["oracle"][2], np.abs(res["oracle"][1]).sum(axis=1), what="row sum")


UNARY_RANGES = {
    "abs": (-10, 10), "neg": (-10, 10), "exp": (-20, 20), "log": (1e-6, 100.0), "sin": (-20, 20),
    "cos": (-20, 20), "tan": (-1.5, 1.5), "leaky_relu": (-5, 5),
}


@pytest.mark.parametrize("op", list(UNARY_RANGES))
@pytest.mark.parametrize("shape", [(4,), (3, 2, 4), (100003,), (300, 1000)])
def test_unary_forward(cuda, oracle, op, shape):
    lo, hi = UNARY_RANGES[op]
    A = rand_uniform(3, shape, lo, hi)
    res = {}
    for be in (cuda, oracle):
        out = be.empty(shape)
        be.forward(op, [be.tensor(A)], out, fval=0.01)
        res[be.name] = out.numpy()
    if op in ("abs", "leaky_relu"):
        assert_bit_equal(res["cuda"], res["oracle"], op)
    elif op == "neg":
        assert np.array_equal(res["cuda"], res["oracle"])
    else:
        assert_ulp(res["cuda"], res["oracle"], 2, op)


def test_unary_special_values(cuda, oracle):
    x = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 3.4e38, -3.4e38,
                  88.7, -103.9, 1e-20], np.float32)
    for op, fval in [("leaky_relu", 0.0), ("leaky_relu", 0.1), ("abs", 0), ("exp", 0), ("neg", 0)]:
        res = {}
        for be in (cuda, oracle):
            out = be.empty(x.shape)
            be.forward(op, [be.tensor(x)], out, fval=fval)
            res[be.name] = out.numpy()
        if op == "exp":
            assert_ulp(res["cuda"], res["oracle"], 2, op)
        elif op == "neg":
            assert np.array_equal(res["cuda"], res["oracle"], equal_nan=True)
        else:
            assert_bit_equal(res["cuda"], res["oracle"], f"{op} {fval}")


def test_unary_strided_views(cuda, oracle):
    A = rand_uniform(5, (31, 45), -3, 3)
    for op in ["exp", "abs", "leaky_relu", "sin"]:
        res = {}
        for be in (cuda, oracle):
            ta = be.tensor(A).transpose(0, 1)          # shape [45,31], strides [1,45]
            out = be.empty((45, 31))
            be.forward(op, [ta], out, fval=0.2)
            res[be.name] = out.numpy()
        if op in ("abs", "leaky_relu"):
            assert_bit_equal(res["cuda"], res["oracle"], op)
        else:
            assert_ulp(res["cuda"], res["oracle"], 2, op)


@pytest.mark.parametrize("op", list(UNARY_RANGES))
def test_unary_backward(cuda, oracle, op):
    lo, hi = UNARY_RANGES[op]
    shape = (129, 65)
    A, G, D0 = rand_uniform(3, shape, lo, hi), rand_normal(4, shape), rand_normal(5, shape)
    res = {}
    for be in (cuda, oracle):
        ta = be.tensor(A, requires_grad=True)
        ta.grad.copy_from(D0)                            # backward accumulates into existing grads
        out = be.empty(shape, requires_grad=True)
        be.forward(op, [ta], out, fval=0.01)
        out.grad.copy_from(G)
        be.backward(op, [ta], out, fval=0.01)
        res[be.name] = ta.grad.numpy()
    if op in ("neg", "leaky_relu", "abs"):
        assert np.array_equal(res["cuda"], res["oracle"])
    else:
        np.testing.assert_allclose(res["cuda"], res["oracle"], rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("shape", [(77, 130), (64, 256), (3, 5, 1024), (4,)])
@pytest.mark.parametrize("op", BINARY)
def test_binary_backward_same_shape(cuda, oracle, op, shape):
    import plast_b200 as pb
    A, B = rand_normal(0, shape), rand_uniform(1, shape, 0.5, 2.0)
    G, DA, DB = rand_normal(2, shape), rand_normal(3, shape), rand_normal(4, shape)
    res = {}
    for be in (cuda, oracle):
        ta, tb = be.tensor(A, requires_grad=True), be.tensor(B, requires_grad=True)
        ta.grad.copy_from(DA); tb.grad.copy_from(DB)
        out = be.empty(shape, requires_grad=True)
        out.grad.copy_from(G)
        be.backward(op, [ta, tb], out)
        res[be.name] = (ta.grad.numpy(), tb.grad.numpy())
    assert_bit_equal(res["cuda"][0], res["oracle"][0], f"{op} da")
    assert_bit_equal(res["cuda"][1], res["oracle"][1], f"{op} db")
    # five dense tensors of one shape with a multiple of four elements: both gradients in one pass
    if int(np.prod(shape)) % 4 == 0:
        assert pb.last_kernel() == "binary_backward_both"


@pytest.mark.parametrize("op", BINARY)
def test_binary_backward_of_a_tensor_with_itself(cuda, oracle, op):
    """x op x: both operands share one gradient buffer, which receives the two terms one after the other
    (include/kernels/kernel_macros.h:301-325); the one-pass kernel must not be taken."""
    shape = (32, 64)
    A, G, DA = rand_uniform(0, shape, 0.5, 2.0), rand_normal(2, shape), rand_normal(3, shape)
    res = {}
    for be in (cuda, oracle):
        ta = be.tensor(A, requires_grad=True)
        ta.grad.copy_from(DA)
        out = be.empty(shape, requires_grad=True)
        out.grad.copy_from(G)
        be.backward(op, [ta, ta], out)
        res[be.name] = ta.grad.numpy()
    assert_bit_equal(res["cuda"], res["oracle"], f"{op}(x, x) dx")


def test_backward_skips_inputs_without_grad(cuda):
    A, B = rand_normal(0, (8, 8)), rand_normal(1, (8, 8))
    ta, tb = cuda.tensor(A), cuda.tensor(B, requires_grad=True)
    out = cuda.empty((8, 8), requires_grad=True)
    out.grad.copy_from(np.ones((8, 8), np.float32))
    cuda.backward("mul", [ta, tb], out)
    assert np.array_equal(tb.grad.numpy(), A)


def test_error_reporting(cuda):
    import plast_b200 as pb
    a, b = cuda.tensor(rand_normal(0, (4, 3))), cuda.tensor(rand_normal(1, (5,)))
    out = cuda.empty((4, 3))
    with pytest.raises(pb.PlastError) as e:
        cuda.forward("add", [a, b], out)
    assert e.value.code == 2                       # shape
    ai = cuda.empty((4, 3), dtype=pb.INT32)
    with pytest.raises(pb.PlastError) as e:
        cuda.forward("exp", [ai], out)
    assert e.value.code == 1                       # dtype: the reference prints and skips too
    with pytest.raises(pb.PlastError):
        cuda.forward("sum", [a], cuda.empty((4,)), dim=5)
    cuda.forward("add", [a, a], out)               # the next good call clears the error
    assert pb.lib.plast_b200_last_error() == 0


@pytest.mark.parametrize("shape,bshape", [((1024, 1024), (1, 1024)), ((37, 64), (64,)), ((5, 7, 128), (5, 7, 128)),
                                          ((33, 1001), (1, 1001)), ((256, 8200), (1, 8200))])
def test_fused_forward_writes_c_and_its_row_sums(cuda, oracle, shape, bshape):
    import ctypes as C
    A, b = rand_uniform(0, shape), rand_uniform(1, bshape)
    ta, tb = cuda.tensor(A), cuda.tensor(b)
    c, s = cuda.empty(shape), cuda.empty(shape[:-1])
    pb.lib.plast_b200_add_leaky_relu_row_sum(C.byref(ta.c), C.byref(tb.c), C.byref(c.c), C.byref(s.c), 0.0)
    pb.check_error()
    oa, ob = oracle.tensor(A), oracle.tensor(b)
    oab, oc = oracle.empty(shape), oracle.empty(shape)
    oracle.forward("add", [oa, ob], oab); oracle.forward("leaky_relu", [oab], oc, fval=0.0)
    osum = oracle.empty(shape[:-1]); oracle.forward("sum", [oc], osum, dim=len(shape) - 1)
    assert_bit_equal(c.numpy(), oc.numpy(), "C of the fused forward")
    assert_sum_close(s.numpy().reshape(shape[:-1]), osum.numpy().reshape(shape[:-1]), np.abs(oc.numpy()).sum(axis=-1), what="row sums")
