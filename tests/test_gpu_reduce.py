"""GPU parity of reductions, argmax, the broadcast-gradient reduce and the fused recipes against
the CPU oracle, through the C ABI.

Bounds: max / min / argmax bit-exact (argmax: lowest index on ties); sums, means, softmax and
gradient reductions |gpu - oracle| <= 1e-5 * sum|terms| (the order of fp32 accumulation differs:
the reference adds left to right, the GPU adds as a tree).
"""
import numpy as np
import pytest

from harness import (FULL_REDUCE, INT32, assert_bit_equal, assert_sum_close, assert_ulp, rand_normal,
                     rand_uniform)

pytestmark = pytest.mark.gpu

REDUCE_SHAPES = [(4,), (2, 3), (3, 2, 4), (7, 33), (33, 7), (5, 1, 9), (128, 1024), (1000, 3),
                 (3, 1000), (17, 5, 64), (6, 8, 5, 5), (2, 3, 4, 5, 6), (70000,), (3, 100000),
                 (64, 16, 1024), (1000, 16, 64), (5, 3, 4096), (40, 64, 260),
                 (5000, 10), (4100, 33), (70, 80, 7), (4096, 48), (100000, 4), (4097, 1), (300, 100), (2000, 256)]


def reduce_both(cuda, oracle, op, A, dim, keepdim, view=None):
    res = {}
    for be in (cuda, oracle):
        ta = be.tensor(A)
        if view is not None:
            ta = view(ta)
        shape = ta.shape
        if dim == FULL_REDUCE:
            out_shape = [1]
        else:
            out_shape = [s for i, s in enumerate(shape) if i != dim] or [1]
            if keepdim:
                out_shape = [1 if i == dim else s for i, s in enumerate(shape)]
        out = be.empty(out_shape, dtype=INT32 if op == "argmax" else 1)
        be.forward(op, [ta], out, dim=dim, keepdim=int(keepdim))
        res[be.name] = (out.numpy(), out.shape)
    assert res["cuda"][1] == res["oracle"][1], "forward must rewrite the output shape like the CPU path"
    return res["cuda"][0], res["oracle"][0]


def abs_sum(A, dim):
    a = np.abs(A.astype(np.float64))
    return a.sum() if dim == FULL_REDUCE else a.sum(axis=dim)


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "argmax"])
@pytest.mark.parametrize("shape", REDUCE_SHAPES)
def test_reduce_all_axes(cuda, oracle, op, shape):
    A = rand_uniform(0, shape)
    for dim in list(range(len(shape))) + [FULL_REDUCE]:
        for keepdim in (False, True):
            got, want = reduce_both(cuda, oracle, op, A, dim, keepdim)
            what = f"{op}{shape} dim={dim} keepdim={keepdim}"
            if op in ("max", "min"):
                assert_bit_equal(got, want, what)
            elif op == "argmax":
                assert np.array_equal(got, want), what
            else:
                n = A.size if dim == FULL_REDUCE else shape[dim]
                scale = abs_sum(A, dim) / (n if op == "mean" else 1)
                assert_sum_close(got.reshape(-1), want.reshape(-1), np.asarray(scale).reshape(-1), what=what)


def test_empty_and_single_element_reductions(cuda, oracle):
    # nothing to reduce: the outputs hold the start value of the CPU loop
    for op, want in (("sum", 0.0), ("max", -np.finfo(np.float32).max), ("min", np.finfo(np.float32).max)):
        got, ref = reduce_both(cuda, oracle, op, np.zeros((4, 0), np.float32), 1, False)
        assert got.shape == (4,) and np.all(got == np.float32(want)) and np.array_equal(got, ref)
    got, _ = reduce_both(cuda, oracle, "mean", np.zeros((4, 0), np.float32), 1, False)
    assert np.all(np.isnan(got))
    # 0-dim and single-element tensors
    for shape in ((), (1,), (1, 1, 1)):
        A = np.float32(3.5).reshape(shape)
        for op in ("sum", "mean", "max", "min"):
            got, ref = reduce_both(cuda, oracle, op, A, FULL_REDUCE, False)
            assert got[0] == 3.5 == ref[0]


def test_full_argmax_of_views_counts_in_logical_order(cuda):
    A = rand_normal(5, (37, 53))
    A[11, 40] = 9.0
    tA = cuda.tensor(A)
    out = cuda.empty((1,), dtype=INT32)
    for view, ref in ((tA, A), (tA.transpose(0, 1), A.T)):
        cuda.forward("argmax", [view], out, dim=FULL_REDUCE)
        assert int(out.numpy()[0]) == int(np.argmax(ref))               # row-major index of the VIEW
    B = rand_normal(6, (5, 7, 9))
    B[3, 2, 8] = B[1, 6, 0] = 11.0                                        # a tie: lowest logical index wins
    tB = cuda.tensor(B)
    for perm in ((2, 0, 1), (1, 2, 0), (0, 2, 1)):
        st = [tB.strides[p] for p in perm]
        sh = [tB.shape[p] for p in perm]
        cuda.forward("argmax", [tB.view(sh, st)], out, dim=FULL_REDUCE)
        assert int(out.numpy()[0]) == int(np.argmax(B.transpose(perm))), perm


def test_argmax_ties_pick_lowest_index(cuda, oracle):
    A = np.zeros((64, 4096), np.float32)
    A[:, 100] = 5.0; A[:, 3000] = 5.0; A[:, 4095] = 5.0
    A[7, 5] = 5.0
    got, want = reduce_both(cuda, oracle, "argmax", A, 1, False)
    assert np.array_equal(got, want)
    assert got[7] == 5 and got[0] == 100
    got, want = reduce_both(cuda, oracle, "argmax", A, 0, False)     # every column ties at row 0..63
    assert np.array_equal(got, want)
    assert np.array_equal(got, np.argmax(A, axis=0).astype(np.int32))


@pytest.mark.parametrize("op", ["sum", "max", "argmax", "mean"])
def test_reduce_on_transposed_view(cuda, oracle, op):
    # config 4's layout in small: shape [M,N], strides [1,M], no copy
    A = rand_uniform(0, (96, 160))
    view = lambda t: t.transpose(0, 1)
    dims = [0, 1] + ([FULL_REDUCE] if op != "argmax" else [])
    for dim in dims:
        got, want = reduce_both(cuda, oracle, op, A, dim, False, view)
        if op == "max":
            assert_bit_equal(got, want, f"{op} dim {dim}")
        elif op == "argmax":
            assert np.array_equal(got, want)
        else:
            At = A.T
            n = At.size if dim == FULL_REDUCE else At.shape[dim]
            scale = abs_sum(At, dim) / (n if op == "mean" else 1)
            assert_sum_close(got.reshape(-1), want.reshape(-1), np.asarray(scale).reshape(-1))


def test_full_reduce_is_reproducible(cuda):
    A = rand_uniform(0, (1 << 22,))
    outs = []
    for _ in range(3):
        out = cuda.empty((1,))
        cuda.forward("sum", [cuda.tensor(A)], out, dim=FULL_REDUCE)
        outs.append(out.numpy())
    assert_bit_equal(outs[0], outs[1]); assert_bit_equal(outs[0], outs[2])
    np.testing.assert_allclose(outs[0][0], A.astype(np.float64).sum(), rtol=0, atol=1e-5 * np.abs(A).sum())


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
@pytest.mark.parametrize("shape,dim", [((7, 33), 1), ((7, 33), 0), ((7, 33), FULL_REDUCE),
                                       ((4, 5, 6), 1), ((300, 200), 1)])
def test_reduce_backward(cuda, oracle, op, shape, dim):
    A = np.round(rand_uniform(0, shape) * 4) / 4          # coarse grid -> plenty of ties for max/min
    D0 = rand_normal(1, shape)
    res = {}
    for be in (cuda, oracle):
        ta = be.tensor(A, requires_grad=True)
        ta.grad.copy_from(D0)
        out_shape = [1] if dim == FULL_REDUCE else ([s for i, s in enumerate(shape) if i != dim] or [1])
        out = be.empty(out_shape, requires_grad=True)
        be.forward(op, [ta], out, dim=dim)
        out.grad.copy_from(rand_normal(2, out_shape))
        be.backward(op, [ta], out, dim=dim)
        res[be.name] = ta.grad.numpy()
    np.testing.assert_allclose(res["cuda"], res["oracle"], rtol=1e-6, atol=1e-7)


def test_max_backward_tie_split(cuda):
    # the reference's CPU rule: gradient / number of ties (its CUDA kernel gives every tie the full grad)
    A = np.array([[1, 3, 3], [2, 2, 2]], np.float32)
    ta = cuda.tensor(A, requires_grad=True)
    out = cuda.empty((2,), requires_grad=True)
    cuda.forward("max", [ta], out, dim=1)
    out.grad.copy_from(np.ones(2, np.float32))
    cuda.backward("max", [ta], out, dim=1)
    np.testing.assert_allclose(ta.grad.numpy(), [[0, .5, .5], [1 / 3, 1 / 3, 1 / 3]], rtol=1e-7)


BCAST_GRAD = [((64, 48), (1, 48)), ((64, 48), (64, 1)), ((64, 48), ()), ((6, 8, 5, 5), (1, 8, 1, 1)),
              ((3, 1, 4), (1, 2, 1)), ((33, 7), (7,)), ((1024, 256), (1, 256)), ((5, 4, 3), (4, 1)),
              # enough (channel x batch) runs for the two-stage path: run sums, then a column sum
              ((64, 64, 16, 16), (1, 64, 1, 1)), ((70, 60, 8, 8), (60, 1, 1))]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("sa,sb", BCAST_GRAD)
def test_broadcast_gradient_reduce(cuda, oracle, op, sa, sb):
    out_shape = tuple(np.broadcast_shapes(sa, sb))
    A = rand_normal(0, sa)
    B = rand_uniform(1, sb, 0.5, 2.0) if sb else np.float32(1.25).reshape(())
    G = rand_normal(2, out_shape)
    DA, DB = rand_normal(3, sa), (rand_normal(4, sb) if sb else np.float32(0.5).reshape(()))
    res = {}
    for be in (cuda, oracle):
        ta, tb = be.tensor(A, requires_grad=True), be.tensor(B, requires_grad=True)
        ta.grad.copy_from(DA); tb.grad.copy_from(DB)
        out = be.empty(out_shape, requires_grad=True)
        out.grad.copy_from(G)
        be.backward(op, [ta, tb], out)
        res[be.name] = (ta.grad.numpy(), tb.grad.numpy())
    # scale of the accumulated terms, per gradient element
    Ab, Bb = np.broadcast_to(A, out_shape).astype(np.float64), np.broadcast_to(B, out_shape).astype(np.float64)
    terms_a = {"add": np.abs(G), "sub": np.abs(G), "mul": np.abs(G * Bb), "div": np.abs(G / Bb)}[op]
    terms_b = {"add": np.abs(G), "sub": np.abs(G), "mul": np.abs(G * Ab), "div": np.abs(G * Ab / (Bb * Bb))}[op]

    def fold(t, shape):
        t = t.astype(np.float64)
        lead = t.ndim - len(shape)
        t = t.sum(axis=tuple(range(lead))) if lead else t
        axes = tuple(i for i, s in enumerate(shape) if s == 1 and t.shape[i] != 1)
        return t.sum(axis=axes, keepdims=True).reshape(shape) if axes else t.reshape(shape)

    assert_sum_close(res["cuda"][0], res["oracle"][0], fold(terms_a, sa) + np.abs(DA), what=f"{op} da")
    assert_sum_close(res["cuda"][1], res["oracle"][1], fold(terms_b, sb) + np.abs(DB), what=f"{op} db")


@pytest.mark.parametrize("cluster,log_tx", [(2, 1), (4, 3), (8, 2), (8, 5), (3, 4)])
def test_column_reduce_combined_inside_a_cluster(cuda, oracle, cluster, log_tx):
    # The chunks of a strip as one thread-block cluster that combines through distributed shared
    # memory (forced through the tuning hook; by default only small inputs take this route). Shapes:
    # ragged chunks, fewer rows than CTAs in the cluster can use, an outer kept dim, a ragged strip.
    import plast_b200 as pb
    pb.lib.plast_b200_tune(0, log_tx)
    pb.lib.plast_b200_tune(10, cluster)
    try:
        for shape, dim in [((1024, 1024), 0), ((1001, 36), 0), ((9, 260), 0), ((5, 77, 128), 1), ((64, 8), 0)]:
            A = rand_uniform(3, shape)
            for op in ("sum", "mean", "max", "argmax"):
                got, want = reduce_both(cuda, oracle, op, A, dim, False)
                what = f"{op}{shape} dim={dim} cluster={cluster} log_tx={log_tx}"
                if op == "max":
                    assert_bit_equal(got, want, what)
                elif op == "argmax":
                    assert np.array_equal(got, want), what
                else:
                    scale = abs_sum(A, dim) / (shape[dim] if op == "mean" else 1)
                    assert_sum_close(got.reshape(-1), want.reshape(-1), np.asarray(scale).reshape(-1), what=what)
    finally:
        pb.lib.plast_b200_tune(0, -1)
        pb.lib.plast_b200_tune(10, -1)


def test_config1_backward_grad_b(cuda, oracle):
    # grad_b = sum_rows(G * (A + b > 0)): leaky_relu(0) backward followed by add backward
    A, b, G = rand_uniform(0, (1024, 1024)), rand_uniform(1, (1, 1024)), rand_normal(2, (1024, 1024))
    res = {}
    for be in (cuda, oracle):
        ta, tb = be.tensor(A), be.tensor(b, requires_grad=True)
        ab = be.empty((1024, 1024), requires_grad=True); be.forward("add", [ta, tb], ab)
        c = be.empty((1024, 1024), requires_grad=True); be.forward("leaky_relu", [ab], c, fval=0.0)
        c.grad.copy_from(G)
        be.backward("leaky_relu", [ab], c, fval=0.0)
        be.backward("add", [ta, tb], ab)
        res[be.name] = tb.grad.numpy()
    want64 = (G.astype(np.float64) * ((A + b) > 0)).sum(axis=0, keepdims=True)
    scale = np.abs(G * ((A + b) > 0)).sum(axis=0, keepdims=True)
    assert_sum_close(res["cuda"], res["oracle"], scale, what="grad_b vs oracle")
    assert_sum_close(res["cuda"], want64, scale, what="grad_b vs fp64")
    # fused node gives the same numbers
    ta, tb = cuda.tensor(A), cuda.tensor(b, requires_grad=True)
    c = cuda.empty((1024, 1024), requires_grad=True)
    cuda.forward("add_leaky_relu", [ta, tb], c, fval=0.0)
    c.grad.copy_from(G)
    cuda.backward("add_leaky_relu", [ta, tb], c, fval=0.0)
    assert_sum_close(tb.grad.numpy(), res["oracle"], scale, what="fused grad_b")


@pytest.mark.parametrize("shape", [(64, 4096), (33, 1000), (8, 10), (5, 16384), (3, 7, 128), (2, 9000),
                                   (1000, 10), (257, 7), (64, 64), (100, 33), (50, 2047), (3, 2049), (700, 1),
                                   (129, 16), (31, 260), (6, 50, 10), (2, 3, 5, 32), (513, 31), (3, 70000), (2, 50257), (3, 65536), (2, 40000), (7, 8196), (4, 12288),
                                   (64, 1001), (10, 8186), (33, 65), (5, 4095), (2, 3, 129), (40, 9)])
def test_softmax_log_softmax(cuda, recipes, shape):
    X = rand_normal(0, shape, std=2.0)
    for op, fn in (("softmax", recipes.softmax), ("log_softmax", recipes.log_softmax)):
        out = cuda.empty(shape)
        cuda.forward(op, [cuda.tensor(X)], out, dim=len(shape) - 1)
        got, want = out.numpy(), fn(X)
        if op == "softmax":
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-30)
        else:
            # log-probabilities: absolute error relative to the row's log-sum-exp scale
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_softmax_over_strided_axis(cuda, recipes):
    X = rand_normal(0, (40, 56), std=2.0)
    out = cuda.empty((40, 56))
    cuda.forward("softmax", [cuda.tensor(X)], out, dim=0)
    np.testing.assert_allclose(out.numpy(), recipes.softmax(X.T.copy()).T, rtol=1e-5)


@pytest.mark.parametrize("rows,cols", [(256, 4096), (100, 10), (37, 1000), (5000, 10), (300, 33), (64, 2047)])
def test_cross_entropy(cuda, recipes, rows, cols):
    X = rand_normal(0, (rows, cols), std=2.0)
    labels = np.random.RandomState(1).randint(0, cols, size=rows).astype(np.int32)
    out = cuda.empty((1,))
    cuda.forward("cross_entropy", [cuda.tensor(X), cuda.tensor(labels)], out)
    want, per_row = recipes.cross_entropy(X, labels)
    assert_sum_close(out.numpy(), want, np.abs(per_row).sum() / rows, what="ce mean")


@pytest.mark.parametrize("rows,cols", [(33, 200), (16, 4096), (5, 1003), (300, 64), (7, 8192), (100, 8), (9, 2048), (3, 8196), (2, 16384), (3, 9000),
                                       (5000, 10), (300, 7), (64, 31), (70, 33), (1000, 1)])
def test_softmax_family_backward(cuda, oracle, rows, cols):
    """Against the reference's OWN backward: the op sequence of plast/nn/functional.py run node by
    node through the CPU kernels, forward and then backward in reverse (harness.cpu_recipe_graph).
    The fused kernels evaluate the closed forms, so the bound is the fp32 accumulation bound of the
    row sums they contain: |gpu - cpu| <= 1e-5 * sum of the |terms| that make up the element."""
    from harness import cpu_recipe_graph
    X, G = rand_normal(0, (rows, cols)), rand_normal(1, (rows, cols))
    x64, g64 = X.astype(np.float64), G.astype(np.float64)
    p = np.exp(x64 - x64.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    scales = {"softmax": p * (np.abs(g64) + (np.abs(g64) * p).sum(1, keepdims=True)),
              "log_softmax": np.abs(g64) + p * np.abs(g64).sum(1, keepdims=True)}
    # The op sequence also sends a gradient through the row maximum (sub -> max backward): the sum
    # of the whole row's gradients, zero in exact arithmetic, lands on the argmax element with the
    # rounding of that sum, so that element's bound carries the row's terms as well.
    top = (np.arange(rows), X.argmax(axis=1))

    def with_max_path(scale):
        scale = scale.copy()
        scale[top] += scale.sum(axis=1)
        return scale
    scales = {k: with_max_path(v) for k, v in scales.items()}
    for op in ("softmax", "log_softmax"):
        _, want = cpu_recipe_graph(oracle, op, X, G)
        tx = cuda.tensor(X, requires_grad=True)
        out = cuda.empty((rows, cols), requires_grad=True)
        cuda.forward(op, [tx], out, dim=1)
        out.grad.copy_from(G)
        cuda.backward(op, [tx], out, dim=1)
        assert_sum_close(tx.grad.numpy(), want, scales[op], what=f"{op} backward vs the op-sequence backward")
        # and against the closed form in fp64
        closed = p * (g64 - (g64 * p).sum(1, keepdims=True)) if op == "softmax" else g64 - p * g64.sum(1, keepdims=True)
        assert_sum_close(tx.grad.numpy(), closed, scales[op], what=f"{op} backward vs fp64")
    labels = np.random.RandomState(2).randint(0, cols, size=rows).astype(np.int32)
    loss_want, want = cpu_recipe_graph(oracle, "cross_entropy", X, labels=labels)
    tx = cuda.tensor(X, requires_grad=True)
    out = cuda.empty((1,), requires_grad=True)
    cuda.forward("cross_entropy", [tx, cuda.tensor(labels)], out)
    np.testing.assert_allclose(out.numpy(), loss_want, rtol=1e-5)
    out.grad.copy_from(np.ones(1, np.float32))
    cuda.backward("cross_entropy", [tx, cuda.tensor(labels)], out)
    onehot = np.eye(cols)[labels]
    ce_scale = with_max_path((p + onehot) / rows)
    assert_sum_close(tx.grad.numpy(), want, ce_scale, what="cross-entropy backward vs the op-sequence backward")
    assert_sum_close(tx.grad.numpy(), (p - onehot) / rows, ce_scale, what="cross-entropy backward vs fp64")


def test_sigmoid_and_chain(cuda, recipes):
    n = 1 << 20
    X, Y = rand_normal(0, (n,)), rand_normal(1, (n,))
    out = cuda.empty((n,))
    cuda.forward("sigmoid", [cuda.tensor(X)], out)
    # exp is <= 2 ulp off glibc's: 1 + e carries up to 2 ulp of [1, 2), the reciprocal lies in
    # (0.5, 1] where an ulp is half as large: up to 4 ulp (also the measured worst case over the
    # 2^28 N(0,1) inputs of the benchmark's configuration 2)
    assert_ulp(out.numpy(), recipes.sigmoid(X), 4, "sigmoid")
    import plast_b200 as pb
    steps = [("neg", 0, 0, 0), ("exp", 2, 0, 0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
             ("mul", 5, 1, 0), ("abs", 0, 0, 0), ("neg", 7, 0, 0), ("exp", 8, 0, 0), ("add", 6, 9, 0)]
    z = cuda.empty((n,))
    pb.chain_forward([cuda.tensor(X), cuda.tensor(Y)], z, steps)
    assert pb.last_kernel() == "chain_precompiled"
    want = recipes.chain(X, Y)
    # z = t + e2 can cancel, so the bound is in ulps of the terms: each exp is <= 2 ulp off the
    # oracle's, which moves t and e2 by <= ~3 ulp each
    x64, y64 = X.astype(np.float64), Y.astype(np.float64)
    terms = np.abs(y64) / (1 + np.exp(-x64)) + np.exp(-np.abs(x64))
    # (measured worst case on the benchmark's 2^28 inputs: 2.69 in these units)
    assert (np.abs(z.numpy().astype(np.float64) - want) <= 3 * 2.0 ** -23 * terms).all(), "fused chain"
    # the same program with one step changed takes the interpreter and must agree with it
    steps2 = steps[:-1] + [("sub", 6, 9, 0)]
    z2 = cuda.empty((n,))
    pb.chain_forward([cuda.tensor(X), cuda.tensor(Y)], z2, steps2)
    # any other program is compiled at run time (NVRTC) or, without the compiler, interpreted
    assert pb.last_kernel() in ("chain_jit", "chain_interpreter")
    # unfused: the nine primitive entry points one after another give bit-identical results
    tx, ty = cuda.tensor(X), cuda.tensor(Y)
    t = [cuda.empty((n,)) for _ in range(9)]
    one = cuda.tensor(np.float32(1.0).reshape(()))
    cuda.forward("neg", [tx], t[0]); cuda.forward("exp", [t[0]], t[1]); cuda.forward("add", [t[1], one], t[2])
    cuda.forward("div", [one, t[2]], t[3]); cuda.forward("mul", [t[3], ty], t[4]); cuda.forward("abs", [tx], t[5])
    cuda.forward("neg", [t[5]], t[6]); cuda.forward("exp", [t[6]], t[7]); cuda.forward("add", [t[4], t[7]], t[8])
    assert_bit_equal(z.numpy(), t[8].numpy(), "fused chain vs nine separate launches")
    cuda.forward("sub", [t[4], t[7]], t[8])
    assert_bit_equal(z2.numpy(), t[8].numpy(), "generic chain vs separate launches")
    # broadcast input, scalar constants, odd length and a third input through the generic chain
    m = 1003
    A, Bv, Cv = rand_normal(2, (7, m)), rand_uniform(3, (1, m), 0.5, 2.0), rand_normal(4, (7, 1))
    prog = [("mul", 0, 1, 0), ("mul_scalar", 3, 0, 0.5), ("rsub_scalar", 4, 0, 2.0), ("leaky_relu", 5, 0, 0.1),
            ("div", 6, 1, 0), ("add", 7, 2, 0), ("sin", 8, 0, 0), ("cos", 9, 0, 0), ("log", 1, 0, 0), ("sub", 10, 11, 0)]
    zz = cuda.empty((7, m))
    ta, tb, tc = cuda.tensor(A), cuda.tensor(Bv), cuda.tensor(Cv)
    pb.chain_forward([ta, tb, tc], zz, prog)
    u = [cuda.empty((7, m)) for _ in range(10)]
    half, two = cuda.tensor(np.float32(0.5).reshape(())), cuda.tensor(np.float32(2.0).reshape(()))
    cuda.forward("mul", [ta, tb], u[0]); cuda.forward("mul", [u[0], half], u[1]); cuda.forward("sub", [two, u[1]], u[2])
    cuda.forward("leaky_relu", [u[2]], u[3], fval=0.1); cuda.forward("div", [u[3], tb], u[4]); cuda.forward("add", [u[4], tc], u[5])
    cuda.forward("sin", [u[5]], u[6]); cuda.forward("cos", [u[6]], u[7])
    lb = cuda.empty((1, m)); cuda.forward("log", [tb], lb); cuda.forward("sub", [u[7], lb], u[8])
    assert_bit_equal(zz.numpy(), u[8].numpy(), "10-step chain vs ten separate launches")


def test_scale_bias_relu_nchw(cuda, oracle):
    # config 5 in small: Y = relu(X * scale + bias), bias-grad = sum_{N,H,W} G * [Y > 0]
    shape, pshape = (6, 16, 14, 14), (1, 16, 1, 1)
    X, S, Bi, G = rand_normal(0, shape), rand_uniform(1, pshape, -.5, .5), rand_uniform(2, pshape, -.5, .5), rand_normal(3, shape)
    res = {}
    for be in (oracle,):
        tx, ts, tb = be.tensor(X, requires_grad=True), be.tensor(S, requires_grad=True), be.tensor(Bi, requires_grad=True)
        m = be.empty(shape, requires_grad=True); be.forward("mul", [tx, ts], m)
        u = be.empty(shape, requires_grad=True); be.forward("add", [m, tb], u)
        y = be.empty(shape, requires_grad=True); be.forward("leaky_relu", [u], y, fval=0.0)
        y.grad.copy_from(G)
        be.backward("leaky_relu", [u], y, fval=0.0); be.backward("add", [m, tb], u); be.backward("mul", [tx, ts], m)
        res = (y.numpy(), tx.grad.numpy(), ts.grad.numpy(), tb.grad.numpy())
    tx, ts, tb = cuda.tensor(X, requires_grad=True), cuda.tensor(S, requires_grad=True), cuda.tensor(Bi, requires_grad=True)
    y = cuda.empty(shape, requires_grad=True)
    cuda.forward("scale_bias_leaky_relu", [tx, ts, tb], y, fval=0.0)
    assert_bit_equal(y.numpy(), res[0], "fused epilogue forward")
    y.grad.copy_from(G)
    cuda.backward("scale_bias_leaky_relu", [tx, ts, tb], y, fval=0.0)
    mask = (res[0] > 0)
    assert_bit_equal(tx.grad.numpy(), res[1], "dx")
    assert_sum_close(ts.grad.numpy(), res[2], np.abs(G * mask * X).sum(axis=(0, 2, 3), keepdims=True), what="dscale")
    assert_sum_close(tb.grad.numpy(), res[3], np.abs(G * mask).sum(axis=(0, 2, 3), keepdims=True), what="dbias")


def test_helpers_fill_pack_view_grads(cuda):
    import ctypes as C
    import plast_b200 as pb
    t = cuda.tensor(rand_normal(0, (1001,)), requires_grad=True)
    pb.lib.ones_cuda(C.byref(t.c), 1001); assert np.all(t.numpy() == 1.0)
    pb.lib.zeros_cuda(C.byref(t.c), 1001); assert np.all(t.numpy() == 0.0)
    pb.lib.set_ones_grad_cuda(C.byref(t.c)); assert np.all(t.grad.numpy() == 1.0)
    pb.lib.zero_grad_cuda(C.byref(t.c)); assert np.all(t.grad.numpy() == 0.0)
    ti = cuda.empty((7,), dtype=INT32)
    pb.lib.ones_cuda(C.byref(ti.c), 7); assert np.all(ti.numpy() == 1)
    A = rand_normal(1, (19, 23))
    ta = cuda.tensor(A)
    dst = cuda.empty((23, 19))
    pb.lib.plast_b200_pack(C.byref(ta.transpose(0, 1).c), dst.c.data); pb.check_error()
    assert_bit_equal(dst.numpy(), A.T.copy(), "pack of a transposed view")
    # reshape / transpose gradient accumulation
    da0, dout = rand_normal(2, (19, 23)), rand_normal(3, (19, 23))
    da = cuda.tensor(da0); do = cuda.tensor(dout)
    pb.lib.reshape_backward_cuda(da.c.data, do.c.data, 19 * 23); pb.check_error()
    assert_bit_equal(da.numpy(), da0 + dout)
    dout_t = rand_normal(4, (23, 19))
    da = cuda.tensor(da0); do = cuda.tensor(dout_t)
    u64x = lambda v: (C.c_uint64 * len(v))(*v)
    pb.lib.transpose_backward_cuda(da.c.data, do.c.data, u64x([19, 23]), u64x([23, 1]), u64x([19, 1]), 2, 0, 1, 19 * 23)
    pb.check_error()
    assert_bit_equal(da.numpy(), da0 + dout_t.T)
