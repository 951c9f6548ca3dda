"""Fused DAGs against the same DAGs run node by node, on the GPU: the graph fusion pass must
change how many kernels run, never what they compute."""
import numpy as np
import pytest

import plast_b200 as pb
from plast_b200 import graph as G
from harness import OracleRecipes, assert_bit_equal, assert_sum_close, rand_normal, rand_uniform

pytestmark = pytest.mark.gpu


def launches(fn):
    before = pb.lib.plast_b200_launch_count()
    fn()
    pb.check_error()
    return pb.lib.plast_b200_launch_count() - before


def build_config2_chain(cuda, x, y):
    tx, ty = cuda.tensor(x), cuda.tensor(y)
    one_a, one_b = cuda.tensor(np.float32(1.0).reshape(())), cuda.tensor(np.float32(1.0).reshape(()))
    t = [cuda.empty(x.shape) for _ in range(9)]
    g = G.Graph()
    g.node("NEG", [tx], t[0]); g.node("EXP", [t[0]], t[1]); g.node("ADD", [one_a, t[1]], t[2])
    g.node("DIV", [one_b, t[2]], t[3]); g.node("MUL", [t[3], ty], t[4])
    g.node("ABS", [tx], t[5]); g.node("NEG", [t[5]], t[6]); g.node("EXP", [t[6]], t[7])
    g.node("ADD", [t[4], t[7]], t[8])
    return g, t[8]


@pytest.mark.parametrize("shape", [(1 << 22,), (1000003,), (37, 129, 5)])
def test_config2_chain_one_launch_bitwise_equal_to_nine(cuda, shape):
    x, y = rand_normal(0, shape), rand_normal(1, shape)
    g, out = build_config2_chain(cuda, x, y)
    dag = g.dag()
    n_unfused = launches(lambda: G.dag_forward(dag))
    want = out.numpy().copy()
    g2, out2 = build_config2_chain(cuda, x, y)
    dag2 = g2.dag()
    assert G.fuse(dag2) == 1 and dag2.count == 1
    G.dag_forward(dag2); pb.check_error()                                 # first run compiles the program
    n_fused = launches(lambda: G.dag_forward(dag2))
    assert_bit_equal(out2.numpy(), want, "fused chain node vs nine nodes")
    assert n_unfused >= 9 and n_fused <= 2                                # body (+ tail for odd lengths)
    assert pb.last_kernel() in ("chain_jit", "chain_interpreter")
    np.testing.assert_allclose(want, OracleRecipes().chain(x.ravel(), y.ravel()).reshape(shape), rtol=3e-6, atol=1e-6)


@pytest.mark.parametrize("kind", ["softmax", "log_softmax"])
def test_softmax_recipes_fused_match_the_node_by_node_run(cuda, kind):
    X = rand_normal(3, (257, 1000), std=2.0)
    Gup = rand_normal(4, (257, 1000))

    def build():
        x = cuda.tensor(X, requires_grad=True)
        mx, se = cuda.empty((257, 1), requires_grad=True), cuda.empty((257, 1), requires_grad=True)
        sh, ex, out = (cuda.empty(X.shape, requires_grad=True) for _ in range(3))
        g = G.Graph()
        g.node("MAX", [x], mx, dim=1, keepdim=1); g.node("SUB", [x, mx], sh); g.node("EXP", [sh], ex)
        g.node("SUM", [ex], se, dim=1, keepdim=1)
        if kind == "softmax":
            g.node("DIV", [ex, se], out)
        else:
            lg = cuda.empty((257, 1), requires_grad=True)
            g.node("LOG", [se], lg); g.node("SUB", [sh, lg], out)
        return g, x, out

    g, x, out = build()
    dag = g.dag()
    G.dag_forward(dag); pb.check_error()
    out.grad.copy_from(Gup)
    G.dag_backward(dag); pb.check_error()
    want, want_dx = out.numpy().copy(), x.grad.numpy().copy()

    g, x, out = build()
    dag = g.dag()
    assert G.fuse(dag) == 1 and dag.count == 1
    assert launches(lambda: G.dag_forward(dag)) == 1
    out.grad.copy_from(Gup)
    assert launches(lambda: G.dag_backward(dag)) == 1
    np.testing.assert_allclose(out.numpy(), want, rtol=2e-6, atol=1e-7)
    scale = np.abs(Gup).sum(axis=1, keepdims=True) * np.ones_like(X)
    assert_sum_close(x.grad.numpy(), want_dx, scale, what=f"{kind} dx through the fused node")


def test_config1_training_graph_fused_epilogue_forward_and_backward(cuda):
    A, b, Gup = rand_uniform(0, (1024, 1024)), rand_uniform(1, (1, 1024)), rand_normal(2, (1024, 1024))

    def build():
        ta, tb = cuda.tensor(A), cuda.tensor(b, requires_grad=True)
        ab, c = cuda.empty(A.shape, requires_grad=True), cuda.empty(A.shape, requires_grad=True)
        s = cuda.empty((1024,), requires_grad=True)
        g = G.Graph()
        g.node("ADD", [ta, tb], ab); g.node("LEAKY_RELU", [ab], c, fval=0.0); g.node("SUM", [c], s, dim=1)
        return g, tb, c, s

    res = []
    for fused in (False, True):
        g, tb, c, s = build()
        dag = g.dag()
        if fused:
            assert G.fuse(dag) == 1 and dag.count == 2
        n_fwd = launches(lambda: G.dag_forward(dag))
        c.grad.copy_from(Gup)
        # backward from C: the row-sum node is skipped so that only the upstream gradient on C counts
        bwd = dag.nodes[0].contents if fused else None
        if fused:
            G.lib.add_leaky_relu_cuda_backward(bwd.inputs, bwd.output, bwd.params)
        else:
            for i in (1, 0):
                n = dag.nodes[i].contents
                name = "leaky_relu" if i == 1 else "add"
                getattr(G.lib, f"{name}_cuda_backward")(n.inputs, n.output, n.params)
        pb.check_error()
        res.append((c.numpy().copy(), s.numpy().copy(), tb.grad.numpy().copy(), n_fwd))
    assert_bit_equal(res[1][0], res[0][0], "relu(A + b)")
    assert_bit_equal(res[1][1], res[0][1], "row sums")
    assert res[1][3] == res[0][3] - 1
    scale = np.abs(Gup).sum(axis=0, keepdims=True)
    assert_sum_close(res[1][2], res[0][2], scale, what="grad_b through the fused node")


def test_config5_epilogue_graph_fuses_to_scale_bias_relu(cuda):
    shape, p = (8, 64, 28, 28), (1, 64, 1, 1)
    X, S, B = rand_normal(0, shape), rand_uniform(1, p, -.5, .5), rand_uniform(2, p, -.5, .5)
    Gup = rand_normal(3, shape)
    res = []
    for fused in (False, True):
        x, sc, bi = cuda.tensor(X), cuda.tensor(S, requires_grad=True), cuda.tensor(B, requires_grad=True)
        t, u, y = (cuda.empty(shape, requires_grad=True) for _ in range(3))
        g = G.Graph()
        g.node("MUL", [x, sc], t); g.node("ADD", [t, bi], u); g.node("LEAKY_RELU", [u], y, fval=0.0)
        dag = g.dag()
        if fused:
            assert G.fuse(dag) == 1 and dag.count == 1
        G.dag_forward(dag); pb.check_error()
        y.grad.copy_from(Gup)
        G.dag_backward(dag); pb.check_error()
        res.append((y.numpy().copy(), sc.grad.numpy().copy(), bi.grad.numpy().copy()))
    assert_bit_equal(res[1][0], res[0][0], "relu(X * scale + bias)")
    gscale = np.abs(Gup).sum(axis=(0, 2, 3), keepdims=True)
    assert_sum_close(res[1][2], res[0][2], gscale, what="bias grad")
    assert_sum_close(res[1][1], res[0][1], np.abs(Gup * X).sum(axis=(0, 2, 3), keepdims=True), what="scale grad")


def test_chain_with_eight_operands_and_constants_in_every_position(cuda):
    shape = (33, 1025)
    xs = [rand_normal(10 + i, shape) for i in range(5)]
    consts = [np.float32(v).reshape(()) for v in (0.5, -1.25, 3.0)]
    res = []
    for fused in (False, True):
        tx = [cuda.tensor(x) for x in xs]
        tc = [cuda.tensor(c) for c in consts]
        t = [cuda.empty(shape) for _ in range(7)]
        g = G.Graph()
        g.node("MUL", [tc[0], tx[0]], t[0]); g.node("ADD", [t[0], tx[1]], t[1]); g.node("SUB", [t[1], tc[1]], t[2])
        g.node("MUL", [t[2], tx[2]], t[3]); g.node("DIV", [t[3], tc[2]], t[4]); g.node("ADD", [t[4], tx[3]], t[5])
        g.node("SUB", [tx[4], t[5]], t[6])
        dag = g.dag()
        if fused:
            assert G.fuse(dag) == 1 and dag.count == 1 and dag.nodes[0].contents.num_inputs == 8
        G.dag_forward(dag); pb.check_error()
        res.append(t[6].numpy().copy())
    assert_bit_equal(res[1], res[0], "eight-operand chain")
    want = xs[4] - (((np.float32(0.5) * xs[0] + xs[1]) - np.float32(-1.25)) * xs[2] / np.float32(3.0) + xs[3])
    assert_bit_equal(res[1], want.astype(np.float32), "eight-operand chain vs numpy")


def build_training_chain(cuda, x, y, bias):
    """z = sigmoid(x) * y + exp(-abs(x)) + bias as ten nodes; x, y and the bias row require grad."""
    tx, ty = cuda.tensor(x, requires_grad=True), cuda.tensor(y, requires_grad=True)
    tb = cuda.tensor(bias, requires_grad=True)
    one_a, one_b = cuda.tensor(np.float32(1.0).reshape(())), cuda.tensor(np.float32(1.0).reshape(()))
    t = [cuda.empty(x.shape, requires_grad=True) for _ in range(10)]
    g = G.Graph()
    g.node("NEG", [tx], t[0]); g.node("EXP", [t[0]], t[1]); g.node("ADD", [one_a, t[1]], t[2])
    g.node("DIV", [one_b, t[2]], t[3]); g.node("MUL", [t[3], ty], t[4])
    g.node("ABS", [tx], t[5]); g.node("NEG", [t[5]], t[6]); g.node("EXP", [t[6]], t[7])
    g.node("ADD", [t[4], t[7]], t[8]); g.node("ADD", [t[8], tb], t[9])
    return g, tx, ty, tb, t[9]


needs_jit = pytest.mark.skipif(not pb.lib.plast_b200_chain_jit_available(),
                               reason="the chain backward needs the run-time compiler")


@needs_jit
@pytest.mark.parametrize("shape", [(64, 1000), (7, 33), (1 << 20,)])
def test_training_chain_fused_backward_equals_node_by_node_backward(cuda, shape):
    x, y = rand_normal(0, shape), rand_normal(1, shape)
    bias = rand_normal(2, (1,) * (len(shape) - 1) + shape[-1:]) if len(shape) > 1 else rand_normal(2, (1,))
    gup = rand_normal(3, shape)
    res = []
    for fused in (False, True):
        g, tx, ty, tb, out = build_training_chain(cuda, x, y, bias)
        dag = g.dag()
        if fused:
            assert G.fuse(dag, G.FUSE_CHAINS_WITH_GRAD) == 1 and dag.count == 1
        G.dag_forward(dag); pb.check_error()
        out.grad.copy_from(gup)
        n_bwd = launches(lambda: G.dag_backward(dag))
        res.append((out.numpy().copy(), tx.grad.numpy().copy(), ty.grad.numpy().copy(), tb.grad.numpy().copy(), n_bwd))
    assert_bit_equal(res[1][0], res[0][0], "forward")
    assert_bit_equal(res[1][1], res[0][1], "x.grad: two contributions, applied in the node order")
    assert_bit_equal(res[1][2], res[0][2], "y.grad")
    red_axes = tuple(range(len(shape) - 1)) if len(shape) > 1 else (0,)
    assert_sum_close(res[1][3], res[0][3], np.abs(gup).sum(axis=red_axes, keepdims=True).reshape(res[0][3].shape),
                     what="bias.grad (reduced over the broadcast dims)")
    assert res[1][4] < res[0][4]                                          # fewer launches than ten backward nodes
    # and against float64 calculus
    x64, y64, g64 = x.astype(np.float64), y.astype(np.float64), gup.astype(np.float64)
    sg = 1 / (1 + np.exp(-x64))
    dx = g64 * (sg * (1 - sg) * y64 - np.sign(x64) * np.exp(-np.abs(x64)))
    np.testing.assert_allclose(res[1][1], dx, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(res[1][2], g64 * sg, rtol=2e-5, atol=2e-6)


@needs_jit
def test_chain_backward_entry_point_with_scalar_opcodes_and_accumulation(cuda):
    n = 4099
    x = rand_uniform(0, (n,), 0.5, 2.0)
    gup = rand_normal(1, (n,))
    steps = [("mul_scalar", 0, 0, 3.0), ("add_scalar", 1, 0, 0.5), ("rdiv_scalar", 2, 0, 2.0), ("rsub_scalar", 3, 0, 1.0),
             ("log", 2, 0, 0.0), ("mul", 4, 5, 0.0)]                        # (1 - 2 / (3x + .5)) * log(3x + .5)
    tx = cuda.tensor(x, requires_grad=True)
    tx.grad.copy_from(np.full(n, 0.25, np.float32))                       # accumulates on top of this
    out = cuda.empty((n,), requires_grad=True)
    pb.chain_forward([tx], out, steps)
    out.grad.copy_from(gup)
    pb.chain_backward([tx], out, steps)
    assert pb.last_kernel() == "chain_backward_jit"
    u = 3 * x.astype(np.float64) + 0.5
    want = 0.25 + gup * 3 * (2 / u ** 2 * np.log(u) + (1 - 2 / u) / u)
    np.testing.assert_allclose(tx.grad.numpy(), want, rtol=2e-5, atol=2e-6)


def test_fused_dag_replayed_as_one_cuda_graph(cuda):
    A, b = rand_uniform(0, (1024, 1024)), rand_uniform(1, (1, 1024))
    ta, tb = cuda.tensor(A), cuda.tensor(b, requires_grad=True)
    ab, c = cuda.empty(A.shape, requires_grad=True), cuda.empty(A.shape, requires_grad=True)
    s = cuda.empty((1024,), requires_grad=True)
    g = G.Graph()
    g.node("ADD", [ta, tb], ab); g.node("LEAKY_RELU", [ab], c, fval=0.0); g.node("SUM", [c], s, dim=1)
    dag = g.dag()
    assert G.fuse(dag) == 1 and dag.count == 2
    G.dag_forward(dag); pb.check_error()
    handle = G.capture(dag); pb.check_error()
    assert handle and G.lib.plast_b200_dag_graph_kernels(handle) == 2
    # new data in the same buffers: the replay computes on it
    A2 = rand_uniform(5, (1024, 1024))
    ta.copy_from(A2)
    assert launches(lambda: G.replay(handle)) == 2
    want_c = np.where(A2 + b > 0, A2 + b, (A2 + b) * np.float32(0.0))
    assert_bit_equal(c.numpy(), want_c.astype(np.float32), "C from the replayed graph")
    G.dag_forward(dag); pb.check_error()
    eager = s.numpy().copy()
    G.replay(handle); pb.check_error()
    assert_bit_equal(s.numpy(), eager, "row sums: replay vs eager")
    # backward recorded without being run, then replayed
    Gup = rand_normal(2, (1024, 1024))
    bwd = G.Graph(); bwd.nodes = [dag.nodes[0].contents]                 # the fused add + relu node only
    bdag = bwd.dag()
    hb = G.capture(bdag, backward=True); pb.check_error()
    c.grad.copy_from(Gup)
    assert np.all(tb.grad.numpy() == 0)                                   # capturing did not execute anything
    G.replay(hb); pb.check_error()
    got = tb.grad.numpy().copy()
    tb.grad.copy_from(np.zeros_like(got))
    G.dag_backward(bdag); pb.check_error()
    assert_bit_equal(got, tb.grad.numpy(), "grad_b: replayed backward vs eager backward")
    G.lib.plast_b200_dag_graph_release(handle); G.lib.plast_b200_dag_graph_release(hb)


def test_capture_refuses_nodes_that_are_not_this_librarys_kernels(cuda):
    import ctypes as C
    x, y = cuda.tensor(rand_normal(0, (16,))), cuda.empty((16,))
    g = G.Graph()
    n = g.node("EXP", [x], y)
    n.op.cuda_forward = C.cast(C.CDLL(None).abs, C.c_void_p).value       # some function of another library
    dag = g.dag()
    assert G.capture(dag) is None
    assert pb.lib.plast_b200_last_error() == 5
    pb.lib.plast_b200_clear_error()
