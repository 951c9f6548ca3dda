"""Pins the CPU oracle (oracle/oracle.c) to the reference:

  * against tests/golden/hotpath.npz, recorded from the reference's own CPU kernels
    (tests/golden/make_golden.py), always;
  * live against oracle/_ref/libplast_ref.so (the reference's CPU sources compiled by
    oracle/Makefile) on more shapes, wherever that build is present.

Rules: elementwise arithmetic, relu, max/min and the sequential sums/means must match the
reference BITWISE (the oracle restates the same accumulation order); libm transcendentals may
differ by 1 ulp between machines (glibc picks FMA / non-FMA variants by CPU); the broadcast
backward of the reference accumulates with `omp atomic` in thread order, so it is compared with
the scaled bound |a - b| <= 1e-5 * sum|terms|.
"""
import numpy as np
import pytest

from golden_cases import cases, run_case
from harness import (FULL_REDUCE, GOLDEN_DIR, OracleRecipes, assert_bit_equal, assert_ulp, rand_normal,
                     rand_uniform)

GOLDEN = np.load(GOLDEN_DIR / "hotpath.npz")
CASES = cases()


def compare(got, want, rule, what):
    if rule == "bits":
        assert_bit_equal(got, want, what)
    elif rule == "values":
        assert np.array_equal(got, want), what
    elif rule in ("ulp2",):
        assert_ulp(got, want, 1, what)
    elif rule == "sum":
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5, err_msg=what)
    else:  # "grad": also covers broadcast reductions, whose reference order is thread-dependent
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-5 * (np.abs(want).max() + 1), err_msg=what)


def test_golden_file_covers_every_case():
    names = {k.split("/")[0] for k in GOLDEN.files}
    assert names == {c["name"] for c in CASES}


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_golden(oracle, case):
    res = run_case(oracle, case)
    for key, got in res.items():
        want = GOLDEN[f"{case['name']}/{key}"]
        if key == "out_shape":
            assert list(got) == list(want), "forward must rewrite the output shape like the reference"
            continue
        rule = case["exact"]
        if key == "out" and case["backward"]:
            rule = "bits" if case["op"] in ("add", "sub", "mul", "div", "max", "min", "abs", "leaky_relu") else \
                ("values" if case["op"] == "neg" else ("ulp2" if case["op"] in ("exp", "log", "sin", "cos", "tan") else "sumseq"))
        if key == "out" and rule in ("sum", "sumseq") and case["op"] in ("sum", "mean"):
            assert_bit_equal(got, want, f"{case['name']}: sequential fp32 accumulation order")
            continue
        compare(got, want, rule, f"{case['name']}/{key}")


LIVE_SHAPES = [(5,), (3, 7), (2, 5, 3), (1, 9), (9, 1), (4, 1, 6), (2, 2, 2, 2, 3), (257, 3), (3, 257)]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_live_binary_vs_reference_build(oracle, ref, op):
    for i, sa in enumerate(LIVE_SHAPES):
        for sb in (sa, (1,) * len(sa), sa[-1:], ()):
            A, B = rand_normal(i, sa), (rand_uniform(i + 50, sb, 0.5, 2) if sb else np.float32(2.0).reshape(()))
            outs = []
            for be in (oracle, ref):
                out = be.empty(np.broadcast_shapes(sa, sb))
                be.forward(op, [be.tensor(A), be.tensor(B)], out)
                outs.append(out.numpy())
            assert_bit_equal(outs[0], outs[1], f"{op} {sa} {sb}")


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
def test_live_reduce_vs_reference_build(oracle, ref, op):
    for i, shape in enumerate(LIVE_SHAPES):
        A = rand_uniform(i, shape)
        for dim in list(range(len(shape))) + [FULL_REDUCE]:
            for keepdim in (0, 1):
                for transposed in (False, True):
                    if transposed and len(shape) < 2:
                        continue
                    outs = []
                    for be in (oracle, ref):
                        t = be.tensor(A)
                        if transposed:
                            t = t.transpose(0, len(shape) - 1)
                        out = be.empty([max(A.size, 1)])
                        be.forward(op, [t], out, dim=dim, keepdim=keepdim)
                        n = 1 if dim == FULL_REDUCE else A.size // t.shape[dim]
                        outs.append((out.storage()[:n].copy(), out.shape))
                    assert_bit_equal(outs[0][0], outs[1][0], f"{op} {shape} dim {dim} T={transposed}")
                    if dim != FULL_REDUCE:
                        assert outs[0][1] == outs[1][1]


def test_live_relu_negative_zero(oracle, ref):
    A = rand_uniform(0, (1024, 1024))
    outs = []
    for be in (oracle, ref):
        out = be.empty(A.shape)
        be.forward("leaky_relu", [be.tensor(A)], out, fval=0.0)
        outs.append(out.numpy())
    assert_bit_equal(outs[0], outs[1])
    assert int((np.signbit(outs[0]) & (outs[0] == 0)).sum()) == int((A < 0).sum())


def test_recipes_equal_the_primitive_chains(ref):
    """softmax / log_softmax / cross_entropy / sigmoid / the 9-op chain of oracle.c, against the
    same op sequences run through the reference's primitive CPU kernels
    (plast/nn/functional.py:42-47, 77-97, 312-333)."""
    rec = OracleRecipes()
    X = rand_normal(0, (33, 130), std=2.0)
    tx = ref.tensor(X)
    m = ref.empty((33, 1)); ref.forward("max", [tx], m, dim=1, keepdim=1)
    sh = ref.empty(X.shape); ref.forward("sub", [tx, m], sh)
    e = ref.empty(X.shape); ref.forward("exp", [sh], e)
    s = ref.empty((33, 1)); ref.forward("sum", [e], s, dim=1, keepdim=1)
    y = ref.empty(X.shape); ref.forward("div", [e, s], y)
    assert_ulp(rec.softmax(X), y.numpy(), 1, "softmax")
    ls = ref.empty((33, 1)); ref.forward("log", [s], ls)
    ly = ref.empty(X.shape); ref.forward("sub", [sh, ls], ly)
    np.testing.assert_allclose(rec.log_softmax(X), ly.numpy(), rtol=0, atol=2e-6)
    labels = np.random.RandomState(1).randint(0, 130, size=33).astype(np.int32)
    onehot = np.zeros(X.shape, np.float32); onehot[np.arange(33), labels] = 1.0
    prod = ref.empty(X.shape); ref.forward("mul", [ref.tensor(onehot), ly], prod)
    rs = ref.empty((33,)); ref.forward("sum", [prod], rs, dim=1)
    neg = ref.empty((33,)); ref.forward("neg", [rs], neg)
    mean = ref.empty((1,)); ref.forward("mean", [neg], mean, dim=FULL_REDUCE)
    got_mean, got_rows = rec.cross_entropy(X, labels)
    np.testing.assert_allclose(got_rows, neg.numpy(), rtol=0, atol=2e-6)
    np.testing.assert_allclose(got_mean, mean.numpy(), rtol=1e-6)
    # sigmoid and the 9-op chain
    n = 10007
    xv, yv = rand_normal(2, (n,)), rand_normal(3, (n,))
    one = ref.tensor(np.float32(1.0).reshape(()))
    t = [ref.empty((n,)) for _ in range(9)]
    tx, ty = ref.tensor(xv), ref.tensor(yv)
    ref.forward("neg", [tx], t[0]); ref.forward("exp", [t[0]], t[1]); ref.forward("add", [t[1], one], t[2])
    ref.forward("div", [one, t[2]], t[3])
    assert_ulp(rec.sigmoid(xv), t[3].numpy(), 1, "sigmoid")
    ref.forward("mul", [t[3], ty], t[4]); ref.forward("abs", [tx], t[5]); ref.forward("neg", [t[5]], t[6])
    ref.forward("exp", [t[6]], t[7]); ref.forward("add", [t[4], t[7]], t[8])
    assert_ulp(rec.chain(xv, yv), t[8].numpy(), 1, "9-op chain")
