"""The five benchmark configurations EXACTLY as stated (shapes, distributions, seeds), every op of
each, compared with the CPU checker on the same inputs at full size:

  1  A[1024,1024] ~ U(-1,1) seed 0, b[1,1024] ~ U(-1,1) seed 1, G ~ N(0,1) seed 2
  2  x, y ~ N(0,1) seeds 0, 1, 2^28 elements; z = sigmoid(x) * y + exp(-abs(x))
  3  X[65536,4096] ~ N(0,2) seed 0, labels ~ U[0,4096) seed 1
  4  X[8192,8192] ~ U(-1,1) seed 0 and its transposed view
  5  X[256,256,56,56] ~ N(0,1) seed 0, scale / bias [1,256,1,1] ~ U(-.5,.5) seeds 1, 2, G ~ N(0,1) seed 3

The checker is the reference's own CPU kernels compiled from its sources (oracle/_ref) where that
build is present, the C restatement (oracle/oracle.c) otherwise; the op sequences are the ones
plast/nn/functional.py builds (24-47, 77-97, 312-333).

Bounds (the benchmark's): bit-exact for add, mul, div, abs, neg, relu, max, argmax; <= 2 ulp for
exp / log; |gpu - cpu| <= 1e-5 * sum|terms| for sums, means and gradient reductions (the CPU adds
left to right, the GPU as a tree; the reference's own broadcast-gradient order is whatever its
atomics give); relative 1e-5 for softmax / log-softmax outputs and the cross-entropy mean. sigmoid
and the nine-op chain are compositions: exp within 2 ulp of glibc's moves 1/(1+e) by up to 4 ulp,
and z = t + e2 can cancel, so their bounds are the measured worst cases stated at the asserts
(sigmoid 4 ulp; chain 3 * 2^-23 * (|t| + |e2|)).

Every test records the largest error it saw; the last test prints the table (and leaves it as
parity_table.json in the run's output folder when that can be written).
"""
import json
import os
import time
from pathlib import Path

import numpy as np
import pytest

import plast_b200 as pb
from harness import FULL_REDUCE, INT32, have_ref, ulp_distance

pytestmark = pytest.mark.gpu

REPORT = {}          # (config, op) -> {"bound": ..., "worst": ..., "unit": ...}
CHUNK = 1 << 24


def record(config, op, worst, bound, unit):
    REPORT[f"{config}:{op}"] = {"config": config, "op": op, "worst": float(worst), "bound": bound, "unit": unit}


@pytest.fixture(scope="module")
def cpu(request):
    """The reference's own CPU kernels where built, else the restatement."""
    return request.getfixturevalue("ref" if have_ref() else "oracle")


def host(cpu, arr, requires_grad=False):
    """CPU-side tensor over `arr` without a copy."""
    arr = np.ascontiguousarray(arr)
    t = pb.Tensor.wrap_pointer(arr.ctypes.data, arr.shape, device="cpu",
                               dtype=INT32 if arr.dtype == np.int32 else pb.FLOAT32, owner=None)
    t._keep = arr
    if requires_grad:
        t.attach_grad()
    return t


def host_empty(shape, requires_grad=False):
    return pb.Tensor(shape, device="cpu", requires_grad=requires_grad)


def host_values(t, shape):
    """The contiguous result of a CPU op as a numpy view (no copy)."""
    n = int(np.prod(shape))
    import ctypes as C
    return np.ctypeslib.as_array(C.cast(t.c.data, C.POINTER(C.c_float)), shape=(n,)).reshape(shape)


def bits_differ(got, want):
    """Number of elements whose bit patterns differ (NaN payloads aside), chunked."""
    g, w = got.reshape(-1), want.reshape(-1)
    bad = 0
    for i in range(0, g.size, CHUNK):
        a, b = g[i:i + CHUNK], w[i:i + CHUNK]
        d = a.view(np.uint32) != b.view(np.uint32)
        d &= ~(np.isnan(a) & np.isnan(b))
        bad += int(d.sum())
    return bad


def values_differ(got, want):
    g, w = got.reshape(-1), want.reshape(-1)
    return sum(int((g[i:i + CHUNK] != w[i:i + CHUNK]).sum()) for i in range(0, g.size, CHUNK))


def max_ulp(got, want):
    g, w = got.reshape(-1), want.reshape(-1)
    worst = 0
    for i in range(0, g.size, CHUNK):
        worst = max(worst, int(ulp_distance(g[i:i + CHUNK], w[i:i + CHUNK]).max()))
    return worst


def max_rel(got, want):
    g, w = got.reshape(-1), want.reshape(-1)
    worst = 0.0
    for i in range(0, g.size, CHUNK):
        a, b = g[i:i + CHUNK].astype(np.float64), w[i:i + CHUNK].astype(np.float64)
        worst = max(worst, float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-30))))
    return worst


def scaled_err(got, want, abs_terms):
    """max |got - want| / sum|terms| (the fp32 accumulation bound is 1e-5 of it)."""
    e = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    return float(np.max(e / np.maximum(np.asarray(abs_terms, np.float64), 1e-300)))


# ---- config 1 ----------------------------------------------------------------------------------------
def test_config1_forward_and_grad_b(cuda, cpu):
    rs = np.random.RandomState
    A = rs(0).uniform(-1, 1, (1024, 1024)).astype(np.float32)
    b = rs(1).uniform(-1, 1, (1, 1024)).astype(np.float32)
    G = rs(2).randn(1024, 1024).astype(np.float32)
    res = {}
    for be in (cuda, cpu):
        ta, tb = be.tensor(A), be.tensor(b, requires_grad=True)
        ab = be.empty(A.shape, requires_grad=True); be.forward("add", [ta, tb], ab)
        c = be.empty(A.shape, requires_grad=True); be.forward("leaky_relu", [ab], c, fval=0.0)
        s = be.empty((1024,)); be.forward("sum", [c], s, dim=1)
        c.grad.copy_from(G)
        be.backward("leaky_relu", [ab], c, fval=0.0)
        be.backward("add", [ta, tb], ab)
        res[be.device] = (ab.numpy(), c.numpy(), s.numpy(), tb.grad.numpy())
    g, w = res["cuda"], res["cpu"]
    assert bits_differ(g[0], w[0]) == 0; record(1, "add (broadcast)", 0, "bit-exact", "elements differing")
    assert bits_differ(g[1], w[1]) == 0; record(1, "relu (incl. -0.0)", 0, "bit-exact", "elements differing")
    e = scaled_err(g[2], w[2], np.abs(w[1]).sum(axis=1)); assert e <= 1e-5
    record(1, "row sum", e, 1e-5, "|gpu-cpu| / sum|x|")
    e = scaled_err(g[3], w[3], np.abs(G * (w[1] > 0)).sum(axis=0, keepdims=True)); assert e <= 1e-5
    record(1, "grad_b (broadcast-gradient reduce)", e, 1e-5, "|gpu-cpu| / sum|terms|")
    # the fused entry points give the same C, s and grad_b
    import ctypes as C
    ta, tb = cuda.tensor(A), cuda.tensor(b, requires_grad=True)
    c, s = cuda.empty(A.shape, requires_grad=True), cuda.empty((1024,))
    pb.lib.plast_b200_add_leaky_relu_row_sum(C.byref(ta.c), C.byref(tb.c), C.byref(c.c), C.byref(s.c), 0.0)
    pb.check_error()
    assert bits_differ(c.numpy(), w[1]) == 0
    assert scaled_err(s.numpy(), w[2], np.abs(w[1]).sum(axis=1)) <= 1e-5
    c.grad.copy_from(G)
    cuda.backward("add_leaky_relu", [ta, tb], c, fval=0.0)
    e = scaled_err(tb.grad.numpy(), w[3], np.abs(G * (w[1] > 0)).sum(axis=0, keepdims=True)); assert e <= 1e-5
    record(1, "fused grad_b", e, 1e-5, "|gpu-cpu| / sum|terms|")


# ---- config 2 ----------------------------------------------------------------------------------------
def test_config2_every_op_and_the_chain_on_2p28_elements(cuda, cpu, recipes):
    n = 1 << 28
    x = np.random.RandomState(0).randn(n).astype(np.float32)
    y = np.random.RandomState(1).randn(n).astype(np.float32)
    tx, ty, tz = cuda.tensor(x), cuda.tensor(y), cuda.empty((n,))
    hx, hy, hz = host(cpu, x), host(cpu, y), host_empty((n,))
    one_d, one_h = cuda.tensor(np.float32(1.0).reshape(())), cpu.tensor(np.float32(1.0).reshape(()))
    want = host_values(hz, (n,))
    exact = [("neg", [tx], [hx]), ("abs", [tx], [hx]), ("add", [tx, one_d], [hx, one_h]),
             ("div", [one_d, tx], [one_h, hx]), ("mul", [tx, ty], [hx, hy]), ("add", [tx, ty], [hx, hy])]
    names = ["neg", "abs", "add_scalar (x + 1.0)", "rdiv_scalar (1.0 / x)", "mul", "add"]
    for (op, di, hi), name in zip(exact, names):
        cuda.forward(op, di, tz); cpu.forward(op, hi, hz)
        # neg: the reference's AVX body gives +0 for -(+0), its scalar path -0: compared as values
        bad = values_differ(tz.numpy(), want) if op == "neg" else bits_differ(tz.numpy(), want)
        assert bad == 0, name
        record(2, name, 0, "bit-exact" if op != "neg" else "equal values", "elements differing")
    cuda.forward("exp", [tx], tz); cpu.forward("exp", [hx], hz)
    u = max_ulp(tz.numpy(), want); assert u <= 2
    record(2, "exp", u, 2, "ulp")
    # sigmoid = neg -> exp -> +1 -> 1/. : exp is within 2 ulp of glibc's; where e = exp(-x) is not
    # small against 1 the sum 1 + e inherits that difference (up to 2 ulp of a value in [1, 2), i.e.
    # 2^-22 relative), and the reciprocal lands in (0.5, 1], where one ulp is 2^-24 relative: up to
    # 4 ulp between the two results. Measured worst case over the 2^28 inputs of this configuration: 4.
    cuda.forward("sigmoid", [tx], tz)
    u = max_ulp(tz.numpy(), recipes.sigmoid(x)); assert u <= 4
    record(2, "sigmoid (4-op recipe)", u, 4, "ulp")
    # the chain: z = t + e2 with t = sigmoid(x) * y, e2 = exp(-|x|); t and e2 can cancel, so the
    # bound is in ulps of the terms: |gpu - cpu| <= k * 2^-23 * (|t| + |e2|); measured worst case over
    # the 2^28 inputs: k = 2.69, asserted: 3
    steps = [("neg", 0, 0, 0), ("exp", 2, 0, 0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
             ("mul", 5, 1, 0), ("abs", 0, 0, 0), ("neg", 7, 0, 0), ("exp", 8, 0, 0), ("add", 6, 9, 0)]
    pb.chain_forward([tx, ty], tz, steps)
    got, ref = tz.numpy(), recipes.chain(x, y)
    worst = 0.0
    for i in range(0, n, CHUNK):
        x64, y64 = x[i:i + CHUNK].astype(np.float64), y[i:i + CHUNK].astype(np.float64)
        terms = np.abs(y64) / (1 + np.exp(-x64)) + np.exp(-np.abs(x64))
        d = np.abs(got[i:i + CHUNK].astype(np.float64) - ref[i:i + CHUNK]) / (2.0 ** -23 * terms)
        worst = max(worst, float(d.max()))
    assert worst <= 3.0
    record(2, "fused chain z = sigmoid(x)*y + exp(-|x|)", worst, 3.0, "|gpu-cpu| / (2^-23 * (|t|+|e2|))")


# ---- config 3 ----------------------------------------------------------------------------------------
def test_config3_row_ops_softmax_and_cross_entropy(cuda, cpu, recipes):
    R, Cn = 65536, 4096
    X = (2.0 * np.random.RandomState(0).randn(R, Cn)).astype(np.float32)
    labels = np.random.RandomState(1).randint(0, Cn, size=R).astype(np.int32)
    tX, hX = cuda.tensor(X), host(cpu, X)
    absrow = np.abs(X).astype(np.float64).sum(axis=1)
    for op in ("sum", "mean", "max"):
        d, h = cuda.empty((R,)), host_empty((R,))
        cuda.forward(op, [tX], d, dim=1); cpu.forward(op, [hX], h, dim=1)
        got, want = d.numpy(), host_values(h, (R,))
        if op == "max":
            assert bits_differ(got, want) == 0
            record(3, "row max", 0, "bit-exact", "elements differing")
        else:
            e = scaled_err(got, want, absrow / (Cn if op == "mean" else 1)); assert e <= 1e-5
            record(3, f"row {op}", e, 1e-5, "|gpu-cpu| / sum|x|")
    idx = cuda.empty((R,), dtype=INT32); cuda.forward("argmax", [tX], idx, dim=1)
    assert np.array_equal(idx.numpy(), np.argmax(X, axis=1).astype(np.int32))   # first occurrence, like the max rule
    record(3, "row argmax", 0, "exact", "indices differing")
    Y = cuda.empty((R, Cn))
    cuda.forward("softmax", [tX], Y, dim=1)
    e = max_rel(Y.numpy(), recipes.softmax(X)); assert e <= 1e-5
    record(3, "softmax", e, 1e-5, "relative")
    cuda.forward("log_softmax", [tX], Y, dim=1)
    e = max_rel(Y.numpy(), recipes.log_softmax(X)); assert e <= 1e-5
    record(3, "log_softmax", e, 1e-5, "relative")
    loss = cuda.empty((1,))
    cuda.forward("cross_entropy", [tX, cuda.tensor(labels)], loss)
    want, per_row = recipes.cross_entropy(X, labels)
    e = abs(float(loss.numpy()[0]) - float(want[0])) / abs(float(want[0])); assert e <= 1e-5
    record(3, "cross-entropy mean", e, 1e-5, "relative")


# ---- config 4 ----------------------------------------------------------------------------------------
def test_config4_column_and_full_reductions_on_both_views(cuda, cpu):
    M = 8192
    X = np.random.RandomState(0).uniform(-1, 1, (M, M)).astype(np.float32)
    tX, hX = cuda.tensor(X), host(cpu, X)
    a64 = np.abs(X).astype(np.float64)
    for name, d_in, h_in, colscale in (("", tX, hX, a64.sum(axis=0)),
                                       (" (transposed view)", tX.transpose(0, 1), hX.transpose(0, 1), a64.sum(axis=1))):
        d, h = cuda.empty((M,)), host_empty((M,))
        cuda.forward("sum", [d_in], d, dim=0); cpu.forward("sum", [h_in], h, dim=0)
        e = scaled_err(d.numpy(), host_values(h, (M,)), colscale); assert e <= 1e-5
        record(4, "sum axis 0" + name, e, 1e-5, "|gpu-cpu| / sum|x|")
        d1, h1 = cuda.empty((1,)), host_empty((1,))
        cuda.forward("sum", [d_in], d1, dim=FULL_REDUCE); cpu.forward("sum", [h_in], h1, dim=FULL_REDUCE)
        e = scaled_err(d1.numpy(), host_values(h1, (1,)), a64.sum()); assert e <= 1e-5
        record(4, "full sum" + name, e, 1e-5, "|gpu-cpu| / sum|x|")
        cuda.forward("max", [d_in], d1, dim=FULL_REDUCE); cpu.forward("max", [h_in], h1, dim=FULL_REDUCE)
        assert bits_differ(d1.numpy(), host_values(h1, (1,))) == 0
        record(4, "full max" + name, 0, "bit-exact", "elements differing")


# ---- config 5 ----------------------------------------------------------------------------------------
def test_config5_nchw_epilogue_forward_and_both_gradients(cuda, cpu):
    shape, pshape = (256, 256, 56, 56), (1, 256, 1, 1)
    X = np.random.RandomState(0).randn(*shape).astype(np.float32)
    S = np.random.RandomState(1).uniform(-.5, .5, pshape).astype(np.float32)
    B = np.random.RandomState(2).uniform(-.5, .5, pshape).astype(np.float32)
    G = np.random.RandomState(3).randn(*shape).astype(np.float32)
    # CPU: mul -> add -> leaky_relu, then the three backward calls in reverse
    hX, hS, hB = host(cpu, X), cpu.tensor(S, requires_grad=True), cpu.tensor(B, requires_grad=True)
    hXS, hU, hY = host_empty(shape, True), host_empty(shape, True), host_empty(shape, False)
    cpu.forward("mul", [hX, hS], hXS); cpu.forward("add", [hXS, hB], hU); cpu.forward("leaky_relu", [hU], hY, fval=0.0)
    hY.grad = host(cpu, G); hY.c.grad = __import__("ctypes").pointer(hY.grad.c)
    cpu.backward("leaky_relu", [hU], hY, fval=0.0); cpu.backward("add", [hXS, hB], hU); cpu.backward("mul", [hX, hS], hXS)
    Yw = host_values(hY, shape)
    # GPU: one fused forward, one fused backward
    tX, tS, tB = cuda.tensor(X), cuda.tensor(S, requires_grad=True), cuda.tensor(B, requires_grad=True)
    tY = cuda.empty(shape, requires_grad=True)
    cuda.forward("scale_bias_leaky_relu", [tX, tS, tB], tY, fval=0.0)
    assert bits_differ(tY.numpy(), Yw) == 0
    record(5, "Y = relu(X*scale + bias)", 0, "bit-exact", "elements differing")
    tY.grad.copy_from(G)
    cuda.backward("scale_bias_leaky_relu", [tX, tS, tB], tY, fval=0.0)
    gm = G * (Yw > 0)
    e = scaled_err(tB.grad.numpy(), hB.grad.numpy(), np.abs(gm).astype(np.float64).sum(axis=(0, 2, 3), keepdims=True))
    assert e <= 1e-5
    record(5, "bias-grad = sum_{N,H,W} G*[Y>0]", e, 1e-5, "|gpu-cpu| / sum|terms|")
    e = scaled_err(tS.grad.numpy(), hS.grad.numpy(), np.abs(gm * X).astype(np.float64).sum(axis=(0, 2, 3), keepdims=True))
    assert e <= 1e-5
    record(5, "scale-grad = sum_{N,H,W} G*[Y>0]*X", e, 1e-5, "|gpu-cpu| / sum|terms|")


def test_zz_print_the_parity_table():
    """Not a check: prints what the tests above measured, one line per op."""
    rows = sorted(REPORT.values(), key=lambda r: (r["config"], r["op"]))
    lines = ["config | op | worst observed | bound | unit"]
    for r in rows:
        lines.append(f"{r['config']} | {r['op']} | {r['worst']:.3g} | {r['bound']} | {r['unit']}")
    print("\n".join(lines))
    out = Path(os.environ.get("GRAFT_REPO_ROOT", Path(__file__).resolve().parent.parent)) / "gpurun_out"
    try:
        out.mkdir(exist_ok=True)
        (out / "parity_table.json").write_text(json.dumps({"checker": "reference" if have_ref() else "restatement",
                                                          "when": time.strftime("%Y-%m-%d"), "rows": rows}, indent=1))
    except OSError:
        pass
