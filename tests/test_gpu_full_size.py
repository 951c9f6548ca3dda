"""The five benchmark configurations at FULL size, checked through properties that need no CPU pass over
the data: idempotence, involution, planted extrema, exact sums of exactly-representable values,
rows of a softmax summing to one, a checksum of checksums. The seeded small-size parity tests
(test_gpu_elementwise / test_gpu_reduce) pin the arithmetic; these pin the indexing, the vector
tails and the multi-CTA combines at the sizes the benchmark runs."""
import numpy as np
import pytest

import plast_b200 as pb
from harness import FULL_REDUCE, INT32, assert_bit_equal

pytestmark = pytest.mark.gpu


def test_config2_chain_2p28_elements(cuda):
    n = 1 << 28
    rs = np.random.RandomState(0)
    x = rs.randn(n).astype(np.float32)
    tx = cuda.tensor(x)
    a, b = cuda.empty((n,)), cuda.empty((n,))
    cuda.forward("abs", [tx], a); cuda.forward("abs", [a], b)          # idempotent
    av = a.numpy()
    assert np.array_equal(av, np.abs(x)) and np.array_equal(b.numpy(), av)
    cuda.forward("neg", [tx], a); cuda.forward("neg", [a], b)          # involution
    assert np.array_equal(b.numpy(), x)
    cuda.forward("leaky_relu", [tx], a, fval=0.0); cuda.forward("leaky_relu", [a], b, fval=0.0)
    assert_bit_equal(b.numpy(), a.numpy(), "relu idempotent (incl. -0.0)")
    # fused chain == the nine primitive launches, bitwise, at full size
    y = np.random.RandomState(1).randn(n).astype(np.float32)
    ty, z = cuda.tensor(y), cuda.empty((n,))
    steps = [("neg", 0, 0, 0), ("exp", 2, 0, 0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
             ("mul", 5, 1, 0), ("abs", 0, 0, 0), ("neg", 7, 0, 0), ("exp", 8, 0, 0), ("add", 6, 9, 0)]
    pb.chain_forward([tx, ty], z, steps)
    one = cuda.tensor(np.float32(1.0).reshape(()))
    cuda.forward("neg", [tx], a); cuda.forward("exp", [a], a); cuda.forward("add", [a, one], a)
    cuda.forward("div", [one, a], a); cuda.forward("mul", [a, ty], a)
    cuda.forward("abs", [tx], b); cuda.forward("neg", [b], b); cuda.forward("exp", [b], b)
    cuda.forward("add", [a, b], b)
    assert_bit_equal(z.numpy(), b.numpy(), "fused chain vs nine launches at 2^28")
    zv = z.numpy()
    sl = slice(123456789, 123456789 + 4096)
    x64, y64 = x[sl].astype(np.float64), y[sl].astype(np.float64)
    np.testing.assert_allclose(zv[sl], y64 / (1 + np.exp(-x64)) + np.exp(-np.abs(x64)), rtol=2e-6, atol=2e-6)


def test_config3_rows_65536x4096(cuda):
    R, Cn = 65536, 4096
    rs = np.random.RandomState(0)
    X = (2.0 * rs.randn(R, Cn)).astype(np.float32)
    planted = rs.randint(0, Cn, size=R)
    X[np.arange(R), planted] = 50.0                                     # unique row maximum
    tX = cuda.tensor(X)
    out = cuda.empty((R,)); cuda.forward("max", [tX], out, dim=1)
    assert np.all(out.numpy() == 50.0)
    idx = cuda.empty((R,), dtype=INT32); cuda.forward("argmax", [tX], idx, dim=1)
    assert np.array_equal(idx.numpy(), planted.astype(np.int32))
    s = cuda.empty((R,)); cuda.forward("sum", [tX], s, dim=1)
    m = cuda.empty((R,)); cuda.forward("mean", [tX], m, dim=1)
    rows = rs.randint(0, R, size=64)
    want = X[rows].astype(np.float64).sum(axis=1)
    scale = np.abs(X[rows]).astype(np.float64).sum(axis=1)
    assert np.all(np.abs(s.numpy()[rows] - want) <= 1e-5 * scale)
    assert np.all(np.abs(m.numpy()[rows] - want / Cn) <= 1e-5 * scale / Cn)
    Y = cuda.empty((R, Cn)); cuda.forward("softmax", [tX], Y, dim=1)
    ysum = cuda.empty((R,)); cuda.forward("sum", [Y], ysum, dim=1)
    np.testing.assert_allclose(ysum.numpy(), 1.0, atol=1e-5)            # rows of a softmax sum to one
    L = cuda.empty((R, Cn)); cuda.forward("log_softmax", [tX], L, dim=1)
    lmax = cuda.empty((R,)); cuda.forward("max", [L], lmax, dim=1)
    # the planted 50.0 dominates: its log-probability is -log(1 + sum exp(x - 50)) ~ -0
    assert np.all(lmax.numpy() <= 0) and np.all(lmax.numpy() > -1e-3)
    labels = cuda.tensor(planted.astype(np.int32))
    loss = cuda.empty((1,)); cuda.forward("cross_entropy", [tX, labels], loss)
    assert 0.0 <= float(loss.numpy()[0]) < 1e-3
    # uniform logits: loss = log(C) whatever the labels
    U = cuda.tensor(np.zeros((R, Cn), np.float32))
    cuda.forward("cross_entropy", [U, labels], loss)
    np.testing.assert_allclose(loss.numpy()[0], np.log(Cn), rtol=1e-6)


def test_config4_8192_square_and_its_transposed_view(cuda):
    M = 8192
    ones = cuda.tensor(np.ones((M, M), np.float32))
    out = cuda.empty((1,))
    for t in (ones, ones.transpose(0, 1)):
        cuda.forward("sum", [t], out, dim=FULL_REDUCE)
        assert out.numpy()[0] == float(M * M)                           # 2^26: every partial is exact
        col = cuda.empty((M,)); cuda.forward("sum", [t], col, dim=0)
        assert np.all(col.numpy() == float(M))
    X = np.random.RandomState(0).uniform(-1, 1, (M, M)).astype(np.float32)
    X[4321, 1234] = 7.0
    tX = cuda.tensor(X)
    tXT = tX.transpose(0, 1)
    res = {}
    for name, t in (("contiguous", tX), ("view", tXT)):
        full = cuda.empty((1,)); cuda.forward("sum", [t], full, dim=FULL_REDUCE)
        mx = cuda.empty((1,)); cuda.forward("max", [t], mx, dim=FULL_REDUCE)
        ax0 = cuda.empty((M,)); cuda.forward("sum", [t], ax0, dim=0)
        tot = cuda.empty((1,)); cuda.forward("sum", [ax0], tot, dim=FULL_REDUCE)   # checksum of checksums
        res[name] = (full.numpy()[0], mx.numpy()[0], ax0.numpy(), tot.numpy()[0])
    truth = X.astype(np.float64).sum()
    scale = np.abs(X).astype(np.float64).sum()
    for name, (full, mx, ax0, tot) in res.items():
        assert mx == 7.0
        assert abs(full - truth) <= 1e-5 * scale and abs(tot - truth) <= 1e-5 * scale, name
    # axis 0 of the view is axis 1 of the tensor
    want = X.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(res["view"][2] - want) <= 1e-5 * np.abs(X).astype(np.float64).sum(axis=1))


def test_config5_nchw_epilogue_256x256x56x56(cuda):
    shape, pshape = (256, 256, 56, 56), (1, 256, 1, 1)
    n = int(np.prod(shape))
    rs = np.random.RandomState(0)
    X = rs.randn(*shape).astype(np.float32)
    S = np.random.RandomState(1).uniform(-.5, .5, pshape).astype(np.float32)
    B = np.random.RandomState(2).uniform(-.5, .5, pshape).astype(np.float32)
    tX = cuda.tensor(X)
    tS, tB = cuda.tensor(S), cuda.tensor(B, requires_grad=True)
    Y = cuda.empty(shape, requires_grad=True)
    cuda.forward("scale_bias_leaky_relu", [tX, tS, tB], Y, fval=0.0)
    # spot-check whole channels bitwise against numpy (mul, add, relu each rounded on their own)
    Yv = Y.numpy()
    for c in (0, 77, 255):
        u = X[:, c] * S[0, c, 0, 0] + B[0, c, 0, 0]
        assert_bit_equal(Yv[:, c], np.where(u > 0, u, u * np.float32(0.0)), f"channel {c}")
    # upstream gradient of ones: bias-grad = number of positive outputs per channel (exact integers)
    Y.grad.copy_from(np.ones(n, np.float32))
    cuda.backward("scale_bias_leaky_relu", [tX, tS, tB], Y, fval=0.0)
    want = (Yv > 0).sum(axis=(0, 2, 3)).astype(np.float32).reshape(pshape)
    assert np.array_equal(tB.grad.numpy(), want)


def test_more_than_2_to_31_elements_use_64_bit_indexing(cuda):
    """8.6 GB per tensor: element offsets no longer fit 32 bits. Everything is generated and checked
    on the device except a handful of small read-backs."""
    import ctypes as C
    R, Cn = (1 << 19) + 1, 4096
    n = R * Cn                                                            # 2^31 + 4096
    x, y = pb.Tensor((R, Cn)), pb.Tensor((R, Cn))
    pb.lib.ones_cuda(C.byref(x.c), n); pb.check_error()
    plant = np.float32([5.0])
    pb.lib.arena_memcpy_h2d_cuda(x.c.data + 4 * (n - 3), plant.ctypes.data, 4)   # beyond offset 2^31
    cuda.forward("add", [x, x], y)                                        # elementwise, 64-bit offsets
    rows = cuda.empty((R,)); cuda.forward("sum", [y], rows, dim=1)
    rv = rows.numpy()
    assert np.all(rv[:-1] == 2.0 * Cn) and rv[-1] == 2.0 * Cn + 8.0
    cols = cuda.empty((Cn,)); cuda.forward("sum", [y], cols, dim=0)
    cv = cols.numpy()
    want = np.full(Cn, 2.0 * R, np.float32); want[Cn - 3] += 8.0          # all exact: integers below 2^24
    assert np.array_equal(cv, want)
    mx = cuda.empty((1,)); cuda.forward("max", [y], mx, dim=FULL_REDUCE)
    assert mx.numpy()[0] == 10.0
    tot = cuda.empty((1,)); cuda.forward("sum", [y], tot, dim=FULL_REDUCE)
    assert abs(float(tot.numpy()[0]) - (2.0 * n + 8.0)) <= 1e-6 * 2.0 * n
    # scalar broadcast and a unary op over the same extent
    two = cuda.tensor(np.float32(2.0).reshape(()))
    cuda.forward("div", [y, two], y); cuda.forward("neg", [y], y)
    cuda.forward("max", [y], mx, dim=FULL_REDUCE)
    assert mx.numpy()[0] == -1.0
    cuda.forward("min", [y], mx, dim=FULL_REDUCE)
    assert mx.numpy()[0] == -5.0
