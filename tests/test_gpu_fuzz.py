"""Seeded random layouts through the C ABI against the CPU oracle: random rank (0-8), extents,
permuted views, broadcast operands (size-1 dims, missing leading dims, stride-0 expands) for the
elementwise ops, and random axes / keepdim over permuted views for the reductions. The fixed cases
of the other GPU tests pin named layouts; this one walks the planner's merge / sort / vector-width
decisions over shapes nobody thought of."""
import numpy as np
import pytest

from harness import FULL_REDUCE, INT32, assert_bit_equal, assert_sum_close, assert_ulp

pytestmark = pytest.mark.gpu

BITWISE = ["add", "sub", "mul", "div"]
UNARY_BIT = ["abs", "neg", "leaky_relu"]
UNARY_ULP = {"exp": (-5, 5), "sin": (-6, 6), "cos": (-6, 6)}


def random_shape(rs, max_ndim=8, max_elems=40000):
    nd = int(rs.randint(0, max_ndim + 1))
    shape = []
    total = 1
    for _ in range(nd):
        s = int(rs.choice([1, 2, 3, 4, 5, 7, 8, 16, 33]))
        if total * s > max_elems:
            s = 1
        shape.append(s)
        total *= s
    return tuple(shape)


def permuted_view(be, arr, perm):
    """Tensor holding `arr` laid out so that view.transpose(perm-order) == arr: the data is stored
    in permuted order and viewed back through strides (no copy on the device)."""
    if arr.ndim < 2:
        return be.tensor(arr)
    stored = np.ascontiguousarray(arr.transpose(perm))
    t = be.tensor(stored)
    inv = np.argsort(perm)
    st = [t.strides[i] for i in inv]
    return t.view(list(arr.shape), st)


def broadcast_operand(rs, shape):
    """A shape that broadcasts to `shape`: some dims collapsed to 1, some leading dims dropped."""
    b = [1 if rs.rand() < 0.4 else s for s in shape]
    drop = int(rs.randint(0, len(b) + 1)) if len(b) and rs.rand() < 0.4 else 0
    while drop and b and b[0] != 1:
        b[0] = 1
    return tuple(b[drop:]) if all(x == 1 for x in b[:drop]) else tuple(b)


@pytest.mark.parametrize("seed", range(40))
def test_elementwise_random_layouts(cuda, oracle, seed):
    rs = np.random.RandomState(1000 + seed)
    shape = random_shape(rs)
    bshape = broadcast_operand(rs, shape)
    A = rs.uniform(-2, 2, shape).astype(np.float32)
    B = (rs.uniform(0.5, 2, bshape) * rs.choice([-1, 1], size=bshape)).astype(np.float32)
    perm = list(rs.permutation(len(shape)))
    op = BITWISE[seed % 4]
    outs = []
    for be in (cuda, oracle):
        ta = permuted_view(be, A, perm)
        tb = be.tensor(B)
        out = be.empty(shape)
        be.forward(op, [ta, tb], out)
        outs.append(out.numpy())
    assert_bit_equal(outs[0], outs[1], f"{op} {shape} perm {perm} b {bshape}")
    # unary on the same view
    uop = (UNARY_BIT + list(UNARY_ULP))[seed % 6]
    outs = []
    for be in (cuda, oracle):
        out = be.empty(shape)
        be.forward(uop, [permuted_view(be, A, perm)], out, fval=0.0 if seed % 2 else 0.1)
        outs.append(out.numpy())
    if uop in UNARY_ULP:
        assert_ulp(outs[0], outs[1], 2, f"{uop} {shape} perm {perm}")
    elif uop == "neg":
        assert np.array_equal(outs[0], outs[1])
    else:
        assert_bit_equal(outs[0], outs[1], f"{uop} {shape} perm {perm}")


@pytest.mark.parametrize("seed", range(40))
def test_reductions_random_layouts(cuda, oracle, seed):
    rs = np.random.RandomState(5000 + seed)
    shape = random_shape(rs, max_ndim=6)
    if len(shape) == 0:
        shape = (int(rs.choice([1, 5, 1000])),)
    A = rs.uniform(-1, 1, shape).astype(np.float32)
    perm = list(rs.permutation(len(shape)))
    dim = int(rs.randint(0, len(shape))) if rs.rand() < 0.7 else FULL_REDUCE
    keepdim = bool(rs.rand() < 0.5)
    op = ["sum", "mean", "max", "min", "argmax"][seed % 5]
    res = []
    for be in (cuda, oracle):
        ta = permuted_view(be, A, perm)
        if dim == FULL_REDUCE:
            out_shape = [1]
        elif keepdim:
            out_shape = [1 if i == dim else s for i, s in enumerate(shape)]
        else:
            out_shape = [s for i, s in enumerate(shape) if i != dim] or [1]
        out = be.empty(out_shape, dtype=INT32 if op == "argmax" else 1)
        be.forward(op, [ta], out, dim=dim, keepdim=int(keepdim))
        res.append(out.numpy().reshape(-1))
    what = f"{op} {shape} perm {perm} dim {dim} keepdim {keepdim}"
    if op == "argmax":
        want = np.argmax(A) if dim == FULL_REDUCE else np.argmax(A, axis=dim)
        assert np.array_equal(res[0], np.asarray(want, dtype=np.int32).reshape(-1)), what
    elif op in ("max", "min"):
        assert_bit_equal(res[0], res[1], what)
    else:
        a64 = np.abs(A.astype(np.float64))
        n = A.size if dim == FULL_REDUCE else shape[dim]
        scale = (a64.sum() if dim == FULL_REDUCE else a64.sum(axis=dim)) / (n if op == "mean" else 1)
        assert_sum_close(res[0], res[1], np.asarray(scale).reshape(-1), what=what)


@pytest.mark.parametrize("seed", range(24))
def test_binary_two_independently_permuted_views(cuda, oracle, seed):
    """Both operands are permuted views with DIFFERENT permutations, so they can be contiguous along
    two different dims, neither of them the output's: the gather-then-tile route, the single-tile
    route and the generic strided kernel all get hit, whatever the extents."""
    rs = np.random.RandomState(9000 + seed)
    nd = int(rs.randint(2, 5))
    shape = tuple(int(rs.choice([3, 8, 12, 17, 32, 40, 64])) for _ in range(nd))
    A = rs.uniform(-2, 2, shape).astype(np.float32)
    B = (rs.uniform(0.5, 2, shape) * rs.choice([-1, 1], size=shape)).astype(np.float32)
    pa, pb_ = list(rs.permutation(nd)), list(rs.permutation(nd))
    op = BITWISE[seed % 4]
    outs = []
    for be in (cuda, oracle):
        out = be.empty(shape)
        be.forward(op, [permuted_view(be, A, pa), permuted_view(be, B, pb_)], out)
        outs.append(out.numpy())
    assert_bit_equal(outs[0], outs[1], f"{op} {shape} perms {pa} {pb_}")


@pytest.mark.parametrize("rows", [7, 64, 200, 1024, 3000])
@pytest.mark.parametrize("cols", [8, 100, 1024, 4100])
def test_column_reductions_of_small_and_medium_matrices(cuda, oracle, rows, cols):
    """Column reductions across the sizes where the geometry changes: narrow strips without a split
    (inputs that fit L2, short reduced dim), one-warp strips with and without a split over CTAs,
    vector and scalar widths, and the three-input gradient prologue on the same shapes."""
    A = np.random.RandomState(rows * 7 + cols).uniform(-1, 1, (rows, cols)).astype(np.float32)
    for op in ("sum", "max"):
        res = []
        for be in (cuda, oracle):
            out = be.empty((cols,))
            be.forward(op, [be.tensor(A)], out, dim=0)
            res.append(out.numpy())
        if op == "max":
            assert_bit_equal(res[0], res[1], f"max {rows}x{cols}")
        else:
            assert_sum_close(res[0], res[1], np.abs(A.astype(np.float64)).sum(axis=0), what=f"sum {rows}x{cols}")
    # grad of a broadcast row through the fused add + leaky_relu backward (three inputs per element)
    b = np.random.RandomState(1).uniform(-1, 1, (1, cols)).astype(np.float32)
    G = np.random.RandomState(2).randn(rows, cols).astype(np.float32)
    ta, tb = oracle.tensor(A), oracle.tensor(b, requires_grad=True)
    ab = oracle.empty(A.shape, requires_grad=True); oracle.forward("add", [ta, tb], ab)
    c = oracle.empty(A.shape, requires_grad=True); oracle.forward("leaky_relu", [ab], c, fval=0.1)
    c.grad.copy_from(G)
    oracle.backward("leaky_relu", [ab], c, fval=0.1); oracle.backward("add", [ta, tb], ab)
    da, db = cuda.tensor(A), cuda.tensor(b, requires_grad=True)
    dc = cuda.empty(A.shape, requires_grad=True)
    cuda.forward("add_leaky_relu", [da, db], dc, fval=0.1)
    dc.grad.copy_from(G)
    cuda.backward("add_leaky_relu", [da, db], dc, fval=0.1)
    scale = np.abs(G.astype(np.float64) * np.where(c.numpy() > 0, 1.0, 0.1)).sum(axis=0, keepdims=True)
    assert_sum_close(db.grad.numpy(), tb.grad.numpy(), scale, what=f"grad of the broadcast row {rows}x{cols}")


def _log_uniform(rs, lo, hi):
    return int(round(np.exp(rs.uniform(np.log(lo), np.log(hi)))))


@pytest.mark.parametrize("seed", range(40))
def test_softmax_family_random_rows(cuda, recipes, seed):
    """Random row counts and row lengths (1 ... 70000, any remainder mod 4) through softmax,
    log-softmax and cross-entropy, dense and as column slices of a wider buffer (rows that start at
    any 4-byte phase, outputs at the same or another phase): every kernel of the family (thread per
    row, slice of a warp, float4 with ragged ends, scalar, cluster per row, two-pass) is reached."""
    rs = np.random.RandomState(7000 + seed)
    cols = _log_uniform(rs, 1, 70000) if seed % 4 else int(rs.choice([1, 2, 3, 5, 8, 31, 33, 64, 65, 127, 1001, 8193]))
    rows = max(1, min(_log_uniform(rs, 1, 6000), 400000 // cols))
    X = (2.0 * rs.randn(rows, cols)).astype(np.float32)
    want_sm, want_ls = recipes.softmax(X), recipes.log_softmax(X)
    layouts = [("dense", 0, 0, 0)]
    if cols > 1:
        layouts.append(("sliced, same phase", int(rs.randint(1, 4)), None, int(rs.randint(0, 5))))
        layouts.append(("sliced, other phase", int(rs.randint(1, 4)), int(rs.randint(0, 4)), int(rs.randint(0, 5))))
    for what, lead, out_lead, pad in layouts:
        # the tensor is columns [lead, lead + cols) of a [rows, lead + cols + pad] buffer
        width = lead + cols + pad
        buf = np.zeros((rows, width), np.float32)
        buf[:, lead:lead + cols] = X
        tb = cuda.tensor(buf)
        x = tb.view([rows, cols], [width, 1], offset=lead) if (lead or pad) else tb
        out_lead = lead if out_lead is None else out_lead
        owidth = out_lead + cols + pad
        for op, want in (("softmax", want_sm), ("log_softmax", want_ls)):
            ob = cuda.tensor(np.full((rows, owidth), 7.0, np.float32))
            o = ob.view([rows, cols], [owidth, 1], offset=out_lead) if (out_lead or pad) else ob
            cuda.forward(op, [x], o, dim=1)
            full = ob.numpy()
            got = full[:, out_lead:out_lead + cols]
            tag = f"{op} [{rows}, {cols}] {what} (lead {lead}/{out_lead}, pad {pad})"
            if op == "softmax":
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-30, err_msg=tag)
            else:
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5, err_msg=tag)
            # nothing outside the rows was written
            assert np.all(full[:, :out_lead] == 7.0) and np.all(full[:, out_lead + cols:] == 7.0), tag
    labels = rs.randint(0, cols, size=rows).astype(np.int32)
    out = cuda.empty((1,))
    cuda.forward("cross_entropy", [cuda.tensor(X), cuda.tensor(labels)], out)
    want, per_row = recipes.cross_entropy(X, labels)
    assert_sum_close(out.numpy(), want, np.abs(per_row).sum() / rows, what=f"cross-entropy mean [{rows}, {cols}]")
