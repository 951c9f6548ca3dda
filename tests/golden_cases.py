"""Case list shared by tests/golden/make_golden.py (which records the reference's outputs) and
the tests that replay the cases on the oracle and on the CUDA library.

A case = one forward (and optionally backward) call of a primitive entry point on seeded inputs:
  name, op, inputs [(kind, seed, shape, lo, hi)], optional view of input 0 ("T" = transpose 0,1),
  params (dim, keepdim, fval), backward flag.
`exact` tells the comparison rule: "bits", "values" (== incl. signed-zero equality),
"ulp2" (transcendentals on the GPU; the CPU oracle must still match the reference bitwise),
"sum" (accumulation order may differ on the GPU), "grad" (gradient accumulation: the reference
build contracts `da + g * x` into one FMA — gcc's default -ffp-contract=fast with -mfma — while
the oracle and the GPU round the product first; compared with rtol 2e-6).
"""
from __future__ import annotations

import numpy as np

from harness import FULL_REDUCE, rand_normal, rand_uniform


def _arr(spec):
    kind, seed, shape, lo, hi = spec
    if kind == "u":
        return rand_uniform(seed, shape, lo, hi)
    if kind == "n":
        return rand_normal(seed, shape, std=hi)
    if kind == "grid":  # coarse values -> ties for max/min
        return (np.round(rand_uniform(seed, shape, lo, hi) * 4) / 4).astype(np.float32)
    raise ValueError(kind)


def cases():
    cs = []

    def add(name, op, inputs, exact, dim=0, keepdim=0, fval=0.0, view=None, backward=False):
        cs.append(dict(name=name, op=op, inputs=inputs, exact=exact, dim=dim, keepdim=keepdim, fval=fval,
                       view=view, backward=backward))

    # binary: the reference's own broadcast pairs (tests/test_ops.py:11-15) + config layouts in small
    pairs = [((4,), (4,)), ((2, 3), (2, 3)), ((3, 2, 4), (3, 2, 4)), ((4,), (1,)), ((2, 3), (1, 3)),
             ((3, 1, 4), (1, 2, 1)), ((64, 48), (1, 48)), ((64, 48), (64, 1)), ((6, 8, 5, 5), (1, 8, 1, 1)),
             ((33, 7), (7,)), ((17,), ()), ((1003,), (1003,))]
    for op in ("add", "sub", "mul", "div"):
        for i, (sa, sb) in enumerate(pairs):
            add(f"{op}_fwd_{i}", op, [("n", 10 + i, sa, 0, 1.0), ("u", 50 + i, sb, 0.5, 2.0)], "bits")
            add(f"{op}_bwd_{i}", op, [("n", 10 + i, sa, 0, 1.0), ("u", 50 + i, sb, 0.5, 2.0)],
                "bits" if (sa == sb and op in ("add", "sub")) else "grad", backward=True)
    # unary
    ranges = {"abs": (-10, 10), "neg": (-10, 10), "exp": (-20, 20), "log": (1e-6, 100.0), "sin": (-20, 20),
              "cos": (-20, 20), "tan": (-1.5, 1.5), "leaky_relu": (-5, 5)}
    for op, (lo, hi) in ranges.items():
        rule = "bits" if op in ("abs", "leaky_relu") else ("values" if op == "neg" else "ulp2")
        for i, shape in enumerate([(4,), (3, 2, 4), (1003,), (37, 29)]):
            add(f"{op}_fwd_{i}", op, [("u", 70 + i, shape, lo, hi)], rule, fval=0.01)
        add(f"{op}_fwd_T", op, [("u", 75, (31, 45), lo, hi)], rule, fval=0.2, view="T")
        add(f"{op}_bwd", op, [("u", 76, (37, 29), lo, hi)], "values" if op in ("neg", "abs") else "grad",
            fval=0.01, backward=True)
    add("relu_fwd", "leaky_relu", [("u", 80, (64, 48), -1, 1)], "bits", fval=0.0)
    add("relu_bwd", "leaky_relu", [("u", 80, (64, 48), -1, 1)], "values", fval=0.0, backward=True)
    # reductions
    for op in ("sum", "mean", "max", "min"):
        rule = "bits" if op in ("max", "min") else "sum"
        for i, shape in enumerate([(4,), (2, 3), (3, 2, 4), (7, 33), (64, 48), (5, 1, 9), (2, 3, 4, 5)]):
            for dim in list(range(len(shape))) + [FULL_REDUCE]:
                for keepdim in (0, 1):
                    add(f"{op}_fwd_{i}_d{dim}_k{keepdim}", op, [("u", 90 + i, shape, -1, 1)], rule, dim=dim, keepdim=keepdim)
        for dim in (0, 1, FULL_REDUCE):
            add(f"{op}_fwd_T_d{dim}", op, [("u", 99, (24, 40), -1, 1)], rule, dim=dim, view="T")
            add(f"{op}_bwd_d{dim}", op, [("grid", 98, (7, 33), -1, 1)], "grad", dim=dim, backward=True)
    return cs


def _out_shape(in_shape, case):
    op, dim, keepdim = case["op"], case["dim"], case["keepdim"]
    if op not in ("sum", "mean", "max", "min", "argmax"):
        return None
    if dim == FULL_REDUCE:
        return [1]
    if keepdim:
        return [1 if i == dim else s for i, s in enumerate(in_shape)]
    return [s for i, s in enumerate(in_shape) if i != dim] or [1]


def run_case(be, case):
    """Runs a case on a backend; returns {key: array} of everything worth comparing."""
    arrs = [_arr(s) if s[2] != () else np.float32(1.25).reshape(()) for s in case["inputs"]]
    grads0 = [rand_normal(200 + i, a.shape) if a.shape else np.float32(0.5).reshape(()) for i, a in enumerate(arrs)]
    ts = [be.tensor(a, requires_grad=case["backward"]) for a in arrs]
    if case["backward"]:
        for t, g in zip(ts, grads0):
            t.grad.copy_from(g)
    ins = list(ts)
    if case["view"] == "T":
        v = ts[0].transpose(0, 1)
        if case["backward"]:
            raise ValueError("view + backward cases are not used")
        ins[0] = v
    in_shape = ins[0].shape
    red = _out_shape(in_shape, case)
    if red is not None:
        out_shape = red
    elif len(arrs) == 2:
        out_shape = list(np.broadcast_shapes(arrs[0].shape, arrs[1].shape))
    else:
        out_shape = in_shape
    out = be.empty(out_shape, requires_grad=case["backward"])
    be.forward(case["op"], ins, out, dim=case["dim"], keepdim=case["keepdim"], fval=case["fval"])
    res = {"out": out.numpy(), "out_shape": np.array(out.shape, np.int64)}
    if case["backward"]:
        out.grad.copy_from(rand_normal(300, tuple(out.shape)))
        be.backward(case["op"], ins, out, dim=case["dim"], keepdim=case["keepdim"], fval=case["fval"])
        for i, t in enumerate(ts):
            res[f"grad{i}"] = t.grad.numpy()
    return res
