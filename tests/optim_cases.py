"""Seeded optimiser runs shared by the golden generator, the oracle pin and the GPU parity test:
three steps of SGD, Adam and AdamW over a handful of parameters (odd sizes, a 0-dim parameter, one
parameter without a gradient, one NULL entry), with a fresh gradient each step."""
import ctypes as C

import numpy as np

from plast_b200 import CTensor, Tensor
from plast_b200 import optim as O

SHAPES = [(1000,), (33, 7), (4097,), (), (2, 3, 5), (1,), (513,)]
NO_GRAD = 4        # index of the parameter that has no grad tensor (skipped by every step)
STEPS = 3
HYPER = {"sgd": dict(lr=0.1),
         "adam": dict(lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8),
         "adamw": dict(lr=2e-3, beta1=0.8, beta2=0.99, epsilon=1e-6, weight_decay=0.05)}


def initial_params():
    rs = np.random.RandomState(42)
    return [np.asarray(rs.randn(*s), dtype=np.float32) for s in SHAPES]


def gradient(step, i):
    rs = np.random.RandomState(1000 * step + i)
    return np.asarray(rs.randn(*SHAPES[i]) * 0.5, dtype=np.float32)


def make_optimizer(kind):
    h = HYPER[kind]
    if kind == "sgd":
        return O.SGD(h["lr"])
    if kind == "adam":
        o = O.Adam()
        o.lr, o.beta1, o.beta2, o.epsilon, o.t = h["lr"], h["beta1"], h["beta2"], h["epsilon"], 0
        return o
    o = O.AdamW()
    o.lr, o.beta1, o.beta2, o.epsilon, o.weight_decay, o.t = (h["lr"], h["beta1"], h["beta2"], h["epsilon"],
                                                            h["weight_decay"], 0)
    return o


def run_through_structs(kind, device, step_fn, before_first_step=None):
    """Drives `step_fn(optimizer, Tensor** params, n)` (the reference's <kind>_step_cpu or this
    library's <kind>_step_cuda) and returns every parameter after every step, plus the final
    moments."""
    params = []
    for i, p0 in enumerate(initial_params()):
        params.append(Tensor.from_numpy(p0, device=device, requires_grad=(i != NO_GRAD)))
    # a NULL entry at the end: skipped by sgd.c:19-21; the reference's Adam set-up loop (adam.c:39-45)
    # dereferences every entry, so only SGD gets one
    plist = params + [None] if kind == "sgd" else params
    opt = make_optimizer(kind)
    if before_first_step:
        before_first_step(opt)
    out = {}
    arr = O.param_array(plist)
    for step in range(1, STEPS + 1):
        for i, p in enumerate(params):
            if p.grad is not None:
                p.grad.copy_from(gradient(step, i))
        step_fn(C.byref(opt), arr, len(plist))
        for i, p in enumerate(params):
            out[f"{kind}/step{step}/p{i}"] = p.numpy().copy()
    if kind != "sgd":
        for i, p in enumerate(params):
            for name, ptrs in (("m", opt.m), ("v", opt.v)):
                t = ptrs[i].contents
                n = max(int(np.prod(SHAPES[i])), 1)
                view = Tensor(SHAPES[i], device=device, _ptr=t.data, _base=opt)
                out[f"{kind}/final/{name}{i}"] = view.numpy().copy().reshape(SHAPES[i]) if n else None
    return out, opt


def run_oracle(kind, lib):
    """The flat-array restatement in oracle/oracle.c, one parameter at a time."""
    f32p = C.POINTER(C.c_float)
    lib.oracle_sgd_step.argtypes = [f32p, f32p, C.c_uint64, C.c_float]
    lib.oracle_adam_step.argtypes = [f32p, f32p, f32p, f32p, C.c_uint64] + [C.c_float] * 4 + [C.c_int]
    lib.oracle_adamw_step.argtypes = [f32p, f32p, f32p, f32p, C.c_uint64] + [C.c_float] * 5 + [C.c_int]
    for fn in (lib.oracle_sgd_step, lib.oracle_adam_step, lib.oracle_adamw_step):
        fn.restype = None
    h = HYPER[kind]
    params = [np.ascontiguousarray(p) for p in initial_params()]
    ms = [np.zeros_like(p) for p in params]
    vs = [np.zeros_like(p) for p in params]
    ptr = lambda a: a.ctypes.data_as(f32p)
    out = {}
    for step in range(1, STEPS + 1):
        for i, p in enumerate(params):
            if i != NO_GRAD:
                g = np.ascontiguousarray(gradient(step, i))
                if kind == "sgd":
                    lib.oracle_sgd_step(ptr(p), ptr(g), p.size, h["lr"])
                elif kind == "adam":
                    lib.oracle_adam_step(ptr(p), ptr(g), ptr(ms[i]), ptr(vs[i]), p.size, h["lr"], h["beta1"],
                                         h["beta2"], h["epsilon"], step)
                else:
                    lib.oracle_adamw_step(ptr(p), ptr(g), ptr(ms[i]), ptr(vs[i]), p.size, h["lr"], h["beta1"],
                                          h["beta2"], h["epsilon"], h["weight_decay"], step)
            out[f"{kind}/step{step}/p{i}"] = p.copy()
    if kind != "sgd":
        for i in range(len(params)):
            out[f"{kind}/final/m{i}"] = ms[i].copy()
            out[f"{kind}/final/v{i}"] = vs[i].copy()
    return out
