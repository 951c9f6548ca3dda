#!/usr/bin/env python
"""Benchmark of the elementwise / reduce hot path: effective HBM GB/s per op.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-per-op]

Headline workload (benchmark configuration 2): the fused chain z = sigmoid(x) * y + exp(-abs(x)) over
2^28 fp32 elements per GPU (x ~ N(0,1) seed 0, y ~ N(0,1) seed 1), one step = one pass = one
launch of plast_b200_chain_forward. Algorithmic bytes per element: 12 (read x, y; write z).
The 3 GiB working set is far larger than L2, so no flush is needed between steps.

For N > 1 (torchrun, one rank per GPU) every rank runs its own 2^28-element shard (weak
scaling, no data-path collective: an elementwise op shards along its outermost dim); time is the
max over ranks of the CUDA-event time; value is the whole-job GB/s.

`--impl reference` times the reference's own CPU kernels (oracle/_ref, else the oracle port) on
the host cores for the same chain, on a bounded sample of the workload.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHARDED_TABLE_LIMIT_S = 240  # wall-clock limit of the multi-GPU per-op table (seconds)
N_ELEMS = 1 << 28
CPU_SAMPLE_ELEMS = 1 << 26    # elements of the 2^28 workload one CPU pass covers (both CPU legs)
BYTES_PER_ELEM = 12
METRIC = "effective_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM traffic of ONE launch of the chain kernel, from an ncu capture of this file's own command at
# --elems 67108864 (dram__bytes_read.sum / dram__bytes_write.sum, three launches averaged; the
# 2^28-element launch holds 3 GiB, beyond what a multi-pass capture may save and restore):
NCU_READ_BYTES_AT_2P26 = 536_909_227      # algorithmic 536 870 912: every operand byte crosses DRAM once
NCU_WRITE_BYTES_AT_2P26 = 224_770_048     # algorithmic 268 435 456: the rest is still dirty in L2 at kernel end
L2_DIRTY_RESIDUE_BYTES = (1 << 28) - NCU_WRITE_BYTES_AT_2P26   # ~44 MB, bounded by L2, does not grow with n

CHAIN_STEPS = [("neg", 0, 0, 0.0), ("exp", 2, 0, 0.0), ("add_scalar", 3, 0, 1.0),
               ("rdiv_scalar", 4, 0, 1.0), ("mul", 5, 1, 0.0), ("abs", 0, 0, 0.0),
               ("neg", 7, 0, 0.0), ("exp", 8, 0, 0.0), ("add", 6, 9, 0.0)]


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- reference / oracle CPU arm -------------------------------------------------------------------
def host_threads() -> int:
    """Cores this process may run on. torchrun exports OMP_NUM_THREADS=1 to its workers, which would
    silently make the CPU arm single-threaded, so the count is set explicitly: in the environment
    (read by libgomp when it starts) and through omp_set_num_threads (if it already has)."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    try:
        gomp = C.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(C.c_int(cores))
    except OSError:
        pass
    return cores


def cpu_backend():
    """The reference's own CPU kernels (oracle/_ref, kind 'reference') where they were built, else
    the oracle port (kind 'port')."""
    sys.path.insert(0, str(ROOT / "tests"))
    cores = host_threads()
    from harness import CpuBackend, have_ref, build_oracle
    if have_ref():
        return CpuBackend("ref"), "reference", cores
    build_oracle()
    return CpuBackend("oracle"), "port", cores


def cpu_chain_baseline(n_sample: int, reps: int):
    """Times the 9-op chain through the reference's CPU entry points (kind 'reference') or the
    oracle port (kind 'port') on n_sample elements; returns (GB/s by the 12 B/el count, info)."""
    be, kind, cores = cpu_backend()
    rs = np.random.RandomState(0)
    x = be.tensor(rs.randn(n_sample).astype(np.float32))
    y = be.tensor(np.random.RandomState(1).randn(n_sample).astype(np.float32))
    one = be.tensor(np.float32(1.0).reshape(()))
    t = [be.empty((n_sample,)) for _ in range(9)]

    def chain():
        be.forward("neg", [x], t[0]); be.forward("exp", [t[0]], t[1]); be.forward("add", [t[1], one], t[2])
        be.forward("div", [one, t[2]], t[3]); be.forward("mul", [t[3], y], t[4]); be.forward("abs", [x], t[5])
        be.forward("neg", [t[5]], t[6]); be.forward("exp", [t[6]], t[7]); be.forward("add", [t[4], t[7]], t[8])

    chain()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        chain()
        times.append(time.perf_counter() - t0)
    best = min(times)
    gbs = BYTES_PER_ELEM * n_sample / best / 1e9
    info = {"value": gbs, "unit": UNIT, "cores": cores, "omp_num_threads": cores, "kind": kind,
            "sample": f"9-op chain (neg,exp,+1,1/.,mul,abs,neg,exp,add) on 2^{int(np.log2(n_sample))} "
                      f"of the 2^28 elements, best of {reps}, {best * 1e3:.1f} ms; contiguous "
                      "elementwise kernels of the reference are single-threaded by construction"}
    return gbs, info, float(np.mean(times))


def cpu_per_op_baselines(rows):
    """Adds the reference's CPU figure to every per-op row: `cpu_baseline_gbps` (by the row's own
    algorithmic byte count, scaled to the sample), `cpu_baseline_ms` and `cpu_baseline_sample`.

    Every row is timed through the reference's own entry points (`<op>_cpu_forward/backward`,
    `*_step_cpu`, `tensor_pack_init`; the oracle port where the reference was not built) as the op
    sequence the reference runs for that row (plast/nn/functional.py:24-47, 77-97, 312-333), with all
    host threads, outputs pre-allocated, best of a few passes, on a bounded sample of the row's
    tensor so that the whole table costs well under a minute."""
    be, kind, cores = cpu_backend()
    import plast_b200 as pb
    FULL = pb.FULL_REDUCE
    rs = np.random.RandomState

    def best(fn, budget=0.8):
        fn()                                           # touches the output pages
        times, t_end = [], time.perf_counter() + budget
        while len(times) < 2 or (time.perf_counter() < t_end and len(times) < 8):
            t0 = time.perf_counter(); fn(); times.append(time.perf_counter() - t0)
        return min(times)

    def U(seed, shape, lo=-1.0, hi=1.0):
        return rs(seed).uniform(lo, hi, shape).astype(np.float32)

    def Nrm(seed, shape, std=1.0):
        return (std * rs(seed).randn(*shape)).astype(np.float32)

    fns = {}     # (config, op) -> (callable, fraction of the row's elements in the sample, sample text)

    # config 1 at full size
    M = 1024
    A, b = be.tensor(U(0, (M, M))), be.tensor(U(1, (1, M)), requires_grad=True)
    AB, Cc, s1 = be.empty((M, M), requires_grad=True), be.empty((M, M), requires_grad=True), be.empty((M,))
    Cc.grad.copy_from(Nrm(2, (M, M)))
    add1 = lambda: be.forward("add", [A, b], AB)
    relu1 = lambda: be.forward("leaky_relu", [AB], Cc, fval=0.0)
    sum1 = lambda: be.forward("sum", [Cc], s1, dim=1)
    full1 = "full size"
    fns[(1, "add_broadcast")] = (add1, 1.0, full1)
    fns[(1, "relu")] = (relu1, 1.0, full1)
    fns[(1, "row_sum")] = (sum1, 1.0, full1)
    fns[(1, "fused_add_relu")] = (lambda: (add1(), relu1()), 1.0, full1 + ", as add -> leaky_relu")
    for name in ("fused_fwd_C_and_row_sum", "forward_dag_as_cuda_graph", "forward_dag_node_by_node"):
        fns[(1, name)] = (lambda: (add1(), relu1(), sum1()), 1.0, full1 + ", as add -> leaky_relu -> sum")
    bwd1 = lambda: (be.backward("leaky_relu", [AB], Cc, fval=0.0), be.backward("add", [A, b], AB))
    fns[(1, "fused_bwd_grad_b")] = (bwd1, 1.0, full1 + ", as leaky_relu backward -> add backward")
    for name in ("forward_and_backward_dag_as_cuda_graph", "forward_and_backward_dag_node_by_node"):
        fns[(1, name)] = (lambda: (add1(), relu1(), sum1(), bwd1()), 1.0,
                          full1 + ", as add -> leaky_relu -> sum, then leaky_relu backward -> add backward")

    # config 2: 2^24 of the 2^28 elements
    n2, full2 = 1 << 24, float(1 << 28)
    x, y = be.tensor(Nrm(0, (n2,))), be.tensor(Nrm(1, (n2,)))
    one = be.tensor(np.float32(1.0).reshape(()))
    t2 = [be.empty((n2,)) for _ in range(4)]
    smp2 = "2^24 of 2^28 elements"
    for op in ("neg", "exp", "abs"):
        fns[(2, op)] = (lambda op=op: be.forward(op, [x], t2[0]), n2 / full2, smp2)
    fns[(2, "neg_with_reference_arena_fill")] = (lambda: (C.memset(t2[0].c.data, 0, n2 * 4), be.forward("neg", [x], t2[0])),
                                                 n2 / full2, smp2 + ", output zero-filled first as the arena does")
    fns[(2, "neg_with_output_fill_skipped")] = (lambda: be.forward("neg", [x], t2[0]), n2 / full2, smp2)
    fns[(2, "add_scalar")] = (lambda: be.forward("add", [x, one], t2[0]), n2 / full2, smp2)
    fns[(2, "rdiv_scalar")] = (lambda: be.forward("div", [one, x], t2[0]), n2 / full2, smp2)
    fns[(2, "mul")] = (lambda: be.forward("mul", [x, y], t2[0]), n2 / full2, smp2)
    fns[(2, "add")] = (lambda: be.forward("add", [x, y], t2[0]), n2 / full2, smp2)

    def sigmoid2():
        be.forward("neg", [x], t2[0]); be.forward("exp", [t2[0]], t2[0])
        be.forward("add", [t2[0], one], t2[0]); be.forward("div", [one, t2[0]], t2[0])

    def chain2():
        sigmoid2(); be.forward("mul", [t2[0], y], t2[1]); be.forward("abs", [x], t2[2])
        be.forward("neg", [t2[2]], t2[2]); be.forward("exp", [t2[2]], t2[2]); be.forward("add", [t2[1], t2[2]], t2[3])

    fns[(2, "sigmoid_fused")] = (sigmoid2, n2 / full2, smp2 + ", as neg -> exp -> +1 -> 1/.")
    for name in ("fused_chain", "chain_as_9_launches", "chain_fused_by_graph_pass"):
        fns[(2, name)] = (chain2, n2 / full2, smp2 + ", as the nine ops")

    # config 3: 2048 of the 65536 rows
    R3, C3 = 2048, 4096
    frac3, smp3 = R3 / 65536.0, "2048 of 65536 rows"
    X3 = be.tensor(Nrm(0, (R3, C3), std=2.0))
    lab3 = rs(1).randint(0, C3, size=R3)
    onehot = np.zeros((R3, C3), np.float32); onehot[np.arange(R3), lab3] = 1.0
    OH = be.tensor(onehot)
    r3, k3 = be.empty((R3,)), [be.empty((R3, 1)) for _ in range(2)]
    W3 = [be.empty((R3, C3)) for _ in range(2)]
    sc3 = be.empty((1,))
    for op in ("sum", "mean", "max"):
        fns[(3, f"row_{op}")] = (lambda op=op: be.forward(op, [X3], r3, dim=1), frac3, smp3)
    X3np = X3.numpy()
    fns[(3, "row_argmax")] = (lambda: np.argmax(X3np, axis=1), frac3,
                              smp3 + "; the reference has no argmax op, numpy.argmax (what its examples call) is timed")

    def softmax3():
        be.forward("max", [X3], k3[0], dim=1, keepdim=1); be.forward("sub", [X3, k3[0]], W3[0])
        be.forward("exp", [W3[0]], W3[0]); be.forward("sum", [W3[0]], k3[1], dim=1, keepdim=1)
        be.forward("div", [W3[0], k3[1]], W3[1])

    def log_softmax3():
        be.forward("max", [X3], k3[0], dim=1, keepdim=1); be.forward("sub", [X3, k3[0]], W3[0])
        be.forward("exp", [W3[0]], W3[1]); be.forward("sum", [W3[1]], k3[1], dim=1, keepdim=1)
        be.forward("log", [k3[1]], k3[1]); be.forward("sub", [W3[0], k3[1]], W3[1])

    def ce3():
        log_softmax3(); be.forward("mul", [W3[1], OH], W3[0]); be.forward("sum", [W3[0]], r3, dim=1)
        be.forward("neg", [r3], r3); be.forward("mean", [r3], sc3, dim=FULL)

    fns[(3, "softmax")] = (softmax3, frac3, smp3 + ", as max -> sub -> exp -> sum -> div")
    fns[(3, "log_softmax")] = (log_softmax3, frac3, smp3 + ", as max -> sub -> exp -> sum -> log -> sub")
    fns[(3, "cross_entropy_mean")] = (ce3, frac3, smp3 + ", as log_softmax -> * one-hot -> sum -> neg -> mean "
                                      "(the one-hot matrix is built outside the timed region)")

    # backward of the three, as the reverse of those op sequences over tensors that carry gradients
    # (src/core/graph.c:57-65 order; the forward pass runs once, outside the timed region)
    def graph3():
        xg = be.tensor(X3np, requires_grad=True)
        m = be.empty((R3, 1), requires_grad=True); be.forward("max", [xg], m, dim=1, keepdim=1)
        sh = be.empty((R3, C3), requires_grad=True); be.forward("sub", [xg, m], sh)
        e = be.empty((R3, C3), requires_grad=True); be.forward("exp", [sh], e)
        s = be.empty((R3, 1), requires_grad=True); be.forward("sum", [e], s, dim=1, keepdim=1)
        head = lambda: (be.backward("sum", [e], s, dim=1, keepdim=1), be.backward("exp", [sh], e),
                        be.backward("sub", [xg, m], sh), be.backward("max", [xg], m, dim=1, keepdim=1))
        return xg, sh, e, s, head

    G3 = Nrm(3, (R3, C3))
    xg, sh, e, s, head = graph3()
    ysm = be.empty((R3, C3), requires_grad=True); be.forward("div", [e, s], ysm); ysm.grad.copy_from(G3)
    fns[(3, "softmax_backward")] = (lambda e=e, s=s, ysm=ysm, head=head: (be.backward("div", [e, s], ysm), head()), frac3,
                                    smp3 + ", as div / sum / exp / sub / max backward")
    xg2, sh2, e2, s2, head2 = graph3()
    ls2 = be.empty((R3, 1), requires_grad=True); be.forward("log", [s2], ls2)
    yls = be.empty((R3, C3), requires_grad=True); be.forward("sub", [sh2, ls2], yls); yls.grad.copy_from(G3)
    lsm_bwd = lambda: (be.backward("sub", [sh2, ls2], yls), be.backward("log", [s2], ls2), head2())
    fns[(3, "log_softmax_backward")] = (lsm_bwd, frac3, smp3 + ", as sub / log / sum / exp / sub / max backward")
    prod = be.empty((R3, C3), requires_grad=True); be.forward("mul", [yls, OH], prod)
    rsum = be.empty((R3,), requires_grad=True); be.forward("sum", [prod], rsum, dim=1)
    ngl = be.empty((R3,), requires_grad=True); be.forward("neg", [rsum], ngl)
    lss = be.empty((1,), requires_grad=True); be.forward("mean", [ngl], lss, dim=FULL)
    lss.grad.copy_from(np.ones(1, np.float32))
    fns[(3, "cross_entropy_backward")] = (lambda: (be.backward("mean", [ngl], lss, dim=FULL), be.backward("neg", [rsum], ngl),
                                                   be.backward("sum", [prod], rsum, dim=1), be.backward("mul", [yls, OH], prod),
                                                   lsm_bwd()), frac3,
                                          smp3 + ", as mean / neg / sum / mul backward, then log_softmax backward")

    # config 4: a 4096 x 4096 corner of the 8192 x 8192 tensor
    M4 = 4096
    frac4, smp4 = (M4 * M4) / float(8192 * 8192), "4096 x 4096 of 8192 x 8192"
    X4 = be.tensor(U(0, (M4, M4)))
    X4T = X4.transpose(0, 1)
    Y4, Z4, c4 = be.tensor(U(1, (M4, M4))), be.empty((M4, M4)), be.empty((M4,))
    for name, tin in (("", X4), ("_transposed_view", X4T)):
        fns[(4, "sum_axis0" + name)] = (lambda tin=tin: be.forward("sum", [tin], c4, dim=0), frac4, smp4)
        fns[(4, "full_sum" + name)] = (lambda tin=tin: be.forward("sum", [tin], sc3, dim=FULL), frac4, smp4)
        fns[(4, "full_max" + name)] = (lambda tin=tin: be.forward("max", [tin], sc3, dim=FULL), frac4, smp4)
    fns[(4, "add_transposed_view_plus_contiguous")] = (lambda: be.forward("add", [X4T, Y4], Z4), frac4, smp4)
    Y4T = Y4.transpose(0, 1)
    fns[(4, "add_of_two_transposed_views")] = (lambda: be.forward("add", [X4T, Y4T], Z4), frac4, smp4)
    I3, J3, K3 = 64, 256, 1024                       # the same 2^24 elements seen as a 3-D tensor
    a3 = X4.view([I3, J3, K3], [1, I3, I3 * J3])
    b3 = Y4.view([I3, J3, K3], [K3 * J3, 1, J3])
    z3 = Z4.view([I3, J3, K3], [J3 * K3, K3, 1])
    fns[(4, "add_inputs_transposed_along_two_different_dims")] = (lambda: be.forward("add", [a3, b3], z3), frac4,
                                                                  smp4 + " seen as [64, 256, 1024]")
    if kind == "reference":
        class Pack(C.Structure):
            _fields_ = [("data", C.c_void_p), ("_buf", C.c_void_p)]
        be.lib.tensor_pack_init.argtypes = [C.POINTER(Pack), C.POINTER(pb.CTensor)]
        be.lib.tensor_pack_release.argtypes = [C.POINTER(Pack)]

        def pack4():
            pk = Pack()
            be.lib.tensor_pack_init(C.byref(pk), C.byref(X4T.c))
            be.lib.tensor_pack_release(C.byref(pk))
        fns[(4, "pack_transposed_view")] = (pack4, frac4, smp4 + ", tensor_pack_init (allocates its buffer per call)")

    # config 5: 4 of the 256 images
    sh5, psh = (4, 256, 56, 56), (1, 256, 1, 1)
    frac5, smp5 = 4 / 256.0, "4 of 256 images"
    X5, S5 = be.tensor(Nrm(0, sh5)), be.tensor(U(1, psh, -.5, .5))
    B5 = be.tensor(U(2, psh, -.5, .5), requires_grad=True)
    XS5, XSB5, Y5 = be.empty(sh5), be.empty(sh5, requires_grad=True), be.empty(sh5, requires_grad=True)
    Y5.grad.copy_from(Nrm(3, sh5))

    def fwd5():
        be.forward("mul", [X5, S5], XS5); be.forward("add", [XS5, B5], XSB5); be.forward("leaky_relu", [XSB5], Y5, fval=0.0)

    fns[(5, "scale_bias_relu_fwd")] = (fwd5, frac5, smp5 + ", as mul -> add -> leaky_relu")
    fns[(5, "bias_grad_masked_reduce")] = (lambda: (be.backward("leaky_relu", [XSB5], Y5, fval=0.0),
                                                    be.backward("add", [XS5, B5], XSB5)),
                                           frac5, smp5 + ", as leaky_relu backward -> add backward (broadcast-gradient reduce)")

    # optimiser steps: 2 of the 12 (matrix, bias) pairs
    if kind == "reference":
        from plast_b200 import optim as O

        class CArena(C.Structure):
            _fields_ = [("current", C.c_void_p), ("device", C.c_int)]
        be.lib.arena_create.argtypes = [C.c_uint64, C.c_int]
        be.lib.arena_create.restype = CArena
        shapes = [(4096, 2048), (4096,)] * 2
        params = []
        for i, sh in enumerate(shapes):
            pt = be.tensor(Nrm(10 + i, sh, 0.1), requires_grad=True)
            pt.grad.copy_from(Nrm(50 + i, sh, 0.01))
            params.append(pt)
        arr = O.param_array(params)
        frac6, smp6 = 2 / 12.0, "2 of the 12 (matrix, bias) pairs"
        n6 = sum(int(np.prod(sh)) for sh in shapes)
        keep = []   # the arena structs the optimisers point at must outlive the timing loop
        for kindname, struct in (("sgd", O.SGD), ("adam", O.Adam), ("adamw", O.AdamW)):
            arenas = [be.lib.arena_create(1 << 20, 0), be.lib.arena_create(n6 * 8 + (1 << 20), 0)]
            keep.append(arenas)
            fn = getattr(be.lib, f"{kindname}_step_cpu")
            fn.argtypes = [C.POINTER(struct), C.POINTER(C.POINTER(pb.CTensor)), C.c_int]
            fn.restype = None
            opt = struct()
            opt.lr = 1e-3
            if kindname != "sgd":
                opt.beta1, opt.beta2, opt.epsilon, opt.t = 0.9, 0.999, 1e-8, 0
                opt.optimizer_arena, opt.data_arena = C.addressof(arenas[0]), C.addressof(arenas[1])
            if kindname == "adamw":
                opt.weight_decay = 0.01
            fns[(6, f"{kindname}_step_24_params")] = (lambda fn=fn, opt=opt, keep=keep: fn(C.byref(opt), arr, len(params)),
                                                      frac6, smp6)

    # tall column sums: 8192 rows of each shape
    for rows7, cols7 in ((65536, 256), (262144, 128), (32768, 512), (16384, 2048), (8192, 1024)):
        X7, o7 = be.tensor(Nrm(20, (8192, cols7))), be.empty((cols7,))
        fns[(7, f"sum_axis0_{rows7}x{cols7}")] = (lambda X7=X7, o7=o7: be.forward("sum", [X7], o7, dim=0), 8192.0 / rows7,
                                                  f"8192 of {rows7} rows")

    for row in rows:
        key = (row.get("config"), row.get("op"))
        if key not in fns or "bytes" not in row:
            continue
        fn, frac, sample = fns[key]
        try:
            sec = best(fn)
        except Exception as exc:   # a baseline that cannot run must not cost the table
            row["cpu_baseline_error"] = str(exc)[:120]
            continue
        row["cpu_baseline_gbps"] = round(row["bytes"] * frac / sec / 1e9, 3)
        row["cpu_baseline_ms"] = round(sec * 1e3, 3)
        row["cpu_baseline_sample"] = f"{sample}; {kind}, {cores} threads"


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = CPU_SAMPLE_ELEMS
    # K + W steps, each one pass of the chain over the sample
    sys.path.insert(0, str(ROOT / "tests"))
    gbs, info, _ = cpu_chain_baseline(n_sample, max(1, args.steps + args.warmup))
    ms = BYTES_PER_ELEM * n_sample / (gbs * 1e9) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 2: fused chain z = sigmoid(x)*y + exp(-abs(x)), fp32, "
                               f"bounded sample of 2^{int(np.log2(n_sample))} of 2^28 elements per step",
                   "l2": "n/a (host)"},
        "cpu_baseline": info,
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- clocks -----------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self._stop = threading.Event()
        self._th = None
        self.max_mhz = None

    def _init_nvml(self) -> bool:
        """NVML handle for the sampled GPU, set up BEFORE the timed region starts."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = None
            try:
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nv, self._h = nv, h
            self._bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                          "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                          "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                          "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            return True
        except Exception:
            self._nv = None
            return False

    def _run_nvml(self) -> bool:
        """NVML queries take well under a millisecond, so even a short timed region is sampled."""
        nv = getattr(self, "_nv", None)
        if nv is None:
            return False
        while True:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for n, b in self._bits.items():
                    if r & b:
                        self.reasons.add(n)
            except Exception:
                pass
            if self._stop.wait(0.002):
                break
        return True

    def _run(self):
        if self._run_nvml():
            return
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:6]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        self._init_nvml()
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=10)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---- our arm ----------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import plast_b200 as pb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG", "WARN")   # a caller that asks for NCCL's log gets it
        # No NVLink multicast objects: the data path has no collective, the tiny exchanges are
        # latency-bound either way, and a rank that left while its memory was bound to a multicast
        # object would fault its peers' GPUs.
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        # a collective that cannot complete raises after this long instead of hanging the job
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=SHARDED_TABLE_LIMIT_S + 60))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # launches go to torch's current stream so torch events bracket them
    pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))

    n = args.elems
    # configuration 2 inputs; rank r draws seeds (2r, 2r+1) so shards differ
    x_h = torch.from_numpy(np.random.RandomState(2 * rank).randn(n).astype(np.float32)).pin_memory()
    y_h = torch.from_numpy(np.random.RandomState(2 * rank + 1).randn(n).astype(np.float32)).pin_memory()
    z_h = torch.empty(n, dtype=torch.float32).pin_memory()
    x_d = torch.empty(n, dtype=torch.float32, device=dev)
    y_d = torch.empty(n, dtype=torch.float32, device=dev)
    z_d = torch.empty(n, dtype=torch.float32, device=dev)
    x_d.copy_(x_h); y_d.copy_(y_h)

    def wrap(t):
        """plast Tensor struct over a torch allocation (no copy)."""
        return pb.Tensor.wrap_pointer(t.data_ptr(), list(t.shape), owner=t)

    X, Y, Z = wrap(x_d), wrap(y_d), wrap(z_d)

    def step():
        pb.chain_forward([X, Y], Z, CHAIN_STEPS, check=False)

    step(); pb.check_error()
    torch.cuda.synchronize()
    # parity spot-check of the timed kernel against the oracle on a slice (outside the timed region)
    if rank == 0:
        sys.path.insert(0, str(ROOT / "tests"))
        from harness import OracleRecipes
        sl = slice(0, 1 << 16)
        xs, ys = x_h[sl].numpy(), y_h[sl].numpy()
        want = OracleRecipes().chain(xs, ys).astype(np.float64)
        got = z_d[sl].cpu().numpy().astype(np.float64)
        x64, y64 = xs.astype(np.float64), ys.astype(np.float64)
        terms = np.abs(y64) / (1 + np.exp(-x64)) + np.exp(-np.abs(x64))  # z = t + e2 may cancel
        assert (np.abs(got - want) <= 3 * 2.0 ** -23 * terms).all(), "bench: fused chain disagrees with the oracle"

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # The timed region (exactly K steps between two events, barrier + synchronise on both sides) is
    # run `--regions` times back to back; the reported time is the MEDIAN region, max over ranks,
    # and every region's time is listed, so a region of a few milliseconds is not a single sample.
    l0 = pb.lib.plast_b200_launch_count()
    region_ms = []
    for _ in range(max(args.regions, 1)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
        region_ms.append(ev0.elapsed_time(ev1))
    launches = int(pb.lib.plast_b200_launch_count() - l0) // max(args.regions, 1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor(region_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    regions_max = [float(v) for v in t.tolist()]
    ms_total = float(np.median(region_ms))          # this rank's kernel time, for the roofline
    ms_total_max = float(np.median(regions_max))
    ms_per_step = ms_total_max / args.steps
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_bytes = BYTES_PER_ELEM * n * world
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----------
    # The library's host-buffer entry point: pinned host arrays in, pinned host array out; chunks
    # are copied in, computed and copied out on three streams at once.
    host_in = [(x_h.data_ptr(), n), (y_h.data_ptr(), n)]
    host_out = (z_h.data_ptr(), n)

    def e2e_step():
        pb.chain_forward_host(host_in, host_out, CHAIN_STEPS, check=False)

    e2e_steps = min(args.steps, 10)
    z_h.zero_()
    e2e_step(); pb.check_error(); barrier()
    if rank == 0:   # the host result of the pipelined call equals the device-resident one
        assert torch.equal(z_h[: 1 << 20], z_d[: 1 << 20].cpu()) and torch.equal(z_h[-(1 << 20):], z_d[-(1 << 20):].cpu()), \
            "bench: host-buffer chain disagrees with the device-resident chain"
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 8 * n, "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
           "call": "plast_b200_chain_forward_host (pinned host buffers; 32 MiB chunks; copy-in, kernel and "
                   "copy-out of successive chunks overlap)"}

    peak, peak_kind = measured_peak()
    achieved = BYTES_PER_ELEM * n / (ms_total / args.steps * 1e-3) / 1e9  # this rank's kernel
    roofline = {"bound": "hbm", "kernel": "ew_kernel<SigmoidMulAddExpNegAbs, vec4, 1-D>",
                "achieved": achieved, "peak": peak, "peak_source": f"of {peak_kind}", "unit": UNIT,
                "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "traffic": None, "algorithmic_bytes_per_launch": BYTES_PER_ELEM * n}
    # per-launch DRAM traffic: measured reads scale with n, writes are the algorithmic bytes less
    # the fixed tail that is still dirty in L2 when the kernel ends
    if n >= (1 << 26):
        scale = n / float(1 << 26)
        roofline["traffic"] = int(NCU_READ_BYTES_AT_2P26 * scale + 4 * n - L2_DIRTY_RESIDUE_BYTES)
        roofline["traffic_source"] = ("ncu dram__bytes_read.sum at 2^26 elements scaled by n/2^26, plus 4 B/element "
                                      "written, minus the ~44 MB of stores ncu saw still dirty in L2 at kernel end")

    per_op = None
    if rank == 0 and world == 1 and not args.no_per_op:
        from plast_b200.opbench import per_op_table
        del x_h, y_h, z_h
        per_op = per_op_table(torch, pb, dev, peak, reps=args.op_reps,
                              configs=tuple(int(c) for c in args.configs.split(",")), chain_elems=args.elems)

    def headline(extra):
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 2: fused chain z = sigmoid(x)*y + exp(-abs(x)) on 2^28 fp32 "
                                   "elements per GPU, x,y ~ N(0,1) (numpy RandomState seeds 0,1)",
                       "algorithmic_bytes_per_element": BYTES_PER_ELEM, "elements_per_gpu": n,
                       "is_baseline_size": n == N_ELEMS,
                       "l2": "working set 3 GiB per GPU > 126 MB L2; no flush needed",
                       "sharding": "elements split across ranks, no collective"},
            "elements_per_s": n * world / (ms_per_step * 1e-3),
            "timed_regions": {"count": len(regions_max), "steps_each": args.steps,
                              "ms_per_step_each": [round(v / args.steps, 5) for v in regions_max],
                              "ms_per_step_min": round(min(regions_max) / args.steps, 5),
                              "ms_per_step_max": round(max(regions_max) / args.steps, 5),
                              "reported": "median region, max over ranks"},
            "roofline": roofline, "cpu_baseline": cpu_info, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks,
        }
        if per_op is not None:
            line["per_op"] = per_op
        line.update(extra)
        return line

    cpu_info = None
    if rank == 0 and world == 1:
        _, cpu_info, _ = cpu_chain_baseline(CPU_SAMPLE_ELEMS, 20)   # about 12 s of CPU work
        if per_op is not None:
            cpu_per_op_baselines(per_op)

    sharded = None
    if world > 1 and not args.no_per_op:
        # Strong scaling of the fixed config 3 / 4 / 5 tensors split across the ranks (local kernel
        # + exchange); every rank takes part. The table watches its own deadline between rows (all
        # ranks agree on it through the process group) and skips what is left, so nobody leaves in
        # the middle of an exchange. The headline above is already measured: should a collective
        # never complete all the same, a watchdog prints the JSON line without the table; it ends
        # no process (the process group's own timeout raises in the stuck rank).
        import threading
        from plast_b200.dist import sharded_reduction_table
        del x_h, y_h, z_h
        printed = threading.Lock()

        def give_up():
            if rank == 0 and printed.acquire(blocking=False):
                print(json.dumps(headline({"sharded_reductions_error": "timed out after %d s" % (SHARDED_TABLE_LIMIT_S + 30)})),
                      flush=True)

        watchdog = threading.Timer(SHARDED_TABLE_LIMIT_S + 30, give_up)
        watchdog.daemon = True
        watchdog.start()
        try:
            sharded = sharded_reduction_table(torch, dist, pb, dev, peak, reps=args.op_reps,
                                              deadline=time.monotonic() + SHARDED_TABLE_LIMIT_S)
        except Exception as exc:  # the table is an extra: never lose the headline to it
            sharded = [{"op": "sharded_table_failed", "error": str(exc)[:200]}]
        watchdog.cancel()
        torch.cuda.synchronize()
        if rank == 0 and not printed.acquire(blocking=False):
            dist.destroy_process_group()
            return  # the watchdog has printed

    if world > 1:
        dist.barrier()   # the other ranks stay quiet while rank 0 writes its one line
    if rank == 0:
        print(json.dumps(headline({"sharded_reductions": sharded} if sharded is not None else {})), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_per_op_only(args):
    import torch
    import plast_b200 as pb
    from plast_b200.opbench import per_op_table
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    peak, kind = measured_peak()
    cfgs = tuple(int(c) for c in args.configs.split(","))
    rows = per_op_table(torch, pb, dev, peak, reps=args.op_reps, configs=cfgs, chain_elems=args.elems)
    print(json.dumps({"per_op": rows, "peak_gbs": peak, "peak_source": f"of {kind}"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--elems", type=int, default=N_ELEMS,
                    help="elements per GPU (default 2^28, the benchmark size; smaller only for profiler captures)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--regions", type=int, default=5, help="how often the K-step timed region is repeated (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-per-op", action="store_true", help="skip the per-op table (configs 1-5 and the optimiser steps)")
    ap.add_argument("--op-reps", type=int, default=10)
    ap.add_argument("--per-op-only", action="store_true",
                    help="only the per-op table (1 GPU); with --op-reps 0 every op is launched 3 times and "
                         "not timed, which is the command the profiler captures use")
    ap.add_argument("--configs", default="1,2,3,4,5,6,7",
                    help="configs of the per-op table (6 = optimiser steps, 7 = column sums of tall matrices)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.per_op_only:
        run_per_op_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
