"""Per-op throughput table for the five benchmark configurations (used by bench.py).

Every row is one entry-point call through the C ABI on device-resident data, timed with CUDA
events on the launch stream (median of `reps`), reported as effective GB/s = algorithmic bytes
(each operand read once, each result written once) / time, and as a fraction of the measured
copy bandwidth and of the 8 TB/s nominal figure. Working sets under 256 MiB have L2 flushed
(a 512 MiB buffer is overwritten) before every timed launch; larger ones need no flush.

Inputs are synthetic with the shapes and value distributions of the configs, generated on the
device (the per-op numbers do not depend on the exact values).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

NOMINAL = 8000.0


def per_op_table(torch, pb, dev, peak_gbs: float, reps: int = 10, configs=(1, 2, 3, 4, 5, 6, 7),
                 chain_elems: int = 1 << 28):
    """chain_elems: length of configuration 2's vectors (2^28 in the benchmark; profiler captures use
    fewer so that the device memory a multi-pass capture has to save stays small)."""
    gen = torch.Generator(device=dev)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    flush_sink = torch.zeros(1, device=dev)
    rows = []

    def read_sweep():
        """Fills L2 with CLEAN lines of another buffer (a write sweep would leave dirty lines whose
        write-back is then billed to the kernel under test)."""
        flush_sink.copy_(flush_buf.view(torch.int32).sum().float().reshape(1))

    # what an event pair around nothing reads after such a sweep (subtract it from cold_ms by eye)
    pair = []
    for _ in range(5):
        read_sweep()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); e1.record(); torch.cuda.synchronize()
        pair.append(e0.elapsed_time(e1))
    empty_pair_ms = float(np.median(pair))

    def wrap(t, shape=None, strides=None, dtype=pb.FLOAT32):
        shape = list(t.shape) if shape is None else shape
        return pb.Tensor.wrap_pointer(t.data_ptr(), shape, strides=strides, dtype=dtype, owner=t)

    def randn(shape, seed, std=1.0):
        gen.manual_seed(seed)
        return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std

    def uniform(shape, seed, lo, hi):
        gen.manual_seed(seed)
        return torch.rand(shape, generator=gen, device=dev, dtype=torch.float32) * (hi - lo) + lo

    def timeit(cfg, name, fn, nbytes, elems, working_set, capture=True):
        flush = working_set < (256 << 20)
        fn(); pb.check_error()
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        kernel = pb.last_kernel()
        # Working sets beyond L2 are timed as `inner` back-to-back launches per event pair, so the
        # few microseconds between an event and the first launch after it are not billed to a 40 us
        # kernel (20 launches for kernels under 100 us, 5 for longer ones); small working sets need
        # the flush before every launch and are timed one launch at a time.
        inner = 1
        if not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); fn(); e1.record()
            torch.cuda.synchronize()
            inner = 20 if e0.elapsed_time(e1) / 2 < 0.1 else 5
        times = []
        for _ in range(reps):
            if flush:
                flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(inner):
                fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / inner)
        if not times:   # --op-reps 0: every op launched, nothing timed (the profiler-capture mode)
            rows.append({"config": cfg, "op": name, "kernel": kernel, "bytes": int(nbytes), "timed": False})
            return
        ms = float(np.median(times))
        gbs = nbytes / (ms * 1e-3) / 1e9
        cold = None
        if not flush and working_set < (1 << 30) and reps > 0:
            # Working sets between L2 and 1 GiB: part of the tensor survives in the 126 MB L2 from one
            # back-to-back launch to the next. cold_ms: ONE launch per event pair after a read sweep
            # of a 512 MiB buffer (includes the event pair's own ~2.6 us; the timer ticks in ~2 us).
            ct = []
            for _ in range(max(reps, 9)):
                read_sweep()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                ct.append(e0.elapsed_time(e1))
            cold = float(np.median(ct))
        row = {"config": cfg, "op": name, "kernel": kernel, "ms": round(ms, 5),
               "bytes": int(nbytes), "GBps": round(gbs, 1), "elements_per_s": elems / (ms * 1e-3),
               "frac_of_measured": round(gbs / peak_gbs, 4), "frac_of_nominal": round(gbs / NOMINAL, 4),
               "l2_flushed": flush, "launches_per_timed_region": inner}
        if cold is not None:
            row["cold_ms"] = round(cold, 5)
            row["cold_GBps"] = round(nbytes / (cold * 1e-3) / 1e9, 1)
            row["empty_event_pair_ms"] = round(empty_pair_ms, 5)
        if flush and reps > 0:
            # Launch-bound sizes: the same call 50 times back to back in the stream (data stays in L2) ...
            bt = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(50):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                bt.append(e0.elapsed_time(e1) / 50)
            row["stream_ms_per_call_l2_resident"] = round(float(np.median(bt)), 5)
        if reps > 0 and capture:
            # ... and the launches replayed from one CUDA graph (no host cost, ~1 us instead of ~4 us
            # between dependent kernels) - what a graph-capturing scheduler sees. 50 launches per
            # graph for the small working sets (data stays in L2), 10 for the large ones.
            n_graph = 50 if flush else 10
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    pb.lib.plast_b200_set_stream(C.c_void_p(side.cuda_stream))
                    fn()
                    with torch.cuda.graph(graph, stream=side):
                        for _ in range(n_graph):
                            fn()
                pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
                torch.cuda.synchronize()
                graph.replay()
                gt = []
                for _ in range(5):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(); graph.replay(); e1.record()
                    torch.cuda.synchronize()
                    gt.append(e0.elapsed_time(e1) / n_graph)
                gms = float(np.median(gt))
                if flush:
                    row["graph_replay_ms_per_launch_l2_resident"] = round(gms, 5)
                    row["graph_replay_GBps_l2_resident"] = round(nbytes / (gms * 1e-3) / 1e9, 1)
                else:
                    row["graph_replay_ms_per_launch"] = round(gms, 5)
                    row["graph_replay_GBps"] = round(nbytes / (gms * 1e-3) / 1e9, 1)
                    row["graph_replay_frac_of_nominal"] = round(nbytes / (gms * 1e-3) / 1e9 / NOMINAL, 4)
            except Exception as exc:  # capture is an extra; never fail the table for it
                pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
                row["graph_replay_error"] = str(exc)[:120]
        rows.append(row)

    F = 4
    if 1 in configs:
        M = N = 1024
        A, b, G = uniform((M, N), 0, -1, 1), uniform((1, N), 1, -1, 1), randn((M, N), 2)
        AB, Cc, s = torch.empty_like(A), torch.empty_like(A), torch.empty(M, device=dev)
        gb = torch.zeros((1, N), device=dev)
        tA, tb, tAB, tC, ts = wrap(A), wrap(b), wrap(AB), wrap(Cc), wrap(s)
        ws = 3 * M * N * F
        timeit(1, "add_broadcast", lambda: pb.forward("add", [tA, tb], tAB, check=False), (2 * M * N + N) * F, M * N, ws)
        timeit(1, "relu", lambda: pb.forward("leaky_relu", [tAB], tC, fval=0.0, check=False), 2 * M * N * F, M * N, ws)
        timeit(1, "row_sum", lambda: pb.forward("sum", [tC], ts, dim=1, check=False), (M * N + M) * F, M * N, ws)
        timeit(1, "fused_add_relu", lambda: pb.forward("add_leaky_relu", [tA, tb], tC, fval=0.0, check=False),
               (2 * M * N + N) * F, M * N, ws)
        timeit(1, "fused_fwd_C_and_row_sum",
               lambda: pb.lib.plast_b200_add_leaky_relu_row_sum(C.byref(tA.c), C.byref(tb.c), C.byref(tC.c), C.byref(ts.c), 0.0),
               (2 * M * N + N + M) * F, M * N, ws)
        # the whole forward graph (fused add + relu node, row-sum node) replayed as ONE CUDA graph
        from . import graph as G1
        g1 = G1.Graph()
        g1.node("ADD", [tA, tb], tAB); g1.node("LEAKY_RELU", [tAB], tC, fval=0.0); g1.node("SUM", [tC], ts, dim=1)
        dag1 = g1.dag()
        G1.fuse(dag1, G1.FUSE_CHAINS_WITH_GRAD)
        G1.dag_forward(dag1)
        h1 = G1.capture(dag1)
        if h1:
            timeit(1, "forward_dag_as_cuda_graph", lambda: G1.replay(h1), (2 * M * N + N + M * N + M) * F, M * N, ws,
                   capture=False)
        timeit(1, "forward_dag_node_by_node", lambda: G1.dag_forward(dag1), (2 * M * N + N + M * N + M) * F, M * N, ws)
        # the whole training step of the configuration (forward C and s, backward from the upstream
        # gradient on C into b.grad) as ONE replayed CUDA graph: fused add + relu, row sum, their two
        # backward nodes (the sum's contributes a zero gradient here)
        gb2, gs2 = torch.zeros((1, N), device=dev), torch.zeros(M, device=dev)
        tb2 = wrap(b); tb2.c.requires_grad = True
        gtb2 = wrap(gb2); tb2.grad = gtb2; tb2.c.grad = C.pointer(gtb2.c)
        tAB2 = wrap(AB); tAB2.c.requires_grad = True
        gAB2 = wrap(torch.zeros_like(A)); tAB2.grad = gAB2; tAB2.c.grad = C.pointer(gAB2.c)
        tC2 = wrap(Cc); tC2.c.requires_grad = True
        gC2 = wrap(G); tC2.grad = gC2; tC2.c.grad = C.pointer(gC2.c)
        ts2 = wrap(s); ts2.c.requires_grad = True
        gts2 = wrap(gs2); ts2.grad = gts2; ts2.c.grad = C.pointer(gts2.c)
        g2 = G1.Graph()
        g2.node("ADD", [tA, tb2], tAB2); g2.node("LEAKY_RELU", [tAB2], tC2, fval=0.0); g2.node("SUM", [tC2], ts2, dim=1)
        dag2 = g2.dag()
        G1.fuse(dag2, G1.FUSE_CHAINS_WITH_GRAD)
        G1.dag_forward(dag2); G1.dag_backward(dag2)
        h2 = G1.capture(dag2, 2)
        step_bytes = (2 * M * N + N + M * N + M) * F + (M * N + M) * F + (2 * M * N + 2 * N) * F
        if h2:
            timeit(1, "forward_and_backward_dag_as_cuda_graph", lambda: G1.replay(h2), step_bytes, M * N, ws, capture=False)
        timeit(1, "forward_and_backward_dag_node_by_node", lambda: (G1.dag_forward(dag2), G1.dag_backward(dag2)),
               step_bytes, M * N, ws)
        tbg = wrap(b); tbg.c.requires_grad = True
        gtb = wrap(gb); tbg.grad = gtb; tbg.c.grad = C.pointer(gtb.c)
        tCg = wrap(Cc); gC = wrap(G); tCg.grad = gC; tCg.c.grad = C.pointer(gC.c)
        timeit(1, "fused_bwd_grad_b", lambda: pb.backward("add_leaky_relu", [tA, tbg], tCg, fval=0.0, check=False),
               (2 * M * N + 2 * N) * F, M * N, ws)
        del A, b, G, AB, Cc, s
    if 2 in configs:
        n = int(chain_elems)
        x, y, z = randn((n,), 0), randn((n,), 1), torch.empty(n, device=dev)
        one = torch.ones((), device=dev)
        tx, ty, tz = wrap(x), wrap(y), wrap(z)
        tone = wrap(one, shape=[])
        ws = 3 * n * F
        for op in ("neg", "exp", "abs"):
            timeit(2, op, lambda op=op: pb.forward(op, [tx], tz, check=False), 2 * n * F, n, ws)
        timeit(2, "add_scalar", lambda: pb.forward("add", [tx, tone], tz, check=False), 2 * n * F, n, ws)
        timeit(2, "rdiv_scalar", lambda: pb.forward("div", [tone, tx], tz, check=False), 2 * n * F, n, ws)
        timeit(2, "mul", lambda: pb.forward("mul", [tx, ty], tz, check=False), 3 * n * F, n, ws)
        timeit(2, "add", lambda: pb.forward("add", [tx, ty], tz, check=False), 3 * n * F, n, ws)
        timeit(2, "sigmoid_fused", lambda: pb.forward("sigmoid", [tx], tz, check=False), 2 * n * F, n, ws)
        # What the reference's arena adds on the caller's side of every op (src/core/arena.c:94-102:
        # each output is zero-filled when allocated, then overwritten by its op): the fill call
        # followed by the op, with the reference's fill policy and with the fill skipped for op
        # outputs (plast_b200_arena_fill_policy). Same 8 algorithmic bytes per element in both rows.
        def neg_after_arena_fill(policy):
            pb.lib.plast_b200_arena_fill_policy(policy)
            pb.lib.arena_memset_cuda(C.c_void_p(z.data_ptr()), 0, n * F)
            pb.lib.plast_b200_arena_fill_policy(0)
            pb.forward("neg", [tx], tz, check=False)
        timeit(2, "neg_with_reference_arena_fill", lambda: neg_after_arena_fill(0), 2 * n * F, n, ws)
        timeit(2, "neg_with_output_fill_skipped", lambda: neg_after_arena_fill(1), 2 * n * F, n, ws)
        steps = [("neg", 0, 0, 0.0), ("exp", 2, 0, 0.0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
                 ("mul", 5, 1, 0.0), ("abs", 0, 0, 0.0), ("neg", 7, 0, 0.0), ("exp", 8, 0, 0.0), ("add", 6, 9, 0.0)]
        timeit(2, "fused_chain", lambda: pb.chain_forward([tx, ty], tz, steps, check=False), 3 * n * F, n, ws)
        # the same chain as nine separate launches (what the reference scheduler issues)
        t = [torch.empty(n, device=dev) for _ in range(4)]
        w = [wrap(v) for v in t]

        def unfused():
            pb.forward("neg", [tx], w[0], check=False); pb.forward("exp", [w[0]], w[0], check=False)
            pb.forward("add", [w[0], tone], w[0], check=False); pb.forward("div", [tone, w[0]], w[0], check=False)
            pb.forward("mul", [w[0], ty], w[1], check=False); pb.forward("abs", [tx], w[2], check=False)
            pb.forward("neg", [w[2]], w[2], check=False); pb.forward("exp", [w[2]], w[2], check=False)
            pb.forward("add", [w[1], w[2]], tz, check=False)
        timeit(2, "chain_as_9_launches", unfused, 3 * n * F, n, ws)
        # the chain as the nine nodes the scheduler holds (the two 1.0 constants are 0-dim tensors),
        # collapsed by the graph fusion pass into one run-time compiled node
        from . import graph as G
        one_b = torch.ones((), device=dev)
        tone_b = wrap(one_b, shape=[])
        t2 = [torch.empty(n, device=dev) for _ in range(8)]              # one buffer per intermediate node
        w2 = [wrap(v) for v in t2]
        gr = G.Graph()
        gr.node("NEG", [tx], w2[0]); gr.node("EXP", [w2[0]], w2[1]); gr.node("ADD", [tone, w2[1]], w2[2])
        gr.node("DIV", [tone_b, w2[2]], w2[3]); gr.node("MUL", [w2[3], ty], w2[4])
        gr.node("ABS", [tx], w2[5]); gr.node("NEG", [w2[5]], w2[6]); gr.node("EXP", [w2[6]], w2[7])
        gr.node("ADD", [w2[4], w2[7]], tz)
        dag = gr.dag()
        if G.fuse(dag) == 1 and dag.count == 1:
            timeit(2, "chain_fused_by_graph_pass", lambda: G.dag_forward(dag), 3 * n * F + 8, n, ws)
        del t2, w2
        del x, y, z, t, w
    if 3 in configs:
        R, Cn = 65536, 4096
        X = randn((R, Cn), 0, std=2.0)
        Y = torch.empty_like(X)
        out = torch.empty(R, device=dev)
        outi = torch.empty(R, device=dev, dtype=torch.int32)
        gen.manual_seed(1)
        labels = torch.randint(0, Cn, (R,), generator=gen, device=dev, dtype=torch.int32)
        loss = torch.empty(1, device=dev)
        tX, tY, tout = wrap(X), wrap(Y), wrap(out)
        touti, tl, tloss = wrap(outi, dtype=pb.INT32), wrap(labels, dtype=pb.INT32), wrap(loss)
        ws = 2 * R * Cn * F
        for op in ("sum", "mean", "max"):
            timeit(3, f"row_{op}", lambda op=op: pb.forward(op, [tX], tout, dim=1, check=False),
                   (R * Cn + R) * F, R * Cn, ws)
        timeit(3, "row_argmax", lambda: pb.forward("argmax", [tX], touti, dim=1, check=False), (R * Cn + R) * F, R * Cn, ws)
        timeit(3, "softmax", lambda: pb.forward("softmax", [tX], tY, dim=1, check=False), 2 * R * Cn * F, R * Cn, ws)
        timeit(3, "log_softmax", lambda: pb.forward("log_softmax", [tX], tY, dim=1, check=False), 2 * R * Cn * F, R * Cn, ws)
        timeit(3, "cross_entropy_mean", lambda: pb.forward("cross_entropy", [tX, tl], tloss, check=False),
               (R * Cn + R) * F + 4, R * Cn, ws)
        # backward of the three (plast/nn/functional.py:77-97, 312-333 run in reverse): dx accumulates,
        # so a pass reads y (or the logits), dy and dx and writes dx
        dY, dX = randn((R, Cn), 3), torch.zeros((R, Cn), device=dev)
        dl = torch.ones(1, device=dev)
        tXg = wrap(X); tXg.c.requires_grad = True
        gX = wrap(dX); tXg.grad = gX; tXg.c.grad = C.pointer(gX.c)
        tYg = wrap(Y); gY = wrap(dY); tYg.grad = gY; tYg.c.grad = C.pointer(gY.c)
        tlg = wrap(loss); gl = wrap(dl); tlg.grad = gl; tlg.c.grad = C.pointer(gl.c)
        pb.forward("softmax", [tX], tY)
        timeit(3, "softmax_backward", lambda: pb.backward("softmax", [tXg], tYg, dim=1, check=False), 4 * R * Cn * F, R * Cn, 4 * R * Cn * F)
        pb.forward("log_softmax", [tX], tY)
        timeit(3, "log_softmax_backward", lambda: pb.backward("log_softmax", [tXg], tYg, dim=1, check=False), 4 * R * Cn * F, R * Cn, 4 * R * Cn * F)
        timeit(3, "cross_entropy_backward", lambda: pb.backward("cross_entropy", [tXg, tl], tlg, check=False), 3 * R * Cn * F, R * Cn, 3 * R * Cn * F)
        del X, Y, dY, dX
    if 4 in configs:
        M = 8192
        X = uniform((M, M), 0, -1, 1)
        out, one = torch.empty(M, device=dev), torch.empty(1, device=dev)
        tX, tout, tone = wrap(X), wrap(out), wrap(one)
        tXT = wrap(X, shape=[M, M], strides=[1, M])
        ws = M * M * F
        for name, tin in (("", tX), ("_transposed_view", tXT)):
            timeit(4, "sum_axis0" + name, lambda tin=tin: pb.forward("sum", [tin], tout, dim=0, check=False),
                   (M * M + M) * F, M * M, ws)
            timeit(4, "full_sum" + name, lambda tin=tin: pb.forward("sum", [tin], tone, dim=pb.FULL_REDUCE, check=False),
                   M * M * F + 4, M * M, ws)
            timeit(4, "full_max" + name, lambda tin=tin: pb.forward("max", [tin], tone, dim=pb.FULL_REDUCE, check=False),
                   M * M * F + 4, M * M, ws)
        # elementwise ops on the transposed view: the view is staged through shared-memory tiles
        Y2, Z2 = uniform((M, M), 1, -1, 1), torch.empty((M, M), device=dev)
        tY2, tZ2 = wrap(Y2), wrap(Z2)
        timeit(4, "add_transposed_view_plus_contiguous", lambda: pb.forward("add", [tXT, tY2], tZ2, check=False),
               3 * M * M * F, M * M, 3 * ws)
        timeit(4, "pack_transposed_view", lambda: pb.lib.plast_b200_pack(C.byref(tXT.c), C.c_void_p(Z2.data_ptr())),
               2 * M * M * F, M * M, 2 * ws)
        tY2T = wrap(Y2, shape=[M, M], strides=[1, M])
        timeit(4, "add_of_two_transposed_views", lambda: pb.forward("add", [tXT, tY2T], tZ2, check=False),
               3 * M * M * F, M * M, 3 * ws)
        # 3-D, the two inputs contiguous along two DIFFERENT dims, neither of them the output's:
        # out[i, j, k] = a.transpose(0, 2) + b.transpose(1, 2) on [128, 512, 1024] (same 2^26 elements)
        I3, J3, K3 = 128, 512, 1024
        t3a = wrap(X, shape=[I3, J3, K3], strides=[1, I3, I3 * J3])          # memory order [K, J, I]
        t3b = wrap(Y2, shape=[I3, J3, K3], strides=[K3 * J3, 1, J3])          # memory order [I, K, J]
        t3z = wrap(Z2, shape=[I3, J3, K3])
        timeit(4, "add_inputs_transposed_along_two_different_dims", lambda: pb.forward("add", [t3a, t3b], t3z, check=False),
               3 * M * M * F, M * M, 3 * ws)
        del X, Y2, Z2
    if 5 in configs:
        shape, pshape = (256, 256, 56, 56), (1, 256, 1, 1)
        n = int(np.prod(shape))
        X, G = randn(shape, 0), randn(shape, 3)
        S, B = uniform(pshape, 1, -.5, .5), uniform(pshape, 2, -.5, .5)
        Y = torch.empty_like(X)
        gS, gB = torch.zeros(pshape, device=dev), torch.zeros(pshape, device=dev)
        tX, tS, tB, tY = wrap(X), wrap(S), wrap(B), wrap(Y)
        ws = 2 * n * F
        timeit(5, "scale_bias_relu_fwd", lambda: pb.forward("scale_bias_leaky_relu", [tX, tS, tB], tY, fval=0.0, check=False),
               2 * n * F + 2048, n, ws)
        tBg = wrap(B); tBg.c.requires_grad = True
        g = wrap(gB); tBg.grad = g; tBg.c.grad = C.pointer(g.c)
        tYg = wrap(Y); gy = wrap(G); tYg.grad = gy; tYg.c.grad = C.pointer(gy.c)
        timeit(5, "bias_grad_masked_reduce", lambda: pb.backward("scale_bias_leaky_relu", [tX, tS, tBg], tYg, fval=0.0, check=False),
               2 * n * F + 1024, n, ws)
        del X, G, Y
    if 6 in configs:
        # Optimiser steps (not one of the reference's benchmark configurations): a parameter set of
        # 12 weight matrices [4096, 2048] and 12 biases [4096], one multi-tensor launch per step.
        from . import optim as O
        shapes = [(4096, 2048), (4096,)] * 12
        ps = [randn(sh, 10 + i, 0.1) for i, sh in enumerate(shapes)]
        gs = [randn(sh, 50 + i, 0.01) for i, sh in enumerate(shapes)]
        params = []
        for p_, g_ in zip(ps, gs):
            tp, tg = wrap(p_), wrap(g_)
            tp.grad = tg; tp.c.grad = C.pointer(tg.c); tp.c.requires_grad = True
            params.append(tp)
        arr = O.param_array(params)
        n = sum(int(np.prod(sh)) for sh in shapes)
        sgd = O.SGD(1e-3)
        timeit(6, "sgd_step_24_params", lambda: pb.lib.sgd_step_cuda(C.byref(sgd), arr, len(params)), 3 * n * F, n, 2 * n * F)
        adam = O.Adam()
        adam.lr, adam.beta1, adam.beta2, adam.epsilon, adam.t = 1e-3, 0.9, 0.999, 1e-8, 0
        timeit(6, "adam_step_24_params", lambda: pb.lib.adam_step_cuda(C.byref(adam), arr, len(params)), 7 * n * F, n, 4 * n * F)
        O.release_state(adam)
        adamw = O.AdamW()
        adamw.lr, adamw.beta1, adamw.beta2, adamw.epsilon, adamw.weight_decay, adamw.t = 1e-3, 0.9, 0.999, 1e-8, 0.01, 0
        timeit(6, "adamw_step_24_params", lambda: pb.lib.adamw_step_cuda(C.byref(adamw), arr, len(params)), 7 * n * F, n, 4 * n * F)
        O.release_state(adamw)
        del ps, gs
    if 7 in configs:
        # Column sums of TALL matrices (not one of the reference's benchmark configurations): the
        # shape of a bias gradient, sum over (batch x positions) rows for a few hundred or thousand
        # features. Few columns leave few strips for the column kernel; see its strip-width rule.
        for rows_, cols_ in ((65536, 256), (262144, 128), (32768, 512), (16384, 2048), (8192, 1024)):
            X = randn((rows_, cols_), 20)
            o = torch.empty(cols_, device=dev)
            tX, to = wrap(X), wrap(o)
            n = rows_ * cols_
            timeit(7, f"sum_axis0_{rows_}x{cols_}", lambda: pb.forward("sum", [tX], to, dim=0, check=False), n * F, n, n * F)
            del X, o
    torch.cuda.synchronize()
    return rows
