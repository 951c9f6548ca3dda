"""Multi-GPU layer of the hot path: one process per GPU, `torch.distributed` for the plumbing.

plast itself has no distributed code (its README lists "MPI + NCCL" as a roadmap item), so this is
new. The path shards naturally:

* elementwise ops, axis reductions over a non-sharded axis, softmax / argmax rows: contiguous
  blocks of the OUTERMOST non-reduced dim per rank, broadcast operands replicated, no
  communication at all;
* reductions that cross the sharded dim (full sum / max / mean, column sums of a row-sharded
  matrix, a bias gradient of a batch-sharded activation, the cross-entropy mean): every rank
  reduces its shard with the single-GPU kernel, then ONE all-reduce of the tiny partial
  (4 bytes .. 32 KiB) over NCCL / NVLink combines them. A mean is the all-reduced SUM divided by
  the GLOBAL count (never a mean of means); an argmax is an all-reduce MAX of the values followed
  by an all-reduce MIN of the indices that attain it.

Everything here works on any backend: the tests run it with `gloo` on CPU tensors (the local
reduce is supplied by the caller), the benchmark with `nccl` on CUDA tensors.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    """Contiguous block [start, start + count) of a dim of length `total` owned by `rank`."""

    start: int
    count: int
    total: int
    rank: int
    world: int


def shard_dim(total: int, rank: int, world: int) -> Shard:
    """Blocks differ by at most one element; the first `total % world` ranks get the extra one.
    Ranks beyond `total` own an empty block (count 0) and contribute the identity."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return Shard(start, count, total, rank, world)


class PeerGroup:
    """The library's own exchange for tiny partials (include/plast_b200_peer.h): every rank stores
    its message into every peer's buffer over NVLink and adds the messages up in rank order, in
    one small kernel. `torch.distributed` only carries the 64-byte IPC handles at set-up.

    Use for messages of at most MAX_FLOATS floats on the GPUs of one box; anything else goes
    through the process group's all-reduce."""

    MAX_FLOATS = 8192
    OPS = {"sum": 0, "max": 1, "min": 2}

    def __init__(self, dist, torch, pb):
        import ctypes as C
        self._C, self._pb, self._dist = C, pb, dist
        lib = pb.lib
        lib.plast_b200_peer_group_begin.argtypes = [C.c_int, C.c_int, C.c_char_p]
        lib.plast_b200_peer_group_begin.restype = C.c_void_p
        lib.plast_b200_peer_group_connect.argtypes = [C.c_void_p, C.c_char_p]
        lib.plast_b200_peer_group_connect.restype = C.c_int
        lib.plast_b200_peer_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int]
        lib.plast_b200_peer_all_reduce.restype = None
        lib.plast_b200_peer_group_status.argtypes = [C.c_void_p]
        lib.plast_b200_peer_group_status.restype = C.c_int
        lib.plast_b200_peer_group_release.argtypes = [C.c_void_p]
        lib.plast_b200_peer_group_release.restype = None
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        handle = C.create_string_buffer(64)
        self._g = lib.plast_b200_peer_group_begin(self.rank, self.world, handle)
        pb.check_error()
        gathered = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle.raw))      # also orders every rank's step 1 before step 2
        if lib.plast_b200_peer_group_connect(self._g, b"".join(gathered)) != 0:
            pb.check_error()
        dist.barrier()                                            # nobody stores before everybody is mapped

    def all_reduce(self, t, op: str = "sum"):
        """In place on a contiguous float32 CUDA tensor of at most MAX_FLOATS elements."""
        assert t.is_contiguous() and t.numel() <= self.MAX_FLOATS and str(t.dtype) == "torch.float32"
        self._pb.lib.plast_b200_peer_all_reduce(self._g, self._C.c_void_p(t.data_ptr()), t.numel(), self.OPS[op])
        self._pb.check_error()
        return t

    def full_reduce(self, t, out, op: str = "sum"):
        """Full reduction of this rank's shard `t` and the exchange of the result in one kernel;
        `t` and `out` are plast_b200.Tensor objects (out holds one float)."""
        C = self._C
        fn = self._pb.lib.plast_b200_peer_full_reduce
        fn.argtypes = [C.c_void_p, C.c_int, C.POINTER(self._pb.CTensor), C.POINTER(self._pb.CTensor)]
        fn.restype = None
        fn(self._g, self.OPS[op], C.byref(t.c), C.byref(out.c))
        self._pb.check_error()
        return out

    def cross_entropy_mean(self, logits, labels, out, global_rows: int):
        """Mean cross-entropy over row-sharded logits with the exchange inside the loss kernel;
        arguments are plast_b200.Tensor objects (labels INT32, out one float)."""
        C = self._C
        fn = self._pb.lib.plast_b200_peer_cross_entropy_mean
        T = C.POINTER(self._pb.CTensor)
        fn.argtypes = [C.c_void_p, T, T, T, C.c_uint64]
        fn.restype = None
        fn(self._g, C.byref(logits.c), C.byref(labels.c), C.byref(out.c), global_rows)
        self._pb.check_error()
        return out

    def reducing(self):
        """Context manager: every final reduction that plast_b200 entry points launch inside the
        block (a sum over the sharded axis, the broadcast-gradient reduce of a backward call) is
        combined across the ranks, inside the reduction kernel where its shape allows it
        (plast_b200_peer_reduce_begin / _end). `exchanges` holds the count afterwards."""
        group = self

        class _Bracket:
            exchanges = 0

            def __enter__(self):
                lib = group._pb.lib
                lib.plast_b200_peer_reduce_begin.argtypes = [group._C.c_void_p]
                lib.plast_b200_peer_reduce_begin.restype = None
                lib.plast_b200_peer_reduce_end.argtypes = [group._C.c_void_p]
                lib.plast_b200_peer_reduce_end.restype = group._C.c_int
                lib.plast_b200_peer_reduce_begin(group._g)
                group._pb.check_error()
                return self

            def __exit__(self, *exc):
                self.exchanges = group._pb.lib.plast_b200_peer_reduce_end(group._g)
                return False

        return _Bracket()

    def status(self) -> int:
        return self._pb.lib.plast_b200_peer_group_status(self._g)

    def close(self):
        if self._g:
            self._dist.barrier()
            self._pb.lib.plast_b200_peer_group_release(self._g)
            self._g = None


_peer_group = None


def use_peer_exchange(group) -> None:
    """Routes all_reduce_sum / max / min of small CUDA tensors through `group` (a PeerGroup), or
    back to the process group with None."""
    global _peer_group
    _peer_group = group


def _peer_ok(t) -> bool:
    return (_peer_group is not None and getattr(t, "is_cuda", False) and t.is_contiguous()
            and t.numel() <= PeerGroup.MAX_FLOATS and str(t.dtype) == "torch.float32")


def all_reduce_sum(dist, t):
    """In place; `t` holds this rank's partial sums (any shape, identical on every rank)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        if _peer_ok(t):
            return _peer_group.all_reduce(t, "sum")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


def all_reduce_max(dist, t):
    if dist.is_initialized() and dist.get_world_size() > 1:
        if _peer_ok(t):
            return _peer_group.all_reduce(t, "max")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t


def all_reduce_min(dist, t):
    if dist.is_initialized() and dist.get_world_size() > 1:
        if _peer_ok(t):
            return _peer_group.all_reduce(t, "min")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return t


def global_mean(dist, local_sum, global_count: int):
    """Mean over all shards = all-reduced sum / global count (src/kernels/cpu/reduce_ops.c:13
    divides the fp32 sum by the count once; so does this)."""
    all_reduce_sum(dist, local_sum)
    local_sum /= float(global_count)
    return local_sum


def global_argmax(dist, torch, local_value, local_index, index_offset: int):
    """Full-tensor argmax across shards, lowest global index on ties.

    local_value / local_index: this rank's maximum and its index inside the shard (tensors of the
    same shape, index dtype int64); index_offset: global index of the shard's first element.
    An empty shard passes value -inf."""
    gmax = local_value.clone()
    all_reduce_max(dist, gmax)
    sentinel = torch.iinfo(torch.int64).max
    cand = torch.where(local_value == gmax, local_index + index_offset,
                       torch.full_like(local_index, sentinel))
    all_reduce_min(dist, cand)
    return gmax, cand


# ---- benchmark of the sharded reductions (rank-parallel, CUDA) -------------------------------------
def sharded_reduction_table(torch, dist, pb, dev, peak_gbs: float, reps: int = 10, deadline=None):
    """Strong-scaling rows: the FIXED tensors of configs 3, 4 and 5 are split across ranks along
    their outermost dim; a step is the local kernel, followed by the all-reduce where the op needs
    one (names ending in +allreduce), timed with CUDA events, max over ranks.

    Rows that use the library's own NVLink exchange (+peer_exchange, _fused_with_exchange) are
    first VERIFIED, outside the timed region: their result is compared with the process group's
    all-reduce of the same per-rank partials (bitwise for max; for sums |a - b| <= 1e-5 * the
    all-reduced sum of |terms|, since the two add the ranks in different orders) and the row
    carries "verified" and the exchange's status word.

    deadline (time.monotonic() value): checked between rows, agreed on by all ranks through the
    process group; rows past it are listed as skipped, so no rank leaves while another is still
    inside an exchange."""
    import time

    import numpy as np

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    gen = torch.Generator(device=dev)
    rows = []

    def wrap(t, shape=None, dtype=pb.FLOAT32):
        return pb.Tensor.wrap_pointer(t.data_ptr(), list(t.shape) if shape is None else shape,
                                      dtype=dtype, owner=t)

    import ctypes as C

    def out_of_time():
        late = torch.tensor([1.0 if (deadline is not None and time.monotonic() > deadline) else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(late, op=dist.ReduceOp.MAX)
        return float(late.item()) > 0

    def timeit(name, fn, total_bytes, check=None):
        if out_of_time():
            rows.append({"op": name, "n_gpus": world, "skipped": "time limit of the table reached"})
            return
        checked = check() if check is not None else {}
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        times = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 5)
        t = torch.tensor([float(np.median(times))], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        gbs = total_bytes / (ms * 1e-3) / 1e9
        row = {"op": name, "n_gpus": world, "ms": round(ms, 5), "GBps": round(gbs, 1),
               "frac_of_measured_aggregate": round(gbs / (peak_gbs * world), 4)}
        row.update(checked)
        # Steps of a few microseconds are bound by the host's call cost when issued one by one; the
        # same 20 steps recorded in a CUDA graph and replayed show what the GPUs and the links need.
        # Every rank must take the same path, so a failure anywhere sends all ranks to the row above.
        ok = torch.ones(1, device=dev)
        graph = None
        main = torch.cuda.current_stream()
        try:
            side = torch.cuda.Stream()
            side.wait_stream(main)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                pb.lib.plast_b200_set_stream(C.c_void_p(side.cuda_stream))
                fn()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        fn()
        except Exception as exc:
            ok.zero_()
            graph = None
            row["graph_replay_error"] = str(exc)[:160]
        pb.lib.plast_b200_set_stream(C.c_void_p(main.cuda_stream))
        torch.cuda.synchronize()
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if graph is not None and float(ok.item()) > 0:
            graph.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            gt = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); graph.replay(); e1.record()
                torch.cuda.synchronize()
                gt.append(e0.elapsed_time(e1) / 20)
            g = torch.tensor([float(np.median(gt))], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(g, op=dist.ReduceOp.MAX)
            gms = float(g.item())
            row["graph_replay_ms"] = round(gms, 5)
            row["graph_replay_GBps"] = round(total_bytes / (gms * 1e-3) / 1e9, 1)
        rows.append(row)

    # config 4: X[8192, 8192], rows sharded; full sum / full max -> 4-byte all-reduce,
    # sum over axis 0 -> 32 KiB all-reduce
    M = 8192
    sh = shard_dim(M, rank, world)
    gen.manual_seed(100 + rank)
    X = torch.rand((max(sh.count, 1), M), generator=gen, device=dev) * 2 - 1
    tX = wrap(X, shape=[sh.count, M])
    one, col = torch.zeros(1, device=dev), torch.zeros(M, device=dev)
    tone, tcol = wrap(one), wrap(col)

    def full_sum():
        pb.forward("sum", [tX], tone, dim=pb.FULL_REDUCE, check=False)
        all_reduce_sum(dist, one)

    def full_max():
        pb.forward("max", [tX], tone, dim=pb.FULL_REDUCE, check=False)
        all_reduce_max(dist, one)

    def sum_axis0():
        pb.forward("sum", [tX], tcol, dim=0, check=False)
        all_reduce_sum(dist, col)

    def verify(run, result, local, op, abs_terms=None):
        """run(): the step under test, leaves its answer in `result`. local(): leaves THIS rank's
        partial in `result` (no exchange). The expected answer is the process group's all-reduce of
        the partials. Returns the fields the row carries."""
        def check():
            if peer is None:
                return {}
            peer_ok = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX}[op]
            local(); torch.cuda.synchronize()
            expect = result.clone()
            dist.all_reduce(expect, op=peer_ok)
            run(); torch.cuda.synchronize()
            got = result.clone()
            if op == "max":
                ok = bool(torch.equal(got, expect))
                worst = 0.0 if ok else 1e30
            else:
                scale = abs_terms().clone()
                dist.all_reduce(scale, op=dist.ReduceOp.SUM)
                worst = float(((got.double() - expect.double()).abs() / (1e-5 * scale.double() + 1e-30)).max().item())
                ok = worst <= 1.0
            flag = torch.tensor([1.0 if ok else 0.0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)          # verified only if every rank agrees
            return {"verified": bool(flag.item() > 0), "max_err_over_bound": round(worst, 4), "peer_status": peer.status()}
        return check

    def local_full(op):
        return lambda: pb.forward(op, [tX], tone, dim=pb.FULL_REDUCE, check=False)

    abs_all = lambda: X.abs().sum().reshape(1)
    abs_cols = lambda: X.abs().sum(dim=0)
    peer = None
    timeit("config4_full_sum+allreduce", full_sum, M * M * 4 + 4)
    timeit("config4_full_max+allreduce", full_max, M * M * 4 + 4)
    timeit("config4_sum_axis0+allreduce", sum_axis0, (M * M + M) * 4)
    # the same three with the library's own NVLink exchange instead of the process group's all-reduce
    if world > 1 and world <= 8:
        try:
            peer = PeerGroup(dist, torch, pb)
        except Exception as exc:  # the table must not die with the exchange
            rows.append({"op": "peer_exchange_unavailable", "n_gpus": world, "error": str(exc)[:200]})
    if peer is not None:
        use_peer_exchange(peer)
        timeit("config4_full_sum+peer_exchange", full_sum, M * M * 4 + 4,
               verify(full_sum, one, local_full("sum"), "sum", abs_all))
        timeit("config4_full_max+peer_exchange", full_max, M * M * 4 + 4, verify(full_max, one, local_full("max"), "max"))
        timeit("config4_sum_axis0+peer_exchange", sum_axis0, (M * M + M) * 4,
               verify(sum_axis0, col, lambda: pb.forward("sum", [tX], tcol, dim=0, check=False), "sum", abs_cols))
        use_peer_exchange(None)
        # ... and with the exchange inside the reduction kernel (one launch per step)
        fused_sum = lambda: peer.full_reduce(tX, tone, "sum")
        fused_max = lambda: peer.full_reduce(tX, tone, "max")
        timeit("config4_full_sum_fused_with_exchange", fused_sum, M * M * 4 + 4,
               verify(fused_sum, one, local_full("sum"), "sum", abs_all))
        timeit("config4_full_max_fused_with_exchange", fused_max, M * M * 4 + 4,
               verify(fused_max, one, local_full("max"), "max"))

        def fused_axis0():
            with peer.reducing():
                pb.forward("sum", [tX], tcol, dim=0, check=False)
        timeit("config4_sum_axis0_fused_with_exchange", fused_axis0, (M * M + M) * 4,
               verify(fused_axis0, col, lambda: pb.forward("sum", [tX], tcol, dim=0, check=False), "sum", abs_cols))
    del X
    # ... and sharded along the KEPT dim instead (columns): every rank sums its own strip of columns
    # of the row-major matrix, a strided view [M, M / world] with row stride M; no exchange at all
    cs = shard_dim(M, rank, world)
    gen.manual_seed(150)
    Xfull = torch.rand((M, M), generator=gen, device=dev) * 2 - 1
    tXc = pb.Tensor.wrap_pointer(Xfull.data_ptr() + 4 * cs.start, [M, cs.count], strides=[M, 1], owner=Xfull)
    colc = torch.zeros(max(cs.count, 1), device=dev)
    tcolc = wrap(colc, shape=[cs.count])
    if cs.count > 0:
        timeit("config4_sum_axis0_column_sharded_no_exchange",
               lambda: pb.forward("sum", [tXc], tcolc, dim=0, check=False), (M * M + M) * 4)
    del Xfull

    # config 3: cross-entropy mean over row-sharded logits -> 4-byte all-reduce of the loss SUM
    R, Cn = 65536, 4096
    sh = shard_dim(R, rank, world)
    gen.manual_seed(200 + rank)
    L = torch.randn((sh.count, Cn), generator=gen, device=dev) * 2.0
    labels = torch.randint(0, Cn, (sh.count,), generator=gen, device=dev, dtype=torch.int32)
    tL, tl = wrap(L), wrap(labels, dtype=pb.INT32)
    loss = torch.zeros(1, device=dev)
    tloss = wrap(loss)

    def ce_mean():
        pb.forward("cross_entropy", [tL, tl], tloss, check=False)  # local mean
        loss.mul_(float(sh.count))                                   # back to the local sum
        global_mean(dist, loss, R)

    def ce_local_share():
        # this rank's share of the global mean: local loss sum / global row count
        pb.forward("cross_entropy", [tL, tl], tloss, check=False)
        loss.mul_(float(sh.count) / float(R))

    # per-row losses are positive, so sum|terms| of the mean is the mean itself
    ce_terms = lambda: (ce_local_share(), loss.clone())[1]
    timeit("config3_cross_entropy_mean+allreduce", ce_mean, (R * Cn + R) * 4 + 4)
    if peer is not None:
        use_peer_exchange(peer)
        timeit("config3_cross_entropy_mean+peer_exchange", ce_mean, (R * Cn + R) * 4 + 4,
               verify(ce_mean, loss, ce_local_share, "sum", ce_terms))
        use_peer_exchange(None)
        ce_fused = lambda: peer.cross_entropy_mean(tL, tl, tloss, R)
        timeit("config3_cross_entropy_mean_fused_with_exchange", ce_fused, (R * Cn + R) * 4 + 4,
               verify(ce_fused, loss, ce_local_share, "sum", ce_terms))
    # row ops of config 3 on the same row shard: independent per row, no collective
    rs, Y = torch.empty(sh.count, device=dev), torch.empty_like(L)
    trs, tY = wrap(rs), wrap(Y)
    timeit("config3_row_sum", lambda: pb.forward("sum", [tL], trs, dim=1, check=False), (R * Cn + R) * 4)
    timeit("config3_softmax", lambda: pb.forward("softmax", [tL], tY, dim=1, check=False), 2 * R * Cn * 4)
    del L, Y

    # config 5: NCHW epilogue, batch-sharded; forward needs no collective, the bias gradient a
    # 1 KiB all-reduce of the per-GPU channel sums
    N, Ch, H, W = 256, 256, 56, 56
    sh = shard_dim(N, rank, world)
    gen.manual_seed(300 + rank)
    X = torch.randn((max(sh.count, 1), Ch, H, W), generator=gen, device=dev)
    G = torch.randn((max(sh.count, 1), Ch, H, W), generator=gen, device=dev)
    S = torch.rand((1, Ch, 1, 1), generator=gen, device=dev) - 0.5
    B = torch.rand((1, Ch, 1, 1), generator=gen, device=dev) - 0.5
    Yv = torch.empty_like(X)
    gB = torch.zeros((1, Ch, 1, 1), device=dev)
    tX5, tS, tB, tY5 = wrap(X), wrap(S), wrap(B), wrap(Yv)
    total = N * Ch * H * W
    timeit("config5_scale_bias_relu_fwd",
           lambda: pb.forward("scale_bias_leaky_relu", [tX5, tS, tB], tY5, fval=0.0, check=False), 2 * total * 4 + 2048)
    import ctypes as C
    tBg = wrap(B); tBg.c.requires_grad = True
    tg = wrap(gB); tBg.grad = tg; tBg.c.grad = C.pointer(tg.c)
    tYg = wrap(Yv); tG = wrap(G); tYg.grad = tG; tYg.c.grad = C.pointer(tG.c)

    # The backward ACCUMULATES into bias.grad; a step that all-reduces the gradient buffer itself
    # needs it zeroed first (one more small kernel), the bracket form exchanges only the new sum.
    def bias_grad():
        gB.zero_()
        pb.backward("scale_bias_leaky_relu", [tX5, tS, tBg], tYg, fval=0.0, check=False)
        all_reduce_sum(dist, gB)

    def bias_grad_local():
        gB.zero_()
        pb.backward("scale_bias_leaky_relu", [tX5, tS, tBg], tYg, fval=0.0, check=False)

    def bias_terms():
        pb.forward("scale_bias_leaky_relu", [tX5, tS, tB], tY5, fval=0.0, check=False)
        return (G.abs() * (Yv > 0)).sum(dim=(0, 2, 3)).reshape(1, Ch, 1, 1)

    timeit("config5_bias_grad+allreduce", bias_grad, 2 * total * 4 + 1024)
    if peer is not None:
        use_peer_exchange(peer)
        timeit("config5_bias_grad+peer_exchange", bias_grad, 2 * total * 4 + 1024,
               verify(bias_grad, gB, bias_grad_local, "sum", bias_terms))
        use_peer_exchange(None)

        def bias_grad_fused():
            with peer.reducing():
                pb.backward("scale_bias_leaky_relu", [tX5, tS, tBg], tYg, fval=0.0, check=False)

        def bias_grad_fused_from_zero():
            gB.zero_()
            bias_grad_fused()
        timeit("config5_bias_grad_fused_with_exchange", bias_grad_fused, 2 * total * 4 + 1024,
               verify(bias_grad_fused_from_zero, gB, bias_grad_local, "sum", bias_terms))
        status = peer.status()
        if status != 0:
            rows.append({"op": "peer_exchange_status", "n_gpus": world, "status": status})
        peer.close()
    del X, G, Yv
    # ... and sharded along the KEPT dim instead (channels): a strided view [N, Ch / world, H, W] of
    # the full activation; every rank reduces its own channels over (N, H, W); no exchange at all
    ch = shard_dim(Ch, rank, world)
    if ch.count > 0 and not out_of_time():
        gen.manual_seed(350)
        Gf = torch.randn((N, Ch, H, W), generator=gen, device=dev)
        Yf = torch.randn((N, Ch, H, W), generator=gen, device=dev)
        Xf = Yf                                                      # only read when the scale needs a gradient
        full_strides = [Ch * H * W, H * W, W, 1]
        view = lambda t: pb.Tensor.wrap_pointer(t.data_ptr() + 4 * ch.start * H * W, [N, ch.count, H, W],
                                                strides=full_strides, owner=t)
        Sc = torch.rand((1, ch.count, 1, 1), generator=gen, device=dev) - 0.5
        Bc = torch.rand((1, ch.count, 1, 1), generator=gen, device=dev) - 0.5
        gBc = torch.zeros((1, ch.count, 1, 1), device=dev)
        tXf, tSc = view(Xf), wrap(Sc)
        tBc = wrap(Bc); tBc.c.requires_grad = True
        tgc = wrap(gBc); tBc.grad = tgc; tBc.c.grad = C.pointer(tgc.c)
        tYf = view(Yf); tGf = view(Gf); tYf.grad = tGf; tYf.c.grad = C.pointer(tGf.c)

        def bias_grad_channels():
            pb.backward("scale_bias_leaky_relu", [tXf, tSc, tBc], tYf, fval=0.0, check=False)
        timeit("config5_bias_grad_channel_sharded_no_exchange", bias_grad_channels, 2 * total * 4 + 1024)
        del Gf, Yf
    torch.cuda.synchronize()
    return rows
