"""One rank of the peer-exchange test (launched by tests/test_gpu_peer.py through torchrun on two or
more GPUs of one box): the library's NVLink exchange against the process group's all-reduce."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import plast_b200 as pb  # noqa: E402
from plast_b200.dist import PeerGroup  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    os.environ["NCCL_DEBUG"] = "WARN"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("nccl", device_id=dev)
    import ctypes as C
    pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    group = PeerGroup(dist, torch, pb)
    gen = torch.Generator(device=dev)
    for it, n in enumerate([1, 5, 1000, 4097, 8192] * 8):
        for op, red in (("sum", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX), ("min", dist.ReduceOp.MIN)):
            gen.manual_seed(1000 * it + rank)
            x = torch.randn(n, generator=gen, device=dev)
            want = x.clone()
            gathered = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(gathered, x)
            acc = gathered[0].clone()
            for g in gathered[1:]:                                        # rank order, like the kernel
                acc = acc + g if op == "sum" else (torch.maximum(acc, g) if op == "max" else torch.minimum(acc, g))
            group.all_reduce(x, op)
            pb.check_error()
            torch.cuda.synchronize()
            assert torch.equal(x, acc), f"rank {rank}: {op} of {n} floats differs from the rank-order result"
            dist.all_reduce(want, op=red)
            assert torch.allclose(x, want, rtol=1e-6, atol=1e-6)
    # the full reduction of a shard with the exchange inside the reduction kernel
    for it, n in enumerate([5, 1 << 16, (1 << 22) + 3, 1 << 23]):
        gen.manual_seed(7000 + 10 * it + rank)
        shard = torch.randn(n, generator=gen, device=dev)
        t_shard = pb.Tensor.wrap_pointer(shard.data_ptr(), [n], owner=shard)
        for op in ("sum", "max", "min"):
            local = pb.Tensor((1,)); pb.forward(op, [t_shard], local, dim=pb.FULL_REDUCE)
            lv = torch.from_numpy(local.numpy().copy()).to(dev)
            gathered = [torch.empty_like(lv) for _ in range(world)]
            dist.all_gather(gathered, lv)
            acc = gathered[0].clone()
            for g in gathered[1:]:
                acc = acc + g if op == "sum" else (torch.maximum(acc, g) if op == "max" else torch.minimum(acc, g))
            out = pb.Tensor((1,))
            group.full_reduce(t_shard, out, op)
            pb.check_error()
            torch.cuda.synchronize()
            assert out.numpy()[0] == acc.item(), f"rank {rank}: fused {op} of {n} floats: {out.numpy()[0]} vs {acc.item()}"
    # mean cross-entropy over row-sharded logits, the exchange inside the loss kernel
    rows_here, cols = 1024 + 8 * rank, 4096
    total_rows = sum(1024 + 8 * r for r in range(world))
    gen.manual_seed(9000 + rank)
    logits = torch.randn((rows_here, cols), generator=gen, device=dev) * 2
    labels = torch.randint(0, cols, (rows_here,), generator=gen, device=dev, dtype=torch.int32)
    t_logits = pb.Tensor.wrap_pointer(logits.data_ptr(), [rows_here, cols], owner=logits)
    t_labels = pb.Tensor.wrap_pointer(labels.data_ptr(), [rows_here], dtype=pb.INT32, owner=labels)
    out = pb.Tensor((1,))
    group.cross_entropy_mean(t_logits, t_labels, out, total_rows)
    pb.check_error()
    torch.cuda.synchronize()
    ref = torch.nn.functional.cross_entropy(logits.double(), labels.long(), reduction="sum")
    dist.all_reduce(ref)
    assert abs(out.numpy()[0] - ref.item() / total_rows) <= 2e-6 * abs(ref.item() / total_rows) + 1e-6, \
        f"rank {rank}: fused cross-entropy mean {out.numpy()[0]} vs {ref.item() / total_rows}"
    assert group.status() == 0
    # reductions that cross the sharded dim, inside the bracket: the column sum of a row-sharded
    # matrix (exchange inside the column-reduce kernel), row sums as a many-output stand-in for the
    # parked route, and the bias / scale gradients of a batch-sharded NCHW activation
    rows_here = 512 + 16 * rank
    gen.manual_seed(11000 + rank)
    Mx = torch.randn((rows_here, 4096), generator=gen, device=dev)
    t_m = pb.Tensor.wrap_pointer(Mx.data_ptr(), [rows_here, 4096], owner=Mx)
    col = torch.zeros(4096, device=dev)
    t_col = pb.Tensor.wrap_pointer(col.data_ptr(), [4096], owner=col)
    pb.forward("sum", [t_m], t_col, dim=0)
    want = col.clone(); dist.all_reduce(want)
    scale = Mx.abs().sum(dim=0); dist.all_reduce(scale)
    with group.reducing() as br:
        pb.forward("sum", [t_m], t_col, dim=0)
    torch.cuda.synchronize()
    assert br.exchanges == 1 and pb.last_kernel().startswith("reduce_cols")
    assert bool(((col - want).abs() <= 1e-5 * scale).all()), f"rank {rank}: fused column sum"
    everyone = [torch.empty_like(col) for _ in range(world)]
    dist.all_gather(everyone, col)
    assert all(torch.equal(everyone[0], e) for e in everyone), "every rank must hold the same bits"
    Mr = torch.randn((3000, 256), generator=gen, device=dev)             # 3000 outputs: the parked route
    t_r = pb.Tensor.wrap_pointer(Mr.data_ptr(), [3000, 256], owner=Mr)
    rs = torch.zeros(3000, device=dev)
    t_rs = pb.Tensor.wrap_pointer(rs.data_ptr(), [3000], owner=rs)
    pb.forward("max", [t_r], t_rs, dim=1)
    want = rs.clone(); dist.all_reduce(want, op=dist.ReduceOp.MAX)
    with group.reducing() as br:
        pb.forward("max", [t_r], t_rs, dim=1)
    torch.cuda.synchronize()
    assert br.exchanges == 1 and torch.equal(rs, want), f"rank {rank}: parked row max"
    nb = 4 + rank
    gen.manual_seed(12000 + rank)
    X5 = torch.randn((nb, 64, 56, 56), generator=gen, device=dev)
    G5 = torch.randn((nb, 64, 56, 56), generator=gen, device=dev)
    gen.manual_seed(12999)
    S5 = torch.rand((1, 64, 1, 1), generator=gen, device=dev) - 0.5
    B5 = torch.rand((1, 64, 1, 1), generator=gen, device=dev) - 0.5
    Y5 = torch.empty_like(X5)
    gS, gB = torch.ones((1, 64, 1, 1), device=dev), torch.full((1, 64, 1, 1), -2.0, device=dev)

    def wrap(t, grad=None):
        w = pb.Tensor.wrap_pointer(t.data_ptr(), list(t.shape), owner=t)
        if grad is not None:
            w.grad = pb.Tensor.wrap_pointer(grad.data_ptr(), list(grad.shape), owner=grad)
            w.c.grad = C.pointer(w.grad.c); w.c.requires_grad = True
        return w
    tX5, tS5, tB5, tY5 = wrap(X5), wrap(S5, gS), wrap(B5, gB), wrap(Y5, G5)
    pb.forward("scale_bias_leaky_relu", [tX5, tS5, tB5], tY5, fval=0.0)
    mask = (Y5 > 0).float()
    wantB = (G5 * mask).sum(dim=(0, 2, 3)).reshape(1, 64, 1, 1); dist.all_reduce(wantB)
    wantS = (G5 * mask * X5).sum(dim=(0, 2, 3)).reshape(1, 64, 1, 1); dist.all_reduce(wantS)
    sclB = (G5 * mask).abs().sum(dim=(0, 2, 3)).reshape(1, 64, 1, 1); dist.all_reduce(sclB)
    sclS = (G5 * mask * X5).abs().sum(dim=(0, 2, 3)).reshape(1, 64, 1, 1); dist.all_reduce(sclS)
    with group.reducing() as br:
        pb.backward("scale_bias_leaky_relu", [tX5, tS5, tB5], tY5, fval=0.0)
    torch.cuda.synchronize()
    assert br.exchanges == 2
    assert bool(((gB - (-2.0 + wantB)).abs() <= 1e-5 * sclB + 1e-6).all()), f"rank {rank}: bias gradient over all ranks"
    assert bool(((gS - (1.0 + wantS)).abs() <= 1e-5 * sclS + 1e-6).all()), f"rank {rank}: scale gradient over all ranks"
    assert group.status() == 0
    # timing: exchange of 1 float and of 8192 floats, against the process group's all-reduce
    def timed(fn, reps=200):
        for _ in range(10):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3
    def graph_timed(fn, inner=50, reps=20):
        """`inner` calls recorded in one CUDA graph and replayed: no host cost per call."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            pb.lib.plast_b200_set_stream(C.c_void_p(side.cuda_stream))
            fn()
            torch.cuda.synchronize(); dist.barrier()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(inner):
                    fn()
        pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize(); dist.barrier()
        graph.replay()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * inner) * 1e3

    for n in (1, 8192):
        x = torch.ones(n, device=dev)
        t_peer = timed(lambda: group.all_reduce(x, "max"))
        t_pg = timed(lambda: dist.all_reduce(x, op=dist.ReduceOp.MAX))
        t_peer_graph = graph_timed(lambda: group.all_reduce(x, "max"))
        assert group.status() == 0 and bool((x == 1).all())
        if rank == 0:
            print(f"exchange of {n} floats on {world} GPUs: peer kernel {t_peer:.1f} us per call from Python, "
                  f"{t_peer_graph:.1f} us replayed from a CUDA graph; process group {t_pg:.1f} us per call", flush=True)
    # a 32 MiB shard (config 4 on eight GPUs): local full sum + all-reduce against the single fused kernel
    shard = torch.randn(1 << 23, device=dev)
    t_shard = pb.Tensor.wrap_pointer(shard.data_ptr(), [1 << 23], owner=shard)
    one = torch.zeros(1, device=dev)
    t_one = pb.Tensor.wrap_pointer(one.data_ptr(), [1], owner=one)

    def two_step():
        pb.forward("sum", [t_shard], t_one, dim=pb.FULL_REDUCE, check=False)
        group.all_reduce(one, "sum")

    def with_process_group():
        pb.forward("sum", [t_shard], t_one, dim=pb.FULL_REDUCE, check=False)
        dist.all_reduce(one, op=dist.ReduceOp.SUM)

    t_fused = graph_timed(lambda: group.full_reduce(t_shard, t_one, "sum"), inner=20)
    t_two = graph_timed(two_step, inner=20)
    t_pg = timed(with_process_group)
    if rank == 0:
        print(f"full sum of a 32 MiB shard on {world} GPUs: one kernel with the exchange inside {t_fused:.1f} us, "
              f"reduce then exchange kernel {t_two:.1f} us (both replayed from a CUDA graph); "
              f"reduce then process-group all-reduce {t_pg:.1f} us per call", flush=True)
    assert group.status() == 0
    group.close()
    dist.barrier()
    if rank == 0:
        print("PEER OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
