"""The N > 1 path on CPU: two `gloo` ranks shard a tensor along its outermost dim, reduce their
shard with the CPU oracle (standing in for the single-GPU kernel), and combine with the helpers of
plast_b200/dist.py. Checked against the unsharded oracle result."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from plast_b200.dist import shard_dim  # noqa: E402


def test_shard_dim_covers_everything_once():
    for total in (0, 1, 7, 8, 65536, 65537):
        for world in (1, 2, 3, 8):
            shards = [shard_dim(total, r, world) for r in range(world)]
            assert shards[0].start == 0 and sum(s.count for s in shards) == total
            for a, b in zip(shards, shards[1:]):
                assert a.start + a.count == b.start
            assert max(s.count for s in shards) - min(s.count for s in shards) <= 1
    with pytest.raises(ValueError):
        shard_dim(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from harness import CpuBackend, FULL_REDUCE, INT32, OracleRecipes, rand_normal, rand_uniform
    from plast_b200 import dist as pd

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = CpuBackend("oracle")
    M, N = 101, 64                                         # ragged split: 51 + 50 rows
    X = rand_uniform(0, (M, N))
    sh = pd.shard_dim(M, rank, world)
    local = X[sh.start:sh.start + sh.count]

    def reduce_local(op, dim, dtype=1, out_shape=(1,)):
        out = oracle.empty(out_shape, dtype=dtype)
        oracle.forward(op, [oracle.tensor(local)], out, dim=dim)
        return out.numpy()

    res = {}
    t = torch.from_numpy(reduce_local("sum", FULL_REDUCE).copy())
    res["full_sum"] = pd.all_reduce_sum(dist, t).numpy()
    t = torch.from_numpy(reduce_local("max", FULL_REDUCE).copy())
    res["full_max"] = pd.all_reduce_max(dist, t).numpy()
    t = torch.from_numpy(reduce_local("sum", FULL_REDUCE).copy())
    res["full_mean"] = pd.global_mean(dist, t, M * N).numpy()
    t = torch.from_numpy(reduce_local("sum", 0, out_shape=(N,)).copy())
    res["sum_axis0"] = pd.all_reduce_sum(dist, t).numpy()
    # row reductions need no communication: each rank owns its rows
    res[f"row_max_{rank}"] = reduce_local("max", 1, out_shape=(sh.count,))
    # full argmax: local (value, index) then max / min all-reduces
    v = torch.from_numpy(reduce_local("max", FULL_REDUCE).copy())
    i = torch.from_numpy(reduce_local("argmax", FULL_REDUCE, dtype=INT32).astype(np.int64))
    gmax, gidx = pd.global_argmax(dist, torch, v, i, sh.start * N)
    res["argmax"] = gidx.numpy()
    # cross-entropy mean over row-sharded logits
    labels = np.random.RandomState(1).randint(0, N, size=M).astype(np.int32)
    mean, per_row = OracleRecipes().cross_entropy(local, labels[sh.start:sh.start + sh.count])
    t = torch.from_numpy(per_row.astype(np.float64).sum(keepdims=True).astype(np.float32))
    res["ce_mean"] = pd.global_mean(dist, t, M).numpy()
    np.savez(Path(out_dir) / f"rank{rank}.npz", **res)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_oracle(tmp_path):
    import torch.multiprocessing as mp
    from harness import CpuBackend, FULL_REDUCE, OracleRecipes, rand_uniform

    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / f"rank{k}.npz") for k in range(world)]
    M, N = 101, 64
    X = rand_uniform(0, (M, N))
    x64 = X.astype(np.float64)
    scale = np.abs(x64).sum()
    for k in range(world):                                  # every rank holds the same result
        assert abs(float(r[k]["full_sum"][0]) - x64.sum()) <= 1e-5 * scale
        assert float(r[k]["full_max"][0]) == X.max()
        assert abs(float(r[k]["full_mean"][0]) - x64.mean()) <= 1e-5 * scale / X.size
        assert np.all(np.abs(r[k]["sum_axis0"] - x64.sum(axis=0)) <= 1e-5 * np.abs(x64).sum(axis=0))
        assert int(r[k]["argmax"][0]) == int(np.argmax(X))
    rows = np.concatenate([r[0]["row_max_0"], r[1]["row_max_1"]])
    assert np.array_equal(rows, X.max(axis=1))
    labels = np.random.RandomState(1).randint(0, N, size=M).astype(np.int32)
    want, per_row = OracleRecipes().cross_entropy(X, labels)
    assert abs(float(r[0]["ce_mean"][0]) - float(want[0])) <= 1e-5 * np.abs(per_row).sum() / M
