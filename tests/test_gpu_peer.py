"""The NVLink peer exchange (include/plast_b200_peer.h). On one GPU: the degenerate one-rank group
and the bounded wait (a group whose other ranks never signal: the kernel gives up, reports which
rank was missing, and the context stays usable). On two or more GPUs: real ranks under torchrun
against the process group's all-reduce."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plast_b200 as pb
from harness import rand_normal

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _lib():
    lib = pb.lib
    lib.plast_b200_peer_group_local.argtypes = [C.c_int, C.c_uint]
    lib.plast_b200_peer_group_local.restype = C.c_void_p
    lib.plast_b200_peer_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int]
    lib.plast_b200_peer_all_reduce.restype = None
    lib.plast_b200_peer_group_status.argtypes = [C.c_void_p]
    lib.plast_b200_peer_group_status.restype = C.c_int
    lib.plast_b200_peer_group_clear_status.argtypes = [C.c_void_p]
    lib.plast_b200_peer_group_release.argtypes = [C.c_void_p]
    return lib


def test_one_rank_group_completes_by_itself(cuda):
    lib = _lib()
    g = lib.plast_b200_peer_group_local(1, 1000)
    pb.check_error()
    x = rand_normal(0, (8192,))
    t = cuda.tensor(x)
    for op in (0, 1, 2, 0, 1):                                            # both parities, several times
        lib.plast_b200_peer_all_reduce(g, t.c.data, 8192, op)
        pb.check_error()
    assert lib.plast_b200_peer_group_status(g) == 0
    assert np.array_equal(t.numpy(), x)
    lib.plast_b200_peer_all_reduce(g, t.c.data, 8193, 0)                  # beyond the message limit
    assert pb.lib.plast_b200_last_error() == 6
    pb.lib.plast_b200_clear_error()
    lib.plast_b200_peer_group_release(g)


def test_wait_for_a_rank_that_never_arrives_runs_out_and_is_reported(cuda):
    lib = _lib()
    g = lib.plast_b200_peer_group_local(3, 2000)                          # ranks 1 and 2 never signal
    pb.check_error()
    x = rand_normal(1, (100,))
    t = cuda.tensor(x)
    lib.plast_b200_peer_all_reduce(g, t.c.data, 100, 0)
    pb.check_error()                                                      # the launch itself is fine
    assert lib.plast_b200_peer_group_status(g) in (2, 3)                  # a wait for rank 1 (or 2) ran out
    assert np.array_equal(t.numpy(), x)                                   # data left as it was
    lib.plast_b200_peer_group_clear_status(g)
    # the context is still usable
    out = cuda.empty((100,))
    cuda.forward("neg", [t], out)
    assert np.array_equal(out.numpy(), -x)
    lib.plast_b200_peer_group_release(g)


def test_full_reduce_with_the_exchange_inside_the_reduction_kernel(cuda):
    lib = _lib()
    lib.plast_b200_peer_full_reduce.argtypes = [C.c_void_p, C.c_int, C.POINTER(pb.CTensor), C.POINTER(pb.CTensor)]
    lib.plast_b200_peer_full_reduce.restype = None
    g = lib.plast_b200_peer_group_local(1, 1000)                          # one rank: publishes to and polls itself
    pb.check_error()
    x = rand_normal(3, (1 << 22,))
    t = cuda.tensor(x)
    for op, name in ((0, "sum"), (1, "max"), (2, "min"), (0, "sum")):
        want = cuda.empty((1,)); cuda.forward(name, [t], want, dim=pb.FULL_REDUCE)
        got = cuda.empty((1,))
        lib.plast_b200_peer_full_reduce(g, op, C.byref(t.c), C.byref(got.c))
        pb.check_error()
        assert pb.last_kernel() == "reduce_seg_with_peer_exchange"
        assert got.numpy()[0] == want.numpy()[0]                          # same kernel, same bits
    small = cuda.tensor(x[:5].copy())                                     # served by another kernel: exchange follows it
    got = cuda.empty((1,))
    lib.plast_b200_peer_full_reduce(g, 1, C.byref(small.c), C.byref(got.c))
    pb.check_error()
    assert pb.last_kernel() == "peer_all_reduce" and got.numpy()[0] == x[:5].max()
    assert lib.plast_b200_peer_group_status(g) == 0
    lib.plast_b200_peer_group_release(g)
    # bounded wait inside the reduction kernel: ranks 1 and 2 never publish
    g = lib.plast_b200_peer_group_local(3, 2000)
    got = cuda.empty((1,))
    lib.plast_b200_peer_full_reduce(g, 1, C.byref(t.c), C.byref(got.c))
    pb.check_error()
    assert lib.plast_b200_peer_group_status(g) == 2
    assert got.numpy()[0] == x.max()                                      # the local value, flagged as unreduced
    lib.plast_b200_peer_group_release(g)


def test_cross_entropy_mean_with_the_exchange_inside_the_loss_kernel(cuda):
    lib = _lib()
    T = C.POINTER(pb.CTensor)
    lib.plast_b200_peer_cross_entropy_mean.argtypes = [C.c_void_p, T, T, T, C.c_uint64]
    lib.plast_b200_peer_cross_entropy_mean.restype = None
    g = lib.plast_b200_peer_group_local(1, 1000)
    pb.check_error()
    for rows, cols in ((512, 4096), (37, 1000), (64, 10)):                # streaming kernel, and two other layouts
        X = rand_normal(rows, (rows, cols), std=2.0)
        lab = np.random.RandomState(1).randint(0, cols, size=rows).astype(np.int32)
        tx, tl = cuda.tensor(X), cuda.tensor(lab)
        want = cuda.empty((1,)); cuda.forward("cross_entropy", [tx, tl], want)
        got = cuda.empty((1,))
        lib.plast_b200_peer_cross_entropy_mean(g, C.byref(tx.c), C.byref(tl.c), C.byref(got.c), rows)
        pb.check_error()
        if cols % 4 == 0 and cols >= 4096:
            assert pb.last_kernel() == "cross_entropy_rows_with_peer_exchange"
            assert got.numpy()[0] == want.numpy()[0]
        np.testing.assert_allclose(got.numpy()[0], want.numpy()[0], rtol=1e-6)
        # a global row count larger than the local one: the sum is divided by it
        lib.plast_b200_peer_cross_entropy_mean(g, C.byref(tx.c), C.byref(tl.c), C.byref(got.c), 4 * rows)
        pb.check_error()
        np.testing.assert_allclose(got.numpy()[0], want.numpy()[0] / 4, rtol=1e-6)
    assert lib.plast_b200_peer_group_status(g) == 0
    lib.plast_b200_peer_group_release(g)


def test_cross_entropy_mean_fallback_layouts_divide_by_the_global_count(cuda):
    """Layouts the streaming kernel does not take (cols % 4 != 0, a logits pointer that is not
    16-byte aligned) write per-row losses and take their mean with a segmented full reduce once
    there are more than 1024 local rows. That reduce must NOT pick up the link armed for the
    cross-entropy kernel: it would exchange the sum and divide by the local row count."""
    lib = _lib()
    T = C.POINTER(pb.CTensor)
    lib.plast_b200_peer_cross_entropy_mean.argtypes = [C.c_void_p, T, T, T, C.c_uint64]
    lib.plast_b200_peer_cross_entropy_mean.restype = None
    g = lib.plast_b200_peer_group_local(1, 1000)
    pb.check_error()
    rows = 4096
    lab = np.random.RandomState(7).randint(0, 1000, size=rows).astype(np.int32)
    tl = cuda.tensor(lab)
    X = rand_normal(11, (rows, 1000), std=2.0)                            # cols % 4 == 0 but see below
    X3 = rand_normal(12, (rows, 1003), std=2.0)                           # cols % 4 != 0
    cases = [("odd columns", cuda.tensor(X3))]
    # a misaligned logits pointer: the matrix starts one float into its allocation
    base = cuda.empty((rows * 1000 + 4,))
    base.copy_from(np.concatenate([np.zeros(1, np.float32), X.ravel(), np.zeros(3, np.float32)]))
    shifted = pb.Tensor.wrap_pointer(base.c.data + 4, (rows, 1000), owner=base)
    cases.append(("misaligned pointer", shifted))
    for what, tx in cases:
        want = cuda.empty((1,)); cuda.forward("cross_entropy", [tx, tl], want)
        assert pb.last_kernel() != "cross_entropy_rows", what
        got = cuda.empty((1,))
        lib.plast_b200_peer_cross_entropy_mean(g, C.byref(tx.c), C.byref(tl.c), C.byref(got.c), rows)
        pb.check_error()
        np.testing.assert_allclose(got.numpy()[0], want.numpy()[0], rtol=1e-6, err_msg=what)
        lib.plast_b200_peer_cross_entropy_mean(g, C.byref(tx.c), C.byref(tl.c), C.byref(got.c), 4 * rows)
        pb.check_error()
        np.testing.assert_allclose(got.numpy()[0], want.numpy()[0] / 4, rtol=1e-6, err_msg=what)
    assert lib.plast_b200_peer_group_status(g) == 0
    lib.plast_b200_peer_group_release(g)


def test_a_local_failure_still_makes_its_call_of_the_exchange_sequence(cuda):
    """A rank whose local kernel cannot run (here: labels of the wrong dtype) still advances the
    sequence counter, so later exchanges of the group do not wait for a packet that never comes,
    and the group's status word says that this exchange carried an invalid value."""
    lib = _lib()
    T = C.POINTER(pb.CTensor)
    lib.plast_b200_peer_cross_entropy_mean.argtypes = [C.c_void_p, T, T, T, C.c_uint64]
    lib.plast_b200_peer_cross_entropy_mean.restype = None
    g = lib.plast_b200_peer_group_local(1, 1000)
    pb.check_error()
    X = rand_normal(5, (64, 4096))
    tx, bad_labels, out = cuda.tensor(X), cuda.tensor(np.zeros(64, np.float32)), cuda.empty((1,))
    lib.plast_b200_peer_cross_entropy_mean(g, C.byref(tx.c), C.byref(bad_labels.c), C.byref(out.c), 64)
    assert pb.lib.plast_b200_last_error() == 1                            # DTYPE: reported to the caller
    pb.lib.plast_b200_clear_error()
    assert lib.plast_b200_peer_group_status(g) == 0x100                   # ... and on the group
    lib.plast_b200_peer_group_clear_status(g)
    x = rand_normal(6, (16,))
    t = cuda.tensor(x)
    lib.plast_b200_peer_all_reduce(g, t.c.data, 16, 0)                    # the sequence is intact
    pb.check_error()
    assert lib.plast_b200_peer_group_status(g) == 0 and np.array_equal(t.numpy(), x)
    lib.plast_b200_peer_group_release(g)


def _bracket(lib):
    lib.plast_b200_peer_reduce_begin.argtypes = [C.c_void_p]
    lib.plast_b200_peer_reduce_begin.restype = None
    lib.plast_b200_peer_reduce_end.argtypes = [C.c_void_p]
    lib.plast_b200_peer_reduce_end.restype = C.c_int


def test_reductions_inside_the_bracket_are_exchanged_fused_or_parked(cuda):
    """One-rank group: the exchange returns the local value, so every result must equal the plain
    call's bits, and the launch count tells which route a reduction took (1 = exchange inside the
    reduction kernel, 3 = reduce into scratch + exchange kernel + store)."""
    lib = _lib(); _bracket(lib)
    g = lib.plast_b200_peer_group_local(1, 1000)
    pb.check_error()

    def launches(fn):
        n0 = pb.lib.plast_b200_launch_count(); fn(); return pb.lib.plast_b200_launch_count() - n0

    A = rand_normal(0, (4096, 2048))
    ta = cuda.tensor(A)
    want = cuda.empty((2048,)); cuda.forward("sum", [ta], want, dim=0)
    got = cuda.empty((2048,))
    lib.plast_b200_peer_reduce_begin(g)
    n = launches(lambda: cuda.forward("sum", [ta], got, dim=0))          # column reduce: strip owners exchange
    assert lib.plast_b200_peer_reduce_end(g) == 1 and n == 1
    assert np.array_equal(got.numpy(), want.numpy())
    for op in ("max", "min"):
        cuda.forward(op, [ta], want, dim=0)
        lib.plast_b200_peer_reduce_begin(g); cuda.forward(op, [ta], got, dim=0)
        assert lib.plast_b200_peer_reduce_end(g) == 1 and np.array_equal(got.numpy(), want.numpy())
    # a small matrix takes narrow strips (two lanes per CTA, no split): the two strip owners exchange
    S = rand_normal(11, (1024, 1024))
    tsm = cuda.tensor(S)
    want = cuda.empty((1024,)); cuda.forward("sum", [tsm], want, dim=0)
    got_s = cuda.empty((1024,))
    lib.plast_b200_peer_reduce_begin(g)
    n = launches(lambda: cuda.forward("sum", [tsm], got_s, dim=0))
    assert lib.plast_b200_peer_reduce_end(g) == 1 and n == 1
    assert np.array_equal(got_s.numpy(), want.numpy())
    # a full reduction: one thread exchanges
    w1, g1 = cuda.empty((1,)), cuda.empty((1,))
    cuda.forward("sum", [ta], w1, dim=pb.FULL_REDUCE)
    lib.plast_b200_peer_reduce_begin(g)
    n = launches(lambda: cuda.forward("sum", [ta], g1, dim=pb.FULL_REDUCE))
    assert lib.plast_b200_peer_reduce_end(g) == 1 and n == 1 and g1.numpy()[0] == w1.numpy()[0]
    # row sums (many outputs, one warp each): parked, exchanged by the stand-alone kernel, stored
    B = rand_normal(1, (3000, 512))
    tb = cuda.tensor(B)
    want = cuda.empty((3000,)); cuda.forward("sum", [tb], want, dim=1)
    got = cuda.empty((3000,))
    lib.plast_b200_peer_reduce_begin(g)
    n = launches(lambda: cuda.forward("sum", [tb], got, dim=1))
    assert lib.plast_b200_peer_reduce_end(g) == 1 and n == 3
    assert np.array_equal(got.numpy(), want.numpy())
    # a backward call: both broadcast gradients are exchanged and ACCUMULATED onto what was there
    shape, pshape = (6, 16, 14, 14), (1, 16, 1, 1)
    X, S, Bi, G = rand_normal(2, shape), rand_normal(3, pshape), rand_normal(4, pshape), rand_normal(5, shape)
    res = []
    for bracket in (False, True):
        tx, ts, tbias = cuda.tensor(X), cuda.tensor(S, requires_grad=True), cuda.tensor(Bi, requires_grad=True)
        y = cuda.empty(shape, requires_grad=True)
        cuda.forward("scale_bias_leaky_relu", [tx, ts, tbias], y, fval=0.0)
        y.grad.copy_from(G)
        ts.grad.copy_from(np.full(16, 2.0, np.float32)); tbias.grad.copy_from(np.full(16, -3.0, np.float32))
        if bracket:
            lib.plast_b200_peer_reduce_begin(g)
        cuda.backward("scale_bias_leaky_relu", [tx, ts, tbias], y, fval=0.0)
        if bracket:
            assert lib.plast_b200_peer_reduce_end(g) == 2
        res.append((ts.grad.numpy(), tbias.grad.numpy()))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])
    # the config-5 shape in small takes the two-stage route: only its second stage is exchanged
    shape, pshape = (32, 128, 28, 28), (1, 128, 1, 1)
    X, S, Bi, G = rand_normal(6, shape), rand_normal(7, pshape), rand_normal(8, pshape), rand_normal(9, shape)
    res = []
    for bracket in (False, True):
        tx, ts, tbias = cuda.tensor(X), cuda.tensor(S), cuda.tensor(Bi, requires_grad=True)
        y = cuda.empty(shape, requires_grad=True)
        cuda.forward("scale_bias_leaky_relu", [tx, ts, tbias], y, fval=0.0)
        y.grad.copy_from(G)
        if bracket:
            lib.plast_b200_peer_reduce_begin(g)
        n = launches(lambda: cuda.backward("scale_bias_leaky_relu", [tx, ts, tbias], y, fval=0.0))
        if bracket:
            assert lib.plast_b200_peer_reduce_end(g) == 1 and n == 2     # rows stage + column stage with the exchange inside
        res.append(tbias.grad.numpy())
    assert np.array_equal(res[0], res[1])
    # an empty shard still makes its call of the sequence (contributing the start value)
    empty = cuda.tensor(np.zeros((0, 64), np.float32))
    got_e = cuda.empty((64,)); got_e.copy_from(np.full(64, 5.0, np.float32))
    lib.plast_b200_peer_reduce_begin(g)
    cuda.forward("sum", [empty], got_e, dim=0)
    assert lib.plast_b200_peer_reduce_end(g) == 1 and np.all(got_e.numpy() == 0.0)
    # what the bracket cannot serve is refused, nothing is launched
    lib.plast_b200_peer_reduce_begin(g)
    n = launches(lambda: pb.forward("mean", [ta], cuda.empty((2048,)), dim=0, check=False))
    assert n == 0 and pb.lib.plast_b200_last_error() == 5
    wide = cuda.tensor(rand_normal(10, (4, 9000)))
    n = launches(lambda: pb.forward("sum", [wide], cuda.empty((9000,)), dim=0, check=False))
    assert n == 0 and pb.lib.plast_b200_last_error() == 5
    assert lib.plast_b200_peer_reduce_end(g) == 0
    pb.lib.plast_b200_clear_error()
    # after the bracket, reductions are local again
    n = launches(lambda: cuda.forward("sum", [tb], got, dim=1))
    assert n == 1
    assert lib.plast_b200_peer_group_status(g) == 0
    lib.plast_b200_peer_group_release(g)
    # bounded wait inside the column reduce: the other ranks never publish
    g = lib.plast_b200_peer_group_local(3, 2000)
    want = cuda.empty((2048,)); cuda.forward("sum", [ta], want, dim=0)
    lib.plast_b200_peer_reduce_begin(g); cuda.forward("sum", [ta], got, dim=0); lib.plast_b200_peer_reduce_end(g)
    assert lib.plast_b200_peer_group_status(g) == 2
    assert np.array_equal(got.numpy(), want.numpy())                      # local values, flagged as unreduced
    lib.plast_b200_peer_group_release(g)


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs of one box")
def test_real_ranks_match_the_process_group():
    n = min(_gpu_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "peer_worker.py")],
                       capture_output=True, text=True, timeout=300, env=env)
    print(p.stdout[-2000:], p.stderr[-2000:])
    assert p.returncode == 0 and "PEER OK" in p.stdout
