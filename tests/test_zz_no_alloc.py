"""sum_axis0_noalloc_cuda_forward — the column sum for callers that cannot allocate device memory
(everything already belongs to their own arena, or an allocation would stall the whole device).

It must give what sum_cuda_forward(dim=0) gives, from a fixed scratch array inside the library:
checked on two calls in a row with different data (the array keeps the first call's partials, so
a stale read would show), then on the limits. This file sorts last on purpose: a run that stops
at the first failure has already run every other test.
"""
import numpy as np
import pytest

import plast_b200 as pb
from harness import assert_sum_close, rand_normal, rand_uniform

pytestmark = pytest.mark.gpu


def column_sums(cuda, A, op="sum_axis0_noalloc", keepdim=0):
    out = cuda.empty((1, A.shape[1]) if keepdim else (A.shape[1],))
    cuda.forward(op, [cuda.tensor(A)], out, dim=0, keepdim=keepdim)
    return out.numpy(), out.shape


@pytest.mark.parametrize("rows,cols", [(4096, 1024), (8192, 8192), (1000, 1000), (777, 3), (5, 16384), (1, 7)])
def test_matches_the_allocating_entry_point_twice_in_a_row(cuda, rows, cols):
    for seed in (0, 1):                                   # second call reuses the scratch array
        A = rand_normal(seed, (rows, cols)) if seed == 0 else rand_uniform(seed, (rows, cols), -3, 5)
        got, shape = column_sums(cuda, A)
        want, want_shape = column_sums(cuda, A, op="sum")
        assert shape == want_shape == [cols]
        scale = np.abs(A.astype(np.float64)).sum(axis=0)  # same bound as the other sum tests
        assert_sum_close(got, want, scale, what=f"{rows}x{cols} call {seed}")
        assert_sum_close(got, A.astype(np.float64).sum(axis=0), scale, what="vs fp64")


def test_no_rows_gives_zeros_like_the_allocating_entry_point(cuda):
    """[0, cols]: nothing to add, every column sum is 0; the output must be written, not left stale."""
    A = np.zeros((0, 8), np.float32)
    out = cuda.empty((8,))
    out.copy_from(np.full(8, 7.0, np.float32))            # stale contents that must disappear
    cuda.forward("sum_axis0_noalloc", [cuda.tensor(A)], out, dim=0)
    want = cuda.empty((8,))
    want.copy_from(np.full(8, 7.0, np.float32))
    cuda.forward("sum", [cuda.tensor(A)], want, dim=0)
    assert np.array_equal(out.numpy(), want.numpy()) and np.all(out.numpy() == 0.0)


def test_keepdim_and_reproducibility(cuda):
    A = rand_normal(2, (3000, 2048))
    a, shape = column_sums(cuda, A, keepdim=1)
    assert shape == [1, 2048]
    b, _ = column_sums(cuda, A, keepdim=1)
    assert np.array_equal(a, b)                           # fixed combine order


def test_rejects_what_it_cannot_hold(cuda):
    too_wide = cuda.empty((2, 16385))
    with pytest.raises(pb.PlastError) as e:
        cuda.forward("sum_axis0_noalloc", [too_wide], cuda.empty((16385,)), dim=0)
    assert e.value.code == 6 and "16384" in str(e.value)  # LIMIT, names the maximum
    A = cuda.tensor(rand_normal(0, (8, 8)))
    with pytest.raises(pb.PlastError) as e:
        cuda.forward("sum_axis0_noalloc", [A], cuda.empty((8,)), dim=1)
    assert e.value.code == 5                               # UNSUPPORTED: only the column sum
    with pytest.raises(pb.PlastError):
        cuda.forward("sum_axis0_noalloc", [A.transpose(0, 1)], cuda.empty((8,)), dim=0)
