"""The host-buffer form of the fused chain (chunks copied in, computed and copied out on three
streams) against the device-resident chain on the same data."""
import numpy as np
import pytest

import plast_b200 as pb
from harness import assert_bit_equal, rand_normal

pytestmark = pytest.mark.gpu

CHUNK = 8 << 20
STEPS = [("neg", 0, 0, 0.0), ("exp", 2, 0, 0.0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
         ("mul", 5, 1, 0.0), ("abs", 0, 0, 0.0), ("neg", 7, 0, 0.0), ("exp", 8, 0, 0.0), ("add", 6, 9, 0.0)]


@pytest.mark.parametrize("n", [1, 1000, CHUNK, CHUNK + 5, 3 * CHUNK + 1, 7 * CHUNK - 3])
def test_host_chain_equals_device_chain(cuda, n):
    x, y = rand_normal(0, (n,)), rand_normal(1, (n,))
    z = np.full(n, np.nan, np.float32)
    pb.chain_forward_host([x, y], z, STEPS)
    pb.synchronize()
    assert pb.last_kernel() == "chain_host_pipeline"
    out = cuda.empty((n,))
    pb.chain_forward([cuda.tensor(x), cuda.tensor(y)], out, STEPS)
    assert_bit_equal(z, out.numpy(), f"host-buffer chain, n = {n}")


def test_one_element_inputs_are_constants_and_calls_can_follow_each_other(cuda):
    n = 2 * CHUNK + 77
    x = rand_normal(2, (n,))
    k = np.float32([1.5])
    prog = [("mul", 0, 1, 0.0), ("sin", 2, 0, 0.0)]
    z1, z2 = np.empty(n, np.float32), np.empty(n, np.float32)
    pb.chain_forward_host([x, k], z1, prog)
    pb.chain_forward_host([z1, k], z2, prog)                              # queued behind the first call
    pb.synchronize()
    out = cuda.empty((n,))
    pb.chain_forward([cuda.tensor(x), cuda.tensor(k.reshape(()))], out, prog)
    assert_bit_equal(z1, out.numpy(), "first call")
    # z1 was still being written by the first call's copies when the second was queued
    pb.chain_forward([cuda.tensor(out.numpy()), cuda.tensor(k.reshape(()))], out, prog)
    assert_bit_equal(z2, out.numpy(), "second call")


def test_bad_sizes_are_rejected():
    x, y, z = np.zeros(10, np.float32), np.zeros(7, np.float32), np.zeros(10, np.float32)
    pb.chain_forward_host([x, y], z, [("add", 0, 1, 0.0)], check=False)
    assert pb.lib.plast_b200_last_error() == 2
    pb.lib.plast_b200_clear_error()
