"""Optimiser steps on the GPU through the reference's own entry-point signatures
(<kind>_step_cuda(optimizer*, Tensor**, int)) against the oracle and the reference's golden runs."""
import ctypes as C

import numpy as np
import pytest

import optim_cases
import plast_b200 as pb
from harness import GOLDEN_DIR, ORACLE_LIB, assert_bit_equal, build_oracle
from plast_b200 import optim as O

pytestmark = pytest.mark.gpu
GOLDEN = np.load(GOLDEN_DIR / "optimizers.npz")


def cuda_step_fn(kind):
    fn = getattr(pb.lib, f"{kind}_step_cuda")

    def call(opt, arr, n):
        fn(opt, arr, n)
        pb.check_error()
    return call


@pytest.mark.parametrize("kind", ["sgd", "adam", "adamw"])
def test_three_steps_match_oracle_bitwise_and_reference_golden(kind):
    build_oracle()
    want = optim_cases.run_oracle(kind, C.CDLL(str(ORACLE_LIB)))
    before = pb.lib.plast_b200_launch_count()
    got, opt = optim_cases.run_through_structs(kind, "cuda", cuda_step_fn(kind))
    assert pb.lib.plast_b200_launch_count() - before == optim_cases.STEPS     # one launch per step
    assert pb.last_kernel() == f"{kind}_multi_tensor"
    assert set(got) == set(want)
    for k in want:
        assert_bit_equal(got[k], want[k].reshape(got[k].shape), k)
        np.testing.assert_allclose(got[k], GOLDEN[k].reshape(got[k].shape), rtol=2e-6, atol=5e-7, err_msg=k)
    if kind != "sgd":
        assert opt.t == optim_cases.STEPS
        O.release_state(opt)


def test_more_parameters_than_one_table_and_unaligned_views():
    rs = np.random.RandomState(0)
    sizes = [int(s) for s in rs.randint(1, 3000, size=130)] + [1 << 20, (1 << 18) + 3]
    params, ref_p, ref_g = [], [], []
    for i, n in enumerate(sizes):
        p0, g0 = rs.randn(n).astype(np.float32), rs.randn(n).astype(np.float32)
        if i % 3 == 1:                                                    # start one element in: 4-byte aligned only
            base = pb.Tensor((n + 1,), requires_grad=True)
            t = pb.Tensor((n,), _ptr=base.c.data + 4, _base=base)
            g = pb.Tensor((n,), _ptr=base.grad.c.data + 4, _base=base)
            t.copy_from(p0); g.copy_from(g0)
            t.grad, t.c.grad, t.c.requires_grad = g, C.pointer(g.c), True
        else:
            t = pb.Tensor.from_numpy(p0, requires_grad=True)
            t.grad.copy_from(g0)
        params.append(t); ref_p.append(p0); ref_g.append(g0)
    opt = O.SGD(0.05)
    before = pb.lib.plast_b200_launch_count()
    O.step(opt, params)
    assert pb.lib.plast_b200_launch_count() - before == 3                 # 132 parameters, 48 per table
    for t, p0, g0 in zip(params, ref_p, ref_g):
        step = np.float32(0.05) * g0
        assert_bit_equal(t.numpy().ravel(), p0 - step, "sgd over many parameters")


def test_errors_and_empty_lists():
    O.step(O.SGD(0.1), [])                                                # nothing to do, no launch
    pb.lib.sgd_step_cuda(None, O.param_array([]), 0)
    assert pb.lib.plast_b200_last_error() == 3                            # NULL optimizer, as sgd.c:12-15 reports
    pb.lib.plast_b200_clear_error()


def test_adam_rejects_a_longer_parameter_list_than_its_moments_cover():
    ps = [pb.Tensor.from_numpy(np.ones(16, np.float32), requires_grad=True) for _ in range(3)]
    opt = O.Adam()
    opt.lr, opt.beta1, opt.beta2, opt.epsilon, opt.t = 1e-3, 0.9, 0.999, 1e-8, 0
    O.step(opt, ps[:2])
    pb.lib.adam_step_cuda(C.byref(opt), O.param_array(ps), 3)
    assert pb.lib.plast_b200_last_error() == 2
    pb.lib.plast_b200_clear_error()
    O.step(opt, ps[:1])                                                   # a shorter list is fine
    O.release_state(opt)
