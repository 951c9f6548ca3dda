"""ctypes mirror of include/plast_b200_optim.h: the optimiser structs of the plast runtime and
the multi-tensor step entry points."""
from __future__ import annotations

import ctypes as C

from . import CTensor, check_error, lib


class SGD(C.Structure):
    """include/optimizers/sgd.h:5-7"""
    _fields_ = [("lr", C.c_float)]


class Adam(C.Structure):
    """include/optimizers/adam.h:5-15"""
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("t", C.c_int), ("m", C.POINTER(C.POINTER(CTensor))), ("v", C.POINTER(C.POINTER(CTensor))),
                ("data_arena", C.c_void_p), ("optimizer_arena", C.c_void_p)]


class AdamW(C.Structure):
    """include/optimizers/adamw.h:5-16"""
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("weight_decay", C.c_float), ("t", C.c_int), ("m", C.POINTER(C.POINTER(CTensor))),
                ("v", C.POINTER(C.POINTER(CTensor))), ("data_arena", C.c_void_p), ("optimizer_arena", C.c_void_p)]


assert C.sizeof(SGD) == 4 and C.sizeof(Adam) == 56 and C.sizeof(AdamW) == 56
assert Adam.t.offset == 16 and Adam.m.offset == 24 and AdamW.t.offset == 20 and AdamW.m.offset == 24

for _name, _struct in (("sgd_step_cuda", SGD), ("adam_step_cuda", Adam), ("adamw_step_cuda", AdamW)):
    getattr(lib, _name).argtypes = [C.POINTER(_struct), C.POINTER(C.POINTER(CTensor)), C.c_int]
    getattr(lib, _name).restype = None
lib.plast_b200_adam_state_release.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(C.POINTER(CTensor))]
lib.plast_b200_adam_state_release.restype = None


def param_array(params):
    """Tensor** for a list of plast_b200.Tensor objects; None entries become NULL."""
    arr = (C.POINTER(CTensor) * max(len(params), 1))()
    for i, p in enumerate(params):
        if p is not None:
            arr[i] = C.pointer(p.c)
    return arr


def step(optimizer, params) -> None:
    """One optimiser step on the GPU over a list of parameters (Tensor objects with .grad)."""
    fn = {SGD: lib.sgd_step_cuda, Adam: lib.adam_step_cuda, AdamW: lib.adamw_step_cuda}[type(optimizer)]
    fn(C.byref(optimizer), param_array(params), len(params))
    check_error()


def release_state(optimizer) -> None:
    if not isinstance(optimizer, SGD) and optimizer.m:
        lib.plast_b200_adam_state_release(optimizer.m, optimizer.v)
        optimizer.m = None
        optimizer.v = None
