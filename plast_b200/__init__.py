"""plast_b200 — sm_100a kernels behind plast's kernel entry points.

The product is the C-ABI shared library ``libplast_b200.so`` (declared in
``include/plast_b200.h``). This package is the thin Python host side used by the tests and the
benchmark: it loads the library with ctypes, mirrors the ``Tensor`` / ``KernelParams`` structs,
and offers small helpers to build tensors in device memory and call an entry point the way
plast's ``execute_forward`` / ``execute_backward`` do (src/core/node.c:22-32).

There is no CPU fallback: if the library is missing or cannot be loaded, importing
:data:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

MAX_NDIM = 8
FULL_REDUCE = MAX_NDIM + 1  # params.dim value for "reduce everything" (plast/tensor.py:601)
INT32, FLOAT32 = 0, 1
CPU, CUDA = 0, 1

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libplast_b200.so"


class KernelParams(C.Structure):
    """include/core/definitions.h:19-23"""

    _fields_ = [("dim", C.c_uint64), ("keepdim", C.c_uint64), ("fval", C.c_float)]


class CTensor(C.Structure):
    """include/core/tensor.h:20-30"""


CTensor._fields_ = [
    ("grad", C.POINTER(CTensor)),
    ("creator", C.c_void_p),
    ("data", C.c_void_p),
    ("shape", C.c_uint64 * MAX_NDIM),
    ("strides", C.c_uint64 * MAX_NDIM),
    ("ndim", C.c_uint64),
    ("dtype", C.c_int),
    ("device", C.c_int),
    ("requires_grad", C.c_bool),
]

assert C.sizeof(KernelParams) == 24
assert C.sizeof(CTensor) == 176
assert CTensor.shape.offset == 24 and CTensor.strides.offset == 88 and CTensor.ndim.offset == 152
assert CTensor.dtype.offset == 160 and CTensor.device.offset == 164
assert CTensor.requires_grad.offset == 168


class ChainStep(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("fval", C.c_float)]


CHAIN_OPCODES = {
    "add": 0, "sub": 1, "mul": 2, "div": 3, "neg": 4, "abs": 5, "exp": 6, "log": 7, "sin": 8,
    "cos": 9, "tan": 10, "leaky_relu": 11, "add_scalar": 12, "rsub_scalar": 13, "mul_scalar": 14,
    "rdiv_scalar": 15,
}

ERROR_NAMES = {0: "OK", 1: "DTYPE", 2: "SHAPE", 3: "NULL", 4: "CUDA", 5: "UNSUPPORTED", 6: "LIMIT"}

FORWARD_OPS = [
    "add", "sub", "mul", "div", "abs", "cos", "sin", "tan", "exp", "log", "neg", "leaky_relu",
    "sum", "mean", "max", "min", "argmax", "softmax", "log_softmax", "cross_entropy", "sigmoid",
    "scale_bias_leaky_relu", "add_leaky_relu",
]
BACKWARD_OPS = [op for op in FORWARD_OPS if op != "argmax"]

_FWD = C.CFUNCTYPE(None, C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams)


def declared_symbols() -> list[str]:
    """Every extern "C" symbol the headers under include/ declare."""
    syms = [f"{op}_cuda_forward" for op in FORWARD_OPS] + [f"{op}_cuda_backward" for op in BACKWARD_OPS]
    syms += [
        "plast_b200_chain_forward", "plast_b200_chain_forward_host", "zeros_cuda", "ones_cuda", "set_ones_grad_cuda", "zero_grad_cuda",
        "reshape_backward_cuda", "transpose_backward_cuda", "arena_alloc_cuda", "arena_free_cuda",
        "arena_memset_cuda", "arena_memcpy_h2d_cuda", "arena_memcpy_d2h_cuda", "arena_memcpy_d2d_cuda",
        "plast_b200_pack", "plast_b200_last_error", "plast_b200_last_error_message",
        "plast_b200_clear_error", "plast_b200_set_stream", "plast_b200_get_stream",
        "plast_b200_set_sync", "plast_b200_launch_count", "plast_b200_last_kernel",
        "plast_b200_release_workspace", "plast_b200_version", "plast_b200_plan_debug",
        "sum_axis0_noalloc_cuda_forward", "plast_b200_chain_source", "plast_b200_chain_try_compile", "plast_b200_tune",
        "plast_b200_arena_fill_policy", "plast_b200_arena_fill_stats",
        "plast_b200_fuse_graph", "plast_b200_fusion_release", "plast_b200_fusion_program",
        "chain_cuda_forward", "chain_cuda_backward",
        "sgd_step_cuda", "adam_step_cuda", "adamw_step_cuda", "plast_b200_adam_state_release",
        "plast_b200_relu_grad_modulate", "plast_b200_bias_grad_reduce", "plast_b200_bias_grad_masked",
        "plast_b200_add_leaky_relu_row_sum", "plast_b200_chain_backward", "plast_b200_chain_backward_source",
        "plast_b200_chain_backward_try_compile", "plast_b200_fuse_graph_ex",
        "plast_b200_dag_capture", "plast_b200_dag_replay", "plast_b200_dag_graph_kernels",
        "plast_b200_dag_graph_release",
        "plast_b200_peer_group_begin", "plast_b200_peer_group_connect", "plast_b200_peer_all_reduce",
        "plast_b200_peer_group_status", "plast_b200_peer_group_clear_status", "plast_b200_peer_group_release",
        "plast_b200_peer_group_local", "plast_b200_chain_jit_available", "plast_b200_peer_full_reduce", "plast_b200_peer_cross_entropy_mean",
        "plast_b200_peer_reduce_begin", "plast_b200_peer_reduce_end",
    ]
    return syms


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m plast_b200.build` "
            "(there is no CPU fallback for the CUDA path)")
    lib = C.CDLL(str(LIB_PATH))
    for op in FORWARD_OPS:
        fn = getattr(lib, f"{op}_cuda_forward")
        fn.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
        fn.restype = None
    for op in BACKWARD_OPS:
        fn = getattr(lib, f"{op}_cuda_backward")
        fn.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
        fn.restype = None
    lib.sum_axis0_noalloc_cuda_forward.argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
    lib.sum_axis0_noalloc_cuda_forward.restype = None
    lib.plast_b200_chain_forward.argtypes = [C.POINTER(C.POINTER(CTensor)), C.c_int, C.POINTER(CTensor),
                                             C.POINTER(ChainStep), C.c_int]
    lib.plast_b200_chain_forward.restype = None
    lib.plast_b200_chain_backward.argtypes = [C.POINTER(C.POINTER(CTensor)), C.c_int, C.POINTER(CTensor),
                                              C.POINTER(ChainStep), C.c_int]
    lib.plast_b200_chain_backward.restype = None
    lib.plast_b200_chain_forward_host.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_int, C.c_void_p,
                                                  C.c_uint64, C.POINTER(ChainStep), C.c_int]
    lib.plast_b200_chain_forward_host.restype = None
    lib.plast_b200_add_leaky_relu_row_sum.argtypes = [C.POINTER(CTensor)] * 4 + [C.c_float]
    lib.plast_b200_add_leaky_relu_row_sum.restype = None
    lib.plast_b200_relu_grad_modulate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_float]
    lib.plast_b200_bias_grad_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
    lib.plast_b200_bias_grad_masked.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_float]
    for name in ("plast_b200_relu_grad_modulate", "plast_b200_bias_grad_reduce", "plast_b200_bias_grad_masked"):
        getattr(lib, name).restype = None
    for name in ("zeros_cuda", "ones_cuda"):
        getattr(lib, name).argtypes = [C.POINTER(CTensor), C.c_uint64]
        getattr(lib, name).restype = None
    for name in ("set_ones_grad_cuda", "zero_grad_cuda"):
        getattr(lib, name).argtypes = [C.POINTER(CTensor)]
        getattr(lib, name).restype = None
    lib.reshape_backward_cuda.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
    lib.reshape_backward_cuda.restype = None
    lib.transpose_backward_cuda.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64),
                                            C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_uint64,
                                            C.c_uint64, C.c_uint64, C.c_uint64]
    lib.transpose_backward_cuda.restype = None
    lib.arena_alloc_cuda.argtypes = [C.c_uint64]
    lib.arena_alloc_cuda.restype = C.c_void_p
    lib.arena_free_cuda.argtypes = [C.c_void_p]
    lib.arena_free_cuda.restype = None
    lib.arena_memset_cuda.argtypes = [C.c_void_p, C.c_int, C.c_uint64]
    lib.arena_memset_cuda.restype = None
    for name in ("arena_memcpy_h2d_cuda", "arena_memcpy_d2h_cuda", "arena_memcpy_d2d_cuda"):
        getattr(lib, name).argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        getattr(lib, name).restype = None
    lib.plast_b200_pack.argtypes = [C.POINTER(CTensor), C.c_void_p]
    lib.plast_b200_pack.restype = None
    lib.plast_b200_last_error.restype = C.c_int
    lib.plast_b200_last_error_message.restype = C.c_char_p
    lib.plast_b200_set_stream.argtypes = [C.c_void_p]
    lib.plast_b200_set_stream.restype = None
    lib.plast_b200_get_stream.restype = C.c_void_p
    lib.plast_b200_set_sync.argtypes = [C.c_int]
    lib.plast_b200_launch_count.restype = C.c_uint64
    lib.plast_b200_last_kernel.restype = C.c_char_p
    lib.plast_b200_version.restype = C.c_char_p
    lib.plast_b200_arena_fill_policy.argtypes = [C.c_int]
    lib.plast_b200_arena_fill_policy.restype = None
    lib.plast_b200_arena_fill_stats.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    lib.plast_b200_arena_fill_stats.restype = None
    lib.plast_b200_tune.argtypes = [C.c_int, C.c_long]
    lib.plast_b200_tune.restype = None
    return lib


class _LazyLib:
    """Loads libplast_b200.so on first attribute access; raises if it cannot."""

    _lib = None

    def __getattr__(self, name):
        if _LazyLib._lib is None:
            _LazyLib._lib = _load()
        return getattr(_LazyLib._lib, name)


lib = _LazyLib()


class PlastError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"plast_b200 error {ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


def contiguous_strides(shape) -> list[int]:
    st, s = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        st[i] = s
        s *= int(shape[i])
    return st


class Tensor:
    """Host-side handle: a ctypes ``Tensor`` struct plus whatever keeps its memory alive.

    ``device='cuda'`` tensors own (or view) device memory obtained from the library's own
    ``arena_alloc_cuda``; ``device='cpu'`` tensors wrap a numpy array and are what the CPU
    checkers (oracle / reference build) consume through the same struct layout.
    """

    def __init__(self, shape, device="cuda", dtype=FLOAT32, strides=None, requires_grad=False,
                 _base=None, _storage_elems=None, _ptr=None):
        shape = [int(s) for s in shape]
        if len(shape) > MAX_NDIM:
            raise ValueError("ndim > MAX_NDIM")
        self.device = device
        self.c = CTensor()
        self.c.ndim = len(shape)
        for i, s in enumerate(shape):
            self.c.shape[i] = s
        st = contiguous_strides(shape) if strides is None else [int(s) for s in strides]
        for i, s in enumerate(st):
            self.c.strides[i] = s
        self.c.dtype = dtype
        self.c.device = CUDA if device == "cuda" else CPU
        self.c.requires_grad = bool(requires_grad)
        self.c.creator = None
        self._base = _base
        self._np = None
        self._dptr = None
        self.grad = None
        n = int(np.prod(shape)) if shape else 1
        self._storage_elems = n if _storage_elems is None else _storage_elems
        if _ptr is not None:
            self.c.data = _ptr          # caller-owned memory; _base keeps its owner alive
        elif _base is None:
            if device == "cuda":
                self._dptr = lib.arena_alloc_cuda(max(self._storage_elems, 1) * 4)
                self.c.data = self._dptr
            else:
                self._np = np.zeros(max(self._storage_elems, 1), dtype=np.float32 if dtype == FLOAT32 else np.int32)
                self.c.data = self._np.ctypes.data
        else:
            self.c.data = _base.c.data
        if requires_grad:
            self.attach_grad()

    # -- construction -------------------------------------------------------------------------
    @staticmethod
    def from_numpy(arr: np.ndarray, device="cuda", requires_grad=False) -> "Tensor":
        shape = np.shape(arr)                      # ascontiguousarray would turn a 0-dim array into [1]
        arr = np.ascontiguousarray(arr)
        dtype = INT32 if arr.dtype == np.int32 else FLOAT32
        if dtype == FLOAT32:
            arr = arr.astype(np.float32, copy=False)
        t = Tensor(shape, device=device, dtype=dtype, requires_grad=requires_grad)
        t.copy_from(arr)
        return t

    @staticmethod
    def wrap_pointer(ptr: int, shape, device="cuda", dtype=FLOAT32, strides=None, owner=None) -> "Tensor":
        """A Tensor struct over memory somebody else owns (e.g. a torch allocation)."""
        return Tensor(shape, device=device, dtype=dtype, strides=strides, _base=owner, _ptr=ptr)

    def attach_grad(self):
        shape = [self.c.shape[i] for i in range(self.c.ndim)]
        g = Tensor(shape, device=self.device, dtype=self.c.dtype)
        g.zero_()
        self.grad = g
        self.c.grad = C.pointer(g.c)
        self.c.requires_grad = True
        return g

    def view(self, shape, strides, offset: int = 0) -> "Tensor":
        """Metadata-only view sharing this tensor's memory (what plast's shape ops produce,
        src/kernels/cpu/shape_ops.c:28-80); `offset` elements into it (a slice: the view's data
        pointer is moved, as plast's Tensor has no offset field)."""
        return Tensor(shape, device=self.device, dtype=self.c.dtype, strides=strides, _base=self,
                      _storage_elems=self._storage_elems, _ptr=int(self.c.data) + 4 * int(offset))

    def transpose(self, a1: int, a2: int) -> "Tensor":
        sh, st = self.shape, self.strides
        sh[a1], sh[a2] = sh[a2], sh[a1]
        st[a1], st[a2] = st[a2], st[a1]
        return self.view(sh, st)

    # -- data movement ------------------------------------------------------------------------
    @property
    def shape(self):
        return [int(self.c.shape[i]) for i in range(self.c.ndim)]

    @property
    def strides(self):
        return [int(self.c.strides[i]) for i in range(self.c.ndim)]

    @property
    def np_dtype(self):
        return np.int32 if self.c.dtype == INT32 else np.float32

    def copy_from(self, arr: np.ndarray):
        arr = np.ascontiguousarray(arr, dtype=self.np_dtype).ravel()
        assert arr.size <= max(self._storage_elems, 1)
        if self.device == "cuda":
            lib.arena_memcpy_h2d_cuda(self.c.data, arr.ctypes.data, arr.size * 4)
        else:
            C.memmove(self.c.data, arr.ctypes.data, arr.size * 4)

    def zero_(self):
        if self.device == "cuda":
            lib.arena_memset_cuda(self.c.data, 0, max(self._storage_elems, 1) * 4)
        else:
            C.memset(self.c.data, 0, max(self._storage_elems, 1) * 4)

    def storage(self) -> np.ndarray:
        """The underlying memory as a flat numpy array (copied to the host for CUDA tensors)."""
        out = np.empty(max(self._storage_elems, 1), dtype=self.np_dtype)
        if self.device == "cuda":
            lib.arena_memcpy_d2h_cuda(out.ctypes.data, self.c.data, out.size * 4)
        else:
            C.memmove(out.ctypes.data, self.c.data, out.size * 4)
        return out

    def numpy(self) -> np.ndarray:
        """Values of the view, in its logical shape."""
        flat = self.storage()
        shape, strides = self.shape, self.strides
        if not shape:
            return flat[:1].reshape(())
        return np.lib.stride_tricks.as_strided(flat, shape=shape, strides=[s * 4 for s in strides]).copy()

    def free(self):
        if self._dptr is not None:
            lib.arena_free_cuda(self._dptr)
            self._dptr = None
        if self.grad is not None:
            self.grad.free()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr_array(tensors):
    arr = (C.POINTER(CTensor) * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = C.pointer(t.c)
    return arr


def check_error():
    code = lib.plast_b200_last_error()
    if code != 0:
        raise PlastError(code, lib.plast_b200_last_error_message().decode())


def forward(op: str, inputs, output: Tensor, dim: int = 0, keepdim: int = 0, fval: float = 0.0,
            check: bool = True):
    """``<op>_cuda_forward(inputs, output, params)``; raises :class:`PlastError` on failure."""
    getattr(lib, f"{op}_cuda_forward")(_ptr_array(inputs), C.byref(output.c),
                                       KernelParams(dim, keepdim, fval))
    if check:
        check_error()
    return output


def backward(op: str, inputs, output: Tensor, dim: int = 0, keepdim: int = 0, fval: float = 0.0,
             check: bool = True):
    """``<op>_cuda_backward(inputs, output, params)``: accumulates into inputs[i].grad."""
    getattr(lib, f"{op}_cuda_backward")(_ptr_array(inputs), C.byref(output.c),
                                        KernelParams(dim, keepdim, fval))
    if check:
        check_error()


def chain_forward(inputs, output: Tensor, steps, check: bool = True):
    """steps: list of (opcode_name, a, b, fval)."""
    arr = (ChainStep * len(steps))()
    for i, (name, a, b, fval) in enumerate(steps):
        arr[i] = ChainStep(CHAIN_OPCODES[name], a, b, fval)
    lib.plast_b200_chain_forward(_ptr_array(inputs), len(inputs), C.byref(output.c), arr, len(steps))
    if check:
        check_error()
    return output


def chain_backward(inputs, output: Tensor, steps, check: bool = True):
    """Accumulates the chain's gradients into inputs[i].grad for every input that requires grad,
    reading output.grad."""
    arr = (ChainStep * len(steps))()
    for i, (name, a, b, fval) in enumerate(steps):
        arr[i] = ChainStep(CHAIN_OPCODES[name], a, b, fval)
    lib.plast_b200_chain_backward(_ptr_array(inputs), len(inputs), C.byref(output.c), arr, len(steps))
    if check:
        check_error()


def chain_forward_host(host_inputs, output, steps, check: bool = True):
    """The chain on host buffers: host_inputs are float32 numpy arrays (or (address, elems) pairs
    for memory owned elsewhere, e.g. a pinned torch tensor) of output.size elements or of 1;
    output likewise. Copies and kernels of successive chunks overlap; returns once everything is
    queued: call synchronize() before reading the output."""
    def addr(a):
        return (a[0], a[1]) if isinstance(a, tuple) else (a.ctypes.data, a.size)
    pairs = [addr(a) for a in host_inputs]
    out_addr, n = addr(output)
    ptrs = (C.c_void_p * len(pairs))(*[p for p, _ in pairs])
    elems = (C.c_uint64 * len(pairs))(*[e for _, e in pairs])
    arr = (ChainStep * len(steps))()
    for i, (name, a, b, fval) in enumerate(steps):
        arr[i] = ChainStep(CHAIN_OPCODES[name], a, b, fval)
    lib.plast_b200_chain_forward_host(ptrs, elems, len(pairs), out_addr, n, arr, len(steps))
    if check:
        check_error()


def synchronize():
    """Blocks until the library's stream has drained (a zero-byte D2H copy on that stream)."""
    lib.arena_memcpy_d2h_cuda(None, None, 0)


def last_kernel() -> str:
    return lib.plast_b200_last_kernel().decode()
