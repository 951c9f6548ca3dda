"""ctypes mirror of the scheduler-side structs (Node, Op, DAG) and the graph fusion pass of
include/plast_b200_graph.h.

The pass only reads and rewrites host structs, so graphs can be built and fused without a GPU;
executing a fused node needs one.
"""
from __future__ import annotations

import ctypes as C

from . import CTensor, ChainStep, KernelParams, lib

# include/core/op.h:8-37
OP_TYPES = ["ADD", "SUB", "MUL", "DIV", "MATMUL", "LEAKY_RELU", "LOG", "EXP", "ABS", "NEG", "SIN", "COS",
            "TAN", "VIEW", "TRANSPOSE", "UNSQUEEZE", "SQUEEZE", "EXPAND", "FLATTEN", "BROADCAST", "MEAN",
            "MIN", "MAX", "SUM", "CONV2D", "MATMUL_RELU", "MATMUL_BIAS_RELU", "CONV_RELU"]
OP = {name: i for i, name in enumerate(OP_TYPES)}
OP.update(FUSED_CHAIN=1000, ADD_LEAKY_RELU=1001, SCALE_BIAS_LEAKY_RELU=1002, SOFTMAX=1003, LOG_SOFTMAX=1004)
# op name -> entry point stem of the primitive ops this library implements
_KERNEL_OF = {"ADD": "add", "SUB": "sub", "MUL": "mul", "DIV": "div", "LEAKY_RELU": "leaky_relu", "LOG": "log",
              "EXP": "exp", "ABS": "abs", "NEG": "neg", "SIN": "sin", "COS": "cos", "TAN": "tan",
              "MEAN": "mean", "MIN": "min", "MAX": "max", "SUM": "sum"}


class COp(C.Structure):
    """include/core/op.h:39-44"""
    _fields_ = [("cpu_forward", C.c_void_p), ("cuda_forward", C.c_void_p),
                ("cpu_backward", C.c_void_p), ("cuda_backward", C.c_void_p)]


class CNode(C.Structure):
    """include/core/node.h:5-14"""
    _fields_ = [("inputs", C.POINTER(C.POINTER(CTensor))), ("output", C.POINTER(CTensor)), ("op", COp),
                ("op_type", C.c_int), ("num_inputs", C.c_int), ("visited", C.c_bool), ("on_stack", C.c_bool),
                ("params", KernelParams)]


class CDAG(C.Structure):
    """include/core/graph.h:8-14"""
    _fields_ = [("nodes", C.POINTER(C.POINTER(CNode))), ("count", C.c_uint32), ("capacity", C.c_uint32),
                ("changed", C.c_bool), ("arena", C.c_void_p)]


assert C.sizeof(COp) == 32 and C.sizeof(CNode) == 88 and C.sizeof(CDAG) == 32
assert CNode.op_type.offset == 48 and CNode.params.offset == 64 and CDAG.arena.offset == 24

lib.plast_b200_fuse_graph.argtypes = [C.POINTER(CDAG)]
lib.plast_b200_fuse_graph.restype = C.c_uint32
lib.plast_b200_fuse_graph_ex.argtypes = [C.POINTER(CDAG), C.c_uint]
lib.plast_b200_fuse_graph_ex.restype = C.c_uint32
FUSE_CHAINS_WITH_GRAD = 1
lib.plast_b200_fusion_release.argtypes = []
lib.plast_b200_fusion_release.restype = None
lib.plast_b200_fusion_program.argtypes = [C.c_uint64, C.POINTER(ChainStep), C.c_int, C.POINTER(C.c_int)]
lib.plast_b200_fusion_program.restype = C.c_int
for _name in ("chain_cuda_forward", "chain_cuda_backward"):
    getattr(lib, _name).argtypes = [C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams]
    getattr(lib, _name).restype = None


lib.plast_b200_dag_capture.argtypes = [C.POINTER(CDAG), C.c_int]
lib.plast_b200_dag_capture.restype = C.c_void_p
lib.plast_b200_dag_replay.argtypes = [C.c_void_p]
lib.plast_b200_dag_replay.restype = None
lib.plast_b200_dag_graph_kernels.argtypes = [C.c_void_p]
lib.plast_b200_dag_graph_kernels.restype = C.c_int
lib.plast_b200_dag_graph_release.argtypes = [C.c_void_p]
lib.plast_b200_dag_graph_release.restype = None


def capture(dag: "CDAG", backward=False):
    """Records the DAG's kernels into a CUDA graph (backward: False / 0 forward pass, True / 1
    backward pass, 2 forward then backward); returns an opaque handle (None on failure, see
    plast_b200.check_error)."""
    return lib.plast_b200_dag_capture(C.byref(dag), int(backward))


def replay(handle) -> None:
    lib.plast_b200_dag_replay(handle)


def symbol_address(name: str) -> int:
    return C.cast(getattr(lib, name), C.c_void_p).value


class Graph:
    """A DAG in the scheduler's own layout, built node by node in topological order (what
    build_dag, src/core/graph.c:52-55, produces)."""

    def __init__(self):
        self.nodes: list[CNode] = []
        self._keep = []

    def node(self, op: str, inputs, output, dim: int = 0, keepdim: int = 0, fval: float = 0.0) -> CNode:
        """inputs / output are plast_b200.Tensor objects (or anything with a .c CTensor)."""
        arr = (C.POINTER(CTensor) * len(inputs))(*[C.pointer(t.c) for t in inputs])
        n = CNode()
        n.inputs = C.cast(arr, C.POINTER(C.POINTER(CTensor)))
        n.output = C.pointer(output.c)
        stem = _KERNEL_OF.get(op)
        if stem:
            n.op.cuda_forward = symbol_address(f"{stem}_cuda_forward")
            n.op.cuda_backward = symbol_address(f"{stem}_cuda_backward")
        n.op_type = OP[op]
        n.num_inputs = len(inputs)
        n.params = KernelParams(dim, keepdim, fval)
        output.c.creator = C.addressof(n)
        self.nodes.append(n)
        self._keep += [arr, inputs, output]
        return n

    def dag(self) -> CDAG:
        arr = (C.POINTER(CNode) * len(self.nodes))(*[C.pointer(n) for n in self.nodes])
        d = CDAG()
        d.nodes = C.cast(arr, C.POINTER(C.POINTER(CNode)))
        d.count = d.capacity = len(self.nodes)
        self._keep.append(arr)
        return d


def fuse(dag: CDAG, flags: int = 0) -> int:
    return lib.plast_b200_fuse_graph_ex(C.byref(dag), flags)


def dag_forward(dag: CDAG) -> None:
    """src/core/graph.c:57-60 for CUDA nodes: run every node's forward kernel in order."""
    fwd = C.CFUNCTYPE(None, C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams)
    for i in range(dag.count):
        n = dag.nodes[i].contents
        fwd(n.op.cuda_forward)(n.inputs, n.output, n.params)


def dag_backward(dag: CDAG) -> None:
    """src/core/graph.c:62-65."""
    bwd = C.CFUNCTYPE(None, C.POINTER(C.POINTER(CTensor)), C.POINTER(CTensor), KernelParams)
    for i in reversed(range(dag.count)):
        n = dag.nodes[i].contents
        bwd(n.op.cuda_backward)(n.inputs, n.output, n.params)


def chain_program(handle: int):
    """(n_inputs, [(opcode, a, b, fval), ...]) of a fused chain node."""
    steps = (ChainStep * 64)()
    n_in = C.c_int(0)
    n = lib.plast_b200_fusion_program(handle, steps, 64, C.byref(n_in))
    return n_in.value, [(steps[i].opcode, steps[i].a, steps[i].b, steps[i].fval) for i in range(n)]
