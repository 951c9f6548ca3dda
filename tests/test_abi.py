"""The drop-in boundary, checked without a GPU: struct layouts, exported symbols, planner."""
import ctypes as C
import os
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

import plast_b200 as pb

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "plast_b200.h"
REF_INCLUDE = Path(os.environ.get("PLAST_REFERENCE", "/root/reference")) / "include"

PROBE = r"""
#include <stdio.h>
#include <stddef.h>
%s
int main(void) {
  printf("%%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%d %%d %%d %%d %%d\n",
         sizeof(Tensor), offsetof(Tensor, grad), offsetof(Tensor, creator), offsetof(Tensor, data),
         offsetof(Tensor, shape), offsetof(Tensor, strides), offsetof(Tensor, ndim),
         offsetof(Tensor, dtype), offsetof(Tensor, device), offsetof(Tensor, requires_grad),
         sizeof(KernelParams), offsetof(KernelParams, dim), offsetof(KernelParams, keepdim),
         offsetof(KernelParams, fval), (int)INT32, (int)FLOAT32, (int)CPU, (int)CUDA, (int)MAX_NDIM);
  return 0;
}
"""
EXPECTED = "176 0 8 16 24 88 152 160 164 168 24 0 8 16 0 1 0 1 8"


def _probe(tmp_path, includes, flags):
    src = tmp_path / "probe.c"
    src.write_text(PROBE % includes)
    exe = tmp_path / "probe"
    subprocess.run(["gcc", "-std=c11", *flags, str(src), "-o", str(exe)], check=True)
    return subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip()


def test_struct_layout_of_our_header(tmp_path):
    assert _probe(tmp_path, '#include "plast_b200.h"', [f"-I{ROOT / 'include'}"]) == EXPECTED


@pytest.mark.skipif(not REF_INCLUDE.exists(), reason="reference headers not on this machine")
def test_struct_layout_matches_reference_headers(tmp_path):
    got = _probe(tmp_path, '#include "core/definitions.h"\n#include "core/tensor.h"', [f"-I{REF_INCLUDE}"])
    assert got == EXPECTED
    # and our header compiles against the reference's own types
    got = _probe(tmp_path, '#define PLAST_B200_USE_REFERENCE_TYPES\n#include "plast_b200.h"',
                 [f"-I{ROOT / 'include'}", f"-I{REF_INCLUDE}"])
    assert got == EXPECTED


def test_ctypes_mirror_matches():
    assert C.sizeof(pb.CTensor) == 176 and C.sizeof(pb.KernelParams) == 24


def _header_functions():
    found = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        text = text[text.index('extern "C" {'):]
        found |= set(re.findall(r"\b([a-z_0-9]+)\s*\([^;{]*\)\s*;", text))
    return found


def test_library_exports_every_declared_symbol():
    declared = _header_functions()
    assert declared == set(pb.declared_symbols()), declared ^ set(pb.declared_symbols())
    lib = C.CDLL(str(pb.LIB_PATH))          # loads without a GPU (CUDA runtime is linked statically)
    missing = [s for s in declared if not hasattr(lib, s)]
    assert not missing, missing
    assert b"sm_100a" in pb.lib.plast_b200_version()
    # the C++-linkage pack wrappers the reference's bindings call (include/kernels/pack.h:17-23)
    syms = subprocess.run(["nm", "-D", "--defined-only", str(pb.LIB_PATH)], capture_output=True, text=True).stdout
    assert "cuda_tensor_pack_init" in syms and "cuda_tensor_pack_release" in syms


def test_every_reference_cuda_entry_point_has_a_replacement():
    """Names bound by the reference's op table for this path: include/kernels/ops/{binary,unary,
    reduce}.h, plus the helper symbols its core links (cuda_tensor_init.h, arena_cuda.h, ...)."""
    ops = ["add", "sub", "mul", "div", "abs", "cos", "sin", "tan", "exp", "log", "neg", "leaky_relu",
           "sum", "mean", "max", "min"]
    want = [f"{o}_cuda_{d}" for o in ops for d in ("forward", "backward")]
    want += ["zeros_cuda", "ones_cuda", "set_ones_grad_cuda", "zero_grad_cuda", "reshape_backward_cuda",
             "transpose_backward_cuda", "arena_alloc_cuda", "arena_free_cuda", "arena_memset_cuda",
             "arena_memcpy_h2d_cuda", "arena_memcpy_d2h_cuda", "arena_memcpy_d2d_cuda"]
    lib = C.CDLL(str(pb.LIB_PATH))
    assert not [s for s in want if not hasattr(lib, s)]


# ---- host planner ---------------------------------------------------------------------------------
def plan(shape, strides, reduced=None, sort_arg=0):
    lib = C.CDLL(str(pb.LIB_PATH))
    nargs, nd = len(strides), len(shape)
    st = (C.c_uint64 * (nargs * 8))()
    for a, row in enumerate(strides):
        for d, v in enumerate(row):
            st[a * 8 + d] = v
    sh = (C.c_uint64 * 8)(*shape)
    red = (C.c_ubyte * 8)(*[int(r) for r in reduced]) if reduced is not None else None
    osz, ost, ored = (C.c_uint64 * 8)(), (C.c_uint64 * (nargs * 8))(), (C.c_ubyte * 8)()
    lib.plast_b200_plan_debug.restype = C.c_int
    n = lib.plast_b200_plan_debug(sh, C.c_uint64(nd), nargs, st, red, sort_arg, osz, ost, ored)
    assert n >= 1
    return ([osz[d] for d in range(n)], [[ost[a * 8 + d] for d in range(n)] for a in range(nargs)],
            [ored[d] for d in range(n)])


def test_planner_merges_contiguous_and_broadcast_dims():
    # same-shape contiguous 4-D -> one dim
    assert plan([6, 8, 5, 5], [[200, 25, 5, 1]] * 3)[0] == [1200]
    # NCHW with a per-channel operand: [HW, C, N], operand strides [0, 1, 0]
    size, st, _ = plan([256, 256, 56, 56], [[802816, 3136, 56, 1], [802816, 3136, 56, 1], [0, 1, 0, 0]])
    assert size == [3136, 256, 256] and st[2] == [0, 1, 0] and st[0] == [1, 3136, 802816]
    # row vector against a matrix, scalar operand, size-1 dims dropped
    assert plan([1024, 1024], [[1024, 1], [1024, 1], [0, 1]])[0] == [1024, 1024]
    assert plan([3, 1, 4], [[4, 4, 1], [4, 4, 1], [0, 0, 0]])[0] == [12]
    assert plan([1, 1], [[1, 1], [1, 1]])[0] == [1]


def test_planner_orders_by_memory_and_keeps_reduced_dims_apart():
    # transposed view [M,N] strides [1,M] reduced over view axis 0 -> memory-contiguous runs are reduced
    size, st, red = plan([8192, 8192], [[0, 1], [1, 8192]], reduced=[1, 0], sort_arg=1)
    assert size == [8192, 8192] and st[1] == [1, 8192] and red == [1, 0]
    # a full reduce of a dense transposed view is one run over its memory
    size, st, red = plan([8192, 8192], [[0, 0], [1, 8192]], reduced=[1, 1], sort_arg=1)
    assert size == [8192 * 8192] and red == [1]
    # NCHW bias gradient: (N, H, W) reduced, C kept -> [HW reduced, C kept, N reduced]
    size, st, red = plan([256, 256, 56, 56], [[0, 1, 0, 0], [802816, 3136, 56, 1]], reduced=[1, 0, 1, 1], sort_arg=1)
    assert size == [3136, 256, 256] and red == [1, 0, 1]
