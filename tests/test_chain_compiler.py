"""The run-time chain compiler, checked without a GPU: the functor generated for a program, and a
trial NVRTC compile of the complete kernel for sm_100a (skipped where libnvrtc is absent)."""
import ctypes as C

import pytest

import plast_b200 as pb

CHAIN = [("neg", 0, 0, 0.0), ("exp", 2, 0, 0.0), ("add_scalar", 3, 0, 1.0), ("rdiv_scalar", 4, 0, 1.0),
         ("mul", 5, 1, 0.0), ("abs", 0, 0, 0.0), ("neg", 7, 0, 0.0), ("exp", 8, 0, 0.0), ("sub", 6, 9, 0.0)]


def steps_array(steps):
    arr = (pb.ChainStep * len(steps))()
    for i, (name, a, b, f) in enumerate(steps):
        arr[i] = pb.ChainStep(pb.CHAIN_OPCODES[name], a, b, f)
    return arr


def lib():
    handle = C.CDLL(str(pb.LIB_PATH))
    handle.plast_b200_chain_source.argtypes = [C.POINTER(pb.ChainStep), C.c_int, C.c_int, C.c_uint, C.c_char_p, C.c_size_t]
    handle.plast_b200_chain_source.restype = C.c_int
    handle.plast_b200_chain_try_compile.argtypes = [C.POINTER(pb.ChainStep), C.c_int, C.c_int, C.c_uint]
    handle.plast_b200_chain_try_compile.restype = C.c_int
    return handle


def test_generated_functor_has_one_rounded_statement_per_step():
    buf = C.create_string_buffer(8192)
    n = lib().plast_b200_chain_source(steps_array(CHAIN), len(CHAIN), 2, 0, buf, len(buf))
    src = buf.value.decode()
    assert n == len(src)
    lines = [l.strip() for l in src.splitlines()]
    assert "const float r0 = x[0];" in lines and "const float r1 = x[1];" in lines
    assert "const float r2 = -r0;" in lines
    assert "const float r3 = expf(r2);" in lines
    assert "const float r4 = r3 + c[2];" in lines            # constants are kernel arguments
    assert "const float r5 = c[3] / r4;" in lines
    assert "const float r6 = r5 * r1;" in lines
    assert "const float r7 = fabsf(r0);" in lines
    assert "const float r10 = r6 - r9;" in lines and "return r10;" in lines
    assert sum(l.startswith("const float r") for l in lines) == 2 + len(CHAIN)


def test_malformed_programs_are_rejected():
    h = lib()
    assert h.plast_b200_chain_source(steps_array([("add", 0, 5, 0.0)]), 1, 2, 0, None, 0) == -1   # register not yet written
    assert h.plast_b200_chain_source(steps_array(CHAIN), len(CHAIN), 9, 0, None, 0) == -1         # too many inputs


def test_every_opcode_compiles_for_sm_100a():
    prog = [("add", 0, 1, 0), ("sub", 2, 0, 0), ("mul", 3, 1, 0), ("div", 4, 1, 0), ("neg", 5, 0, 0), ("abs", 6, 0, 0),
            ("exp", 7, 0, 0), ("log", 8, 0, 0), ("sin", 9, 0, 0), ("cos", 10, 0, 0), ("tan", 11, 0, 0),
            ("leaky_relu", 12, 0, 0.1), ("add_scalar", 13, 0, 1.0), ("rsub_scalar", 14, 0, 2.0),
            ("mul_scalar", 15, 0, 0.5), ("rdiv_scalar", 16, 0, 3.0)]
    rc = lib().plast_b200_chain_try_compile(steps_array(prog), len(prog), 2, 0)
    if rc == -2:
        pytest.skip("libnvrtc not available on this machine")
    assert rc == 0


def test_one_element_constants_are_read_through_pointers_and_compile():
    # the nine nodes of z = sigmoid(x) * y + exp(-abs(x)) as the graph holds them: inputs x, 1.0, 1.0, y
    prog = [("neg", 0, 0, 0), ("exp", 4, 0, 0), ("add", 1, 5, 0), ("div", 2, 6, 0), ("mul", 7, 3, 0),
            ("abs", 0, 0, 0), ("neg", 9, 0, 0), ("exp", 10, 0, 0), ("add", 8, 11, 0)]
    buf = C.create_string_buffer(8192)
    h = lib()
    assert h.plast_b200_chain_source(steps_array(prog), len(prog), 4, 0b0110, buf, len(buf)) > 0
    lines = [l.strip() for l in buf.value.decode().splitlines()]
    assert "const float r0 = x[0];" in lines and "const float r3 = x[1];" in lines
    assert "const float r1 = __ldg(sp[0]);" in lines and "const float r2 = __ldg(sp[1]);" in lines
    assert h.plast_b200_chain_source(steps_array(prog), len(prog), 4, 0b1111, None, 0) == -1   # no operand left
    rc = h.plast_b200_chain_try_compile(steps_array(prog), len(prog), 4, 0b0110)
    if rc == -2:
        pytest.skip("libnvrtc not available on this machine")
    assert rc == 0


def backward_source(prog, n_inputs, mask, wrt, accumulate):
    h = lib()
    h.plast_b200_chain_backward_source.argtypes = [C.POINTER(pb.ChainStep), C.c_int, C.c_int, C.c_uint, C.c_int,
                                                   C.c_int, C.c_char_p, C.c_size_t]
    h.plast_b200_chain_backward_source.restype = C.c_int
    buf = C.create_string_buffer(16384)
    n = h.plast_b200_chain_backward_source(steps_array(prog), len(prog), n_inputs, mask, wrt, accumulate, buf, len(buf))
    return n, [l.strip() for l in buf.value.decode().splitlines()]


def test_backward_functor_sweeps_the_steps_in_reverse_with_one_rounding_per_contribution():
    # z = (x * y) + exp(x): r2 = r0 * r1, r3 = exp(r0), r4 = r2 + r3
    prog = [("mul", 0, 1, 0), ("exp", 0, 0, 0), ("add", 2, 3, 0)]
    n, lines = backward_source(prog, 2, 0, 0, 1)
    assert n > 0
    assert "const float g = x[0];" in lines and "const float r0 = x[1];" in lines and "const float r1 = x[2];" in lines
    assert "float a0 = x[3];" in lines                      # starts from the current gradient of x
    assert "float a1 = 0.0f;" in lines and "float a4 = g;" in lines
    body = [l for l in lines if l.startswith("a")]
    assert body == ["a2 = a2 + a4; a3 = a3 + a4;",           # add
                    "a0 = a0 + a3 * r3;",                    # exp: g * exp(x), the forward value reused
                    "a0 = a0 + a2 * r1; a1 = a1 + a2 * r0;"]  # mul
    assert "return a0;" in lines
    n, lines = backward_source(prog, 2, 0, 1, 0)            # w.r.t. y, no accumulation operand
    assert "float a1 = 0.0f;" in lines and "return a1;" in lines
    assert backward_source(prog, 2, 0, 2, 0)[0] == -1       # no such input


def test_every_opcode_backward_compiles_for_sm_100a():
    prog = [("add", 0, 1, 0), ("sub", 2, 0, 0), ("mul", 3, 1, 0), ("div", 4, 1, 0), ("neg", 5, 0, 0), ("abs", 6, 0, 0),
            ("exp", 7, 0, 0), ("log", 8, 0, 0), ("sin", 9, 0, 0), ("cos", 10, 0, 0), ("tan", 11, 0, 0),
            ("leaky_relu", 12, 0, 0.1), ("add_scalar", 13, 0, 1.0), ("rsub_scalar", 14, 0, 2.0),
            ("mul_scalar", 15, 0, 0.5), ("rdiv_scalar", 16, 0, 3.0)]
    h = lib()
    h.plast_b200_chain_backward_try_compile.argtypes = [C.POINTER(pb.ChainStep), C.c_int, C.c_int, C.c_uint, C.c_int, C.c_int]
    h.plast_b200_chain_backward_try_compile.restype = C.c_int
    for wrt, acc in ((0, 1), (1, 0)):
        rc = h.plast_b200_chain_backward_try_compile(steps_array(prog), len(prog), 2, 0, wrt, acc)
        if rc == -2:
            pytest.skip("libnvrtc not available on this machine")
        assert rc == 0
