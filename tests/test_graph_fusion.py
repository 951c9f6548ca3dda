"""The graph fusion pass (include/plast_b200_graph.h) on DAGs in the scheduler's own struct layout.
The pass only reads and rewrites host structs, so none of this needs a GPU; the fused nodes are
executed by tests/test_gpu_graph_fusion.py and by the drop-in check."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import pytest

import plast_b200 as pb
from plast_b200 import graph as G

ROOT = Path(__file__).resolve().parent.parent
REF_INCLUDE = Path(os.environ.get("PLAST_REFERENCE", "/root/reference")) / "include"


def T(shape, requires_grad=False, device="cuda"):
    # the data pointer is never dereferenced by the pass, and no grad buffer is needed
    t = pb.Tensor(shape, device=device, _ptr=0x1000)
    t.c.requires_grad = requires_grad
    return t


def ops_of(dag):
    return [dag.nodes[i].contents.op_type for i in range(dag.count)]


def test_config2_chain_of_nine_nodes_becomes_one_program():
    n = (1 << 20,)
    x, y, one_a, one_b = T(n), T(n), T(()), T(())
    g = G.Graph()
    t = [T(n) for _ in range(9)]
    g.node("NEG", [x], t[0]); g.node("EXP", [t[0]], t[1]); g.node("ADD", [one_a, t[1]], t[2])
    g.node("DIV", [one_b, t[2]], t[3]); g.node("MUL", [t[3], y], t[4])
    g.node("ABS", [x], t[5]); g.node("NEG", [t[5]], t[6]); g.node("EXP", [t[6]], t[7])
    g.node("ADD", [t[4], t[7]], t[8])
    dag = g.dag()
    assert G.fuse(dag) == 1 and dag.count == 1 and dag.changed
    node = dag.nodes[0].contents
    assert node.op_type == G.OP["FUSED_CHAIN"] and node.num_inputs == 4
    assert node.op.cuda_forward == G.symbol_address("chain_cuda_forward")
    assert C.addressof(node.output.contents) == C.addressof(t[8].c)
    assert t[8].c.creator == C.addressof(node)
    ins = [C.addressof(node.inputs[k].contents) for k in range(4)]
    assert ins == [C.addressof(v.c) for v in (x, one_a, one_b, y)]        # order of first use
    n_in, steps = G.chain_program(node.params.dim)
    op = pb.CHAIN_OPCODES
    assert n_in == 4
    assert [(s[0], s[1], s[2]) for s in steps] == [
        (op["neg"], 0, 0), (op["exp"], 4, 4), (op["add"], 1, 5), (op["div"], 2, 6), (op["mul"], 7, 3),
        (op["abs"], 0, 0), (op["neg"], 9, 9), (op["exp"], 10, 10), (op["add"], 8, 11)]


def test_softmax_and_log_softmax_recipes_become_single_nodes():
    for kind in ("softmax", "log_softmax"):
        x = T((64, 128), requires_grad=True)
        mx, sh, ex, se = T((64, 1), True), T((64, 128), True), T((64, 128), True), T((64, 1), True)
        out = T((64, 128), True)
        g = G.Graph()
        g.node("MAX", [x], mx, dim=1, keepdim=1); g.node("SUB", [x, mx], sh); g.node("EXP", [sh], ex)
        g.node("SUM", [ex], se, dim=1, keepdim=1)
        if kind == "softmax":
            g.node("DIV", [ex, se], out)
        else:
            lg = T((64, 1), True)
            g.node("LOG", [se], lg); g.node("SUB", [sh, lg], out)
        loss = T((1,), True)
        g.node("SUM", [out], loss, dim=9)
        dag = g.dag()
        assert G.fuse(dag) == 1
        assert ops_of(dag) == [G.OP[kind.upper()], G.OP["SUM"]]
        node = dag.nodes[0].contents
        assert node.op.cuda_forward == G.symbol_address(f"{kind}_cuda_forward")
        assert node.op.cuda_backward == G.symbol_address(f"{kind}_cuda_backward")
        assert node.num_inputs == 1 and node.params.dim == 1
        assert C.addressof(node.inputs[0].contents) == C.addressof(x.c)


def test_softmax_is_left_alone_when_an_intermediate_has_another_reader():
    x = T((64, 128), True)
    mx, sh, ex, se, out = T((64, 1), True), T((64, 128), True), T((64, 128), True), T((64, 1), True), T((64, 128), True)
    extra = T((64, 128), True)
    g = G.Graph()
    g.node("MAX", [x], mx, dim=1, keepdim=1); g.node("SUB", [x, mx], sh); g.node("EXP", [sh], ex)
    g.node("SUM", [ex], se, dim=1, keepdim=1); g.node("DIV", [ex, se], out)
    g.node("MUL", [out, sh], extra)                                       # reads the shifted logits too
    dag = g.dag()
    assert G.fuse(dag) == 0 and dag.count == 6


def test_training_graphs_use_the_epilogues_that_have_a_backward():
    A, b = T((256, 512)), T((1, 512), requires_grad=True)
    ab, c, s = T((256, 512), True), T((256, 512), True), T((256,), True)
    g = G.Graph()
    g.node("ADD", [A, b], ab); g.node("LEAKY_RELU", [ab], c, fval=0.0); g.node("SUM", [c], s, dim=1)
    dag = g.dag()
    assert G.fuse(dag) == 1 and ops_of(dag) == [G.OP["ADD_LEAKY_RELU"], G.OP["SUM"]]
    node = dag.nodes[0].contents
    assert node.op.cuda_backward == G.symbol_address("add_leaky_relu_cuda_backward")
    # bias on the left, product on the right: both operand orders match
    X, sc, bi = T((8, 16, 4, 4)), T((1, 16, 1, 1), True), T((1, 16, 1, 1), True)
    t, u, y = T((8, 16, 4, 4), True), T((8, 16, 4, 4), True), T((8, 16, 4, 4), True)
    g = G.Graph()
    g.node("MUL", [sc, X], t); g.node("ADD", [bi, t], u); g.node("LEAKY_RELU", [u], y, fval=0.01)
    dag = g.dag()
    assert G.fuse(dag) == 1 and ops_of(dag) == [G.OP["SCALE_BIAS_LEAKY_RELU"]]
    node = dag.nodes[0].contents
    assert [C.addressof(node.inputs[k].contents) for k in range(3)] == [C.addressof(v.c) for v in (sc, X, bi)]
    assert abs(node.params.fval - 0.01) < 1e-9


def test_chain_keeps_a_result_that_someone_outside_the_group_reads():
    x = T((32, 64))
    t, s, u, out = T((32, 64)), T((32, 1)), T((32, 64)), T((32, 64))
    g = G.Graph()
    g.node("EXP", [x], t); g.node("SUM", [t], s, dim=1, keepdim=1); g.node("NEG", [t], u); g.node("ADD", [u, s], out)
    dag = g.dag()
    assert G.fuse(dag) == 1
    assert ops_of(dag) == [G.OP["EXP"], G.OP["SUM"], G.OP["FUSED_CHAIN"]]
    n_in, steps = G.chain_program(dag.nodes[2].contents.params.dim)
    assert n_in == 2 and [s_[0] for s_ in steps] == [pb.CHAIN_OPCODES["neg"], pb.CHAIN_OPCODES["add"]]


def test_nothing_is_fused_on_cpu_tensors_or_through_requires_grad():
    x, t, out = T((16,), device="cpu"), T((16,), device="cpu"), T((16,), device="cpu")
    g = G.Graph()
    g.node("EXP", [x], t); g.node("NEG", [t], out)
    dag = g.dag()
    assert G.fuse(dag) == 0 and dag.count == 2
    x, t, out = T((16,), True), T((16,), True), T((16,), True)
    g = G.Graph()
    g.node("EXP", [x], t); g.node("NEG", [t], out)
    dag = g.dag()
    assert G.fuse(dag) == 0 and dag.count == 2


def test_group_respects_the_input_and_step_limits():
    shape = (128,)
    acc = T(shape)
    g = G.Graph()
    first = T(shape)
    g.node("NEG", [T(shape)], first)
    cur = first
    for _ in range(12):                                                   # 12 more external operands
        nxt = T(shape)
        g.node("ADD", [cur, T(shape)], nxt)
        cur = nxt
    dag = g.dag()
    made = G.fuse(dag)
    assert made >= 1
    for i in range(dag.count):
        n = dag.nodes[i].contents
        if n.op_type == G.OP["FUSED_CHAIN"]:
            n_in, steps = G.chain_program(n.params.dim)
            assert n_in <= 8 and len(steps) <= 24 and n.num_inputs == n_in
    # topological order survives: every input produced in the DAG is produced earlier
    seen = set()
    for i in range(dag.count):
        n = dag.nodes[i].contents
        for k in range(n.num_inputs):
            t = n.inputs[k].contents
            if t.creator:
                assert t.creator in seen or all(t.creator != C.addressof(dag.nodes[j].contents) for j in range(dag.count))
        seen.add(C.addressof(n))


@pytest.mark.skipif(not REF_INCLUDE.exists(), reason="reference headers not on this machine")
def test_node_and_dag_layout_match_reference_headers(tmp_path):
    probe = r'''
#include <stdio.h>
#include <stddef.h>
%s
int main(void) {
  printf("%%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%d %%d %%d %%d\n", sizeof(Op), sizeof(Node),
         offsetof(Node, inputs), offsetof(Node, output), offsetof(Node, op), offsetof(Node, op_type),
         offsetof(Node, num_inputs), offsetof(Node, params), sizeof(DAG), offsetof(DAG, count),
         offsetof(DAG, changed), offsetof(DAG, arena), (int)ADD, (int)LEAKY_RELU, (int)SUM, (int)CONV_RELU);
  return 0;
}'''
    out = []
    for inc, flags in (('#include "plast_b200_graph.h"', [f"-I{ROOT / 'include'}"]),
                       ('#include "core/graph.h"', [f"-I{REF_INCLUDE}"]),
                       ('#define PLAST_B200_USE_REFERENCE_TYPES\n#include "plast_b200_graph.h"',
                        [f"-I{ROOT / 'include'}", f"-I{REF_INCLUDE}"])):
        src = tmp_path / "p.c"
        src.write_text(probe % inc)
        subprocess.run(["gcc", "-std=c11", *flags, str(src), "-o", str(tmp_path / "p")], check=True)
        out.append(subprocess.run([str(tmp_path / "p")], check=True, capture_output=True, text=True).stdout.strip())
    assert out[0] == out[1] == out[2] == "32 88 0 8 16 48 52 64 32 8 16 24 0 5 23 27"


def test_training_chains_are_fused_only_when_a_backward_can_be_generated():
    x, t, out = T((16,), True), T((16,), True), T((16,), True)
    for tensor in (x, t, out):                       # the pass wants grad buffers on tensors that require grad
        g_ = pb.Tensor((16,), device="cuda", _ptr=0x2000)
        tensor.grad, tensor.c.grad = g_, C.pointer(g_.c)
    g = G.Graph()
    g.node("EXP", [x], t); g.node("NEG", [t], out)
    dag = g.dag()
    assert G.fuse(dag) == 0 and dag.count == 2                            # default: forward-only groups
    can = bool(pb.lib.plast_b200_chain_jit_available())                   # needs libnvrtc AND the driver library
    assert G.fuse(dag, G.FUSE_CHAINS_WITH_GRAD) == (1 if can else 0)
    if can:
        node = dag.nodes[0].contents
        assert node.op_type == G.OP["FUSED_CHAIN"]
        assert node.op.cuda_backward == G.symbol_address("chain_cuda_backward")
