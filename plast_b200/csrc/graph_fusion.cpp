// Graph-level fusion over the scheduler's DAG (host code only): pattern rewrites to the fused
// recipes that have a backward, then grouping of the remaining forward-only elementwise nodes
// into chain programs. The reference's pass for comparison: src/scheduler/fusion.c:28-224
// (matmul / conv + leaky_relu only; it puts the fused node in the first matched slot, which is
// right for a straight chain; a group with several branches needs the LAST slot, after every
// producer of its external operands).
#include "common.cuh"
#include "plast_b200_graph.h"

#include <string.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace pb {
bool chain_jit_available(); // chain_jit.cu
namespace {

struct Program {
  int n_inputs;
  std::vector<PlastChainStep> steps;
};
struct Owned {
  Node *node;
  Tensor **inputs;
};

std::mutex g_mutex;
std::vector<Program> g_programs; // handle = index + 1
std::vector<Owned> g_owned;

bool same_shape(const Tensor *a, const Tensor *b) {
  if (a->ndim != b->ndim) return false;
  for (u64 d = 0; d < a->ndim; ++d)
    if (a->shape[d] != b->shape[d]) return false;
  return true;
}
bool on_gpu_f32(const Tensor *t) { return t && t->device == CUDA && t->dtype == FLOAT32; }

int chain_opcode(OP_TYPE t) {
  switch ((int)t) {
  case ADD: return PLAST_CHAIN_ADD;
  case SUB: return PLAST_CHAIN_SUB;
  case MUL: return PLAST_CHAIN_MUL;
  case DIV: return PLAST_CHAIN_DIV;
  case NEG: return PLAST_CHAIN_NEG;
  case ABS: return PLAST_CHAIN_ABS;
  case EXP: return PLAST_CHAIN_EXP;
  case LOG: return PLAST_CHAIN_LOG;
  case SIN: return PLAST_CHAIN_SIN;
  case COS: return PLAST_CHAIN_COS;
  case TAN: return PLAST_CHAIN_TAN;
  case LEAKY_RELU: return PLAST_CHAIN_LEAKY_RELU;
  default: return -1;
  }
}
int arity(OP_TYPE t) { return (int)t <= (int)DIV ? 2 : 1; }

// The working view of a DAG: node list with tombstones, and who reads each produced tensor.
struct Graph {
  std::vector<Node *> nodes; // nullptr = removed
  std::unordered_map<const Node *, int> index;
  std::unordered_map<const Tensor *, std::vector<int>> readers;

  explicit Graph(DAG *dag) : nodes(dag->nodes, dag->nodes + dag->count) { rebuild(); }
  void rebuild() {
    index.clear();
    readers.clear();
    for (int i = 0; i < (int)nodes.size(); ++i) {
      Node *n = nodes[i];
      if (!n) continue;
      index[n] = i;
      for (int k = 0; k < n->num_inputs; ++k) readers[n->inputs[k]].push_back(i);
    }
  }
  // The node of this DAG that produced t, if any.
  int producer(const Tensor *t) const {
    if (!t || !t->creator) return -1;
    auto it = index.find(t->creator);
    if (it == index.end() || nodes[it->second]->output != t) return -1;
    return it->second;
  }
  Node *producer_node(const Tensor *t, OP_TYPE want) const {
    const int i = producer(t);
    if (i < 0 || nodes[i]->op_type != want || nodes[i]->num_inputs != arity_of(want)) return nullptr;
    return on_gpu_f32(nodes[i]->output) ? nodes[i] : nullptr;
  }
  static int arity_of(OP_TYPE t) {
    switch ((int)t) {
    case ADD: case SUB: case MUL: case DIV: return 2;
    default: return 1;
    }
  }
  // True when every reader of t in this DAG is one of `allowed`.
  bool read_only_by(const Tensor *t, std::initializer_list<const Node *> allowed) const {
    auto it = readers.find(t);
    if (it == readers.end()) return false;
    for (int r : it->second) {
      bool ok = false;
      for (const Node *a : allowed) ok = ok || nodes[r] == a;
      if (!ok) return false;
    }
    return true;
  }
};

Node *make_node(int op_type, ForwardKernel fwd, BackwardKernel bwd, const std::vector<Tensor *> &inputs,
                Tensor *output, KernelParams params) {
  Node *n = new Node();
  Tensor **in = new Tensor *[inputs.size()];
  std::copy(inputs.begin(), inputs.end(), in);
  n->inputs = in;
  n->num_inputs = (int)inputs.size();
  n->output = output;
  n->op.cpu_forward = nullptr;
  n->op.cpu_backward = nullptr;
  n->op.cuda_forward = fwd;
  n->op.cuda_backward = bwd;
  memcpy(&n->op_type, &op_type, sizeof(int)); // a value past the enum's range: no enum cast
  n->visited = false;
  n->on_stack = false;
  n->params = params;
  output->creator = n;
  std::lock_guard<std::mutex> lock(g_mutex);
  g_owned.push_back({n, in});
  return n;
}

// Puts `fused` in the slot of `last` (the member with the highest index: every producer of an
// external operand comes before it, every reader of the result after it) and removes the rest.
void replace(Graph &g, const std::vector<Node *> &members, Node *last, Node *fused) {
  for (Node *m : members) g.nodes[g.index[m]] = nullptr;
  g.nodes[g.index[last]] = fused;
  g.rebuild();
}

bool is_keepdim_reduce(const Node *n, u64 dim) { return n->params.dim == dim && n->params.keepdim != 0; }

// exp(x - max(x)) with its row sum: the common front of softmax and log_softmax
// (plast/nn/functional.py:77-97). Fills the five handles when the shapes and axes agree.
struct SoftmaxFront {
  Node *mx, *sh, *ex, *se;
  Tensor *x;
  u64 dim;
};
bool match_front(const Graph &g, const Tensor *sum_out, SoftmaxFront *f) {
  f->se = g.producer_node(sum_out, SUM);
  if (!f->se) return false;
  f->dim = f->se->params.dim;
  if (f->se->params.keepdim == 0) return false;
  f->ex = g.producer_node(f->se->inputs[0], EXP);
  if (!f->ex) return false;
  f->sh = g.producer_node(f->ex->inputs[0], SUB);
  if (!f->sh) return false;
  f->x = f->sh->inputs[0];
  f->mx = g.producer_node(f->sh->inputs[1], MAX);
  if (!f->mx || f->mx->inputs[0] != f->x || !is_keepdim_reduce(f->mx, f->dim)) return false;
  if (!on_gpu_f32(f->x) || f->dim >= f->x->ndim) return false;
  if (!same_shape(f->x, f->sh->output) || !same_shape(f->x, f->ex->output)) return false;
  if (!same_shape(f->mx->output, f->se->output)) return false;
  return g.read_only_by(f->mx->output, {f->sh});
}

u32 fuse_softmax_family(Graph &g) {
  u32 made = 0;
  for (int i = 0; i < (int)g.nodes.size(); ++i) {
    Node *n = g.nodes[i];
    if (!n || n->num_inputs != 2 || !on_gpu_f32(n->output)) continue;
    SoftmaxFront f;
    if (n->op_type == DIV) {
      // exp_x / sum(exp_x)
      if (!match_front(g, n->inputs[1], &f) || n->inputs[0] != f.ex->output) continue;
      if (!same_shape(n->output, f.x)) continue;
      if (!g.read_only_by(f.se->output, {n}) || !g.read_only_by(f.ex->output, {f.se, n}) ||
          !g.read_only_by(f.sh->output, {f.ex}))
        continue;
      Node *fused = make_node(PLAST_OP_SOFTMAX, softmax_cuda_forward, softmax_cuda_backward, {f.x},
                              n->output, KernelParams{f.dim, 0, 0.0f});
      replace(g, {f.mx, f.sh, f.ex, f.se, n}, n, fused);
      ++made;
    } else if (n->op_type == SUB) {
      // shifted - log(sum(exp(shifted)))
      Node *lg = g.producer_node(n->inputs[1], LOG);
      if (!lg || !match_front(g, lg->inputs[0], &f) || n->inputs[0] != f.sh->output) continue;
      if (!same_shape(n->output, f.x)) continue;
      if (!g.read_only_by(lg->output, {n}) || !g.read_only_by(f.se->output, {lg}) ||
          !g.read_only_by(f.ex->output, {f.se}) || !g.read_only_by(f.sh->output, {f.ex, n}))
        continue;
      Node *fused = make_node(PLAST_OP_LOG_SOFTMAX, log_softmax_cuda_forward, log_softmax_cuda_backward,
                              {f.x}, n->output, KernelParams{f.dim, 0, 0.0f});
      replace(g, {f.mx, f.sh, f.ex, f.se, lg, n}, n, fused);
      ++made;
    }
  }
  return made;
}

// leaky_relu(a + b) and leaky_relu(v * scale + bias). Addition and multiplication commute
// bitwise, so either operand order matches. These carry a backward, so they are applied to
// training graphs too; the intermediates' grad buffers are then never touched.
u32 fuse_relu_epilogues(Graph &g) {
  u32 made = 0;
  for (int i = 0; i < (int)g.nodes.size(); ++i) {
    Node *n = g.nodes[i];
    if (!n || n->op_type != LEAKY_RELU || n->num_inputs != 1 || !on_gpu_f32(n->output)) continue;
    Node *add = g.producer_node(n->inputs[0], ADD);
    if (!add || !same_shape(add->output, n->output) || !g.read_only_by(add->output, {n})) continue;
    // forward-only graphs are left to the chain pass, which can take in more than these nodes
    if (!n->output->requires_grad && !add->output->requires_grad) continue;
    if (!on_gpu_f32(add->inputs[0]) || !on_gpu_f32(add->inputs[1])) continue;
    Node *fused = nullptr;
    for (int side = 0; side < 2 && !fused; ++side) {
      Node *mul = g.producer_node(add->inputs[side], MUL);
      if (!mul || !same_shape(mul->output, n->output) || !g.read_only_by(mul->output, {add})) continue;
      if (!on_gpu_f32(mul->inputs[0]) || !on_gpu_f32(mul->inputs[1])) continue;
      fused = make_node(PLAST_OP_SCALE_BIAS_LEAKY_RELU, scale_bias_leaky_relu_cuda_forward,
                        scale_bias_leaky_relu_cuda_backward,
                        {mul->inputs[0], mul->inputs[1], add->inputs[1 - side]}, n->output, n->params);
      replace(g, {mul, add, n}, n, fused);
    }
    if (!fused) {
      fused = make_node(PLAST_OP_ADD_LEAKY_RELU, add_leaky_relu_cuda_forward, add_leaky_relu_cuda_backward,
                        {add->inputs[0], add->inputs[1]}, n->output, n->params);
      replace(g, {add, n}, n, fused);
    }
    ++made;
  }
  return made;
}

bool g_with_grad = false; // set for the duration of one pass (under g_pass_mutex)
std::mutex g_pass_mutex;

bool chain_member(const Node *n) {
  if (!n || chain_opcode(n->op_type) < 0 || n->num_inputs != arity(n->op_type)) return false;
  if (!on_gpu_f32(n->output) || (n->output->requires_grad && !g_with_grad)) return false;
  for (int k = 0; k < n->num_inputs; ++k)
    if (!on_gpu_f32(n->inputs[k]) || (n->inputs[k]->requires_grad && !g_with_grad)) return false;
  // with gradients, every tensor that takes part needs its grad buffer at backward time
  if (n->output->requires_grad && !n->output->grad) return false;
  return true;
}

// External operands of a member set, in order of first use by the members in DAG order.
std::vector<Tensor *> external_inputs(const Graph &g, const std::vector<int> &members) {
  std::vector<Tensor *> ext;
  for (int m : members)
    for (int k = 0; k < g.nodes[m]->num_inputs; ++k) {
      Tensor *t = g.nodes[m]->inputs[k];
      const int p = g.producer(t);
      if (p >= 0 && std::binary_search(members.begin(), members.end(), p)) continue;
      if (std::find(ext.begin(), ext.end(), t) == ext.end()) ext.push_back(t);
    }
  return ext;
}

u32 fuse_chains(Graph &g) {
  u32 made = 0;
  for (int i = (int)g.nodes.size() - 1; i >= 0; --i) {
    Node *root = g.nodes[i];
    if (!chain_member(root)) continue;
    std::vector<int> members{i}; // kept sorted
    bool grew = true;
    while (grew) {
      grew = false;
      for (size_t mi = 0; mi < members.size() && !grew; ++mi) {
        const Node *m = g.nodes[members[mi]];
        for (int k = 0; k < m->num_inputs && !grew; ++k) {
          const Tensor *t = m->inputs[k];
          const int p = g.producer(t);
          if (p < 0 || std::binary_search(members.begin(), members.end(), p)) continue;
          if (!chain_member(g.nodes[p]) || !same_shape(t, root->output)) continue;
          bool inside = true;
          for (int r : g.readers[t]) inside = inside && std::binary_search(members.begin(), members.end(), r);
          if (!inside || (int)members.size() + 1 > PLAST_CHAIN_MAX_STEPS) continue;
          std::vector<int> trial = members;
          trial.insert(std::upper_bound(trial.begin(), trial.end(), p), p);
          if ((int)external_inputs(g, trial).size() > PLAST_CHAIN_MAX_INPUTS) continue;
          members.swap(trial);
          grew = true;
        }
      }
    }
    if (members.size() < 2) continue;
    const std::vector<Tensor *> ext = external_inputs(g, members);
    if (ext.empty() || (int)ext.size() > PLAST_CHAIN_MAX_INPUTS) continue;
    Program prog;
    prog.n_inputs = (int)ext.size();
    auto reg_of = [&](const Tensor *t) {
      const int p = g.producer(t);
      if (p >= 0) {
        auto it = std::lower_bound(members.begin(), members.end(), p);
        if (it != members.end() && *it == p) return prog.n_inputs + (int)(it - members.begin());
      }
      return (int)(std::find(ext.begin(), ext.end(), t) - ext.begin());
    };
    for (int m : members) {
      const Node *n = g.nodes[m];
      PlastChainStep s = {};
      s.opcode = chain_opcode(n->op_type);
      s.a = reg_of(n->inputs[0]);
      s.b = n->num_inputs > 1 ? reg_of(n->inputs[1]) : s.a;
      s.fval = n->params.fval;
      prog.steps.push_back(s);
    }
    u64 handle;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      g_programs.push_back(prog);
      handle = g_programs.size();
    }
    Node *fused = make_node(PLAST_OP_FUSED_CHAIN, chain_cuda_forward, chain_cuda_backward, ext,
                            root->output, KernelParams{handle, 0, 0.0f});
    std::vector<Node *> gone;
    for (int m : members) gone.push_back(g.nodes[m]);
    replace(g, gone, root, fused);
    ++made;
  }
  return made;
}

} // namespace
} // namespace pb

using namespace pb;

extern "C" {

u32 plast_b200_fuse_graph(DAG *dag) { return plast_b200_fuse_graph_ex(dag, 0u); }

u32 plast_b200_fuse_graph_ex(DAG *dag, unsigned flags) {
  if (!dag || !dag->nodes || dag->count < 2) return 0;
  std::lock_guard<std::mutex> pass_lock(g_pass_mutex);
  g_with_grad = (flags & PLAST_B200_FUSE_CHAINS_WITH_GRAD) != 0 && chain_jit_available();
  for (u32 i = 0; i < dag->count; ++i)
    if (!dag->nodes[i] || !dag->nodes[i]->output || !dag->nodes[i]->inputs) return 0;
  Graph g(dag);
  u32 made = fuse_softmax_family(g);
  made += fuse_relu_epilogues(g);
  made += fuse_chains(g);
  if (!made) return 0;
  u32 w = 0;
  for (Node *n : g.nodes)
    if (n) dag->nodes[w++] = n;
  dag->count = w;
  dag->changed = true;
  return made;
}

void plast_b200_fusion_release(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (Owned &o : g_owned) {
    delete[] o.inputs;
    delete o.node;
  }
  g_owned.clear();
  g_programs.clear();
}

int plast_b200_fusion_program(u64 handle, PlastChainStep *steps, int max_steps, int *n_inputs) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (handle == 0 || handle > g_programs.size()) return 0;
  const Program &p = g_programs[handle - 1];
  if (n_inputs) *n_inputs = p.n_inputs;
  for (int s = 0; steps && s < (int)p.steps.size() && s < max_steps; ++s) steps[s] = p.steps[s];
  return (int)p.steps.size();
}

void chain_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  Program prog;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (params.dim == 0 || params.dim > g_programs.size()) {
      begin_call();
      set_error(PLAST_B200_ERR_SHAPE, "chain: unknown program handle %llu", (unsigned long long)params.dim);
      return;
    }
    prog = g_programs[params.dim - 1];
  }
  plast_b200_chain_forward(inputs, prog.n_inputs, output, prog.steps.data(), (int)prog.steps.size());
}

void chain_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  Program prog;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (params.dim == 0 || params.dim > g_programs.size()) {
      begin_call();
      set_error(PLAST_B200_ERR_SHAPE, "chain: unknown program handle %llu", (unsigned long long)params.dim);
      return;
    }
    prog = g_programs[params.dim - 1];
  }
  plast_b200_chain_backward(inputs, prog.n_inputs, output, prog.steps.data(), (int)prog.steps.size());
}

} // extern "C"
