/*
 * plast_b200_graph.h — graph-level fusion for the plast scheduler: a pass over the scheduler's
 * topologically sorted DAG that replaces groups of elementwise / softmax nodes by single nodes
 * whose kernels are this library's fused entry points.
 *
 * The reference scheduler runs a graph node by node (src/scheduler/scheduler.c:16-52,
 * src/core/graph.c:57-65) and its own fusion pass only knows matmul / conv + leaky_relu
 * (src/scheduler/fusion.c:28-90). plast_b200_fuse_graph is called where that pass is called
 * (scheduler.c:33, right after fusion_optimize(dag)) or on any DAG made by build_dag().
 *
 * Node, Op, OP_TYPE and DAG restate include/core/node.h:5-14, include/core/op.h:8-44 and
 * include/core/graph.h:8-14; define PLAST_B200_USE_REFERENCE_TYPES to compile against the
 * reference's own headers instead.
 */
#ifndef PLAST_B200_GRAPH_H
#define PLAST_B200_GRAPH_H

#include "plast_b200.h"

#ifdef PLAST_B200_USE_REFERENCE_TYPES
#include "core/graph.h"
#include "core/node.h"
#include "core/op.h"
#else

typedef uint32_t u32;

/* include/core/op.h:5-6 */
typedef void (*ForwardKernel)(const Tensor **inputs, Tensor *output, KernelParams params);
typedef void (*BackwardKernel)(Tensor **inputs, const Tensor *output, KernelParams params);

/* include/core/op.h:8-37 */
typedef enum OP_TYPE {
  ADD, SUB, MUL, DIV, MATMUL, LEAKY_RELU, LOG, EXP, ABS, NEG, SIN, COS, TAN,
  VIEW, TRANSPOSE, UNSQUEEZE, SQUEEZE, EXPAND, FLATTEN, BROADCAST,
  MEAN, MIN, MAX, SUM, CONV2D, MATMUL_RELU, MATMUL_BIAS_RELU, CONV_RELU
} OP_TYPE;

/* include/core/op.h:39-44 — 32 bytes */
typedef struct Op {
  ForwardKernel cpu_forward;
  ForwardKernel cuda_forward;
  BackwardKernel cpu_backward;
  BackwardKernel cuda_backward;
} Op;

/* include/core/node.h:5-14 — 88 bytes:
 * inputs@0 output@8 op@16 op_type@48 num_inputs@52 visited@56 on_stack@57 params@64 */
typedef struct Node {
  Tensor **inputs;
  Tensor *output;
  Op op;
  OP_TYPE op_type;
  int num_inputs;
  bool visited;
  bool on_stack;
  KernelParams params;
} Node;

struct Arena;

/* include/core/graph.h:8-14 — 32 bytes: nodes@0 count@8 capacity@12 changed@16 arena@24 */
typedef struct DAG {
  Node **nodes;
  u32 count;
  u32 capacity;
  bool changed;
  struct Arena *arena;
} DAG;

#endif /* PLAST_B200_USE_REFERENCE_TYPES */

/* op_type values of the nodes the pass creates (past the end of the reference's enum). */
#define PLAST_OP_FUSED_CHAIN 1000
#define PLAST_OP_ADD_LEAKY_RELU 1001
#define PLAST_OP_SCALE_BIAS_LEAKY_RELU 1002
#define PLAST_OP_SOFTMAX 1003
#define PLAST_OP_LOG_SOFTMAX 1004

#ifdef __cplusplus
extern "C" {
#endif

/* Rewrites dag->nodes in place (order stays topological, dag->count shrinks, dag->changed is
 * set) and returns the number of fused nodes it created. Only nodes whose output is a FLOAT32
 * CUDA tensor are touched. An intermediate result disappears only when every node of the DAG
 * that reads it is fused into the same node; like the reference's matmul + relu fusion, its
 * buffer is then never written. Rewrites, in this order:
 *   max(keepdim) -> sub -> exp -> sum(keepdim) -> div          => softmax      (fwd + bwd)
 *   max(keepdim) -> sub -> exp -> sum(keepdim) -> log -> sub   => log_softmax  (fwd + bwd)
 *   mul -> add -> leaky_relu                                   => scale_bias_leaky_relu (fwd + bwd)
 *   add -> leaky_relu                                          => add_leaky_relu (fwd + bwd)
 *   any connected group of add sub mul div neg abs exp log sin cos tan leaky_relu nodes of one
 *   shape, none of which requires grad                          => one chain node (forward only)
 * The fused node's output tensor is the last node's output (its creator is re-pointed to the
 * fused node, as fusion.c:159-160 does). Fused nodes are owned by the library
 * (plast_b200_fusion_release frees them; call it only when no DAG refers to them any more). */
u32 plast_b200_fuse_graph(DAG *dag);
void plast_b200_fusion_release(void);

/* plast_b200_fuse_graph(dag) is plast_b200_fuse_graph_ex(dag, 0). With
 * PLAST_B200_FUSE_CHAINS_WITH_GRAD the last rule also takes groups whose tensors require grad:
 * the chain node's backward (plast_b200_chain_backward) recomputes the group inside one kernel per
 * differentiated input instead of reading saved intermediates, so the gradients of the
 * intermediates are never materialised. Only taken when the run-time compiler is available. */
#define PLAST_B200_FUSE_CHAINS_WITH_GRAD 1u
u32 plast_b200_fuse_graph_ex(DAG *dag, unsigned flags);

/* Kernel of a PLAST_OP_FUSED_CHAIN node: params.dim is the handle of the program the pass
 * registered; inputs are the group's external operands. The backward runs
 * plast_b200_chain_backward on the same program (nothing to do when no input requires grad). */
void chain_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void chain_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);

/* A DAG as one CUDA graph. plast_b200_dag_capture records the kernels of every node (backward == 0:
 * forward order; 1: reverse order with the nodes' backward kernels; 2: the forward pass followed by
 * the backward pass, a whole training step whose upstream gradient is already in place) WITHOUT
 * running them and returns a handle; plast_b200_dag_replay launches the whole recording on the library
 * stream. This is what the scheduler's JIT mode wants for a cached DAG it executes again and again
 * on the same tensors (src/scheduler/scheduler.c:17-27): per replay one launch instead of one
 * per node, which is the bound for small graphs. Every node must be a CUDA node whose kernel is
 * an entry point of this library (anything else returns NULL with PLAST_B200_ERR_UNSUPPORTED);
 * run the DAG once the ordinary way first so that run-time compiled chains and the scratch
 * workspace exist. The recording holds the tensors' addresses: it is valid while they are. */
typedef struct PlastDagGraph PlastDagGraph;
PlastDagGraph *plast_b200_dag_capture(DAG *dag, int backward);
void plast_b200_dag_replay(PlastDagGraph *graph);
int plast_b200_dag_graph_kernels(const PlastDagGraph *graph);
void plast_b200_dag_graph_release(PlastDagGraph *graph);

/* Test hook: copies the program behind a chain handle; returns its step count (0 = unknown
 * handle) and stores its input count. */
int plast_b200_fusion_program(u64 handle, PlastChainStep *steps, int max_steps, int *n_inputs);

#ifdef __cplusplus
}
#endif

#endif /* PLAST_B200_GRAPH_H */
