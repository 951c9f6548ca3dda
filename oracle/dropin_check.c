/*
 * dropin_check.c — TEST INFRASTRUCTURE: proves that the reference's own runtime drives
 * libplast_b200.so unchanged.
 *
 * This file is compiled by oracle/Makefile together with the REFERENCE's sources where they lie
 * (src/core/{tensor,arena,arena_cpu,node,op,graph}.c, src/scheduler/{scheduler,jit,fusion}.c,
 * src/kernels/cpu/*.c with -DCUDA_AVAILABLE, plus its matmul / conv CUDA objects, which are out of
 * this repository's scope) and linked against libplast_b200.so INSTEAD of the reference's
 * src/kernels/cuda/{binary,unary,reduce,shape}_ops.cu, cuda_tensor_init.cu, cuda_pack.cu and
 * src/core/arena_cuda.cu. The result, oracle/_ref/dropin_check, builds graphs the way the
 * reference's main.c does (arena_create, init, arena_node_alloc(get_op_impl(OP)), schedule) and
 * runs each graph twice: device = CPU (the reference's own kernels) and device = CUDA (the
 * reference's op table dispatching into this library). It compares the two and exits non-zero on
 * a mismatch.
 *
 * Graphs: (1) benchmark configuration 1 in small: C = relu(A + b), s = sum(C, axis 1), backward from an
 * upstream gradient on C into b.grad (leaky_relu backward, then the broadcast-gradient reduce of
 * add backward); (2) the softmax recipe of plast/nn/functional.py:77-86 as five nodes;
 * (3) reductions over a transposed view made by the reference's transpose node;
 * (4) z = sigmoid(x) * y + exp(-abs(x)) as the nine nodes plast/tensor.py builds (the two 1.0
 * constants are 0-dim tensors).
 * (4b) is (4) with requires_grad on every tensor and a backward pass from an upstream gradient.
 * On CUDA, (1), (2), (4) and (4b) run a second time on fresh graphs that go through build_dag, this
 * library's plast_b200_fuse_graph (the call a maintainer adds after fusion_optimize in
 * src/scheduler/scheduler.c:33) and the reference's dag_forward / dag_backward: the fused DAGs
 * must have 2, 1 and 1 nodes and give the results of the node-by-node runs.
 * (5) CUDA only: the arena's zero-fill (src/core/arena.c:94-102). The nine-node training chain runs
 * node by node twice in an arena whose memory was dirtied first: once as the reference allocates
 * (every allocation filled, gradients filled a second time by zeros_cuda, src/core/tensor.c:82-90)
 * and once with the three-line caller patch this library offers: plast_b200_arena_fill_policy(SKIP)
 * around the allocation of an op's output. Results and gradients must be the same bits, every
 * gradient buffer must still start at zero, and the fill counters must show the outputs skipped.
 */
#include "core/arena.h"
#include "core/graph.h"
#include "core/node.h"
#include "core/op.h"
#include "core/tensor.h"
#include "scheduler/jit.h"
#include "scheduler/scheduler.h"

#define PLAST_B200_USE_REFERENCE_TYPES
#include "plast_b200_graph.h"

#include <math.h>
#include <stdio.h>
#include <time.h>
#include <stdlib.h>
#include <string.h>

void arena_memcpy_h2d_cuda(void *dest, const void *src, u64 size);
void arena_memcpy_d2h_cuda(void *dest, const void *src, u64 size);

typedef struct {
  Arena meta, data;
  DEVICE dev;
  Scheduler *sched;
  bool skip_output_fill;     /* (5): allocate op outputs without the arena's zero-fill */
  Tensor *outputs[64];       /* (5): every op output allocated through node1 / node2 */
  int n_outputs;
} Ctx;

static Tensor *mk(Ctx *c, const u64 *shape, u64 nd, bool rg) {
  u64 sh[MAX_NDIM];
  memcpy(sh, shape, nd * sizeof(u64));
  return init(&c->meta, &c->data, c->dev, FLOAT32, sh, nd, rg, NULL);
}
/* An op's output: its forward kernel overwrites every element, so the arena's fill is wasted on
 * it. This is the whole caller-side patch: the policy call before and after the allocation. */
static Tensor *mk_output(Ctx *c, const u64 *shape, u64 nd, bool rg) {
  if (c->skip_output_fill) plast_b200_arena_fill_policy(PLAST_B200_ARENA_SKIP_FILL);
  Tensor *t = mk(c, shape, nd, rg);
  if (c->skip_output_fill) plast_b200_arena_fill_policy(PLAST_B200_ARENA_FILL);
  if (c->n_outputs < 64) c->outputs[c->n_outputs++] = t;
  return t;
}
static void upload(Ctx *c, void *dst, const float *src, u64 n) {
  if (c->dev == CUDA) arena_memcpy_h2d_cuda(dst, src, n * 4);
  else memcpy(dst, src, n * 4);
}
static void download(Ctx *c, float *dst, const void *src, u64 n) {
  if (c->dev == CUDA) arena_memcpy_d2h_cuda(dst, src, n * 4);
  else memcpy(dst, src, n * 4);
}
static Tensor *node1(Ctx *c, OP_TYPE op, Tensor *a, const u64 *shape, u64 nd, bool rg, KernelParams p) {
  Tensor *out = mk_output(c, shape, nd, rg);
  Tensor **in = (Tensor **)arena_alloc(&c->meta, sizeof(Tensor *), 8);
  in[0] = a;
  arena_node_alloc(&c->meta, in, 1, out, get_op_impl(op), op, p);
  return out;
}
static Tensor *node2(Ctx *c, OP_TYPE op, Tensor *a, Tensor *b, const u64 *shape, u64 nd, bool rg) {
  Tensor *out = mk_output(c, shape, nd, rg);
  Tensor **in = (Tensor **)arena_alloc(&c->meta, 2 * sizeof(Tensor *), 8);
  in[0] = a;
  in[1] = b;
  arena_node_alloc(&c->meta, in, 2, out, get_op_impl(op), op, (KernelParams){0, 0, 0.0f});
  return out;
}

enum { M = 64, N = 48, R = 33, K = 130, CH = 4099 };
typedef struct {
  float ab[M * N], c[M * N], s[M], grad_b[N];
  float softmax[R * K];
  float tsum0[R], tmax_full[1], tsum1[K];
  float chain[CH];
  /* the same graphs after plast_b200_fuse_graph (CUDA only) */
  float f_c[M * N], f_s[M], f_grad_b[N], f_softmax[R * K], f_chain[CH];
  unsigned f_nodes[3], f_launches[3];
  /* the chain as a training graph: gradients of x and y, node by node and (CUDA) fused */
  float chain_dx[CH], chain_dy[CH], f_chain_dx[CH], f_chain_dy[CH];
  unsigned f_train_nodes, f_train_bwd_launches;
  /* (5) the training chain in a dirtied arena: [0] every allocation filled, [1] op outputs unfilled */
  float fill_z[2][CH], fill_dx[2][CH], fill_dy[2][CH];
  int fill_grads_nonzero[2];
  unsigned long long fill_filled[2], fill_skipped[2];
  /* config 1's fused forward DAG (2 nodes): the reference's dag_forward against one CUDA-graph replay */
  float replay_s[M];
  double us_node_by_node, us_replay;
  int replay_kernels;
} Results;

static Tensor *config1_graph(Ctx *c, const float *A, const float *b, Tensor **tb_out, Tensor **cc_out) {
  Tensor *tA = mk(c, (u64[]){M, N}, 2, false);
  Tensor *tb = mk(c, (u64[]){1, N}, 2, true);
  upload(c, tA->data, A, M * N);
  upload(c, tb->data, b, N);
  Tensor *ab = node2(c, ADD, tA, tb, (u64[]){M, N}, 2, true);
  Tensor *cc = node1(c, LEAKY_RELU, ab, (u64[]){M, N}, 2, true, (KernelParams){0, 0, 0.0f});
  *tb_out = tb;
  *cc_out = cc;
  return node1(c, SUM, cc, (u64[]){M}, 1, true, (KernelParams){1, 0, 0.0f});
}
static Tensor *softmax_graph(Ctx *c, Tensor *tX) {
  Tensor *mx = node1(c, MAX, tX, (u64[]){R, 1}, 2, false, (KernelParams){1, 1, 0.0f});
  Tensor *sh = node2(c, SUB, tX, mx, (u64[]){R, K}, 2, false);
  Tensor *ex = node1(c, EXP, sh, (u64[]){R, K}, 2, false, (KernelParams){0, 0, 0.0f});
  Tensor *se = node1(c, SUM, ex, (u64[]){R, 1}, 2, false, (KernelParams){1, 1, 0.0f});
  return node2(c, DIV, ex, se, (u64[]){R, K}, 2, false);
}
static Tensor *chain_graph_rg(Ctx *c, const float *x, const float *y, bool rg, Tensor **tx_out, Tensor **ty_out);
static Tensor *chain_graph(Ctx *c, const float *x, const float *y) {
  Tensor *tx, *ty;
  return chain_graph_rg(c, x, y, false, &tx, &ty);
}
static Tensor *chain_graph_rg(Ctx *c, const float *x, const float *y, bool rg, Tensor **tx_out, Tensor **ty_out) {
  const KernelParams none = {0, 0, 0.0f};
  const float one = 1.0f;
  Tensor *tx = mk(c, (u64[]){CH}, 1, rg), *ty = mk(c, (u64[]){CH}, 1, rg);
  *tx_out = tx;
  *ty_out = ty;
  Tensor *one_a = mk(c, NULL, 0, false), *one_b = mk(c, NULL, 0, false);
  upload(c, tx->data, x, CH);
  upload(c, ty->data, y, CH);
  upload(c, one_a->data, &one, 1);
  upload(c, one_b->data, &one, 1);
  Tensor *nx = node1(c, NEG, tx, (u64[]){CH}, 1, rg, none);
  Tensor *e = node1(c, EXP, nx, (u64[]){CH}, 1, rg, none);
  Tensor *d = node2(c, ADD, one_a, e, (u64[]){CH}, 1, rg);
  Tensor *sg = node2(c, DIV, one_b, d, (u64[]){CH}, 1, rg);
  Tensor *t = node2(c, MUL, sg, ty, (u64[]){CH}, 1, rg);
  Tensor *ax = node1(c, ABS, tx, (u64[]){CH}, 1, rg, none);
  Tensor *nax = node1(c, NEG, ax, (u64[]){CH}, 1, rg, none);
  Tensor *e2 = node1(c, EXP, nax, (u64[]){CH}, 1, rg, none);
  return node2(c, ADD, t, e2, (u64[]){CH}, 1, rg);
}
/* What schedule() does in JIT mode (scheduler.c:29-33) with this library's pass added. */
static DAG *fused_dag(Ctx *c, Tensor *root, unsigned *n_nodes) {
  DAG *dag = alloc_dag(MIN_DAG_CAPACITY);
  dag->arena = &c->meta;
  build_dag(dag, root->creator);
  plast_b200_fuse_graph(dag);
  *n_nodes = dag->count;
  return dag;
}

static float frand(unsigned *st) {
  *st = *st * 1664525u + 1013904223u;
  /* scaled by a value with a full mantissa so that sums really depend on the order of addition */
  return ((float)((*st >> 8) & 0xffff) / 32768.0f - 1.0f) * 0.7317519f;
}

/* (5): see the header comment. */
static void run_arena_fill(Results *res, const float *CX, const float *CY, const float *CG) {
  for (int pass = 0; pass < 2; ++pass) {
    Ctx c;
    memset(&c, 0, sizeof(c));
    c.dev = CUDA;
    c.meta = arena_create(Mib(4), CPU);
    c.data = arena_create(Mib(16), CUDA);
    c.sched = init_scheduler(jit_create(16));
    /* dirty the block, then hand it out again from the start */
    Tensor *junk = mk(&c, (u64[]){Mib(3)}, 1, false);
    ones(junk, Mib(3));
    arena_reset(&c.data);
    c.skip_output_fill = pass == 1;
    u64 f0, s0, f1, s1;
    plast_b200_arena_fill_stats(&f0, &s0);
    Tensor *gx, *gy;
    Tensor *gz = chain_graph_rg(&c, CX, CY, true, &gx, &gy);
    plast_b200_arena_fill_stats(&f1, &s1);
    res->fill_filled[pass] = f1 - f0;
    res->fill_skipped[pass] = s1 - s0;
    /* every gradient buffer of an op output starts at zero although its memory was dirty */
    static float g[CH];
    res->fill_grads_nonzero[pass] = 0;
    for (int i = 0; i < c.n_outputs; ++i) {
      download(&c, g, c.outputs[i]->grad->data, CH);
      for (int j = 0; j < CH; ++j) res->fill_grads_nonzero[pass] += g[j] != 0.0f;
    }
    schedule(c.sched, gz->creator, FORWARD, &c.meta);
    download(&c, res->fill_z[pass], gz->data, CH);
    upload(&c, gz->grad->data, CG, CH);
    schedule(c.sched, gz->creator, BACKWARD, &c.meta);
    download(&c, res->fill_dx[pass], gx->grad->data, CH);
    download(&c, res->fill_dy[pass], gy->grad->data, CH);
    arena_release(&c.data);
    arena_release(&c.meta);
  }
}

static void run(DEVICE dev, Results *res) {
  Ctx c;
  memset(&c, 0, sizeof(c));
  c.dev = dev;
  c.meta = arena_create(Mib(4), CPU); /* metadata always lives on the host */
  c.data = arena_create(Mib(16), dev);
  c.sched = init_scheduler(jit_create(16));
  unsigned st = 12345;
  static float A[M * N], b[N], G[M * N], X[R * K], CX[CH], CY[CH], CG[CH];
  for (int i = 0; i < M * N; ++i) A[i] = frand(&st);
  for (int i = 0; i < N; ++i) b[i] = frand(&st);
  for (int i = 0; i < M * N; ++i) G[i] = frand(&st) * 3.0f;
  for (int i = 0; i < R * K; ++i) X[i] = frand(&st) * 4.0f;
  for (int i = 0; i < CH; ++i) CX[i] = frand(&st) * 6.0f;
  for (int i = 0; i < CH; ++i) CY[i] = frand(&st);
  for (int i = 0; i < CH; ++i) CG[i] = frand(&st) * 2.0f;

  /* (1) config 1 */
  Tensor *tb, *cc;
  Tensor *s = config1_graph(&c, A, b, &tb, &cc);
  Tensor *ab = cc->creator->inputs[0];
  schedule(c.sched, s->creator, FORWARD, &c.meta);
  download(&c, res->ab, ab->data, M * N);
  download(&c, res->c, cc->data, M * N);
  download(&c, res->s, s->data, M);
  upload(&c, cc->grad->data, G, M * N); /* upstream gradient on C */
  schedule(c.sched, cc->creator, BACKWARD, &c.meta);
  download(&c, res->grad_b, tb->grad->data, N);

  /* (2) softmax = max(keepdim) -> sub -> exp -> sum(keepdim) -> div */
  Tensor *tX = mk(&c, (u64[]){R, K}, 2, false);
  upload(&c, tX->data, X, R * K);
  Tensor *sm = softmax_graph(&c, tX);
  schedule(c.sched, sm->creator, FORWARD, &c.meta);
  download(&c, res->softmax, sm->data, R * K);

  /* (4) the nine-node chain */
  Tensor *z = chain_graph(&c, CX, CY);
  schedule(c.sched, z->creator, FORWARD, &c.meta);
  download(&c, res->chain, z->data, CH);

  /* (4b) the same chain with requires_grad everywhere: backward from an upstream gradient on z */
  {
    Tensor *gx, *gy;
    Tensor *gz = chain_graph_rg(&c, CX, CY, true, &gx, &gy);
    schedule(c.sched, gz->creator, FORWARD, &c.meta);
    upload(&c, gz->grad->data, CG, CH);
    schedule(c.sched, gz->creator, BACKWARD, &c.meta);
    download(&c, res->chain_dx, gx->grad->data, CH);
    download(&c, res->chain_dy, gy->grad->data, CH);
  }

  if (dev == CUDA) {
    {
      Tensor *gx, *gy;
      Tensor *gz = chain_graph_rg(&c, CX, CY, true, &gx, &gy);
      DAG *dg = alloc_dag(MIN_DAG_CAPACITY);
      dg->arena = &c.meta;
      build_dag(dg, gz->creator);
      plast_b200_fuse_graph_ex(dg, PLAST_B200_FUSE_CHAINS_WITH_GRAD);
      res->f_train_nodes = dg->count;
      dag_forward(dg);
      upload(&c, gz->grad->data, CG, CH);
      const u64 before_bwd = plast_b200_launch_count();
      dag_backward(dg);
      res->f_train_bwd_launches = (unsigned)(plast_b200_launch_count() - before_bwd);
      download(&c, res->f_chain_dx, gx->grad->data, CH);
      download(&c, res->f_chain_dy, gy->grad->data, CH);
      dag_release(dg);
    }
    Tensor *ftb, *fcc;
    Tensor *fs = config1_graph(&c, A, b, &ftb, &fcc);
    DAG *d1 = fused_dag(&c, fs, &res->f_nodes[0]);
    u64 before = plast_b200_launch_count();
    dag_forward(d1);
    res->f_launches[0] = (unsigned)(plast_b200_launch_count() - before);
    download(&c, res->f_c, fcc->data, M * N);
    download(&c, res->f_s, fs->data, M);
    {
      /* the same two-node DAG recorded once and replayed; timings are per execution of the DAG */
      PlastDagGraph *rec = plast_b200_dag_capture(d1, 0);
      res->replay_kernels = plast_b200_dag_graph_kernels(rec);
      const int reps = 2000;
      float sink[1];
      struct timespec t0, t1;
      for (int i = 0; i < 50; ++i) dag_forward(d1);
      download(&c, sink, fs->data, 1);
      clock_gettime(CLOCK_MONOTONIC, &t0);
      for (int i = 0; i < reps; ++i) dag_forward(d1);
      download(&c, sink, fs->data, 1);
      clock_gettime(CLOCK_MONOTONIC, &t1);
      res->us_node_by_node = ((t1.tv_sec - t0.tv_sec) * 1e6 + (t1.tv_nsec - t0.tv_nsec) * 1e-3) / reps;
      if (rec) {
        for (int i = 0; i < 50; ++i) plast_b200_dag_replay(rec);
        download(&c, sink, fs->data, 1);
        clock_gettime(CLOCK_MONOTONIC, &t0);
        for (int i = 0; i < reps; ++i) plast_b200_dag_replay(rec);
        download(&c, sink, fs->data, 1);
        clock_gettime(CLOCK_MONOTONIC, &t1);
        res->us_replay = ((t1.tv_sec - t0.tv_sec) * 1e6 + (t1.tv_nsec - t0.tv_nsec) * 1e-3) / reps;
        download(&c, res->replay_s, fs->data, M);
        plast_b200_dag_graph_release(rec);
      }
    }
    upload(&c, fcc->grad->data, G, M * N);
    execute_backward(fcc->creator); /* the fused add + leaky_relu node */
    download(&c, res->f_grad_b, ftb->grad->data, N);
    dag_release(d1);

    Tensor *fsm = softmax_graph(&c, tX);
    DAG *d2 = fused_dag(&c, fsm, &res->f_nodes[1]);
    before = plast_b200_launch_count();
    dag_forward(d2);
    res->f_launches[1] = (unsigned)(plast_b200_launch_count() - before);
    download(&c, res->f_softmax, fsm->data, R * K);
    dag_release(d2);

    Tensor *fz = chain_graph(&c, CX, CY);
    DAG *d3 = fused_dag(&c, fz, &res->f_nodes[2]);
    before = plast_b200_launch_count();
    dag_forward(d3);
    res->f_launches[2] = (unsigned)(plast_b200_launch_count() - before);
    download(&c, res->f_chain, fz->data, CH);
    dag_release(d3);
  }

  /* (3) reductions over the transposed view [K, R] of X (strides [1, K], no copy) */
  Tensor *xt = node1(&c, TRANSPOSE, tX, (u64[]){K, R}, 2, false, (KernelParams){0, 1, 0.0f});
  Tensor *t0 = node1(&c, SUM, xt, (u64[]){R}, 1, false, (KernelParams){0, 0, 0.0f});
  schedule(c.sched, t0->creator, FORWARD, &c.meta);
  download(&c, res->tsum0, t0->data, R);
  Tensor *t1 = node1(&c, SUM, xt, (u64[]){K}, 1, false, (KernelParams){1, 0, 0.0f});
  schedule(c.sched, t1->creator, FORWARD, &c.meta);
  download(&c, res->tsum1, t1->data, K);
  Tensor *tm = node1(&c, MAX, xt, (u64[]){1}, 1, false, (KernelParams){MAX_NDIM + 1, 0, 0.0f});
  schedule(c.sched, tm->creator, FORWARD, &c.meta);
  download(&c, res->tmax_full, tm->data, 1);

  arena_release(&c.data);
  arena_release(&c.meta);
  if (dev == CUDA) run_arena_fill(res, CX, CY, CG);
}

static int same_bits(const char *what, const float *a, const float *b, int n) {
  int bad = 0;
  for (int i = 0; i < n; ++i) bad += memcmp(&a[i], &b[i], 4) != 0;
  printf("%-28s %s (%d of %d differ bitwise)\n", what, bad ? "MISMATCH" : "bit-exact", bad, n);
  return bad;
}
static int close_to(const char *what, const float *a, const float *b, int n, float scale) {
  float worst = 0;
  for (int i = 0; i < n; ++i) worst = fmaxf(worst, fabsf(a[i] - b[i]));
  const int bad = !(worst <= 1e-5f * scale);
  printf("%-28s %s (max |diff| %.3g, bound %.3g)\n", what, bad ? "MISMATCH" : "ok", worst, 1e-5f * scale);
  return bad;
}

int main(void) {
  static Results cpu, gpu;
  run(CPU, &cpu);
  run(CUDA, &gpu);
  int bad = 0;
  bad += same_bits("A + b", cpu.ab, gpu.ab, M * N);
  bad += same_bits("relu(A + b)", cpu.c, gpu.c, M * N);
  bad += close_to("sum(C, axis 1)", cpu.s, gpu.s, M, (float)N);
  bad += close_to("grad_b (broadcast reduce)", cpu.grad_b, gpu.grad_b, N, 3.0f * M);
  bad += close_to("softmax (5 nodes)", cpu.softmax, gpu.softmax, R * K, 1.0f);
  bad += close_to("sum(X.T, axis 0)", cpu.tsum0, gpu.tsum0, R, 4.0f * K);
  bad += close_to("sum(X.T, axis 1)", cpu.tsum1, gpu.tsum1, K, 4.0f * R);
  bad += same_bits("max(X.T)", cpu.tmax_full, gpu.tmax_full, 1);
  bad += close_to("chain (9 nodes)", cpu.chain, gpu.chain, CH, 2.0f);
  printf("fused DAGs: config 1 %u nodes / %u launches, softmax %u / %u, chain %u / %u\n", gpu.f_nodes[0],
         gpu.f_launches[0], gpu.f_nodes[1], gpu.f_launches[1], gpu.f_nodes[2], gpu.f_launches[2]);
  if (gpu.f_nodes[0] != 2 || gpu.f_nodes[1] != 1 || gpu.f_nodes[2] != 1 || gpu.f_launches[0] != 2 ||
      gpu.f_launches[1] != 1 || gpu.f_launches[2] > 2) {
    printf("fused DAG sizes                MISMATCH\n");
    ++bad;
  }
  printf("config 1 forward DAG (2 fused nodes, %d x %d): node by node %.2f us, one CUDA-graph replay (%d kernels) %.2f us\n",
         M, N, gpu.us_node_by_node, gpu.replay_kernels, gpu.us_replay);
  if (gpu.replay_kernels != 2) {
    printf("CUDA-graph recording           MISMATCH\n");
    ++bad;
  }
  bad += same_bits("replayed: sum(C, axis 1)", gpu.f_s, gpu.replay_s, M);
  bad += same_bits("fused: relu(A + b)", gpu.c, gpu.f_c, M * N);
  bad += same_bits("fused: sum(C, axis 1)", gpu.s, gpu.f_s, M);
  bad += close_to("fused: grad_b", cpu.grad_b, gpu.f_grad_b, N, 3.0f * M);
  bad += close_to("fused: softmax", cpu.softmax, gpu.f_softmax, R * K, 1.0f);
  bad += same_bits("fused: chain vs 9 nodes", gpu.chain, gpu.f_chain, CH);
  bad += close_to("chain dx (9 backward nodes)", cpu.chain_dx, gpu.chain_dx, CH, 4.0f);
  bad += close_to("chain dy (9 backward nodes)", cpu.chain_dy, gpu.chain_dy, CH, 4.0f);
  printf("fused training chain: %u node, %u backward launches\n", gpu.f_train_nodes, gpu.f_train_bwd_launches);
  if (gpu.f_train_nodes != 1 || gpu.f_train_bwd_launches > 4) {
    printf("fused training chain size      MISMATCH\n");
    ++bad;
  }
  bad += same_bits("fused: chain dx", gpu.chain_dx, gpu.f_chain_dx, CH);
  bad += same_bits("fused: chain dy", gpu.chain_dy, gpu.f_chain_dy, CH);
  bad += same_bits("arena: chain, all filled", gpu.chain, gpu.fill_z[0], CH);
  bad += same_bits("arena: chain, outputs unfilled", gpu.chain, gpu.fill_z[1], CH);
  bad += same_bits("arena: dx, outputs unfilled", gpu.fill_dx[0], gpu.fill_dx[1], CH);
  bad += same_bits("arena: dy, outputs unfilled", gpu.fill_dy[0], gpu.fill_dy[1], CH);
  printf("arena fill, nine-node training chain of %d elements: as the reference allocates %llu bytes filled by the "
         "arena, %llu skipped; with the caller patch %llu filled, %llu skipped; non-zero gradient words at start: %d / %d\n",
         CH, gpu.fill_filled[0], gpu.fill_skipped[0], gpu.fill_filled[1], gpu.fill_skipped[1],
         gpu.fill_grads_nonzero[0], gpu.fill_grads_nonzero[1]);
  /* nine outputs, data and gradient twin each, are not filled by the arena any more */
  if (gpu.fill_grads_nonzero[0] || gpu.fill_grads_nonzero[1] || gpu.fill_skipped[0] != 0 ||
      gpu.fill_skipped[1] != (unsigned long long)9 * 2 * CH * 4 ||
      gpu.fill_filled[0] != gpu.fill_filled[1] + gpu.fill_skipped[1]) {
    printf("arena fill policy              MISMATCH\n");
    ++bad;
  }
  printf(bad ? "DROPIN FAILED\n" : "DROPIN OK\n");
  return bad ? 1 : 0;
}
