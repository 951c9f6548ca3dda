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
 * (3) reductions over a transposed view made by the reference's transpose node.
 */
#include "core/arena.h"
#include "core/graph.h"
#include "core/node.h"
#include "core/op.h"
#include "core/tensor.h"
#include "scheduler/jit.h"
#include "scheduler/scheduler.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

void arena_memcpy_h2d_cuda(void *dest, const void *src, u64 size);
void arena_memcpy_d2h_cuda(void *dest, const void *src, u64 size);

typedef struct {
  Arena meta, data;
  DEVICE dev;
  Scheduler *sched;
} Ctx;

static Tensor *mk(Ctx *c, const u64 *shape, u64 nd, bool rg) {
  u64 sh[MAX_NDIM];
  memcpy(sh, shape, nd * sizeof(u64));
  return init(&c->meta, &c->data, c->dev, FLOAT32, sh, nd, rg, NULL);
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
  Tensor *out = mk(c, shape, nd, rg);
  Tensor **in = (Tensor **)arena_alloc(&c->meta, sizeof(Tensor *), 8);
  in[0] = a;
  arena_node_alloc(&c->meta, in, 1, out, get_op_impl(op), op, p);
  return out;
}
static Tensor *node2(Ctx *c, OP_TYPE op, Tensor *a, Tensor *b, const u64 *shape, u64 nd, bool rg) {
  Tensor *out = mk(c, shape, nd, rg);
  Tensor **in = (Tensor **)arena_alloc(&c->meta, 2 * sizeof(Tensor *), 8);
  in[0] = a;
  in[1] = b;
  arena_node_alloc(&c->meta, in, 2, out, get_op_impl(op), op, (KernelParams){0, 0, 0.0f});
  return out;
}

enum { M = 64, N = 48, R = 33, K = 130 };
typedef struct {
  float ab[M * N], c[M * N], s[M], grad_b[N];
  float softmax[R * K];
  float tsum0[R], tmax_full[1], tsum1[K];
} Results;

static float frand(unsigned *st) {
  *st = *st * 1664525u + 1013904223u;
  /* scaled by a value with a full mantissa so that sums really depend on the order of addition */
  return ((float)((*st >> 8) & 0xffff) / 32768.0f - 1.0f) * 0.7317519f;
}

static void run(DEVICE dev, Results *res) {
  Ctx c;
  c.dev = dev;
  c.meta = arena_create(Mib(4), CPU); /* metadata always lives on the host */
  c.data = arena_create(Mib(16), dev);
  c.sched = init_scheduler(jit_create(16));
  unsigned st = 12345;
  static float A[M * N], b[N], G[M * N], X[R * K];
  for (int i = 0; i < M * N; ++i) A[i] = frand(&st);
  for (int i = 0; i < N; ++i) b[i] = frand(&st);
  for (int i = 0; i < M * N; ++i) G[i] = frand(&st) * 3.0f;
  for (int i = 0; i < R * K; ++i) X[i] = frand(&st) * 4.0f;

  /* (1) config 1 */
  Tensor *tA = mk(&c, (u64[]){M, N}, 2, false);
  Tensor *tb = mk(&c, (u64[]){1, N}, 2, true);
  upload(&c, tA->data, A, M * N);
  upload(&c, tb->data, b, N);
  Tensor *ab = node2(&c, ADD, tA, tb, (u64[]){M, N}, 2, true);
  Tensor *cc = node1(&c, LEAKY_RELU, ab, (u64[]){M, N}, 2, true, (KernelParams){0, 0, 0.0f});
  Tensor *s = node1(&c, SUM, cc, (u64[]){M}, 1, true, (KernelParams){1, 0, 0.0f});
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
  Tensor *mx = node1(&c, MAX, tX, (u64[]){R, 1}, 2, false, (KernelParams){1, 1, 0.0f});
  Tensor *sh = node2(&c, SUB, tX, mx, (u64[]){R, K}, 2, false);
  Tensor *ex = node1(&c, EXP, sh, (u64[]){R, K}, 2, false, (KernelParams){0, 0, 0.0f});
  Tensor *se = node1(&c, SUM, ex, (u64[]){R, 1}, 2, false, (KernelParams){1, 1, 0.0f});
  Tensor *sm = node2(&c, DIV, ex, se, (u64[]){R, K}, 2, false);
  schedule(c.sched, sm->creator, FORWARD, &c.meta);
  download(&c, res->softmax, sm->data, R * K);

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
  printf(bad ? "DROPIN FAILED\n" : "DROPIN OK\n");
  return bad ? 1 : 0;
}
