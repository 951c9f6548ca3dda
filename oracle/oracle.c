/*
 * oracle.c — CPU restatement of plast's elementwise / reduce hot path. TEST INFRASTRUCTURE ONLY:
 * it is the checker the CUDA kernels are compared with; nothing in the shipped library calls it.
 *
 * Each function states, in plain scalar C, what the reference's CPU kernels compute and in which
 * order they accumulate, and cites the reference file:line it follows. The restatement is pinned
 * against the reference itself: tests/test_oracle_pins.py runs it against the reference's CPU
 * sources compiled into oracle/_ref/ (when that build is present) and against the golden vectors
 * under tests/golden/ that were generated from that build.
 *
 * Same calling convention as the library (include/plast_b200.h) but every pointer is host memory
 * and the entry points are named oracle_<op>_forward / oracle_<op>_backward.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off; no -ffast-math, so fp32
 * accumulation order is exactly the loop order written here).
 */
#include "plast_b200.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- index helpers: src/kernels/cpu/cpu_utils.c:4-17 ------------------------------------- */
static inline void unravel(u64 linear, const u64 *shape, u64 ndim, u64 *coords) {
  for (u64 i = ndim; i-- > 0;) {
    coords[i] = linear % shape[i];
    linear /= shape[i];
  }
}
static inline u64 dot_offset(const u64 *coords, const u64 *strides, u64 ndim) {
  u64 off = 0;
  for (u64 i = 0; i < ndim; ++i) off += coords[i] * strides[i];
  return off;
}
/* include/kernels/kernel_macros.h:156-168: right-aligned, size-1 dims read offset 0 */
static inline u64 bcast_offset(const u64 *coords, u64 coords_ndim, const u64 *strides,
                               const u64 *shape, u64 ndim) {
  u64 off = 0;
  long shift = (long)coords_ndim - (long)ndim;
  for (u64 j = 0; j < ndim; ++j) {
    u64 c = coords[j + shift];
    if (shape[j] == 1) c = 0;
    off += c * strides[j];
  }
  return off;
}
static u64 count(const Tensor *t) { /* src/core/tensor.c:44-50 */
  u64 n = 1;
  for (u64 i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}

/* ---- scalar functors ------------------------------------------------------------------------ */
enum { B_ADD, B_SUB, B_MUL, B_DIV };
enum { U_ABS, U_COS, U_SIN, U_TAN, U_EXP, U_LOG, U_NEG, U_LRELU };

/* src/kernels/cpu/binary_ops.c:18-60 */
static inline float bin_f(int op, float x, float y) {
  switch (op) {
  case B_ADD: return x + y;
  case B_SUB: return x - y;
  case B_MUL: return x * y;
  default: return x / y;
  }
}
static inline float bin_ga(int op, float g, float x, float y) {
  (void)x;
  switch (op) {
  case B_ADD: return g;
  case B_SUB: return g;
  case B_MUL: return g * y;
  default: return g / y;
  }
}
static inline float bin_gb(int op, float g, float x, float y) {
  switch (op) {
  case B_ADD: return g;
  case B_SUB: return -g;
  case B_MUL: return g * x;
  default: return -g * x / (y * y);
  }
}
/* src/kernels/cpu/unary_ops.c:9-31. neg is -x here (the reference's AVX body computes 0-x, its
 * scalar tail and strided path -x: they differ only in the sign of a zero result). */
static inline float un_f(int op, float x, float alpha) {
  switch (op) {
  case U_ABS: return fabsf(x);
  case U_COS: return cosf(x);
  case U_SIN: return sinf(x);
  case U_TAN: return tanf(x);
  case U_EXP: return expf(x);
  case U_LOG: return logf(x);
  case U_NEG: return -x;
  default: return x > 0 ? x : x * alpha;
  }
}
static inline float un_g(int op, float g, float x, float alpha) {
  switch (op) {
  case U_ABS: return x > 0 ? g : (x < 0 ? -g : 0.0f);
  case U_COS: return g * (-sinf(x));
  case U_SIN: return g * cosf(x);
  case U_TAN: { float t = tanf(x); float tt = t * t; return g * (1.0f + tt); }
  case U_EXP: return g * expf(x);
  case U_LOG: return g * (1.0f / x);
  case U_NEG: return -g;
  default: return x > 0 ? g : g * alpha;
  }
}

/* ---- binary: include/kernels/kernel_macros.h:191-242 (forward), 244-325 (backward) ---------- */
static void binary_forward(int op, const Tensor **in, Tensor *out) {
  const Tensor *a = in[0], *b = in[1];
  const float *ad = (const float *)a->data, *bd = (const float *)b->data;
  float *cd = (float *)out->data;
  u64 n = count(out);
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n; ++i) {
    u64 c[MAX_NDIM];
    unravel(i, out->shape, out->ndim, c);
    u64 ao = bcast_offset(c, out->ndim, a->strides, a->shape, a->ndim);
    u64 bo = bcast_offset(c, out->ndim, b->strides, b->shape, b->ndim);
    cd[dot_offset(c, out->strides, out->ndim)] = bin_f(op, ad[ao], bd[bo]);
  }
}
/* The reference accumulates with `omp atomic` in thread order (kernel_macros.h:283-299); this
 * restatement fixes the order to i = 0..n-1. Gradient buffers are indexed with the operand's
 * own strides and shape (kernel_macros.h:313-318). */
static void binary_backward(int op, Tensor **in, const Tensor *out) {
  const Tensor *a = in[0], *b = in[1];
  const Tensor *dout = out->grad;
  const float *ad = (const float *)a->data, *bd = (const float *)b->data;
  const float *gd = (const float *)dout->data;
  float *da = a->requires_grad ? (float *)a->grad->data : NULL;
  float *db = b->requires_grad ? (float *)b->grad->data : NULL;
  u64 n = count(dout);
  for (u64 i = 0; i < n; ++i) {
    u64 c[MAX_NDIM];
    unravel(i, dout->shape, dout->ndim, c);
    float g = gd[dot_offset(c, dout->strides, dout->ndim)];
    u64 ao = bcast_offset(c, dout->ndim, a->strides, a->shape, a->ndim);
    u64 bo = bcast_offset(c, dout->ndim, b->strides, b->shape, b->ndim);
    if (da) da[ao] += bin_ga(op, g, ad[ao], bd[bo]);
    if (db) db[bo] += bin_gb(op, g, ad[ao], bd[bo]);
  }
}

/* ---- unary: include/kernels/kernel_macros.h:19-138 ------------------------------------------ */
static void unary_forward(int op, const Tensor **in, Tensor *out, float alpha) {
  const Tensor *a = in[0];
  const float *ad = (const float *)a->data;
  float *cd = (float *)out->data;
  u64 n = count(a);
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n; ++i) {
    u64 c[MAX_NDIM];
    unravel(i, a->shape, a->ndim, c);
    cd[dot_offset(c, out->strides, a->ndim)] = un_f(op, ad[dot_offset(c, a->strides, a->ndim)], alpha);
  }
}
static void unary_backward(int op, Tensor **in, const Tensor *out, float alpha) {
  const Tensor *a = in[0];
  if (!a->requires_grad) return;
  const float *ad = (const float *)a->data;
  const float *gd = (const float *)out->grad->data;
  float *da = (float *)a->grad->data;
  u64 n = count(a);
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n; ++i) {
    u64 c[MAX_NDIM];
    unravel(i, a->shape, a->ndim, c);
    float g = gd[dot_offset(c, out->grad->strides, a->ndim)];
    float x = ad[dot_offset(c, a->strides, a->ndim)];
    da[dot_offset(c, a->grad->strides, a->ndim)] += un_g(op, g, x, alpha);
  }
}

/* ---- reductions: src/kernels/cpu/reduce_ops.c ----------------------------------------------- */
enum { R_SUM, R_MEAN, R_MAX, R_MIN };

static inline float red_init(int op) { /* reduce_ops.c:265-278 */
  return op == R_MAX ? -FLT_MAX : (op == R_MIN ? FLT_MAX : 0.0f);
}
static inline float red_step(int op, float acc, float x) { /* reduce_ops.c:8-10 */
  switch (op) {
  case R_MAX: return acc > x ? acc : x;
  case R_MIN: return acc < x ? acc : x;
  default: return acc + x;
  }
}
static inline float red_post(int op, float acc, u64 n) { /* reduce_ops.c:12-15 */
  return op == R_MEAN ? acc / n : acc;
}
/* src/kernels/cpu/cpu_utils.c:121-154 */
static void reduced_shape(const Tensor *a, u64 dim, int keepdim, u64 *shape, u64 *ndim,
                          u64 *strides) {
  u64 nd = 0;
  if (keepdim) {
    for (u64 i = 0; i < a->ndim; ++i) shape[i] = (i == dim) ? 1 : a->shape[i];
    nd = a->ndim;
  } else {
    for (u64 i = 0; i < a->ndim; ++i)
      if (i != dim) shape[nd++] = a->shape[i];
    if (nd == 0) { shape[0] = 1; nd = 1; }
  }
  *ndim = nd;
  u64 s = 1;
  for (long i = (long)nd - 1; i >= 0; --i) { strides[i] = s; s *= shape[i]; }
}
/* include/kernels/kernel_macros.h:171-188 */
static inline void out_to_in_coords(const u64 *cc, u64 *ac, u64 a_ndim, u64 dim, int keepdim) {
  for (u64 j = 0; j < a_ndim; ++j) {
    if (j == dim) ac[j] = 0;
    else if (keepdim) ac[j] = cc[j];
    else ac[j] = (j < dim) ? cc[j] : cc[j - 1];
  }
}

/* reduce_ops.c:24-87. Full reduce: one left-to-right chain in row-major order of the view.
 * Axis reduce: one left-to-right chain along `dim` per output; output written at its linear
 * index (the output is freshly allocated, contiguous). */
static void reduce_forward(int op, const Tensor **in, Tensor *out, KernelParams p) {
  const Tensor *a = in[0];
  const float *ad = (const float *)a->data;
  float *cd = (float *)out->data;
  if (p.dim == PLAST_FULL_REDUCE) {
    u64 n = count(a);
    float acc = red_init(op);
    u64 c[MAX_NDIM];
    for (u64 i = 0; i < n; ++i) {
      unravel(i, a->shape, a->ndim, c);
      acc = red_step(op, acc, ad[dot_offset(c, a->strides, a->ndim)]);
    }
    cd[0] = red_post(op, acc, n);
    return;
  }
  u64 dim = p.dim;
  int keepdim = p.keepdim != 0;
  reduced_shape(a, dim, keepdim, out->shape, &out->ndim, out->strides);
  u64 n_out = count(out), len = a->shape[dim];
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n_out; ++i) {
    u64 cc[MAX_NDIM], ac[MAX_NDIM];
    unravel(i, out->shape, out->ndim, cc);
    out_to_in_coords(cc, ac, a->ndim, dim, keepdim);
    u64 base = dot_offset(ac, a->strides, a->ndim);
    float acc = red_init(op);
    for (u64 k = 0; k < len; ++k) acc = red_step(op, acc, ad[base + k * a->strides[dim]]);
    cd[i] = red_post(op, acc, len);
  }
}

/* reduce_ops.c:90-154 (sum, mean) and 157-262 (max, min: gradient / number of ties) */
static void reduce_backward(int op, Tensor **in, const Tensor *out, KernelParams p) {
  const Tensor *a = in[0];
  if (!a->requires_grad) return;
  const float *ad = (const float *)a->data;
  const float *cd = (const float *)out->data;
  const float *gd = (const float *)out->grad->data;
  float *da = (float *)a->grad->data;
  const u64 *das = a->grad->strides;
  int is_ext = (op == R_MAX || op == R_MIN);
  if (p.dim == PLAST_FULL_REDUCE) {
    u64 n = count(a);
    u64 c[MAX_NDIM];
    if (!is_ext) {
      float g = (op == R_MEAN) ? gd[0] / n : gd[0];
      for (u64 i = 0; i < n; ++i) {
        unravel(i, a->shape, a->ndim, c);
        da[dot_offset(c, das, a->ndim)] += g;
      }
      return;
    }
    float ext = red_init(op);
    for (u64 i = 0; i < n; ++i) {
      unravel(i, a->shape, a->ndim, c);
      ext = red_step(op, ext, ad[dot_offset(c, a->strides, a->ndim)]);
    }
    u64 ties = 0;
    for (u64 i = 0; i < n; ++i) {
      unravel(i, a->shape, a->ndim, c);
      if (ad[dot_offset(c, a->strides, a->ndim)] == ext) ties++;
    }
    if (ties == 0) return;
    float g = gd[0];
    g /= ties;
    for (u64 i = 0; i < n; ++i) {
      unravel(i, a->shape, a->ndim, c);
      if (ad[dot_offset(c, a->strides, a->ndim)] == ext) da[dot_offset(c, das, a->ndim)] += g;
    }
    return;
  }
  u64 dim = p.dim;
  int keepdim = p.keepdim != 0;
  u64 n_out = count(out), len = a->shape[dim];
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n_out; ++i) {
    u64 cc[MAX_NDIM], ac[MAX_NDIM];
    unravel(i, out->shape, out->ndim, cc);
    u64 co = dot_offset(cc, out->strides, out->ndim);
    out_to_in_coords(cc, ac, a->ndim, dim, keepdim);
    u64 abase = dot_offset(ac, a->strides, a->ndim);
    u64 gbase = dot_offset(ac, das, a->ndim);
    if (!is_ext) {
      float g = (op == R_MEAN) ? gd[co] / len : gd[co];
      for (u64 k = 0; k < len; ++k) da[gbase + k * das[dim]] += g;
    } else {
      float ext = cd[co], g = gd[co];
      u64 ties = 0;
      for (u64 k = 0; k < len; ++k)
        if (ad[abase + k * a->strides[dim]] == ext) ties++;
      if (ties == 0) continue;
      g /= ties;
      for (u64 k = 0; k < len; ++k)
        if (ad[abase + k * a->strides[dim]] == ext) da[gbase + k * das[dim]] += g;
    }
  }
}

/* argmax: absent from the reference's op table; first occurrence of the maximum found with the
 * reference's max rule (start at -FLT_MAX, replace only on strictly greater). */
void oracle_argmax_forward(const Tensor **in, Tensor *out, KernelParams p) {
  const Tensor *a = in[0];
  const float *ad = (const float *)a->data;
  i32 *cd = (i32 *)out->data;
  if (p.dim == PLAST_FULL_REDUCE) {
    u64 n = count(a);
    float best = 0.0f;
    u64 at = 0;
    u64 c[MAX_NDIM];
    for (u64 i = 0; i < n; ++i) {
      unravel(i, a->shape, a->ndim, c);
      float x = ad[dot_offset(c, a->strides, a->ndim)];
      if (i == 0 || x > best) { best = x; at = i; }
    }
    cd[0] = (i32)at;
    return;
  }
  u64 dim = p.dim;
  int keepdim = p.keepdim != 0;
  reduced_shape(a, dim, keepdim, out->shape, &out->ndim, out->strides);
  u64 n_out = count(out), len = a->shape[dim];
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n_out; ++i) {
    u64 cc[MAX_NDIM], ac[MAX_NDIM];
    unravel(i, out->shape, out->ndim, cc);
    out_to_in_coords(cc, ac, a->ndim, dim, keepdim);
    u64 base = dot_offset(ac, a->strides, a->ndim);
    float best = ad[base];
    u64 at = 0;
    for (u64 k = 1; k < len; ++k) {
      float x = ad[base + k * a->strides[dim]];
      if (x > best) { best = x; at = k; }
    }
    cd[i] = (i32)at;
  }
}

/* ---- exported primitive entry points --------------------------------------------------------- */
#define ORACLE_BINARY(name, OP)                                                                    \
  void oracle_##name##_forward(const Tensor **in, Tensor *out, KernelParams p) {                   \
    (void)p;                                                                                       \
    binary_forward(OP, in, out);                                                                   \
  }                                                                                                \
  void oracle_##name##_backward(Tensor **in, const Tensor *out, KernelParams p) {                  \
    (void)p;                                                                                       \
    binary_backward(OP, in, out);                                                                  \
  }
ORACLE_BINARY(add, B_ADD)
ORACLE_BINARY(sub, B_SUB)
ORACLE_BINARY(mul, B_MUL)
ORACLE_BINARY(div, B_DIV)

#define ORACLE_UNARY(name, OP)                                                                     \
  void oracle_##name##_forward(const Tensor **in, Tensor *out, KernelParams p) {                   \
    unary_forward(OP, in, out, p.fval);                                                            \
  }                                                                                                \
  void oracle_##name##_backward(Tensor **in, const Tensor *out, KernelParams p) {                  \
    unary_backward(OP, in, out, p.fval);                                                           \
  }
ORACLE_UNARY(abs, U_ABS)
ORACLE_UNARY(cos, U_COS)
ORACLE_UNARY(sin, U_SIN)
ORACLE_UNARY(tan, U_TAN)
ORACLE_UNARY(exp, U_EXP)
ORACLE_UNARY(log, U_LOG)
ORACLE_UNARY(neg, U_NEG)
ORACLE_UNARY(leaky_relu, U_LRELU)

#define ORACLE_REDUCE(name, OP)                                                                    \
  void oracle_##name##_forward(const Tensor **in, Tensor *out, KernelParams p) {                   \
    reduce_forward(OP, in, out, p);                                                                \
  }                                                                                                \
  void oracle_##name##_backward(Tensor **in, const Tensor *out, KernelParams p) {                  \
    reduce_backward(OP, in, out, p);                                                               \
  }
ORACLE_REDUCE(sum, R_SUM)
ORACLE_REDUCE(mean, R_MEAN)
ORACLE_REDUCE(max, R_MAX)
ORACLE_REDUCE(min, R_MIN)

/* ---- composite recipes: the op sequences of plast/nn/functional.py, one rounding per op ------ */
/* All recipes below take a contiguous [rows, cols] problem described by the caller: `x` points
 * at rows*cols floats with the softmax axis innermost. */

/* functional.py:77-86: max(keepdim) -> sub -> exp -> sum(keepdim) -> div */
void oracle_softmax_rows(const float *x, float *y, u64 rows, u64 cols) {
#pragma omp parallel for schedule(static)
  for (u64 r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float m = -FLT_MAX;
    for (u64 j = 0; j < cols; ++j) m = m > xr[j] ? m : xr[j];
    float s = 0.0f;
    for (u64 j = 0; j < cols; ++j) {
      float sh = xr[j] - m;
      float e = expf(sh);
      yr[j] = e;
      s = s + e;
    }
    for (u64 j = 0; j < cols; ++j) yr[j] = yr[j] / s;
  }
}
/* functional.py:89-97: max -> sub -> exp -> sum -> log -> sub */
void oracle_log_softmax_rows(const float *x, float *y, u64 rows, u64 cols) {
#pragma omp parallel for schedule(static)
  for (u64 r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float m = -FLT_MAX;
    for (u64 j = 0; j < cols; ++j) m = m > xr[j] ? m : xr[j];
    float s = 0.0f;
    for (u64 j = 0; j < cols; ++j) {
      float sh = xr[j] - m;
      s = s + expf(sh);
    }
    float lse = logf(s);
    for (u64 j = 0; j < cols; ++j) {
      float sh = xr[j] - m;
      yr[j] = sh - lse;
    }
  }
}
/* functional.py:312-333, 391-396 with reduction="mean": log_softmax(dim=1) -> one-hot * ->
 * sum(dim=1) -> neg -> mean. Multiplying by the one-hot row and summing left to right leaves
 * exactly log_softmax[label] (all other terms are +-0), so the label indexes the row here.
 * per_row (may be NULL) receives the per-sample losses. */
void oracle_cross_entropy_rows(const float *x, const i32 *labels, float *per_row, float *mean_out,
                               u64 rows, u64 cols) {
  float *loss = per_row ? per_row : (float *)malloc(rows * sizeof(float));
#pragma omp parallel for schedule(static)
  for (u64 r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float m = -FLT_MAX;
    for (u64 j = 0; j < cols; ++j) m = m > xr[j] ? m : xr[j];
    float s = 0.0f;
    for (u64 j = 0; j < cols; ++j) {
      float sh = xr[j] - m;
      s = s + expf(sh);
    }
    float lse = logf(s);
    float sh = xr[labels[r]] - m;
    float lp = sh - lse;
    /* one-hot(1.0) * lp, summed after zeros: 0.0f + lp */
    float picked = 0.0f + 1.0f * lp;
    loss[r] = -picked;
  }
  float acc = 0.0f;
  for (u64 r = 0; r < rows; ++r) acc = acc + loss[r];
  *mean_out = acc / rows;
  if (!per_row) free(loss);
}
/* functional.py:42-47: neg -> exp -> (+ 1.0) -> (1.0 / .) */
void oracle_sigmoid(const float *x, float *y, u64 n) {
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n; ++i) {
    float nx = -x[i];
    float e = expf(nx);
    float d = e + 1.0f;
    y[i] = 1.0f / d;
  }
}
/* The 9-op chain of the 2^28-element benchmark: z = sigmoid(x) * y + exp(-abs(x)), each op
 * rounded to fp32 on its own (neg, exp, +1, 1/., mul; abs, neg, exp; add). */
void oracle_sigmoid_mul_add_exp_neg_abs(const float *x, const float *y, float *z, u64 n) {
#pragma omp parallel for schedule(static)
  for (u64 i = 0; i < n; ++i) {
    float nx = -x[i];
    float e = expf(nx);
    float d = e + 1.0f;
    float sg = 1.0f / d;
    float t = sg * y[i];
    float ax = fabsf(x[i]);
    float nax = -ax;
    float e2 = expf(nax);
    z[i] = t + e2;
  }
}

/* ---- optimiser steps (flat float arrays, one parameter per call) ---------------------------------
 * src/optimizers/cpu/sgd.c:23-30 */
void oracle_sgd_step(float *data, const float *grad, u64 n, float lr) {
  for (u64 j = 0; j < n; ++j) data[j] -= lr * grad[j];
}
/* src/optimizers/cpu/adam.c:48-49: the bias-corrected step size of step t (t >= 1). sqrt is the
 * double function there, so the expression is evaluated in double and rounded to float once. */
float oracle_adam_lr_t(float lr, float beta1, float beta2, int t) {
  float lr_t = lr * sqrt(1.0f - powf(beta2, t)) / (1.0f - powf(beta1, t));
  return lr_t;
}
/* src/optimizers/cpu/adam.c:62-66; t is the step count AFTER the increment of adam.c:28. */
void oracle_adam_step(float *data, const float *grad, float *m_data, float *v_data, u64 n, float lr,
                      float beta1, float beta2, float epsilon, int t) {
  const float lr_t = oracle_adam_lr_t(lr, beta1, beta2, t);
  for (u64 j = 0; j < n; ++j) {
    m_data[j] = beta1 * m_data[j] + (1.0f - beta1) * grad[j];
    v_data[j] = beta2 * v_data[j] + (1.0f - beta2) * grad[j] * grad[j];
    data[j] -= lr_t * m_data[j] / (sqrtf(v_data[j]) + epsilon);
  }
}
/* src/optimizers/cpu/adamw.c:64-71: decoupled weight decay, then the Adam update. */
void oracle_adamw_step(float *data, const float *grad, float *m_data, float *v_data, u64 n, float lr,
                       float beta1, float beta2, float epsilon, float weight_decay, int t) {
  const float lr_t = oracle_adam_lr_t(lr, beta1, beta2, t);
  for (u64 j = 0; j < n; ++j) {
    data[j] -= lr * weight_decay * data[j];
    m_data[j] = beta1 * m_data[j] + (1.0f - beta1) * grad[j];
    v_data[j] = beta2 * v_data[j] + (1.0f - beta2) * grad[j] * grad[j];
    data[j] -= lr_t * m_data[j] / (sqrtf(v_data[j]) + epsilon);
  }
}

/* ---- backward pieces of the fused GEMM epilogues ---------------------------------------------------
 * src/kernels/cpu/fused_ops.c:105-109 (relu_grad_modulate_contig_kernel; its CUDA twin is
 * src/kernels/cuda/matmul_relu.cu:137-144). Pinned by tests/golden/epilogue_pieces.npz, recorded
 * through the reference's matmul_bias_relu_cpu_backward. */
void oracle_relu_grad_modulate(const float *dout, const float *out_data, float *dc, u64 n, float alpha) {
  for (u64 i = 0; i < n; ++i) {
    float o = out_data[i];
    dc[i] = dout[i] * (o > 0.0f ? 1.0f : alpha);
  }
}
/* src/kernels/cpu/fused_ops.c:288-299: dbias is zeroed, then every dc_mod[row][col] is added to
 * dbias[col], rows in order (the CUDA twin, src/kernels/cuda/matmul_bias_relu.cu:143-151, adds in
 * whatever order its atomics give). */
void oracle_bias_grad_reduce(const float *dc_mod, float *dbias, u64 num_elements, u64 cols) {
  for (u64 c = 0; c < cols; ++c) dbias[c] = 0.0f;
  for (u64 i = 0; i < num_elements; ++i) dbias[i % cols] += dc_mod[i];
}

const char *oracle_version(void) { return "plast-oracle 1"; }
