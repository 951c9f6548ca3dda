// Entry points of the binary and unary elementwise ops (forward and backward).
#include "ew_engine.cuh"
#include "functors.cuh"
#include "grad_accum.cuh"

namespace pb {

static bool float_only(const Tensor *t, const char *op) {
  if (t->dtype != FLOAT32) {
    // include/kernels/kernel_macros.h:12-14: message on stderr, nothing computed
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", op, (int)t->dtype);
    return false;
  }
  return true;
}

// ---- unary -----------------------------------------------------------------------------------------
// Iteration space is the INPUT's shape; the output is indexed with its own strides over the same
// coordinates (include/kernels/kernel_macros.h:19-32, 84-93).
template <class F>
static void unary_forward(const char *name, const Tensor **inputs, Tensor *output, const F &f) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name)) return;
  const Tensor *a = inputs[0];
  if (!float_only(a, name)) return;
  u64 st[2][MAX_NDIM] = {};
  for (u64 d = 0; d < a->ndim; ++d) {
    st[0][d] = output->strides[d];
    st[1][d] = a->strides[d];
  }
  IterPlan plan;
  make_plan(&plan, a->shape, a->ndim, 2, st, nullptr, 0);
  const float *ins[1] = {(const float *)a->data};
  launch_ew<F, 1>(plan, (float *)output->data, ins, f);
  end_call();
}

// da[coords] += g(dout[coords], a[coords]) (kernel_macros.h:34-49, 95-110); nothing to do when
// the input does not require a gradient.
template <class B>
static void unary_backward(const char *name, Tensor **inputs, const Tensor *output, const B &f) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name, false)) return;
  const Tensor *a = inputs[0];
  if (!float_only(a, name)) return;
  if (!a->requires_grad) return;
  if (!a->grad || !a->grad->data || !output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: missing grad tensor", name);
    return;
  }
  u64 st[4][MAX_NDIM] = {};
  for (u64 d = 0; d < a->ndim; ++d) {
    st[0][d] = a->grad->strides[d];      // written
    st[1][d] = output->grad->strides[d]; // g
    st[2][d] = a->strides[d];            // a
    st[3][d] = a->grad->strides[d];      // old value
  }
  IterPlan plan;
  make_plan(&plan, a->shape, a->ndim, 4, st, nullptr, 0);
  const float *ins[3] = {(const float *)output->grad->data, (const float *)a->data,
                         (const float *)a->grad->data};
  launch_ew<B, 3>(plan, (float *)a->grad->data, ins, f);
  end_call();
}

// ---- binary ------------------------------------------------------------------------------------------
template <class F>
static void binary_forward(const char *name, const Tensor **inputs, Tensor *output, const F &f) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(inputs[1], name) ||
      !check_tensor(output, name))
    return;
  const Tensor *a = inputs[0], *b = inputs[1];
  if (!float_only(a, name)) return;
  u64 st[3][MAX_NDIM] = {};
  for (u64 d = 0; d < output->ndim; ++d) st[0][d] = output->strides[d];
  if (!broadcast_strides(a, output->shape, output->ndim, st[1]) ||
      !broadcast_strides(b, output->shape, output->ndim, st[2])) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: operand shape does not broadcast to the output shape", name);
    return;
  }
  IterPlan plan;
  make_plan(&plan, output->shape, output->ndim, 3, st, nullptr, 0);
  const float *ins[2] = {(const float *)a->data, (const float *)b->data};
  launch_ew<F, 2>(plan, (float *)output->data, ins, f);
  end_call();
}

// One operand's share of a binary backward: grad(operand) += term(g, p, q). `sel` names which of
// {a, b} feed p and q, so a term only streams the tensors it needs (add/sub read g alone).
// The gradient buffer is indexed with the operand's own strides and shape
// (include/kernels/kernel_macros.h:313-318): dims the operand broadcasts over collapse onto one
// address, which makes this the broadcast-gradient reduce.
template <class Term, int NIN>
static void binary_backward_one(const char *name, const Tensor *a, const Tensor *b,
                                const Tensor *dout, int which, int p_sel, int q_sel) {
  const Tensor *t = which == 0 ? a : b;
  if (!t->requires_grad) return;
  if (!t->grad || !t->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: operand requires grad but has no grad tensor", name);
    return;
  }
  u64 ab[2][MAX_NDIM] = {};
  if (!broadcast_strides(a, dout->shape, dout->ndim, ab[0]) ||
      !broadcast_strides(b, dout->shape, dout->ndim, ab[1])) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: operand shape does not broadcast to the gradient shape", name);
    return;
  }
  const Tensor *src[2] = {a, b};
  u64 in_st[3][MAX_NDIM] = {};
  const float *ins[3] = {(const float *)dout->data, nullptr, nullptr};
  for (u64 d = 0; d < dout->ndim; ++d) in_st[0][d] = dout->strides[d];
  const int sel[2] = {p_sel, q_sel};
  for (int k = 0; k < NIN - 1; ++k) {
    for (u64 d = 0; d < dout->ndim; ++d) in_st[k + 1][d] = ab[sel[k]][d];
    ins[k + 1] = (const float *)src[sel[k]]->data;
  }
  accumulate_grad<Term, NIN>(dout->shape, dout->ndim, (float *)t->grad->data, ab[which], in_st, ins,
                             Term{});
}

// ---- both gradients of a binary op in one pass --------------------------------------------------------
// When both operands want a gradient and nothing broadcasts (five dense tensors of one shape), the
// two accumulations share their reads: dout (and a, b for mul / div) cross HBM once instead of
// once per operand. Same terms, same `old + term` rounding as the one-operand passes.
struct BothAdd {
  static constexpr bool kNeedsAB = false;
  __device__ __forceinline__ static float ta(float g, float, float) { return g; }
  __device__ __forceinline__ static float tb(float g, float, float) { return g; }
};
struct BothSub {
  static constexpr bool kNeedsAB = false;
  __device__ __forceinline__ static float ta(float g, float, float) { return g; }
  __device__ __forceinline__ static float tb(float g, float, float) { return -g; }
};
struct BothMul {
  static constexpr bool kNeedsAB = true;
  __device__ __forceinline__ static float ta(float g, float, float b) { return g * b; }
  __device__ __forceinline__ static float tb(float g, float a, float) { return g * a; }
};
struct BothDiv {
  static constexpr bool kNeedsAB = true;
  __device__ __forceinline__ static float ta(float g, float, float b) { return g / b; }
  __device__ __forceinline__ static float tb(float g, float a, float b) { return -g * a / (b * b); }
};

template <class T>
__global__ void __launch_bounds__(256)
binary_backward_both_kernel(const float4 *__restrict__ g, const float4 *__restrict__ a, const float4 *__restrict__ b,
                            float4 *__restrict__ da, float4 *__restrict__ db, u64 nvec) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int kItems = 2; // float4 per thread and tensor: up to ten loads in flight
  const u64 first = (u64)blockIdx.x * (256 * kItems) + threadIdx.x;
  float4 vg[kItems], va[kItems], vb[kItems], oa[kItems], ob[kItems];
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const u64 j = first + (u64)i * 256;
    if (j < nvec) {
      vg[i] = __ldcs(g + j);
      if (T::kNeedsAB) {
        va[i] = __ldcs(a + j);
        vb[i] = __ldcs(b + j);
      }
      oa[i] = __ldcs(da + j);
      ob[i] = __ldcs(db + j);
    }
  }
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const u64 j = first + (u64)i * 256;
    if (j < nvec) {
      const float4 x = T::kNeedsAB ? va[i] : vg[i], y = T::kNeedsAB ? vb[i] : vg[i];
      oa[i].x += T::ta(vg[i].x, x.x, y.x); oa[i].y += T::ta(vg[i].y, x.y, y.y);
      oa[i].z += T::ta(vg[i].z, x.z, y.z); oa[i].w += T::ta(vg[i].w, x.w, y.w);
      ob[i].x += T::tb(vg[i].x, x.x, y.x); ob[i].y += T::tb(vg[i].y, x.y, y.y);
      ob[i].z += T::tb(vg[i].z, x.z, y.z); ob[i].w += T::tb(vg[i].w, x.w, y.w);
      __stcs(da + j, oa[i]);
      __stcs(db + j, ob[i]);
    }
  }
}

// Takes the fused pass when it applies; false = the caller runs the two one-operand passes.
template <class T>
static bool binary_backward_both(const Tensor *a, const Tensor *b, const Tensor *dout) {
  if (!a->requires_grad || !b->requires_grad || !a->grad || !b->grad || !a->grad->data || !b->grad->data) return false;
  const Tensor *five[5] = {a, b, dout, a->grad, b->grad};
  const u64 n = numel(dout);
  if (n == 0 || (n & 3)) return false;
  for (const Tensor *t : five) {
    if (t->ndim != dout->ndim || ((uintptr_t)t->data & 15)) return false;
    u64 expect = 1; // dense row-major, dim 0 included
    for (u64 d = dout->ndim; d-- > 0;) {
      if (t->shape[d] != dout->shape[d]) return false;
      if (t->shape[d] > 1 && t->strides[d] != expect) return false;
      expect *= t->shape[d];
    }
  }
  // gradient buffers that alias each other (x * x) or an input must go through the ordered passes
  const void *p[5] = {a->data, b->data, dout->data, a->grad->data, b->grad->data};
  for (int i = 0; i < 5; ++i)
    for (int j = i + 1; j < 5; ++j)
      if (p[i] == p[j] && (i >= 3 || j >= 3)) return false;
  const u64 nvec = n >> 2, per_cta = 256 * 2;
  const u64 grid = (nvec + per_cta - 1) / per_cta;
  if (grid > 0x7fffffffull) return false;
  launch_k(binary_backward_both_kernel<T>, dim3((unsigned)grid), dim3(256), 0, stream(), (const float4 *)dout->data,
           (const float4 *)a->data, (const float4 *)b->data, (float4 *)a->grad->data, (float4 *)b->grad->data, nvec);
  count_launch();
  note_kernel("binary_backward_both");
  return true;
}

static bool binary_backward_begin(const char *name, Tensor **inputs, const Tensor *output) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(inputs[1], name) ||
      !check_tensor(output, name, false))
    return false;
  if (!float_only(inputs[0], name)) return false;
  if (!inputs[0]->requires_grad && !inputs[1]->requires_grad) return false;
  if (!output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: output has no grad tensor", name);
    return false;
  }
  return true;
}

} // namespace pb

using namespace pb;

extern "C" {

#define PB_BINARY_FWD(name, F)                                                                    \
  void name##_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams) {                  \
    binary_forward(#name, inputs, output, F{});                                                    \
  }
PB_BINARY_FWD(add, AddF)
PB_BINARY_FWD(sub, SubF)
PB_BINARY_FWD(mul, MulF)
PB_BINARY_FWD(div, DivF)

// src/kernels/cpu/binary_ops.c:18-60 gradient terms
void add_cuda_backward(Tensor **in, const Tensor *out, KernelParams) {
  if (!binary_backward_begin("add", in, out)) return;
  if (binary_backward_both<BothAdd>(in[0], in[1], out->grad)) {
    end_call();
    return;
  }
  binary_backward_one<GradPass, 1>("add", in[0], in[1], out->grad, 0, 0, 0);
  if (!failed()) binary_backward_one<GradPass, 1>("add", in[0], in[1], out->grad, 1, 0, 0);
  end_call();
}
void sub_cuda_backward(Tensor **in, const Tensor *out, KernelParams) {
  if (!binary_backward_begin("sub", in, out)) return;
  if (binary_backward_both<BothSub>(in[0], in[1], out->grad)) {
    end_call();
    return;
  }
  binary_backward_one<GradPass, 1>("sub", in[0], in[1], out->grad, 0, 0, 0);
  if (!failed()) binary_backward_one<GradNeg, 1>("sub", in[0], in[1], out->grad, 1, 0, 0);
  end_call();
}
void mul_cuda_backward(Tensor **in, const Tensor *out, KernelParams) {
  if (!binary_backward_begin("mul", in, out)) return;
  if (binary_backward_both<BothMul>(in[0], in[1], out->grad)) {
    end_call();
    return;
  }
  binary_backward_one<GradMul, 2>("mul", in[0], in[1], out->grad, 0, /*p=b*/ 1, 0);
  if (!failed()) binary_backward_one<GradMul, 2>("mul", in[0], in[1], out->grad, 1, /*p=a*/ 0, 0);
  end_call();
}
void div_cuda_backward(Tensor **in, const Tensor *out, KernelParams) {
  if (!binary_backward_begin("div", in, out)) return;
  if (binary_backward_both<BothDiv>(in[0], in[1], out->grad)) {
    end_call();
    return;
  }
  binary_backward_one<GradDiv, 2>("div", in[0], in[1], out->grad, 0, /*p=b*/ 1, 0);
  if (!failed()) binary_backward_one<GradDivB, 3>("div", in[0], in[1], out->grad, 1, /*p=a*/ 0, /*q=b*/ 1);
  end_call();
}

#define PB_UNARY(name, F, B)                                                                       \
  void name##_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams) {                  \
    unary_forward(#name, inputs, output, F{});                                                     \
  }                                                                                                \
  void name##_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams) {                 \
    unary_backward(#name, inputs, output, B{});                                                    \
  }
PB_UNARY(abs, AbsF, AbsB)
PB_UNARY(cos, CosF, CosB)
PB_UNARY(sin, SinF, SinB)
PB_UNARY(tan, TanF, TanB)
PB_UNARY(exp, ExpF, ExpB)
PB_UNARY(log, LogF, LogB)
PB_UNARY(neg, NegF, NegB)

void leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  unary_forward("leaky_relu", inputs, output, LeakyReluF{params.fval});
}
void leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  unary_backward("leaky_relu", inputs, output, LeakyReluB{params.fval});
}

} // extern "C"
