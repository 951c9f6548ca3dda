// Fused elementwise recipes and the generic fused chain.
//
//   sigmoid                 neg -> exp -> +1 -> 1/.        (plast/nn/functional.py:42-47)
//   add_leaky_relu          add -> leaky_relu
//   scale_bias_leaky_relu   mul -> add -> leaky_relu
//   plast_b200_chain_forward  any straight-line program of elementwise steps
//
// Every step is rounded to fp32 on its own (-fmad=false), so a fused result is bit-identical to
// running the primitive ops one after another; the gain is that intermediates never touch HBM.
#include "ew_engine.cuh"
#include "functors.cuh"
#include "grad_accum.cuh"

namespace pb {

// ---- fixed recipes ------------------------------------------------------------------------------------
struct SigmoidF {
  __device__ __forceinline__ float operator()(const float *x) const {
    const float nx = -x[0];
    const float e = expf(nx);
    const float d = e + 1.0f;
    return 1.0f / d;
  }
};
struct SigmoidB { // x = {g, y, old}: dy/dx = y (1 - y)
  __device__ __forceinline__ float operator()(const float *x) const {
    return x[2] + x[0] * (x[1] * (1.0f - x[1]));
  }
};
struct AddLeakyF { // x = {a, b}
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float u = x[0] + x[1];
    return u > 0.0f ? u : u * alpha;
  }
};
struct ScaleBiasLeakyF { // x = {v, scale, bias}
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float t = x[0] * x[1];
    const float u = t + x[2];
    return u > 0.0f ? u : u * alpha;
  }
};
// Gradient terms. The pre-activation u is recomputed from the inputs (exact for any slope);
// du = g * (u > 0 ? 1 : slope) is what leaky_relu's backward hands to the add / mul backward
// (src/kernels/cpu/unary_ops.c:234-262, binary_ops.c:18-49).
struct AddLeakyGrad { // x = {g, a, b}
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float u = x[1] + x[2];
    return x[0] * (u > 0.0f ? 1.0f : alpha);
  }
};
struct SblBiasGrad { // x = {g, v, scale, bias} -> du
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float t = x[1] * x[2];
    const float u = t + x[3];
    return x[0] * (u > 0.0f ? 1.0f : alpha);
  }
};
struct SblScaleGrad { // du * v
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float t = x[1] * x[2];
    const float u = t + x[3];
    return (x[0] * (u > 0.0f ? 1.0f : alpha)) * x[1];
  }
};
struct SblInputGrad { // du * scale
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    const float t = x[1] * x[2];
    const float u = t + x[3];
    return (x[0] * (u > 0.0f ? 1.0f : alpha)) * x[2];
  }
};

// ---- C = leaky_relu(A + b) and s = sum(C, last axis) in one pass -------------------------------------
// One warp per row of a contiguous [rows, cols] matrix (cols % 4 == 0, 16-byte aligned): each lane
// loads float4s of A and of b's row (b is [cols]-like and stays in L1 / L2), stores C and keeps a
// running sum; a shuffle tree finishes the row. C is bit-identical to the two-op sequence; s is a
// tree sum of exactly those values.
constexpr int kRowSumThreads = 256;
__global__ void __launch_bounds__(kRowSumThreads)
add_leaky_relu_row_sum_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ c,
                              float *__restrict__ s, u64 rows, u64 cols, u64 b_row_stride, float alpha) {
  pdl_wait();
  pdl_launch_dependents();
  const unsigned lane = threadIdx.x & 31;
  const u64 warps = (u64)gridDim.x * (kRowSumThreads / 32);
  const u64 nvec = cols >> 2;
  for (u64 row = (u64)blockIdx.x * (kRowSumThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const float4 *ar = reinterpret_cast<const float4 *>(a + row * cols);
    const float4 *br = reinterpret_cast<const float4 *>(b + row * b_row_stride);
    float4 *cr = reinterpret_cast<float4 *>(c + row * cols);
    float acc = 0.0f;
    for (u64 j0 = 0; j0 < nvec; j0 += 8 * 32) {
      float4 va[8], vb[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const u64 j = j0 + lane + (u64)u * 32;
        if (j < nvec) {
          va[u] = __ldcs(ar + j);
          vb[u] = __ldg(br + j);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const u64 j = j0 + lane + (u64)u * 32;
        if (j < nvec) {
          float4 r;
          float t;
          t = va[u].x + vb[u].x; r.x = t > 0.0f ? t : t * alpha;
          t = va[u].y + vb[u].y; r.y = t > 0.0f ? t : t * alpha;
          t = va[u].z + vb[u].z; r.z = t > 0.0f ? t : t * alpha;
          t = va[u].w + vb[u].w; r.w = t > 0.0f ? t : t * alpha;
          __stcs(cr + j, r);
          acc += (r.x + r.y) + (r.z + r.w);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s[row] = acc;
  }
}

// ---- generic chain -------------------------------------------------------------------------------------
struct ChainProgram {
  int n_inputs, n_steps;
  unsigned char opcode[PLAST_CHAIN_MAX_STEPS], a[PLAST_CHAIN_MAX_STEPS], b[PLAST_CHAIN_MAX_STEPS];
  float fval[PLAST_CHAIN_MAX_STEPS];
};

__device__ __forceinline__ float chain_step(int opcode, float p, float q, float f) {
  switch (opcode) {
  case PLAST_CHAIN_ADD: return p + q;
  case PLAST_CHAIN_SUB: return p - q;
  case PLAST_CHAIN_MUL: return p * q;
  case PLAST_CHAIN_DIV: return p / q;
  case PLAST_CHAIN_NEG: return -p;
  case PLAST_CHAIN_ABS: return fabsf(p);
  case PLAST_CHAIN_EXP: return expf(p);
  case PLAST_CHAIN_LOG: return logf(p);
  case PLAST_CHAIN_SIN: return sinf(p);
  case PLAST_CHAIN_COS: return cosf(p);
  case PLAST_CHAIN_TAN: return tan_accurate(p);
  case PLAST_CHAIN_LEAKY_RELU: return p > 0.0f ? p : p * f;
  case PLAST_CHAIN_ADD_SCALAR: return p + f;
  case PLAST_CHAIN_RSUB_SCALAR: return f - p;
  case PLAST_CHAIN_MUL_SCALAR: return p * f;
  default: return f / p; // PLAST_CHAIN_RDIV_SCALAR
  }
}

// Interpreter: the program is uniform across threads, so the switch never diverges; the register
// file is a small per-thread array.
template <int NIN> struct ChainInterp {
  ChainProgram prog;
  __device__ __forceinline__ float operator()(const float *x) const {
    float reg[PLAST_CHAIN_MAX_INPUTS + PLAST_CHAIN_MAX_STEPS];
#pragma unroll
    for (int i = 0; i < NIN; ++i) reg[i] = x[i];
    for (int s = 0; s < prog.n_steps; ++s)
      reg[NIN + s] = chain_step(prog.opcode[s], reg[prog.a[s]], reg[prog.b[s]], prog.fval[s]);
    return reg[NIN + prog.n_steps - 1];
  }
};

// z = sigmoid(x) * y + exp(-abs(x)) as the nine primitive steps, compiled ahead of time; chosen
// when a submitted program is exactly this sequence.
struct SigmoidMulAddExpNegAbs { // x = {x, y}
  __device__ __forceinline__ float operator()(const float *x) const {
    const float nx = -x[0];
    const float e = expf(nx);
    const float d = e + 1.0f;
    const float sg = 1.0f / d;
    const float t = sg * x[1];
    const float ax = fabsf(x[0]);
    const float nax = -ax;
    const float e2 = expf(nax);
    return t + e2;
  }
};
static bool is_sigmoid_mul_add_exp_neg_abs(const ChainProgram &p) {
  static const int ops[9] = {PLAST_CHAIN_NEG, PLAST_CHAIN_EXP, PLAST_CHAIN_ADD_SCALAR,
                             PLAST_CHAIN_RDIV_SCALAR, PLAST_CHAIN_MUL, PLAST_CHAIN_ABS,
                             PLAST_CHAIN_NEG, PLAST_CHAIN_EXP, PLAST_CHAIN_ADD};
  static const int as[9] = {0, 2, 3, 4, 5, 0, 7, 8, 6};
  static const int bs[9] = {0, 0, 0, 0, 1, 0, 0, 0, 9};
  if (p.n_inputs != 2 || p.n_steps != 9) return false;
  for (int s = 0; s < 9; ++s) {
    if (p.opcode[s] != ops[s] || p.a[s] != as[s]) return false;
    if ((ops[s] == PLAST_CHAIN_MUL || ops[s] == PLAST_CHAIN_ADD) && p.b[s] != bs[s]) return false;
  }
  return p.fval[2] == 1.0f && p.fval[3] == 1.0f;
}

// chain_jit.cu
struct ChainProgramView {
  int n_inputs, n_steps;
  const unsigned char *opcode, *a, *b;
  const float *fval;
  unsigned scalar_mask; // filled by the compiler from the plan
  int wrt;              // -1 forward; else backward with respect to this input
  bool accumulate;      // backward: the last operand is the input's current gradient
};
bool launch_chain_jit(const ChainProgramView &p, const IterPlan &plan, float *out, const float *const *ins);
bool chain_jit_available();

static bool read_program(const PlastChainStep *steps, int n_steps, int n_inputs, ChainProgram *prog) {
  if (n_inputs < 1 || n_inputs > PLAST_CHAIN_MAX_INPUTS || n_steps < 1 || n_steps > PLAST_CHAIN_MAX_STEPS) {
    set_error(PLAST_B200_ERR_LIMIT, "chain: %d inputs / %d steps (limits %d / %d)", n_inputs, n_steps,
              PLAST_CHAIN_MAX_INPUTS, PLAST_CHAIN_MAX_STEPS);
    return false;
  }
  prog->n_inputs = n_inputs;
  prog->n_steps = n_steps;
  for (int s = 0; s < n_steps; ++s) {
    const PlastChainStep &st = steps[s];
    const bool binary = st.opcode <= PLAST_CHAIN_DIV;
    if (st.opcode < 0 || st.opcode > PLAST_CHAIN_RDIV_SCALAR || st.a < 0 || st.a >= n_inputs + s ||
        (binary && (st.b < 0 || st.b >= n_inputs + s))) {
      set_error(PLAST_B200_ERR_SHAPE, "chain: step %d is malformed (opcode %d, a %d, b %d)", s,
                st.opcode, st.a, st.b);
      return false;
    }
    prog->opcode[s] = (unsigned char)st.opcode;
    prog->a[s] = (unsigned char)st.a;
    prog->b[s] = (unsigned char)(binary ? st.b : st.a);
    prog->fval[s] = st.fval;
  }
  return true;
}

static bool float_only(const Tensor *t, const char *op) {
  if (t->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", op, (int)t->dtype);
    return false;
  }
  return true;
}

// out = f(inputs...) with every input broadcast against the output shape.
template <class F, int NIN>
static void fused_forward(const char *name, const Tensor **inputs, Tensor *output, const F &f) {
  u64 st[NIN + 1][MAX_NDIM] = {};
  const float *ins[NIN];
  for (u64 d = 0; d < output->ndim; ++d) st[0][d] = output->strides[d];
  for (int a = 0; a < NIN; ++a) {
    if (!check_tensor(inputs[a], name) || !float_only(inputs[a], name)) return;
    if (!broadcast_strides(inputs[a], output->shape, output->ndim, st[a + 1])) {
      set_error(PLAST_B200_ERR_SHAPE, "%s: input %d does not broadcast to the output shape", name, a);
      return;
    }
    ins[a] = (const float *)inputs[a]->data;
  }
  IterPlan plan;
  make_plan(&plan, output->shape, output->ndim, NIN + 1, st, nullptr, 0);
  launch_ew<F, NIN>(plan, (float *)output->data, ins, f);
}

// grad(inputs[which]) += term(g, inputs...), reduced over the dims inputs[which] broadcasts.
template <class Term, int NOPS>
static void fused_backward_one(const char *name, Tensor **inputs, const Tensor *output, int which,
                               const Term &term) {
  const Tensor *t = inputs[which];
  if (!t->requires_grad) return;
  if (!t->grad || !t->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: input %d requires grad but has no grad tensor", name, which);
    return;
  }
  const Tensor *dout = output->grad;
  u64 in_st[NOPS + 1][MAX_NDIM] = {};
  const float *ins[NOPS + 1];
  for (u64 d = 0; d < dout->ndim; ++d) in_st[0][d] = dout->strides[d];
  ins[0] = (const float *)dout->data;
  for (int a = 0; a < NOPS; ++a) {
    if (!broadcast_strides(inputs[a], dout->shape, dout->ndim, in_st[a + 1])) {
      set_error(PLAST_B200_ERR_SHAPE, "%s: input %d does not broadcast to the gradient shape", name, a);
      return;
    }
    ins[a + 1] = (const float *)inputs[a]->data;
  }
  accumulate_grad<Term, NOPS + 1>(dout->shape, dout->ndim, (float *)t->grad->data, in_st[which + 1],
                                  in_st, ins, term);
}

static bool fused_backward_begin(const char *name, Tensor **inputs, int n, const Tensor *output) {
  begin_call();
  if (!inputs || !check_tensor(output, name, false)) return false;
  bool any = false;
  for (int a = 0; a < n; ++a) {
    if (!check_tensor(inputs[a], name) || !float_only(inputs[a], name)) return false;
    any = any || inputs[a]->requires_grad;
  }
  if (!any) return false;
  if (!output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: output has no grad tensor", name);
    return false;
  }
  return true;
}

} // namespace pb

using namespace pb;

extern "C" {

void sigmoid_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams) {
  begin_call();
  if (!inputs || !check_tensor(output, "sigmoid")) return;
  fused_forward<SigmoidF, 1>("sigmoid", inputs, output, SigmoidF{});
  end_call();
}
void sigmoid_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], "sigmoid") || !check_tensor(output, "sigmoid")) return;
  const Tensor *a = inputs[0];
  if (!a->requires_grad) return;
  if (!a->grad || !a->grad->data || !output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "sigmoid: missing grad tensor");
    return;
  }
  u64 st[4][MAX_NDIM] = {};
  for (u64 d = 0; d < a->ndim; ++d) {
    st[0][d] = a->grad->strides[d];
    st[1][d] = output->grad->strides[d];
    st[2][d] = output->strides[d];
    st[3][d] = a->grad->strides[d];
  }
  IterPlan plan;
  make_plan(&plan, a->shape, a->ndim, 4, st, nullptr, 0);
  const float *ins[3] = {(const float *)output->grad->data, (const float *)output->data,
                         (const float *)a->grad->data};
  launch_ew<SigmoidB, 3>(plan, (float *)a->grad->data, ins, SigmoidB{});
  end_call();
}

void add_leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  begin_call();
  if (!inputs || !check_tensor(output, "add_leaky_relu")) return;
  fused_forward<AddLeakyF, 2>("add_leaky_relu", inputs, output, AddLeakyF{params.fval});
  end_call();
}
void add_leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  if (!fused_backward_begin("add_leaky_relu", inputs, 2, output)) return;
  const AddLeakyGrad term{params.fval};
  fused_backward_one<AddLeakyGrad, 2>("add_leaky_relu", inputs, output, 0, term);
  if (!failed()) fused_backward_one<AddLeakyGrad, 2>("add_leaky_relu", inputs, output, 1, term);
  end_call();
}

void scale_bias_leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  begin_call();
  if (!inputs || !check_tensor(output, "scale_bias_leaky_relu")) return;
  fused_forward<ScaleBiasLeakyF, 3>("scale_bias_leaky_relu", inputs, output,
                                    ScaleBiasLeakyF{params.fval});
  end_call();
}
void scale_bias_leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  const char *name = "scale_bias_leaky_relu";
  if (!fused_backward_begin(name, inputs, 3, output)) return;
  fused_backward_one<SblInputGrad, 3>(name, inputs, output, 0, SblInputGrad{params.fval});
  if (!failed()) fused_backward_one<SblScaleGrad, 3>(name, inputs, output, 1, SblScaleGrad{params.fval});
  if (!failed()) fused_backward_one<SblBiasGrad, 3>(name, inputs, output, 2, SblBiasGrad{params.fval});
  end_call();
}

void plast_b200_add_leaky_relu_row_sum(const Tensor *a, const Tensor *b, Tensor *c, Tensor *s, float slope) {
  const char *name = "add_leaky_relu_row_sum";
  begin_call();
  if (!check_tensor(a, name) || !check_tensor(b, name) || !check_tensor(c, name) || !check_tensor(s, name)) return;
  if (!float_only(a, name) || !float_only(b, name) || !float_only(c, name) || !float_only(s, name)) return;
  if (a->ndim < 1 || c->ndim != a->ndim) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: a and c must have the same rank >= 1", name);
    return;
  }
  for (u64 d = 0; d < a->ndim; ++d)
    if (a->shape[d] != c->shape[d]) {
      set_error(PLAST_B200_ERR_SHAPE, "%s: a and c differ in dim %llu", name, (unsigned long long)d);
      return;
    }
  const u64 cols = a->shape[a->ndim - 1];
  const u64 rows = cols ? numel(a) / cols : 0;
  if (numel(s) != rows) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: s holds %llu elements, the matrix has %llu rows", name,
              (unsigned long long)numel(s), (unsigned long long)rows);
    return;
  }
  // b: one row for all (any shape of cols elements, e.g. [1, cols] or [cols]) or a's own shape
  const bool b_row = numel(b) == cols && b->ndim >= 1 && b->shape[b->ndim - 1] == cols;
  const bool b_full = numel(b) == numel(a) && b->ndim == a->ndim && b->shape[b->ndim - 1] == cols;
  auto dense = [](const Tensor *t) {
    u64 expect = 1;
    for (u64 d = t->ndim; d-- > 0;) {
      if (t->shape[d] == 1) continue;
      if (t->strides[d] != expect) return false;
      expect *= t->shape[d];
    }
    return true;
  };
  const bool aligned = ((((uintptr_t)a->data) | ((uintptr_t)b->data) | ((uintptr_t)c->data)) & 15) == 0;
  const bool fast = (b_row || b_full) && dense(a) && dense(b) && dense(c) && dense(s) && cols % 4 == 0 &&
                    aligned && rows > 0;
  if (!fast) {
    // any other layout: the two entry points one after the other
    const Tensor *in2[2] = {a, b};
    KernelParams p = {0, 0, slope};
    add_leaky_relu_cuda_forward(in2, c, p);
    if (failed()) return;
    const Tensor *in1[1] = {c};
    KernelParams q = {a->ndim - 1, 0, 0.0f};
    Tensor s_copy = *s; // the reduction rewrites its output's shape; the caller's header stays as given
    sum_cuda_forward(in1, &s_copy, q);
    return;
  }
  const u64 warps_per_cta = kRowSumThreads / 32;
  u64 blocks = (rows + warps_per_cta - 1) / warps_per_cta;
  const u64 cap = (u64)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  launch_k(add_leaky_relu_row_sum_kernel, dim3((unsigned)blocks), dim3(kRowSumThreads), 0, stream(),
           (const float *)a->data, (const float *)b->data, (float *)c->data, (float *)s->data, rows, cols,
           b_full ? cols : (u64)0, slope);
  count_launch();
  note_kernel("add_leaky_relu_row_sum");
  end_call();
}

void plast_b200_chain_forward(const Tensor **inputs, int n_inputs, Tensor *output,
                              const PlastChainStep *steps, int n_steps) {
  const char *name = "chain";
  begin_call();
  if (!inputs || !steps || !check_tensor(output, name)) {
    if (!inputs || !steps) set_error(PLAST_B200_ERR_NULL, "chain: NULL inputs or steps");
    return;
  }
  ChainProgram prog = {};
  if (!read_program(steps, n_steps, n_inputs, &prog)) return;
  if (is_sigmoid_mul_add_exp_neg_abs(prog)) {
    fused_forward<SigmoidMulAddExpNegAbs, 2>(name, inputs, output, SigmoidMulAddExpNegAbs{});
    if (!failed()) note_kernel("chain_precompiled");
    end_call();
    return;
  }
  // Run-time compiled functor (NVRTC), same rounding as the interpreter; falls through to the
  // interpreter when the compiler is unavailable.
  {
    u64 st[PLAST_CHAIN_MAX_INPUTS + 1][MAX_NDIM] = {};
    const float *ins[PLAST_CHAIN_MAX_INPUTS] = {};
    for (u64 d = 0; d < output->ndim; ++d) st[0][d] = output->strides[d];
    bool ok = true;
    for (int a = 0; ok && a < n_inputs; ++a) {
      if (!check_tensor(inputs[a], name) || !float_only(inputs[a], name)) return;
      if (!broadcast_strides(inputs[a], output->shape, output->ndim, st[a + 1])) {
        set_error(PLAST_B200_ERR_SHAPE, "%s: input %d does not broadcast to the output shape", name, a);
        return;
      }
      ins[a] = (const float *)inputs[a]->data;
    }
    IterPlan plan;
    make_plan(&plan, output->shape, output->ndim, n_inputs + 1, st, nullptr, 0);
    const ChainProgramView view{n_inputs, n_steps, prog.opcode, prog.a, prog.b, prog.fval, 0u, -1, false};
    if (launch_chain_jit(view, plan, (float *)output->data, ins)) {
      note_kernel("chain_jit");
      end_call();
      return;
    }
  }
  switch (n_inputs) {
#define PB_INTERP(N) case N: fused_forward<ChainInterp<N>, N>(name, inputs, output, ChainInterp<N>{prog}); break;
    PB_INTERP(1) PB_INTERP(2) PB_INTERP(3) PB_INTERP(4) PB_INTERP(5) PB_INTERP(6) PB_INTERP(7)
  default: fused_forward<ChainInterp<8>, 8>(name, inputs, output, ChainInterp<8>{prog}); break;
#undef PB_INTERP
  }
  if (!failed()) note_kernel("chain_interpreter");
  end_call();
}

// Backward of a fused chain: for every input that requires grad, one run-time compiled kernel
// recomputes the chain's registers from the inputs and sweeps the steps in reverse, applying each
// gradient contribution in the order and with the rounding of the node-by-node backward
// (functors.cuh), so full-shape inputs receive bit-identical gradients. An input that broadcasts
// gets its per-element adjoint written to a stream-ordered scratch buffer, which the
// broadcast-gradient reduce then sums into its gradient.
void plast_b200_chain_backward(Tensor **inputs, int n_inputs, const Tensor *output,
                               const PlastChainStep *steps, int n_steps) {
  const char *name = "chain backward";
  begin_call();
  if (!inputs || !steps || !check_tensor(output, name, false)) {
    if (!inputs || !steps) set_error(PLAST_B200_ERR_NULL, "chain backward: NULL inputs or steps");
    return;
  }
  ChainProgram prog = {};
  if (!read_program(steps, n_steps, n_inputs, &prog)) return;
  bool any = false;
  for (int a = 0; a < n_inputs; ++a) {
    if (!check_tensor(inputs[a], name) || !float_only(inputs[a], name)) return;
    any = any || inputs[a]->requires_grad;
  }
  if (!any) return;
  const Tensor *dout = output->grad;
  if (!dout || !dout->data) {
    set_error(PLAST_B200_ERR_NULL, "chain backward: output has no grad tensor");
    return;
  }
  if (!chain_jit_available()) {
    set_error(PLAST_B200_ERR_UNSUPPORTED, "chain backward needs the run-time compiler (libnvrtc and libcuda)");
    return;
  }
  const u64 nd = dout->ndim;
  for (int w = 0; w < n_inputs && !failed(); ++w) {
    Tensor *t = inputs[w];
    if (!t->requires_grad) continue;
    if (!t->grad || !t->grad->data) {
      set_error(PLAST_B200_ERR_NULL, "chain backward: input %d requires grad but has no grad tensor", w);
      return;
    }
    // operand strides aligned to the upstream gradient's shape: [target, g, inputs..., current grad]
    u64 st[PLAST_CHAIN_MAX_INPUTS + 3][MAX_NDIM] = {};
    const float *ins[PLAST_CHAIN_MAX_INPUTS + 2] = {};
    for (u64 d = 0; d < nd; ++d) st[1][d] = dout->strides[d];
    ins[0] = (const float *)dout->data;
    for (int a = 0; a < n_inputs; ++a) {
      if (!broadcast_strides(inputs[a], dout->shape, nd, st[a + 2])) {
        set_error(PLAST_B200_ERR_SHAPE, "chain backward: input %d does not broadcast to the gradient shape", a);
        return;
      }
      ins[a + 1] = (const float *)inputs[a]->data;
    }
    // does input w cover the whole iteration space (no broadcast dim of extent > 1)?
    u64 gst[MAX_NDIM] = {};
    Tensor as_grad = *t; // the operand's shape with its gradient's strides
    for (u64 d = 0; d < t->ndim; ++d) as_grad.strides[d] = t->grad->strides[d];
    broadcast_strides(&as_grad, dout->shape, nd, gst);
    bool full = true;
    for (u64 d = 0; d < nd; ++d) full = full && !(gst[d] == 0 && dout->shape[d] > 1);
    ChainProgramView view{n_inputs, n_steps, prog.opcode, prog.a, prog.b, prog.fval, 0u, w, full};
    IterPlan plan;
    if (full) {
      for (u64 d = 0; d < nd; ++d) {
        st[0][d] = gst[d];
        st[n_inputs + 2][d] = gst[d];
      }
      ins[n_inputs + 1] = (const float *)t->grad->data;
      make_plan(&plan, dout->shape, nd, n_inputs + 3, st, nullptr, 0);
      if (!launch_chain_jit(view, plan, (float *)t->grad->data, ins)) {
        set_error(PLAST_B200_ERR_CUDA, "chain backward: the gradient kernel for input %d could not be built or launched", w);
        return;
      }
    } else {
      float *scratch = nullptr;
      PB_CUDA(scratch_alloc_async((void **)&scratch, numel(dout) * sizeof(float)));
      u64 cs = 1;
      for (u64 d = nd; d-- > 0;) {
        st[0][d] = cs;
        cs *= dout->shape[d];
      }
      make_plan(&plan, dout->shape, nd, n_inputs + 2, st, nullptr, 0);
      if (!launch_chain_jit(view, plan, scratch, ins)) {
        cudaFreeAsync(scratch, stream());
        set_error(PLAST_B200_ERR_CUDA, "chain backward: the gradient kernel for input %d could not be built or launched", w);
        return;
      }
      u64 in_st[1][MAX_NDIM] = {};
      for (u64 d = 0; d < nd; ++d) in_st[0][d] = st[0][d];
      const float *rins[1] = {scratch};
      accumulate_grad<GradPass, 1>(dout->shape, nd, (float *)t->grad->data, gst, in_st, rins, GradPass{});
      cudaFreeAsync(scratch, stream());
    }
  }
  if (!failed()) note_kernel("chain_backward_jit");
  end_call();
}

} // extern "C"
