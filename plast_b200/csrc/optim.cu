// Optimiser steps: SGD, Adam and AdamW as one multi-tensor launch per step.
//
// A step touches every parameter once: 12 B/element for SGD (read p and g, write p), 28 B/element
// for Adam / AdamW (read p, g, m, v; write p, m, v). The reference launches one scalar kernel per
// parameter for SGD and has no CUDA Adam at all (src/optimizers/cuda/*.cu); here a table of up
// to kMaxTensors parameters travels in the kernel arguments, each CTA takes one 4096-element
// chunk of one parameter (found by binary search over the chunk prefix sums) and moves it with
// the widest vectors the four pointers allow. Models with more parameters take more launches.
#include "common.cuh"
#include "plast_b200_optim.h"

#include <math.h>
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

namespace pb {

constexpr int kMaxTensors = 48;
constexpr int kOptThreads = 256;
constexpr int kOptChunk = kOptThreads * 16; // elements per CTA

struct OptTable {
  float *p[kMaxTensors];
  const float *g[kMaxTensors];
  float *m[kMaxTensors];
  float *v[kMaxTensors];
  u64 n[kMaxTensors];
  unsigned int first_chunk[kMaxTensors + 1];
  unsigned char vec[kMaxTensors]; // 4, 2 or 1 floats per access
  int count;
};

struct SgdRule {
  float lr;
  static constexpr bool kMoments = false;
  __device__ __forceinline__ void operator()(float &p, float g, float &, float &) const {
    const float step = lr * g;
    p = p - step;
  }
};
struct AdamRule {
  float lr_t, beta1, beta2, one_minus_beta1, one_minus_beta2, epsilon, decay; // decay = lr * weight_decay
  bool decoupled_decay;
  static constexpr bool kMoments = true;
  __device__ __forceinline__ void operator()(float &p, float g, float &m, float &v) const {
    if (decoupled_decay) {
      const float d = decay * p;
      p = p - d;
    }
    const float m1 = beta1 * m;
    const float m2 = one_minus_beta1 * g;
    m = m1 + m2;
    const float v1 = beta2 * v;
    const float v2 = (one_minus_beta2 * g) * g;
    v = v1 + v2;
    const float num = lr_t * m;
    const float den = sqrtf(v) + epsilon;
    p = p - num / den;
  }
};

template <int VEC> struct VecT;
template <> struct VecT<4> { using type = float4; };
template <> struct VecT<2> { using type = float2; };
template <> struct VecT<1> { using type = float; };

template <class Rule, int VEC>
__device__ __forceinline__ void update_chunk(const Rule &rule, float *p, const float *g, float *m, float *v,
                                             u64 begin, u64 end) {
  using V = typename VecT<VEC>::type;
  const u64 nvec = (end - begin) / VEC;
  V *pv = reinterpret_cast<V *>(p + begin);
  const V *gv = reinterpret_cast<const V *>(g + begin);
  V *mv = Rule::kMoments ? reinterpret_cast<V *>(m + begin) : nullptr;
  V *vv = Rule::kMoments ? reinterpret_cast<V *>(v + begin) : nullptr;
  for (u64 i = threadIdx.x; i < nvec; i += kOptThreads) {
    V P = pv[i];
    const V G = __ldcs(gv + i);
    V M = {}, Vv = {};
    if (Rule::kMoments) {
      M = mv[i];
      Vv = vv[i];
    }
    float *pf = reinterpret_cast<float *>(&P);
    const float *gf = reinterpret_cast<const float *>(&G);
    float *mf = reinterpret_cast<float *>(&M);
    float *vf = reinterpret_cast<float *>(&Vv);
#pragma unroll
    for (int k = 0; k < VEC; ++k) rule(pf[k], gf[k], mf[k], vf[k]);
    pv[i] = P;
    if (Rule::kMoments) {
      mv[i] = M;
      vv[i] = Vv;
    }
  }
  // ragged end of the tensor (fewer than VEC elements)
  const u64 done = begin + nvec * VEC;
  if (threadIdx.x < end - done) {
    const u64 j = done + threadIdx.x;
    float P = p[j], M = 0.0f, Vv = 0.0f;
    if (Rule::kMoments) {
      M = m[j];
      Vv = v[j];
    }
    rule(P, g[j], M, Vv);
    p[j] = P;
    if (Rule::kMoments) {
      m[j] = M;
      v[j] = Vv;
    }
  }
}

template <class Rule>
__global__ void __launch_bounds__(kOptThreads) optimizer_step_kernel(const __grid_constant__ OptTable tab,
                                                                     const Rule rule) {
  // which tensor owns this chunk: last t with first_chunk[t] <= blockIdx.x
  int lo = 0, hi = tab.count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tab.first_chunk[mid] <= blockIdx.x) lo = mid; else hi = mid - 1;
  }
  const int t = lo;
  const u64 begin = (u64)(blockIdx.x - tab.first_chunk[t]) * kOptChunk;
  const u64 end = begin + kOptChunk < tab.n[t] ? begin + kOptChunk : tab.n[t];
  float *p = tab.p[t];
  const float *g = tab.g[t];
  float *m = tab.m[t], *v = tab.v[t];
  switch (tab.vec[t]) {
  case 4: update_chunk<Rule, 4>(rule, p, g, m, v, begin, end); break;
  case 2: update_chunk<Rule, 2>(rule, p, g, m, v, begin, end); break;
  default: update_chunk<Rule, 1>(rule, p, g, m, v, begin, end); break;
  }
}

static int widest_vector(const void *a, const void *b, const void *c, const void *d) {
  const uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d;
  return (bits & 15) == 0 ? 4 : ((bits & 7) == 0 ? 2 : 1);
}

// Walks the parameter list, fills tables of up to kMaxTensors entries and launches each.
template <class Rule>
static void multi_tensor_step(const char *name, const Rule &rule, Tensor **parameters, int num_parameters,
                              Tensor **m, Tensor **v) {
  OptTable tab;
  tab.count = 0;
  tab.first_chunk[0] = 0;
  auto flush = [&]() {
    if (tab.count == 0) return true;
    const unsigned int blocks = tab.first_chunk[tab.count];
    optimizer_step_kernel<Rule><<<blocks, kOptThreads, 0, stream()>>>(tab, rule);
    count_launch();
    note_kernel(name);
    tab.count = 0;
    return cudaPeekAtLastError() == cudaSuccess;
  };
  for (int i = 0; i < num_parameters; ++i) {
    Tensor *param = parameters[i];
    if (!param || !param->grad) continue; // sgd.c:19-21, adam.c:53-55
    if (param->dtype != FLOAT32) {
      set_error(PLAST_B200_ERR_DTYPE, "%s: parameter %d is not FLOAT32", name, i);
      return;
    }
    if (!param->data || !param->grad->data) {
      set_error(PLAST_B200_ERR_NULL, "%s: parameter %d has no data or grad buffer", name, i);
      return;
    }
    const u64 n = numel(param);
    if (n == 0) continue;
    const u64 chunks = (n + kOptChunk - 1) / kOptChunk;
    if (chunks > 0x7fffffffull) {
      set_error(PLAST_B200_ERR_LIMIT, "%s: parameter %d is too large for one launch", name, i);
      return;
    }
    if (tab.count == kMaxTensors || (u64)tab.first_chunk[tab.count] + chunks > 0x7fffffffull)
      if (!flush()) break;
    const int k = tab.count++;
    tab.p[k] = (float *)param->data;
    tab.g[k] = (const float *)param->grad->data;
    tab.m[k] = m ? (float *)m[i]->data : nullptr;
    tab.v[k] = v ? (float *)v[i]->data : nullptr;
    tab.n[k] = n;
    tab.vec[k] = (unsigned char)widest_vector(tab.p[k], tab.g[k], tab.m[k], tab.v[k]);
    tab.first_chunk[k + 1] = tab.first_chunk[k] + (unsigned int)chunks;
  }
  flush();
}

// ---- Adam moments owned by the library --------------------------------------------------------------
struct MomentState {
  Tensor **m, **v;
  Tensor *structs;
  void *slab;
  int n; // parameters the moments were created for
};
static std::mutex g_state_mutex;
static std::unordered_map<Tensor **, MomentState> g_states; // keyed by the m array

// adam.c:30-46: m[i], v[i] = zeros like parameters[i].
static bool create_moments(const char *name, Tensor **parameters, int n, Tensor ***m_out, Tensor ***v_out) {
  MomentState st = {};
  st.m = (Tensor **)calloc((size_t)n > 0 ? n : 1, sizeof(Tensor *));
  st.v = (Tensor **)calloc((size_t)n > 0 ? n : 1, sizeof(Tensor *));
  st.structs = (Tensor *)calloc((size_t)(2 * n > 0 ? 2 * n : 1), sizeof(Tensor));
  if (!st.m || !st.v || !st.structs) {
    set_error(PLAST_B200_ERR_CUDA, "%s: out of host memory for the moment tensors", name);
    free(st.m); free(st.v); free(st.structs);
    return false;
  }
  u64 bytes = 0;
  auto padded = [](u64 nbytes) { return (nbytes + 255) & ~(u64)255; };
  for (int i = 0; i < n; ++i)
    if (parameters[i]) bytes += 2 * padded(numel(parameters[i]) * sizeof(float));
  if (cudaMalloc(&st.slab, bytes ? bytes : 256) != cudaSuccess) {
    set_error(PLAST_B200_ERR_CUDA, "%s: cannot allocate %llu bytes for the moments", name, (unsigned long long)bytes);
    free(st.m); free(st.v); free(st.structs);
    return false;
  }
  if (cudaMemsetAsync(st.slab, 0, bytes ? bytes : 256, stream()) != cudaSuccess) {
    set_error(PLAST_B200_ERR_CUDA, "%s: cannot zero the moments", name);
    cudaFree(st.slab);
    free(st.m); free(st.v); free(st.structs);
    return false;
  }
  char *cursor = (char *)st.slab;
  for (int i = 0; i < n; ++i) {
    if (!parameters[i]) continue;
    for (int which = 0; which < 2; ++which) {
      Tensor *t = &st.structs[2 * i + which];
      t->data = cursor;
      t->ndim = parameters[i]->ndim;
      u64 stride = 1;
      for (u64 d = t->ndim; d-- > 0;) {
        t->shape[d] = parameters[i]->shape[d];
        t->strides[d] = stride;
        stride *= t->shape[d];
      }
      t->dtype = parameters[i]->dtype;
      t->device = parameters[i]->device;
      t->requires_grad = false;
      cursor += padded(numel(parameters[i]) * sizeof(float));
      (which == 0 ? st.m : st.v)[i] = t;
    }
  }
  st.n = n;
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    g_states[st.m] = st;
  }
  *m_out = st.m;
  *v_out = st.v;
  return true;
}

// Moments made by this library cover a fixed number of parameters; a later step with a longer list
// would index past them (the reference has the same limit, silently).
static bool moments_cover(const char *name, Tensor **m, int num_parameters) {
  std::lock_guard<std::mutex> lock(g_state_mutex);
  auto it = g_states.find(m);
  if (it == g_states.end() || num_parameters <= it->second.n) return true;
  set_error(PLAST_B200_ERR_SHAPE, "%s: %d parameters, but the moments were created for %d", name, num_parameters,
            it->second.n);
  return false;
}

// adam.c:48-49: float * double sqrt / float, evaluated in double and rounded to float once.
static float bias_corrected_lr(float lr, float beta1, float beta2, int t) {
  // (in C, sqrt is the double function; C++ would pick the float overload without the cast)
  const double root = sqrt((double)(1.0f - powf(beta2, (float)t)));
  return (float)((double)lr * root / (double)(1.0f - powf(beta1, (float)t)));
}

} // namespace pb

using namespace pb;

extern "C" {

void sgd_step_cuda(SGD *optimizer, Tensor **parameters, int num_parameters) {
  begin_call();
  if (!optimizer) {
    set_error(PLAST_B200_ERR_NULL, "SGD is NULL"); // sgd.c:12-15
    return;
  }
  if (!parameters && num_parameters > 0) {
    set_error(PLAST_B200_ERR_NULL, "sgd: parameters is NULL");
    return;
  }
  multi_tensor_step("sgd_multi_tensor", SgdRule{optimizer->lr}, parameters, num_parameters, nullptr, nullptr);
  end_call();
}

void adam_step_cuda(Adam *optimizer, Tensor **parameters, int num_parameters) {
  begin_call();
  if (!optimizer) {
    set_error(PLAST_B200_ERR_NULL, "Adam is NULL");
    return;
  }
  if (!parameters && num_parameters > 0) {
    set_error(PLAST_B200_ERR_NULL, "adam: parameters is NULL");
    return;
  }
  optimizer->t++;
  if (!optimizer->m && !create_moments("adam", parameters, num_parameters, &optimizer->m, &optimizer->v)) return;
  if (!moments_cover("adam", optimizer->m, num_parameters)) return;
  AdamRule rule = {};
  rule.lr_t = bias_corrected_lr(optimizer->lr, optimizer->beta1, optimizer->beta2, optimizer->t);
  rule.beta1 = optimizer->beta1;
  rule.beta2 = optimizer->beta2;
  rule.one_minus_beta1 = 1.0f - optimizer->beta1;
  rule.one_minus_beta2 = 1.0f - optimizer->beta2;
  rule.epsilon = optimizer->epsilon;
  rule.decoupled_decay = false;
  multi_tensor_step("adam_multi_tensor", rule, parameters, num_parameters, optimizer->m, optimizer->v);
  end_call();
}

void adamw_step_cuda(AdamW *optimizer, Tensor **parameters, int num_parameters) {
  begin_call();
  if (!optimizer) {
    set_error(PLAST_B200_ERR_NULL, "AdamW is NULL");
    return;
  }
  if (!parameters && num_parameters > 0) {
    set_error(PLAST_B200_ERR_NULL, "adamw: parameters is NULL");
    return;
  }
  optimizer->t++;
  if (!optimizer->m && !create_moments("adamw", parameters, num_parameters, &optimizer->m, &optimizer->v)) return;
  if (!moments_cover("adamw", optimizer->m, num_parameters)) return;
  AdamRule rule = {};
  rule.lr_t = bias_corrected_lr(optimizer->lr, optimizer->beta1, optimizer->beta2, optimizer->t);
  rule.beta1 = optimizer->beta1;
  rule.beta2 = optimizer->beta2;
  rule.one_minus_beta1 = 1.0f - optimizer->beta1;
  rule.one_minus_beta2 = 1.0f - optimizer->beta2;
  rule.epsilon = optimizer->epsilon;
  rule.decay = optimizer->lr * optimizer->weight_decay; // adamw.c:66: lr * weight_decay * data, left to right
  rule.decoupled_decay = true;
  multi_tensor_step("adamw_multi_tensor", rule, parameters, num_parameters, optimizer->m, optimizer->v);
  end_call();
}

void plast_b200_adam_state_release(Tensor **m, Tensor **v) {
  (void)v;
  MomentState st = {};
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    auto it = g_states.find(m);
    if (it == g_states.end()) return;
    st = it->second;
    g_states.erase(it);
  }
  cudaStreamSynchronize(stream());
  cudaFree(st.slab);
  free(st.structs);
  free(st.m);
  free(st.v);
}

} // extern "C"
