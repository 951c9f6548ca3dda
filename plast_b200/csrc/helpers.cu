// Symbols the reference's core, arena, shape ops and Python extension link against:
// fills, arena memory calls, view-gradient accumulation and the strided -> contiguous pack.
#include <atomic>
#include "ew_engine.cuh"
#include "functors.cuh"
#include "grad_accum.cuh"

#include <stdlib.h>

namespace pb {

struct CopyF { __device__ __forceinline__ float operator()(const float *x) const { return x[0]; } };
struct AccF { __device__ __forceinline__ float operator()(const float *x) const { return x[1] + x[0]; } };

// 16-byte stores; value is a 32-bit pattern so int32 and float32 share the kernel.
__global__ void __launch_bounds__(256) fill_kernel(unsigned int *p, unsigned int value, u64 n) {
  const u64 stride = (u64)gridDim.x * blockDim.x;
  u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x;
  // head until 16-byte aligned
  const u64 head = (((uintptr_t)p) & 15) ? ((16 - (((uintptr_t)p) & 15)) >> 2) : 0;
  const u64 h = head < n ? head : n;
  if (i < h) p[i] = value;
  uint4 *q = reinterpret_cast<uint4 *>(p + h);
  const u64 nv = (n - h) >> 2;
  const uint4 v = make_uint4(value, value, value, value);
  for (u64 j = i; j < nv; j += stride) q[j] = v;
  const u64 tail_begin = h + (nv << 2);
  if (tail_begin + i < n && i < 4) p[tail_begin + i] = value;
}

void fill32(void *data, unsigned int pattern, u64 n) {
  if (n == 0) return;
  u64 blocks = (n / 4 + 255) / 256;
  const u64 cap = (u64)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  fill_kernel<<<(unsigned)blocks, 256, 0, stream()>>>((unsigned int *)data, pattern, n);
  count_launch();
  note_kernel("fill32");
}

// dout * (y > 0 ? 1 : slope): the gradient a leaky_relu epilogue hands to what it is fused onto.
struct ReluGradModulate { // x = {dout, y}
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    return x[0] * (x[1] > 0.0f ? 1.0f : alpha);
  }
};

// Column sums of a contiguous [num_elements / cols, cols] matrix of Term values, written to dbias.
template <class Term, int NIN>
static void column_sums(const char *name, const float *const *ins, float *dbias, u64 num_elements, u64 cols,
                        const Term &term) {
  if (cols == 0 || num_elements % cols != 0) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: %llu elements are not rows of %llu columns", name,
              (unsigned long long)num_elements, (unsigned long long)cols);
    return;
  }
  if (num_elements == 0) {
    fill32(dbias, 0u, cols);
    return;
  }
  const u64 shape[2] = {num_elements / cols, cols};
  const bool reduced[2] = {true, false};
  u64 st[NIN + 1][MAX_NDIM] = {};
  st[0][1] = 1; // target: one value per column
  for (int a = 0; a < NIN; ++a) {
    st[a + 1][0] = cols;
    st[a + 1][1] = 1;
  }
  IterPlan plan;
  make_plan(&plan, shape, 2, NIN + 1, st, reduced, 1);
  launch_reduce<SumOp, Term, NIN>(plan, dbias, ins, term, SumOp{}, /*accumulate=*/false, 0.0f);
}

static unsigned int one_pattern(DTYPE dt) {
  if (dt == INT32) return 1u;
  const float f = 1.0f;
  unsigned int u;
  memcpy(&u, &f, 4);
  return u;
}

} // namespace pb

using namespace pb;

extern "C" {

// src/kernels/cuda/cuda_tensor_init.cu:19-95
void zeros_cuda(Tensor *t, u64 num_elements) {
  begin_call();
  if (!check_tensor(t, "zeros")) return;
  fill32(t->data, 0u, num_elements);
  end_call();
}
void ones_cuda(Tensor *t, u64 num_elements) {
  begin_call();
  if (!check_tensor(t, "ones")) return;
  fill32(t->data, one_pattern(t->dtype), num_elements);
  end_call();
}
void set_ones_grad_cuda(Tensor *t) {
  begin_call();
  if (!check_tensor(t, "set_ones_grad", false)) return;
  if (!t->grad || !t->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "set_ones_grad: tensor has no grad");
    return;
  }
  fill32(t->grad->data, one_pattern(t->dtype), numel(t));
  end_call();
}
// src/optimizers/cuda/zero_grad.cu:11-25
void zero_grad_cuda(Tensor *t) {
  begin_call();
  if (!t || !t->grad || !t->grad->data) return;
  fill32(t->grad->data, 0u, numel(t->grad));
  end_call();
}

// src/kernels/cuda/shape_ops_cuda.cu:38-43: da[i] += dout[i]
void reshape_backward_cuda(float *da, const float *dout, u64 num_elements) {
  begin_call();
  if (!da || !dout) {
    set_error(PLAST_B200_ERR_NULL, "reshape_backward: NULL pointer");
    return;
  }
  const u64 shape[1] = {num_elements};
  u64 st[3][MAX_NDIM] = {};
  st[0][0] = st[1][0] = st[2][0] = 1;
  IterPlan plan;
  make_plan(&plan, shape, 1, 3, st, nullptr, 0);
  const float *ins[2] = {dout, da};
  launch_ew<AccF, 2>(plan, da, ins, AccF{});
  end_call();
}

// src/kernels/cuda/shape_ops_cuda.cu:45-70 (src/kernels/cpu/shape_ops.c:82-120): for every
// coordinate of a, da[coords . da_strides] += dout[swap(coords) . dout_strides]. Each da element
// is written once, so no atomics are needed; shape/stride arrays are host memory.
void transpose_backward_cuda(float *da, const float *dout, const u64 *a_shape,
                             const u64 *da_strides, const u64 *dout_strides, u64 ndim, u64 axis1,
                             u64 axis2, u64 num_elements) {
  begin_call();
  (void)num_elements;
  if (!da || !dout || !a_shape || !da_strides || !dout_strides) {
    set_error(PLAST_B200_ERR_NULL, "transpose_backward: NULL pointer");
    return;
  }
  if (ndim > MAX_NDIM || axis1 >= ndim || axis2 >= ndim) {
    set_error(PLAST_B200_ERR_SHAPE, "transpose_backward: bad ndim/axes");
    return;
  }
  u64 st[3][MAX_NDIM] = {};
  for (u64 d = 0; d < ndim; ++d) {
    u64 od = d == axis1 ? axis2 : (d == axis2 ? axis1 : d);
    st[0][d] = da_strides[d];
    st[1][d] = dout_strides[od];
    st[2][d] = da_strides[d];
  }
  IterPlan plan;
  make_plan(&plan, a_shape, ndim, 3, st, nullptr, 0);
  const float *ins[2] = {dout, da};
  launch_ew<AccF, 2>(plan, da, ins, AccF{});
  end_call();
}

// src/core/arena_cuda.cu:13-32. Allocation failures are fatal there (exit); here too, because the
// arena has no way to report them.
#define PB_FATAL(expr)                                                                             \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess) {                                                                       \
      fprintf(stderr, "CUDA Error: %s %s %d\n", cudaGetErrorString(_e), __FILE__, __LINE__);       \
      exit(EXIT_FAILURE);                                                                          \
    }                                                                                              \
  } while (0)

void *arena_alloc_cuda(u64 size) {
  void *p = nullptr;
  PB_FATAL(cudaMalloc(&p, size ? size : 1));
  return p;
}
void arena_free_cuda(void *ptr) { PB_FATAL(cudaFree(ptr)); }
// The reference's arena zero-fills EVERY allocation (src/core/arena.c:94-102), also the output of
// a forward op that is about to be overwritten (+4 bytes per element of HBM traffic on top of the
// op's own 8-12) and the gradient twin that src/core/tensor.c:82-90 zeroes again through
// zeros_cuda. The fill is stream-ordered on the library stream, so it never races the kernels
// around it and never stalls the host; and the caller can switch it off around allocations whose
// first use is a full overwrite (plast_b200_arena_fill_policy): gradients are still zeroed, once,
// by zeros_cuda.
static thread_local int t_fill_policy = PLAST_B200_ARENA_FILL;
static std::atomic<unsigned long long> g_fill_bytes{0}, g_fill_skipped_bytes{0};
void arena_memset_cuda(void *ptr, int value, u64 size) {
  if (t_fill_policy == PLAST_B200_ARENA_SKIP_FILL && value == 0) {
    g_fill_skipped_bytes.fetch_add(size, std::memory_order_relaxed);
    return;
  }
  g_fill_bytes.fetch_add(size, std::memory_order_relaxed);
  PB_FATAL(cudaMemsetAsync(ptr, value, size, stream()));
}
void plast_b200_arena_fill_policy(int policy) {
  t_fill_policy = policy == PLAST_B200_ARENA_SKIP_FILL ? PLAST_B200_ARENA_SKIP_FILL : PLAST_B200_ARENA_FILL;
}
void plast_b200_arena_fill_stats(u64 *filled_bytes, u64 *skipped_bytes) {
  if (filled_bytes) *filled_bytes = g_fill_bytes.load(std::memory_order_relaxed);
  if (skipped_bytes) *skipped_bytes = g_fill_skipped_bytes.load(std::memory_order_relaxed);
}
void arena_memcpy_h2d_cuda(void *dest, const void *src, u64 size) {
  PB_FATAL(cudaMemcpyAsync(dest, src, size, cudaMemcpyHostToDevice, stream()));
  PB_FATAL(cudaStreamSynchronize(stream()));
}
void arena_memcpy_d2h_cuda(void *dest, const void *src, u64 size) {
  PB_FATAL(cudaMemcpyAsync(dest, src, size, cudaMemcpyDeviceToHost, stream()));
  PB_FATAL(cudaStreamSynchronize(stream()));
}
void arena_memcpy_d2d_cuda(void *dest, const void *src, u64 size) {
  PB_FATAL(cudaMemcpyAsync(dest, src, size, cudaMemcpyDeviceToDevice, stream()));
}

// ---- backward pieces of the reference's fused GEMM / conv epilogues ---------------------------------
// src/kernels/cuda/matmul_relu.cu:137-150 (launch_relu_grad_modulate_cuda):
// dc[i] = dout[i] * (out[i] > 0 ? 1 : alpha), 128-bit accesses.
void plast_b200_relu_grad_modulate(const float *dout, const float *out_data, float *dc, u64 num_elements,
                                   float alpha) {
  begin_call();
  if (!dout || !out_data || !dc) {
    set_error(PLAST_B200_ERR_NULL, "relu_grad_modulate: NULL pointer");
    return;
  }
  const u64 shape[1] = {num_elements};
  u64 st[3][MAX_NDIM] = {};
  st[0][0] = st[1][0] = st[2][0] = 1;
  IterPlan plan;
  make_plan(&plan, shape, 1, 3, st, nullptr, 0);
  const float *ins[2] = {dout, out_data};
  launch_ew<ReluGradModulate, 2>(plan, dc, ins, ReluGradModulate{alpha});
  end_call();
}
// src/kernels/cuda/matmul_bias_relu.cu:143-151, 219-223: dbias[c] = sum over rows of dc_mod[r, c]
// (the reference zeroes dbias and then issues one float atomic per element; here a deterministic
// tree sum overwrites dbias).
void plast_b200_bias_grad_reduce(const float *dc_mod, float *dbias, u64 num_elements, u64 cols) {
  begin_call();
  if (!dc_mod || !dbias) {
    set_error(PLAST_B200_ERR_NULL, "bias_grad_reduce: NULL pointer");
    return;
  }
  const float *ins[1] = {dc_mod};
  column_sums<CopyF, 1>("bias_grad_reduce", ins, dbias, num_elements, cols, CopyF{});
  end_call();
}
// Both steps in one pass, without the dc_mod buffer (and the cudaMalloc / cudaFree around it,
// matmul_bias_relu.cu:177-179, 226): dbias[c] = sum_r dout[r, c] * (out[r, c] > 0 ? 1 : alpha).
void plast_b200_bias_grad_masked(const float *dout, const float *out_data, float *dbias, u64 num_elements,
                                 u64 cols, float alpha) {
  begin_call();
  if (!dout || !out_data || !dbias) {
    set_error(PLAST_B200_ERR_NULL, "bias_grad_masked: NULL pointer");
    return;
  }
  const float *ins[2] = {dout, out_data};
  column_sums<ReluGradModulate, 2>("bias_grad_masked", ins, dbias, num_elements, cols, ReluGradModulate{alpha});
  end_call();
}

// Strided gather into a contiguous buffer (src/kernels/cuda/cuda_pack.cu:5-27), through the
// elementwise engine so contiguous inner runs move as 128-bit vectors.
void plast_b200_pack(const Tensor *t, void *dst) {
  begin_call();
  if (!check_tensor(t, "pack") || !dst) {
    if (!dst) set_error(PLAST_B200_ERR_NULL, "pack: dst is NULL");
    return;
  }
  u64 st[2][MAX_NDIM] = {};
  u64 s = 1;
  for (u64 d = t->ndim; d-- > 0;) {
    st[0][d] = s;
    s *= t->shape[d];
    st[1][d] = t->strides[d];
  }
  IterPlan plan;
  make_plan(&plan, t->shape, t->ndim, 2, st, nullptr, 0);
  const float *ins[1] = {(const float *)t->data};
  launch_ew<CopyF, 1>(plan, (float *)dst, ins, CopyF{});
  end_call();
}

} // extern "C"

// include/kernels/pack.h:17-23 (C++ linkage in the reference). Contiguous tensors are passed
// through; otherwise a buffer is allocated, filled by the gather and released by ..._release.
struct CudaTensorPack {
  void *data;
  void *_d_buf;
};
void cuda_tensor_pack_init(CudaTensorPack *p, const Tensor *t) {
  p->data = nullptr;
  p->_d_buf = nullptr;
  if (ref_is_contiguous(t)) {
    p->data = t->data;
    return;
  }
  const u64 bytes = numel(t) * sizeof(float);
  if (cudaMalloc(&p->_d_buf, bytes ? bytes : 1) != cudaSuccess) {
    p->_d_buf = nullptr;
    return;
  }
  plast_b200_pack(t, p->_d_buf);
  if (plast_b200_last_error() != PLAST_B200_OK) {
    cudaFree(p->_d_buf);
    p->_d_buf = nullptr;
    return;
  }
  p->data = p->_d_buf;
}
void cuda_tensor_pack_release(CudaTensorPack *p) {
  if (p->_d_buf) {
    cudaFree(p->_d_buf);
    p->_d_buf = nullptr;
  }
  p->data = nullptr;
}
