// Shared host-side plumbing of libplast_b200: error state, stream, launch accounting, the
// per-device scratch workspace, and small device helpers used by every kernel file.
#pragma once

#include "plast_b200.h"

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace pb {

// ---- error state (thread local; entry points return void like the reference's) ---------------
void set_error(int code, const char *fmt, ...);
void begin_call();                 // clears the error of the previous call on this thread
void note_kernel(const char *name); // remembers the kernel family for plast_b200_last_kernel()
bool failed();

cudaStream_t stream();
void count_launch(int n = 1);
bool sync_enabled(); // plast_b200_set_sync state
void end_call(); // optional device sync (plast_b200_set_sync) + launch error check

#define PB_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess) {                                                                       \
      pb::set_error(PLAST_B200_ERR_CUDA, "CUDA error at %s:%d: '%s': %s", __FILE__, __LINE__,      \
                    #expr, cudaGetErrorString(_e));                                                \
      return;                                                                                      \
    }                                                                                              \
  } while (0)

#define PB_CUDA_RET(expr, ret)                                                                     \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess) {                                                                       \
      pb::set_error(PLAST_B200_ERR_CUDA, "CUDA error at %s:%d: '%s': %s", __FILE__, __LINE__,      \
                    #expr, cudaGetErrorString(_e));                                                \
      return ret;                                                                                  \
    }                                                                                              \
  } while (0)

// ---- per-device scratch ------------------------------------------------------------------------
// Reductions that split one output over several CTAs park their partials here and elect the
// last-arriving CTA (a ticket counter) to combine them. One buffer per device, allocated on
// first use and kept; counters live at the front, start at zero and are reset by the CTA that
// consumes them, so no launch ever needs a memset.
struct Workspace {
  unsigned int *counters; // kCounters tickets
  float *partials;        // kPartialFloats floats
  float *parked;          // kParkedFloats floats: a local result waiting for its cross-GPU exchange
};
constexpr size_t kCounters = 1 << 16;
constexpr size_t kPartialFloats = (size_t)8 << 20; // 32 MiB
constexpr size_t kParkedFloats = 8192;             // = PLAST_B200_PEER_MAX_FLOATS
bool get_workspace(Workspace *ws);

int sm_count();

// Stream-ordered scratch on the library stream (cudaMallocAsync from the device's default pool;
// release with cudaFreeAsync). The first call on a device tells the pool to keep freed memory
// instead of returning it to the driver at the next synchronisation, so that a kernel sequence
// that needs scratch every call (gathering a transposed operand, the argmax of a view) does not
// pay a device allocation each time. plast_b200_release_workspace trims the pool.
cudaError_t scratch_alloc_async(void **p, size_t bytes);

// Geometry knobs a test or a tuning run may override (plast_b200_tune); negative = built-in choice.
enum TuneKey {
  kTuneColsLogTx = 0, kTuneColsCtasPerSm = 1, kTuneColsMinBatches = 2, kTuneSegCtasPerSm = 3, kTuneTinyRowCols = 4,
  kTuneColsTileMajor = 5, kTuneColsPrefetch = 6, kTuneColsPrefetchUntil = 7, kTuneSegPrefetch = 8, kTuneSegLogTx = 9, kTuneColsCluster = 10, kTuneTile3Shape = 11, kTuneKeys = 12
};
long tuned(int key);

// ---- launches ------------------------------------------------------------------------------------
// Kernels in a stream cost ~4 us from the end of one to the start of the next, a tenth of the time a
// 268 MB tensor needs at HBM speed. The streaming kernels of this library are therefore launched
// with programmatic stream serialization: the grid may become resident while its predecessor in the
// stream is still draining, and waits (pdl_wait(), the first statement of every such kernel, before
// any global memory access) until that predecessor has completed and its writes are visible. The
// early start hides launch latency and block scheduling only; ordering of memory is unchanged.
// PLAST_B200_PDL=0 in the environment turns the attribute off (plain stream order).
bool pdl_enabled();

// `cluster` > 1 launches thread-block clusters of that many consecutive CTAs along x (the grid must
// be a multiple of it).
template <class... KArgs, class... Args>
inline cudaError_t launch_kc(unsigned cluster, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t s, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <class... KArgs, class... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                            Args &&...args) {
  return launch_kc(1u, kernel, grid, block, smem, s, static_cast<Args &&>(args)...);
}

// Frees the staging buffers, streams and events of the host-buffer chain (host_pipeline.cu).
void release_host_pipeline();

// Fills n 32-bit words with a bit pattern on the library stream (helpers.cu).
void fill32(void *data, unsigned int pattern, u64 n);

// ---- tensor helpers ------------------------------------------------------------------------------
inline u64 numel(const Tensor *t) {
  u64 n = 1;
  for (u64 i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}
// src/core/tensor.c:32-42: the stride of dim 0 is never examined.
inline bool ref_is_contiguous(const Tensor *t) {
  if (t->ndim == 0) return true;
  u64 expect = 1;
  for (u64 i = t->ndim - 1; i > 0; --i) {
    if (t->strides[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}
bool check_tensor(const Tensor *t, const char *what, bool need_data = true);

} // namespace pb
