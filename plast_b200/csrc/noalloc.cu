// sum_axis0_noalloc_cuda_forward: the column sum (reduce over axis 0 of a contiguous [rows, cols]
// fp32 matrix — the shape of a bias / broadcast gradient) for callers that must not allocate.
//
// Who needs this: code that runs where cudaMalloc is forbidden or fatal — a caller that has
// already handed all device memory to its own arena (plast's data arena grabs its capacity up
// front, src/core/arena.c:7-27), a latency-critical serving loop that must never hit the
// allocator's device-wide synchronisation, or a host thread that is inside a region where
// allocation calls are rejected. The regular reductions of this library keep their split-K
// partials in a workspace obtained with cudaMalloc on first use; this variant keeps them in a
// fixed array that is part of the library image instead.
//
// The price is a hard size limit and shared state:
//   * cols <= kNoAllocMaxCols (16384) and rows < 2^31; larger inputs are rejected with
//     PLAST_B200_ERR_LIMIT and nothing is launched;
//   * every GPU that uses the library holds the ~1 MiB array until the process exits. With CUDA's
//     default lazy module loading the driver claims that memory when the array is first touched,
//     which is the first call of this entry point on the device, not the moment the library is
//     loaded. A caller that is about to hand ALL device memory to its own arena must therefore
//     make one call (any small input will do) BEFORE that grab, or run with
//     CUDA_MODULE_LOADING=EAGER; afterwards no call needs memory from the driver;
//   * all calls on a device share the array and it keeps the previous call's contents: the ticket
//     counters are cleared at the start of every call, partials are always written before they
//     are read. Two calls whose kernels overlap on the GPU (different streams) race on it — issue
//     them on one stream;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress). Make that first call outside any stream capture.
// No cudaMalloc, cudaFree or other allocating call is made here.
#include "common.cuh"

namespace pb {

constexpr int kNoAllocMaxCols = 16384;
constexpr int kNoAllocMaxSplits = 16;
constexpr int kNoAllocThreads = 256;
constexpr int kNoAllocStripCols = kNoAllocThreads * 4;                   // float4 per thread
constexpr int kNoAllocMaxStrips = kNoAllocMaxCols / kNoAllocStripCols;   // 16
constexpr size_t kNoAllocCounterBytes = 256;                             // >= kNoAllocMaxStrips tickets
constexpr size_t kNoAllocScratchBytes =
    kNoAllocCounterBytes + (size_t)kNoAllocMaxSplits * kNoAllocMaxCols * sizeof(float); // 1 MiB + 256 B

// Ticket counters (first 256 bytes) followed by partials[split][col]. In host code this name is
// only a handle for cudaGetSymbolAddress; kernels receive the looked-up device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// One CTA sums rows [r0, r1) of a 1024-column strip; each thread owns 4 adjacent columns.
__global__ void __launch_bounds__(kNoAllocThreads)
sum_axis0_noalloc_kernel(const float *__restrict__ x, float *__restrict__ out, unsigned rows,
                         unsigned cols, unsigned splits, unsigned char *scratch) {
  unsigned int *counters = reinterpret_cast<unsigned int *>(scratch);
  float *partials = reinterpret_cast<float *>(scratch + kNoAllocCounterBytes);
  const unsigned strip = blockIdx.x, split = blockIdx.y;
  const unsigned col = strip * kNoAllocStripCols + threadIdx.x * 4;
  const unsigned per = (rows + splits - 1) / splits;
  const unsigned r0 = split * per;
  const unsigned r1 = r0 + per < rows ? r0 + per : rows;
  const bool vec = (cols & 3u) == 0 && ((uintptr_t)x & 15u) == 0;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (col < cols) {
    if (vec) { // whole float4 inside the row (cols % 4 == 0 and col % 4 == 0)
      const float4 *p = reinterpret_cast<const float4 *>(x + (size_t)r0 * cols + col);
      const size_t step = cols / 4;
      unsigned r = r0;
      for (; r + 4 <= r1; r += 4) { // four independent loads in flight
        const float4 a = __ldcs(p), b = __ldcs(p + step), c = __ldcs(p + 2 * step), d = __ldcs(p + 3 * step);
        p += 4 * step;
        acc[0] += (a.x + b.x) + (c.x + d.x);
        acc[1] += (a.y + b.y) + (c.y + d.y);
        acc[2] += (a.z + b.z) + (c.z + d.z);
        acc[3] += (a.w + b.w) + (c.w + d.w);
      }
      for (; r < r1; ++r) {
        const float4 a = __ldcs(p);
        p += step;
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      }
    } else {
      for (unsigned r = r0; r < r1; ++r)
        for (int k = 0; k < 4; ++k)
          if (col + k < cols) acc[k] += x[(size_t)r * cols + col + k];
    }
  }
  if (splits == 1) {
    if (col < cols)
      for (int k = 0; k < 4; ++k)
        if (col + k < cols) out[col + k] = acc[k];
    return;
  }
  if (col < cols)
    for (int k = 0; k < 4; ++k)
      if (col + k < cols) partials[(size_t)split * kNoAllocMaxCols + col + k] = acc[k];
  // last CTA of this strip to arrive adds the partials in split order (reproducible)
  __shared__ bool is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[strip], 1u) == splits - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (col < cols)
    for (int k = 0; k < 4; ++k)
      if (col + k < cols) {
        float s = 0.0f;
        for (unsigned c = 0; c < splits; ++c) s += __ldcg(&partials[(size_t)c * kNoAllocMaxCols + col + k]);
        out[col + k] = s;
      }
}

// Device address of the scratch array, looked up once per device with that device current.
static unsigned char *noalloc_scratch_address() {
  constexpr int kMaxDevices = 64;
  static unsigned char *addr[kMaxDevices] = {};
  int dev = 0;
  PB_CUDA_RET(cudaGetDevice(&dev), nullptr);
  if (dev < 0 || dev >= kMaxDevices) {
    set_error(PLAST_B200_ERR_LIMIT, "sum_axis0_noalloc: device ordinal %d beyond %d", dev, kMaxDevices);
    return nullptr;
  }
  if (!addr[dev]) {
    void *p = nullptr;
    PB_CUDA_RET(cudaGetSymbolAddress(&p, g_noalloc_scratch), nullptr);
    addr[dev] = static_cast<unsigned char *>(p);
  }
  return addr[dev];
}

} // namespace pb

using namespace pb;

extern "C" void sum_axis0_noalloc_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  const char *name = "sum_axis0_noalloc";
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name)) return;
  const Tensor *a = inputs[0];
  if (a->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", name, (int)a->dtype);
    return;
  }
  if (a->ndim != 2 || params.dim != 0 || a->strides[1] != 1 || a->strides[0] != a->shape[1]) {
    set_error(PLAST_B200_ERR_UNSUPPORTED,
              "%s: needs a contiguous 2-D tensor and dim 0 (use sum_cuda_forward otherwise)", name);
    return;
  }
  const u64 rows = a->shape[0], cols = a->shape[1];
  if (cols > (u64)kNoAllocMaxCols || rows > 0x7fffffffull) {
    set_error(PLAST_B200_ERR_LIMIT,
              "%s: %llu x %llu exceeds the built-in scratch (at most %d columns, fewer than 2^31 rows)",
              name, (unsigned long long)rows, (unsigned long long)cols, kNoAllocMaxCols);
    return;
  }
  // same output metadata as sum_cuda_forward (src/kernels/cpu/reduce_ops.c:80-81)
  if (params.keepdim) {
    output->ndim = 2;
    output->shape[0] = 1; output->shape[1] = cols;
    output->strides[0] = cols; output->strides[1] = 1;
  } else {
    output->ndim = 1;
    output->shape[0] = cols;
    output->strides[0] = 1;
  }
  if (cols == 0) return;
  if (rows == 0) {
    // nothing to add: every column sum is the start value of the CPU loop, 0
    // (src/kernels/cpu/reduce_ops.c:53), exactly what sum_cuda_forward stores for an empty input
    PB_CUDA(cudaMemsetAsync(output->data, 0, cols * sizeof(float), stream()));
    end_call();
    return;
  }
  unsigned char *scratch = noalloc_scratch_address();
  if (!scratch) return;
  const unsigned strips = (unsigned)((cols + kNoAllocStripCols - 1) / kNoAllocStripCols);
  // enough CTAs to fill the GPU, at least 64 rows each, at most kNoAllocMaxSplits partial rows
  u64 splits = ((u64)sm_count() * 4 + strips - 1) / strips;
  if (splits > rows / 64) splits = rows / 64;
  if (splits > (u64)kNoAllocMaxSplits) splits = kNoAllocMaxSplits;
  if (splits < 1) splits = 1;
  cudaStream_t s = stream();
  if (splits > 1) PB_CUDA(cudaMemsetAsync(scratch, 0, kNoAllocCounterBytes, s)); // tickets start at zero
  sum_axis0_noalloc_kernel<<<dim3(strips, (unsigned)splits), kNoAllocThreads, 0, s>>>(
      (const float *)a->data, (float *)output->data, (unsigned)rows, (unsigned)cols, (unsigned)splits, scratch);
  count_launch();
  note_kernel("sum_axis0_noalloc");
  end_call();
}
