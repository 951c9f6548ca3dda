// Host-buffer form of the fused chain: inputs and output live in (pinned) host memory.
//
// A caller that holds its data on the host pays PCIe for 8-12 bytes per element, ~100x the HBM
// time of the kernel, so the only thing that matters is keeping both directions of the link busy
// at once. The work is cut into chunks; chunk c is copied in on one side stream while chunk c-1
// runs on the library stream and chunk c-2 is copied out on a second side stream (three staging
// slots on the device, reused round-robin under events). With n floats per operand the step then
// costs max(bytes in, bytes out) / link rate instead of their sum.
#include "common.cuh"

#include <mutex>

namespace pb {
namespace {

constexpr int kSlots = 3;
constexpr u64 kChunkElems = (u64)8 << 20; // 32 MiB per operand per slot

struct HostPipe {
  bool ready = false;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, in_done[kSlots] = {}, kernel_done[kSlots] = {}, out_done[kSlots] = {};
  float *staging = nullptr; // kSlots x (PLAST_CHAIN_MAX_INPUTS + 1) x kChunkElems floats, grown on demand
  int staged_operands = 0;
  float *constants = nullptr; // one float per operand, for one-element inputs
};
constexpr int kMaxDevices = 64;
std::mutex g_pipe_mutex;
HostPipe g_pipe[kMaxDevices];

void destroy(HostPipe &p) {
  if (p.staging) cudaFree(p.staging);
  if (p.constants) cudaFree(p.constants);
  if (p.in) cudaStreamDestroy(p.in);
  if (p.out) cudaStreamDestroy(p.out);
  if (p.start) cudaEventDestroy(p.start);
  for (int s = 0; s < kSlots; ++s) {
    if (p.in_done[s]) cudaEventDestroy(p.in_done[s]);
    if (p.kernel_done[s]) cudaEventDestroy(p.kernel_done[s]);
    if (p.out_done[s]) cudaEventDestroy(p.out_done[s]);
  }
  p = HostPipe{};
}

HostPipe *get_pipe(int operands) {
  int dev = 0;
  PB_CUDA_RET(cudaGetDevice(&dev), nullptr);
  if (dev < 0 || dev >= kMaxDevices) {
    set_error(PLAST_B200_ERR_LIMIT, "device ordinal %d beyond %d", dev, kMaxDevices);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_pipe_mutex);
  HostPipe &p = g_pipe[dev];
  if (!p.ready) {
    // non-blocking: the library stream may be the legacy default stream, which would otherwise
    // serialise with every other stream
    PB_CUDA_RET(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking), nullptr);
    PB_CUDA_RET(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking), nullptr);
    PB_CUDA_RET(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming), nullptr);
    for (int s = 0; s < kSlots; ++s) {
      PB_CUDA_RET(cudaEventCreateWithFlags(&p.in_done[s], cudaEventDisableTiming), nullptr);
      PB_CUDA_RET(cudaEventCreateWithFlags(&p.kernel_done[s], cudaEventDisableTiming), nullptr);
      PB_CUDA_RET(cudaEventCreateWithFlags(&p.out_done[s], cudaEventDisableTiming), nullptr);
    }
    PB_CUDA_RET(cudaMalloc(&p.constants, PLAST_CHAIN_MAX_INPUTS * sizeof(float)), nullptr);
    p.ready = true;
  }
  if (p.staged_operands < operands) {
    if (p.staging) {
      PB_CUDA_RET(cudaDeviceSynchronize(), nullptr);
      cudaFree(p.staging);
      p.staging = nullptr;
      p.staged_operands = 0;
    }
    PB_CUDA_RET(cudaMalloc(&p.staging, (size_t)kSlots * operands * kChunkElems * sizeof(float)), nullptr);
    p.staged_operands = operands;
  }
  return &p;
}

} // namespace

void release_host_pipeline() {
  std::lock_guard<std::mutex> lock(g_pipe_mutex);
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) return;
  for (int d = 0; d < kMaxDevices; ++d)
    if (g_pipe[d].ready) {
      cudaSetDevice(d);
      cudaDeviceSynchronize();
      destroy(g_pipe[d]);
    }
  cudaSetDevice(cur);
}

} // namespace pb

using namespace pb;

extern "C" void plast_b200_chain_forward_host(const float *const *host_inputs, const u64 *input_elems,
                                              int n_inputs, float *host_output, u64 n,
                                              const PlastChainStep *steps, int n_steps) {
  begin_call();
  if (!host_inputs || !input_elems || !host_output || !steps) {
    set_error(PLAST_B200_ERR_NULL, "chain (host buffers): NULL argument");
    return;
  }
  if (n_inputs < 1 || n_inputs > PLAST_CHAIN_MAX_INPUTS) {
    set_error(PLAST_B200_ERR_LIMIT, "chain (host buffers): %d inputs (limit %d)", n_inputs, PLAST_CHAIN_MAX_INPUTS);
    return;
  }
  int n_streamed = 0;
  for (int a = 0; a < n_inputs; ++a) {
    if (!host_inputs[a] || (input_elems[a] != n && input_elems[a] != 1)) {
      set_error(PLAST_B200_ERR_SHAPE, "chain (host buffers): input %d must hold %llu elements or 1", a,
                (unsigned long long)n);
      return;
    }
    n_streamed += input_elems[a] == n && n != 1;
  }
  if (n == 0) return;
  HostPipe *p = get_pipe(n_streamed + 1);
  if (!p) return;
  cudaStream_t lib = stream();
  // everything already queued on the library stream (an earlier call may still use the slots)
  PB_CUDA(cudaEventRecord(p->start, lib));
  PB_CUDA(cudaStreamWaitEvent(p->in, p->start, 0));
  PB_CUDA(cudaStreamWaitEvent(p->out, p->start, 0));
  // one-element operands travel once
  Tensor in_t[PLAST_CHAIN_MAX_INPUTS] = {};
  const Tensor *in_ptr[PLAST_CHAIN_MAX_INPUTS];
  int slot_of_input[PLAST_CHAIN_MAX_INPUTS];
  for (int a = 0, k = 0; a < n_inputs; ++a) {
    in_t[a].dtype = FLOAT32;
    in_t[a].device = CUDA;
    in_ptr[a] = &in_t[a];
    if (input_elems[a] == n && n != 1) {
      slot_of_input[a] = k++;
      in_t[a].ndim = 1;
      in_t[a].strides[0] = 1;
    } else {
      slot_of_input[a] = -1;
      in_t[a].ndim = 0;
      in_t[a].data = p->constants + a;
      PB_CUDA(cudaMemcpyAsync(p->constants + a, host_inputs[a], sizeof(float), cudaMemcpyHostToDevice, p->in));
    }
  }
  const int operands = n_streamed + 1;
  const u64 n_chunks = (n + kChunkElems - 1) / kChunkElems;
  Tensor out_t = {};
  out_t.dtype = FLOAT32;
  out_t.device = CUDA;
  out_t.ndim = 1;
  out_t.strides[0] = 1;
  for (u64 c = 0; c < n_chunks; ++c) {
    const int slot = (int)(c % kSlots);
    const u64 begin = c * kChunkElems;
    const u64 len = n - begin < kChunkElems ? n - begin : kChunkElems;
    float *base = p->staging + (size_t)slot * operands * kChunkElems;
    // copy in: the slot's operand buffers are free once the kernel of chunk c - kSlots has run
    if (c >= kSlots) PB_CUDA(cudaStreamWaitEvent(p->in, p->kernel_done[slot], 0));
    for (int a = 0; a < n_inputs; ++a) {
      if (slot_of_input[a] < 0) continue;
      float *dst = base + (size_t)slot_of_input[a] * kChunkElems;
      PB_CUDA(cudaMemcpyAsync(dst, host_inputs[a] + begin, len * sizeof(float), cudaMemcpyHostToDevice, p->in));
      in_t[a].data = dst;
      in_t[a].shape[0] = len;
    }
    PB_CUDA(cudaEventRecord(p->in_done[slot], p->in));
    // compute on the library stream: needs the inputs, and the slot's result buffer copied out
    PB_CUDA(cudaStreamWaitEvent(lib, p->in_done[slot], 0));
    if (c >= kSlots) PB_CUDA(cudaStreamWaitEvent(lib, p->out_done[slot], 0));
    out_t.data = base + (size_t)n_streamed * kChunkElems;
    out_t.shape[0] = len;
    plast_b200_chain_forward(in_ptr, n_inputs, &out_t, steps, n_steps);
    if (failed()) break; // nothing was launched for this chunk; earlier chunks drain normally
    PB_CUDA(cudaEventRecord(p->kernel_done[slot], lib));
    // copy out
    PB_CUDA(cudaStreamWaitEvent(p->out, p->kernel_done[slot], 0));
    PB_CUDA(cudaMemcpyAsync(host_output + begin, out_t.data, len * sizeof(float), cudaMemcpyDeviceToHost, p->out));
    PB_CUDA(cudaEventRecord(p->out_done[slot], p->out));
  }
  // the library stream is done when the last copies out are: the caller synchronises one stream
  const int err = plast_b200_last_error();
  for (int s = 0; s < kSlots && (u64)s < n_chunks; ++s) cudaStreamWaitEvent(lib, p->out_done[s], 0);
  if (err == PLAST_B200_OK) note_kernel("chain_host_pipeline");
}
