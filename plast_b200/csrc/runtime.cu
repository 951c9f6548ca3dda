// Library state: last-error record, launch stream, launch counter, per-device scratch.
#include "common.cuh"
#include "peer_link.cuh"

#include <atomic>
#include <mutex>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

namespace pb {

namespace {
thread_local int t_err = PLAST_B200_OK;
thread_local char t_msg[512] = "";
thread_local const char *t_kernel = "";
std::atomic<cudaStream_t> g_stream{nullptr};
std::atomic<int> g_sync{0};
std::atomic<unsigned long long> g_launches{0};

constexpr int kMaxDevices = 64;
std::mutex g_ws_mutex;
Workspace g_ws[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
} // namespace

namespace {
thread_local const PeerLink *t_link = nullptr;
thread_local float t_link_count = 0.0f;
thread_local bool t_link_armed = false, t_link_taken = false;
thread_local PeerConsumer t_link_consumer = kPeerFullReduce;
thread_local int t_link_suspended = 0, t_bracket_exchanges = 0;
} // namespace
void arm_peer_link(const PeerLink *device_link, PeerConsumer consumer, float global_count) {
  t_link = device_link;
  t_link_consumer = consumer;
  t_link_count = global_count;
  t_link_armed = true;
  t_link_taken = false;
  t_bracket_exchanges = 0;
}
bool take_peer_link(PeerConsumer consumer, const PeerLink **out, float *global_count) {
  if (!t_link_armed || t_link_taken || consumer != t_link_consumer) return false;
  *out = t_link;
  if (global_count) *global_count = t_link_count;
  t_link_taken = true;
  return true;
}
bool disarm_peer_link() {
  const bool taken = t_link_taken;
  t_link_armed = t_link_taken = false;
  t_link = nullptr;
  return taken;
}
bool peer_bracket_open() { return t_link_armed && t_link_consumer == kPeerEveryReduction && t_link_suspended == 0; }
const PeerLink *peer_bracket_take() {
  t_link_taken = true;
  ++t_bracket_exchanges;
  return t_link;
}
int peer_bracket_exchanges() { return t_bracket_exchanges; }
PeerSuspend::PeerSuspend() { ++t_link_suspended; }
PeerSuspend::~PeerSuspend() { --t_link_suspended; }

void set_error(int code, const char *fmt, ...) {
  if (t_err != PLAST_B200_OK) return; // keep the first error of a call
  t_err = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_msg, sizeof(t_msg), fmt, ap);
  va_end(ap);
  fprintf(stderr, "plast: %s\n", t_msg);
}
void begin_call() {
  t_err = PLAST_B200_OK;
  t_msg[0] = 0;
  t_kernel = "";
}
void note_kernel(const char *name) { t_kernel = name; }
bool failed() { return t_err != PLAST_B200_OK; }
cudaStream_t stream() { return g_stream.load(std::memory_order_relaxed); }
bool sync_enabled() { return g_sync.load(std::memory_order_relaxed) != 0; }
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

void end_call() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(PLAST_B200_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return;
  }
  if (g_sync.load(std::memory_order_relaxed)) {
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess)
      set_error(PLAST_B200_ERR_CUDA, "device synchronize failed: %s", cudaGetErrorString(e));
  }
}

namespace {
std::atomic<long> g_tune[kTuneKeys];
struct TuneInit {
  TuneInit() {
    for (int i = 0; i < kTuneKeys; ++i) g_tune[i].store(-1);
  }
} g_tune_init;
} // namespace
long tuned(int key) { return key >= 0 && key < kTuneKeys ? g_tune[key].load(std::memory_order_relaxed) : -1; }

bool pdl_enabled() {
  static const bool on = [] {
    const char *e = getenv("PLAST_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

cudaError_t scratch_alloc_async(void **p, size_t bytes) {
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && !configured[dev]) {
    cudaMemPool_t pool = nullptr;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
      unsigned long long keep_all = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep_all);
    }
    cudaGetLastError();
    configured[dev] = true;
  }
  return cudaMallocAsync(p, bytes ? bytes : 1, stream());
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

bool get_workspace(Workspace *ws) {
  int dev = 0;
  PB_CUDA_RET(cudaGetDevice(&dev), false);
  if (dev < 0 || dev >= kMaxDevices) {
    set_error(PLAST_B200_ERR_LIMIT, "device ordinal %d beyond %d", dev, kMaxDevices);
    return false;
  }
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  if (!g_ws[dev].counters) {
    void *p = nullptr;
    size_t bytes = kCounters * sizeof(unsigned int) + (kPartialFloats + kParkedFloats) * sizeof(float);
    PB_CUDA_RET(cudaMalloc(&p, bytes), false);
    cudaError_t e = cudaMemset(p, 0, kCounters * sizeof(unsigned int));
    if (e != cudaSuccess) {
      cudaFree(p);
      set_error(PLAST_B200_ERR_CUDA, "workspace memset failed: %s", cudaGetErrorString(e));
      return false;
    }
    g_ws[dev].counters = (unsigned int *)p;
    g_ws[dev].partials = (float *)((char *)p + kCounters * sizeof(unsigned int));
    g_ws[dev].parked = g_ws[dev].partials + kPartialFloats;
  }
  *ws = g_ws[dev];
  return true;
}

bool check_tensor(const Tensor *t, const char *what, bool need_data) {
  if (!t) {
    set_error(PLAST_B200_ERR_NULL, "%s: tensor is NULL", what);
    return false;
  }
  if (t->ndim > MAX_NDIM) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: ndim %llu exceeds %d", what, (unsigned long long)t->ndim,
              MAX_NDIM);
    return false;
  }
  if (need_data && !t->data && numel(t) > 0) {
    set_error(PLAST_B200_ERR_NULL, "%s: data pointer is NULL", what);
    return false;
  }
  return true;
}

} // namespace pb

extern "C" {

int plast_b200_last_error(void) { return pb::t_err; }
const char *plast_b200_last_error_message(void) { return pb::t_msg; }
void plast_b200_clear_error(void) { pb::begin_call(); }
void plast_b200_set_stream(void *s) { pb::g_stream.store((cudaStream_t)s); }
void *plast_b200_get_stream(void) { return (void *)pb::g_stream.load(); }
void plast_b200_set_sync(int on) { pb::g_sync.store(on ? 1 : 0); }
u64 plast_b200_launch_count(void) { return (u64)pb::g_launches.load(); }
const char *plast_b200_last_kernel(void) { return pb::t_kernel; }
const char *plast_b200_version(void) { return "plast_b200 0.1 (sm_100a)"; }

void plast_b200_tune(int key, long value) {
  if (key >= 0 && key < pb::kTuneKeys) pb::g_tune[key].store(value);
}

void plast_b200_release_workspace(void) {
  pb::release_host_pipeline();
  std::lock_guard<std::mutex> lock(pb::g_ws_mutex);
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) return;
  for (int d = 0; d < pb::kMaxDevices; ++d) {
    if (pb::g_ws[d].counters) {
      cudaSetDevice(d);
      cudaMemPool_t pool = nullptr;
      if (cudaDeviceGetDefaultMemPool(&pool, d) == cudaSuccess) {
        cudaDeviceSynchronize();
        cudaMemPoolTrimTo(pool, 0);
      }
      cudaFree(pb::g_ws[d].counters);
      pb::g_ws[d] = pb::Workspace{};
    }
  }
  cudaSetDevice(cur);
}

} // extern "C"
