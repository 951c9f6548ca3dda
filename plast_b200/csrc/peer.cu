// All-reduce of tiny partials over NVLink peer memory: see include/plast_b200_peer.h.
//
// Layout of one rank's exchange buffer (all ranks use the same layout):
//   data  [2 parities][world slots][kMaxFloats]   slot r of parity q holds rank r's message of
//                                                 every call whose sequence number has parity q
//   flags [2 parities][world]                     flag r of parity q = sequence number of the
//                                                 last message rank r completed into this buffer
// A call with sequence number s: (1) store my message into slot `rank` of parity s&1 of EVERY
// rank's buffer, (2) fence, then store s into flag `rank` of every buffer, (3) wait until all
// `world` flags of MY buffer show s, (4) add the slots of my buffer in rank order. Two parities
// are enough: a rank can only begin call s + 2 after completing s + 1, which needs every peer's
// flag for s + 1, which a peer raises only after it has read everything of call s.
#include "common.cuh"
#include "plast_b200_peer.h"

#include <string.h>

namespace pb {

constexpr int kPeerThreads = 1024;
constexpr unsigned kMaxFloats = PLAST_B200_PEER_MAX_FLOATS;
constexpr int kMaxWorld = PLAST_B200_PEER_MAX_WORLD;

struct PeerPtrs {
  float *data[kMaxWorld];
  unsigned int *flags[kMaxWorld];
};

__device__ __forceinline__ unsigned int load_flag(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_flag(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPeerThreads)
peer_all_reduce_kernel(PeerPtrs peers, int rank, int world, float *inout, unsigned n, unsigned int *seq_counter,
                       int op, unsigned int *status, unsigned max_spins) {
  // The sequence number lives on the device and advances once per launch, so a launch recorded in
  // a CUDA graph stays correct however often the graph is replayed (every rank makes the same
  // sequence of launches, so the counters agree). 0 is what empty flags hold and is skipped.
  __shared__ unsigned seq_shared;
  if (threadIdx.x == 0) {
    unsigned next = *seq_counter + 1u;
    if (next == 0u) next = 2u; // wrapped: keep the parities alternating
    *seq_counter = next;
    seq_shared = next;
  }
  __syncthreads();
  const unsigned seq = seq_shared;
  const unsigned par = seq & 1u;
  const size_t my_slot = ((size_t)par * world + rank) * kMaxFloats;
  // (1) my message into everybody's buffer (plain stores; peer addresses go over NVLink)
  for (unsigned i = threadIdx.x; i < n; i += kPeerThreads) {
    const float v = inout[i];
    for (int p = 0; p < world; ++p) peers.data[p][my_slot + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  // (2) tell everybody it is complete
  if (threadIdx.x < (unsigned)world) store_flag(peers.flags[threadIdx.x] + par * world + rank, seq);
  // (3) wait for everybody's message in MY buffer; every wait is bounded
  __shared__ int gave_up;
  if (threadIdx.x == 0) gave_up = 0;
  __syncthreads();
  if (threadIdx.x < (unsigned)world) {
    const unsigned int *f = peers.flags[rank] + par * world + threadIdx.x;
    unsigned spins = 0;
    while (load_flag(f) != seq) {
      if (++spins > max_spins) {
        atomicCAS(status, 0u, 1u + threadIdx.x); // remember the first rank that never arrived
        gave_up = 1;
        break;
      }
      __nanosleep(256);
    }
  }
  __syncthreads();
  if (gave_up) return; // data stays unreduced; the host reads `status`
  // (4) combine in rank order: the same bits on every rank. L1 may hold lines of an earlier
  // call with this parity, so the slots are read past it.
  const float *mine = peers.data[rank] + (size_t)par * world * kMaxFloats;
  for (unsigned i = threadIdx.x; i < n; i += kPeerThreads) {
    float acc = __ldcg(mine + i);
    for (int p = 1; p < world; ++p) {
      const float v = __ldcg(mine + (size_t)p * kMaxFloats + i);
      acc = op == PLAST_B200_PEER_SUM ? acc + v : (op == PLAST_B200_PEER_MAX ? (acc > v ? acc : v) : (acc < v ? acc : v));
    }
    inout[i] = acc;
  }
}

constexpr size_t kDataBytes = (size_t)2 * kMaxWorld * kMaxFloats * sizeof(float);
constexpr size_t kFlagBytes = (size_t)2 * kMaxWorld * sizeof(unsigned int);
constexpr size_t kBufferBytes = kDataBytes + 256; // flags live after the data, 256-byte aligned

} // namespace pb

struct PlastPeerGroup {
  int rank, world;
  void *local;                       // this rank's buffer (cudaMalloc)
  void *mapped[pb::kMaxWorld];       // peers' buffers (IPC mappings; mapped[rank] == local)
  bool opened[pb::kMaxWorld];
  void *fake[pb::kMaxWorld];         // test groups: local stand-ins for the other ranks
  unsigned max_spins;
  unsigned int *status_dev;          // device words: [0] set by the kernel on a give-up, [1] the sequence counter
  bool connected;
};

using namespace pb;

static PeerPtrs layout(const PlastPeerGroup *g) {
  PeerPtrs p = {};
  for (int r = 0; r < g->world; ++r) {
    p.data[r] = (float *)g->mapped[r];
    p.flags[r] = (unsigned int *)((char *)g->mapped[r] + kDataBytes);
  }
  return p;
}

static PlastPeerGroup *new_group(int rank, int world) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
    set_error(PLAST_B200_ERR_LIMIT, "peer group: rank %d / world %d (at most %d ranks)", rank, world, kMaxWorld);
    return nullptr;
  }
  PlastPeerGroup *g = new PlastPeerGroup();
  memset(g, 0, sizeof(*g));
  g->rank = rank;
  g->world = world;
  g->max_spins = 1u << 22; // x 256 ns sleeps: about a second
  if (cudaMalloc(&g->local, kBufferBytes) != cudaSuccess || cudaMemset(g->local, 0, kBufferBytes) != cudaSuccess ||
      cudaMalloc((void **)&g->status_dev, 2 * sizeof(unsigned int)) != cudaSuccess ||
      cudaMemset(g->status_dev, 0, 2 * sizeof(unsigned int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    set_error(PLAST_B200_ERR_CUDA, "peer group: cannot allocate the exchange buffer: %s",
              cudaGetErrorString(cudaGetLastError()));
    if (g->local) cudaFree(g->local);
    if (g->status_dev) cudaFree(g->status_dev);
    delete g;
    return nullptr;
  }
  g->mapped[rank] = g->local;
  return g;
}

extern "C" {

PlastPeerGroup *plast_b200_peer_group_begin(int rank, int world, unsigned char handle[PLAST_B200_IPC_HANDLE_BYTES]) {
  begin_call();
  static_assert(sizeof(cudaIpcMemHandle_t) == PLAST_B200_IPC_HANDLE_BYTES, "IPC handle size");
  if (!handle) {
    set_error(PLAST_B200_ERR_NULL, "peer group: handle is NULL");
    return nullptr;
  }
  PlastPeerGroup *g = new_group(rank, world);
  if (!g) return nullptr;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, g->local) != cudaSuccess) {
    set_error(PLAST_B200_ERR_CUDA, "peer group: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
    plast_b200_peer_group_release(g);
    return nullptr;
  }
  memcpy(handle, &h, sizeof(h));
  return g;
}

int plast_b200_peer_group_connect(PlastPeerGroup *g, const unsigned char *all_handles) {
  begin_call();
  if (!g || !all_handles) {
    set_error(PLAST_B200_ERR_NULL, "peer group connect: NULL argument");
    return 1;
  }
  for (int r = 0; r < g->world; ++r) {
    if (r == g->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, all_handles + (size_t)r * PLAST_B200_IPC_HANDLE_BYTES, sizeof(h));
    if (cudaIpcOpenMemHandle(&g->mapped[r], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      set_error(PLAST_B200_ERR_CUDA, "peer group connect: cannot map the buffer of rank %d: %s", r,
                cudaGetErrorString(cudaGetLastError()));
      return 1;
    }
    g->opened[r] = true;
  }
  g->connected = true;
  return 0;
}

PlastPeerGroup *plast_b200_peer_group_local(int world, unsigned max_spins) {
  begin_call();
  PlastPeerGroup *g = new_group(0, world);
  if (!g) return nullptr;
  for (int r = 1; r < world; ++r) {
    if (cudaMalloc(&g->fake[r], kBufferBytes) != cudaSuccess || cudaMemset(g->fake[r], 0, kBufferBytes) != cudaSuccess) {
      set_error(PLAST_B200_ERR_CUDA, "peer group: cannot allocate a stand-in buffer");
      plast_b200_peer_group_release(g);
      return nullptr;
    }
    g->mapped[r] = g->fake[r];
  }
  cudaDeviceSynchronize();
  g->max_spins = max_spins ? max_spins : 1u;
  g->connected = true;
  return g;
}

void plast_b200_peer_all_reduce(PlastPeerGroup *g, float *data, u64 n, int op) {
  begin_call();
  if (!g || !data) {
    set_error(PLAST_B200_ERR_NULL, "peer all-reduce: NULL argument");
    return;
  }
  if (!g->connected) {
    set_error(PLAST_B200_ERR_UNSUPPORTED, "peer all-reduce: the group is not connected");
    return;
  }
  if (n > kMaxFloats || op < PLAST_B200_PEER_SUM || op > PLAST_B200_PEER_MIN) {
    set_error(PLAST_B200_ERR_LIMIT, "peer all-reduce: %llu floats (limit %u) / op %d", (unsigned long long)n,
              kMaxFloats, op);
    return;
  }
  if (n == 0) return;
  peer_all_reduce_kernel<<<1, kPeerThreads, 0, stream()>>>(layout(g), g->rank, g->world, data, (unsigned)n,
                                                           g->status_dev + 1, op, g->status_dev, g->max_spins);
  count_launch();
  note_kernel("peer_all_reduce");
  end_call();
}

int plast_b200_peer_group_status(PlastPeerGroup *g) {
  if (!g) return -1;
  unsigned int s = 0;
  if (cudaStreamSynchronize(stream()) != cudaSuccess ||
      cudaMemcpy(&s, g->status_dev, sizeof(s), cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  return (int)s;
}

void plast_b200_peer_group_clear_status(PlastPeerGroup *g) {
  if (g) cudaMemsetAsync(g->status_dev, 0, sizeof(unsigned int), stream());
}

void plast_b200_peer_group_release(PlastPeerGroup *g) {
  if (!g) return;
  cudaStreamSynchronize(stream());
  for (int r = 0; r < g->world; ++r) {
    if (g->opened[r]) cudaIpcCloseMemHandle(g->mapped[r]);
    if (g->fake[r]) cudaFree(g->fake[r]);
  }
  if (g->local) cudaFree(g->local);
  if (g->status_dev) cudaFree(g->status_dev);
  delete g;
}

} // extern "C"
