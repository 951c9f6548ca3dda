// All-reduce of tiny partials over NVLink peer memory: see include/plast_b200_peer.h.
//
// One rank's exchange buffer (the same layout on every rank):
//   packets [2 parities][world slots][kMaxFloats] of 8 bytes: {value bits, sequence number}
// slot r of parity q receives rank r's message of every call whose sequence number has parity q.
// A call with sequence number s: (1) store {value, s} for every element into slot `rank` of
// parity s & 1 of EVERY rank's buffer (one naturally aligned 8-byte store per element and peer:
// it arrives whole, so the packet validates itself and no fence or separate flag is needed),
// (2) for every element poll slot 0 .. world-1 of MY buffer until its packet carries s, and add
// the values in rank order. Two parities are enough: a rank can only begin call s + 2 after
// completing s + 1, which needs every peer's packets of s + 1, which a peer sends only after its
// kernel of call s, and with it all its reads of parity s & 1, has finished.
#include "common.cuh"
#include "peer_link.cuh"

#include <string.h>

namespace pb {

constexpr int kPeerThreads = 1024;
constexpr unsigned kMaxFloats = PLAST_B200_PEER_MAX_FLOATS;
constexpr int kMaxWorld = PLAST_B200_PEER_MAX_WORLD;

// The mapped buffers arrive through a pointer to the group's PeerLink in device memory: a table
// passed by value and indexed with a run-time rank would be copied to every thread's local stack.
__global__ void __launch_bounds__(kPeerThreads)
peer_all_reduce_kernel(const PeerLink *__restrict__ link, float *inout, unsigned n, int op) {
  const int rank = link->rank, world = link->world;
  unsigned int *words = link->words;
  const unsigned max_spins = peer_spin_limit(*link);
  // words[0]: status (set on a give-up), words[1]: sequence counter, words[2]: CTA ticket.
  // The sequence number lives on the device and advances once per launch, so a launch recorded in
  // a CUDA graph stays correct however often the graph is replayed (every rank makes the same
  // sequence of launches, so the counters agree). Every CTA reads the counter when it starts; the
  // CTA that finishes last stores the new value, after all the others have read the old one.
  // 0 is what an empty buffer holds and is skipped.
  unsigned seq = words[1] + 1u;
  if (seq == 0u) seq = 2u; // wrapped: keep the parities alternating
  const size_t parity_base = (size_t)(seq & 1u) * world * kMaxFloats;
  const unsigned i = blockIdx.x * kPeerThreads + threadIdx.x; // one element per thread
  // (1) my message into everybody's buffer
  if (i < n) {
    const unsigned long long pkt = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(inout[i]);
    for (int p = 0; p < world; ++p) store_packet(link->packets[p] + parity_base + (size_t)rank * kMaxFloats + i, pkt);
  }
  // (2) everybody's message out of MY buffer, added in rank order: the same bits on every rank.
  // Every poll loop is bounded; a give-up leaves the element untouched and records the missing rank.
  if (i < n) {
    const unsigned long long *mine = link->packets[rank] + parity_base + i;
    float acc = 0.0f;
    bool complete = true;
    for (int p = 0; p < world && complete; ++p) {
      const unsigned long long *slot = mine + (size_t)p * kMaxFloats;
      unsigned long long pkt = load_packet(slot);
      unsigned spins = 0;
      while ((unsigned)(pkt >> 32) != seq) {
        if (++spins > max_spins) {
          atomicCAS(&words[0], 0u, 1u + (unsigned)p);
          complete = false;
          break;
        }
        __nanosleep(64);
        pkt = load_packet(slot);
      }
      const float v = __uint_as_float((unsigned)pkt);
      acc = p == 0 ? v : peer_combine(op, acc, v);
    }
    if (complete) inout[i] = acc;
  }
  // last CTA out advances the sequence counter and re-arms the ticket
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&words[2], 1u) == gridDim.x - 1) {
      words[2] = 0;
      words[1] = seq;
    }
  }
}

constexpr size_t kBufferBytes = (size_t)2 * kMaxWorld * kMaxFloats * sizeof(unsigned long long);

} // namespace pb

struct PlastPeerGroup {
  int rank, world;
  void *local;                       // this rank's buffer (cudaMalloc)
  void *mapped[pb::kMaxWorld];       // peers' buffers (IPC mappings; mapped[rank] == local)
  bool opened[pb::kMaxWorld];
  void *fake[pb::kMaxWorld];         // test groups: local stand-ins for the other ranks
  unsigned max_spins;
  pb::PeerLink *link_dev;            // the link as kernels see it (device memory), made when connected
  unsigned int *status_dev;          // device words: [0] set by the kernel on a give-up, [1] sequence counter, [2] CTA ticket
  bool connected;
};

using namespace pb;

static PlastPeerGroup *new_group(int rank, int world) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
    set_error(PLAST_B200_ERR_LIMIT, "peer group: rank %d / world %d (at most %d ranks)", rank, world, kMaxWorld);
    return nullptr;
  }
  PlastPeerGroup *g = new PlastPeerGroup();
  memset(g, 0, sizeof(*g));
  g->rank = rank;
  g->world = world;
  g->max_spins = 1u << 23; // polls of ~100 ns each: about a second
  if (cudaMalloc(&g->local, kBufferBytes) != cudaSuccess || cudaMemset(g->local, 0, kBufferBytes) != cudaSuccess ||
      cudaMalloc((void **)&g->status_dev, 4 * sizeof(unsigned int)) != cudaSuccess ||
      cudaMemset(g->status_dev, 0, 4 * sizeof(unsigned int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
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

static PeerLink link_of(const PlastPeerGroup *g) {
  PeerLink link = {};
  for (int r = 0; r < g->world; ++r) link.packets[r] = (unsigned long long *)g->mapped[r];
  link.words = g->status_dev;
  link.rank = g->rank;
  link.world = g->world;
  link.max_spins = g->max_spins;
  return link;
}
// Called once every peer is mapped: the device copy of the link that fused kernels read.
static bool publish_link(PlastPeerGroup *g) {
  const PeerLink link = link_of(g);
  if (!g->link_dev && cudaMalloc((void **)&g->link_dev, sizeof(PeerLink)) != cudaSuccess) return false;
  return cudaMemcpy(g->link_dev, &link, sizeof(PeerLink), cudaMemcpyHostToDevice) == cudaSuccess;
}

__global__ void scale_one_kernel(float *v, float factor) { v[0] = v[0] * factor; }
__global__ void raise_status_kernel(unsigned int *words, unsigned code) { atomicCAS(&words[0], 0u, code); }

__global__ void add_parked_kernel(float *dst, const float *parked, unsigned n, bool accumulate) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = accumulate ? dst[i] + parked[i] : parked[i];
}

namespace pb {
void launch_peer_exchange(const PeerLink *device_link, float *data, unsigned n, int op) {
  if (n == 0) return;
  const unsigned blocks = (n + kPeerThreads - 1) / kPeerThreads; // at most 8, all resident at once
  peer_all_reduce_kernel<<<blocks, kPeerThreads, 0, stream()>>>(device_link, data, n, op);
  count_launch();
}
void launch_add_parked(float *dst, const float *parked, unsigned n, bool accumulate) {
  if (n == 0) return;
  add_parked_kernel<<<(n + 255) / 256, 256, 0, stream()>>>(dst, parked, n, accumulate);
  count_launch();
}
} // namespace pb

// One call of the exchange sequence on the library stream (arguments already checked).
static void launch_exchange(PlastPeerGroup *g, float *data, unsigned n, int op) {
  launch_peer_exchange(g->link_dev, data, n, op);
}
// The local part of a fused call failed on THIS rank (the error is already recorded). The peers
// still make their call of the sequence, so this rank makes it too, with whatever the output
// holds, and raises the group's status word: packets are matched on the sequence number, and a
// rank that skipped a call would leave every later exchange of every rank waiting until it times
// out. The result of this exchange is not valid on any rank; the status word says so.
static void keep_sequence_after_local_failure(PlastPeerGroup *g, Tensor *output, int op) {
  if (!output || !output->data) return;
  raise_status_kernel<<<1, 1, 0, stream()>>>(g->status_dev, (unsigned)PLAST_B200_PEER_STATUS_LOCAL_FAILURE);
  launch_exchange(g, (float *)output->data, 1, op);
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
  if (!publish_link(g)) {
    set_error(PLAST_B200_ERR_CUDA, "peer group connect: cannot store the link on the device");
    return 1;
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
  if (!publish_link(g)) {
    set_error(PLAST_B200_ERR_CUDA, "peer group: cannot store the link on the device");
    plast_b200_peer_group_release(g);
    return nullptr;
  }
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
  launch_exchange(g, data, (unsigned)n, op);
  note_kernel("peer_all_reduce");
  end_call();
}

// Full reduction of this rank's shard AND the exchange of its result in one kernel: the last CTA
// of the local reduction (the one that combines the per-CTA partials) publishes the value to every
// peer, polls for theirs and stores the combined result. Shards the single-output kernel does not
// serve (a few elements, an empty shard) reduce locally and then run the stand-alone exchange, so
// every rank always makes exactly one call of the exchange sequence.
void plast_b200_peer_full_reduce(PlastPeerGroup *g, int op, const Tensor *input, Tensor *output) {
  begin_call();
  if (!g || !input || !output) {
    set_error(PLAST_B200_ERR_NULL, "peer full reduce: NULL argument");
    return;
  }
  if (!g->connected || op < PLAST_B200_PEER_SUM || op > PLAST_B200_PEER_MIN) {
    set_error(PLAST_B200_ERR_UNSUPPORTED, "peer full reduce: group not connected or unknown op %d", op);
    return;
  }
  const Tensor *ins[1] = {input};
  const KernelParams full = {PLAST_FULL_REDUCE, 0, 0.0f};
  arm_peer_link(g->link_dev, kPeerFullReduce, 0.0f);
  if (op == PLAST_B200_PEER_SUM) sum_cuda_forward(ins, output, full);
  else if (op == PLAST_B200_PEER_MAX) max_cuda_forward(ins, output, full);
  else min_cuda_forward(ins, output, full);
  const bool fused = disarm_peer_link();
  if (fused) { // the kernel that took the link made this call of the sequence
    if (!failed()) note_kernel("reduce_seg_with_peer_exchange");
    return;
  }
  if (failed()) {
    keep_sequence_after_local_failure(g, output, op);
    return;
  }
  launch_exchange(g, (float *)output->data, 1, op);
  note_kernel("peer_all_reduce");
  end_call();
}

// Cross-entropy mean over row-sharded logits: this rank's rows go through the streaming
// cross-entropy kernel, whose last CTA exchanges the loss sum and divides by the global row count.
// Layouts that kernel does not take compute the local mean first, turn it back into a sum,
// exchange it with the stand-alone kernel and divide.
void plast_b200_peer_cross_entropy_mean(PlastPeerGroup *g, const Tensor *logits, const Tensor *labels,
                                        Tensor *output, u64 global_rows) {
  begin_call();
  if (!g || !logits || !labels || !output || !output->data) {
    set_error(PLAST_B200_ERR_NULL, "peer cross entropy: NULL argument");
    return;
  }
  if (!g->connected || global_rows == 0 || logits->ndim != 2) {
    set_error(PLAST_B200_ERR_UNSUPPORTED, "peer cross entropy: group not connected, no rows, or logits not [N, C]");
    return;
  }
  const Tensor *ins[2] = {logits, labels};
  const KernelParams none = {0, 0, 0.0f};
  const u64 local_rows = logits->shape[0];
  bool fused = false;
  if (local_rows > 0) {
    arm_peer_link(g->link_dev, kPeerCrossEntropy, (float)global_rows);
    cross_entropy_cuda_forward(ins, output, none);
    fused = disarm_peer_link();
    if (failed()) {
      if (!fused) keep_sequence_after_local_failure(g, output, PLAST_B200_PEER_SUM);
      return;
    }
  } else {
    fill32(output->data, 0u, 1); // an empty shard contributes a zero sum
  }
  if (fused) {
    note_kernel("cross_entropy_rows_with_peer_exchange");
    return;
  }
  if (local_rows > 0) {
    scale_one_kernel<<<1, 1, 0, stream()>>>((float *)output->data, (float)local_rows); // mean -> sum
    count_launch();
  }
  launch_exchange(g, (float *)output->data, 1, PLAST_B200_PEER_SUM);
  scale_one_kernel<<<1, 1, 0, stream()>>>((float *)output->data, 1.0f / (float)global_rows);
  count_launch();
  end_call();
}

// Bracket mode: every final reduction the entry points of this thread launch until _end is combined
// across the ranks (reduce_engine.cuh decides per launch whether the exchange runs inside the
// reduction kernel or right behind it).
void plast_b200_peer_reduce_begin(PlastPeerGroup *g) {
  begin_call();
  if (!g || !g->connected) {
    set_error(g ? PLAST_B200_ERR_UNSUPPORTED : PLAST_B200_ERR_NULL, "peer reduce begin: no connected group");
    return;
  }
  arm_peer_link(g->link_dev, kPeerEveryReduction, 0.0f);
}
int plast_b200_peer_reduce_end(PlastPeerGroup *g) {
  (void)g;
  const int n = peer_bracket_exchanges();
  disarm_peer_link();
  return n;
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
  if (g->link_dev) cudaFree(g->link_dev);
  delete g;
}

} // extern "C"
