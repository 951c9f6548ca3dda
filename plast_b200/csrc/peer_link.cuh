// What a kernel needs to take part in the NVLink packet exchange (include/plast_b200_peer.h): the
// mapped buffers of every rank, this rank's control words, and the one-element exchange a single
// thread can run at the end of a reduction, so that the local reduce and the cross-GPU combine
// are ONE kernel. Protocol and buffer layout are those of peer.cu.
#pragma once

#include "plast_b200_peer.h"

namespace pb {

struct PeerLink {
  unsigned long long *packets[PLAST_B200_PEER_MAX_WORLD]; // every rank's buffer, as mapped here
  unsigned int *words; // [0] status, [1] sequence counter, [2] CTA ticket of the exchange kernel
  int rank, world;
  unsigned max_spins;
};
// Kernels receive a POINTER to the link (in device memory, NULL = no exchange): a by-value copy
// would be indexed dynamically (packets[p]) and end up on every thread's local stack.

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long load_packet(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_packet(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float peer_combine(int op, float a, float b) {
  return op == PLAST_B200_PEER_SUM ? a + b : (op == PLAST_B200_PEER_MAX ? (a > b ? a : b) : (a < b ? a : b));
}

// One exchange of ONE float, run by a single thread of the last CTA of a reduction (the grid has
// nothing else left to do, so nothing waits on this thread but the kernel's end). Counts as one
// call of the exchange sequence: same sequence counter, same slots (element 0), so fused and
// stand-alone exchanges can be mixed as long as every rank makes the same sequence of calls.
// Returns the combined value; on a give-up (bounded wait ran out) records the missing rank in
// words[0] and returns the local value.
__device__ __forceinline__ float peer_exchange_scalar(const PeerLink &link, float v, int op) {
  unsigned seq = link.words[1] + 1u;
  if (seq == 0u) seq = 2u;
  const size_t parity_base = (size_t)(seq & 1u) * link.world * PLAST_B200_PEER_MAX_FLOATS;
  const unsigned long long pkt = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
  for (int p = 0; p < link.world; ++p)
    store_packet(link.packets[p] + parity_base + (size_t)link.rank * PLAST_B200_PEER_MAX_FLOATS, pkt);
  const unsigned long long *mine = link.packets[link.rank] + parity_base;
  float acc = 0.0f;
  bool complete = true;
  for (int p = 0; p < link.world && complete; ++p) {
    const unsigned long long *slot = mine + (size_t)p * PLAST_B200_PEER_MAX_FLOATS;
    unsigned long long got = load_packet(slot);
    unsigned spins = 0;
    while ((unsigned)(got >> 32) != seq) {
      if (++spins > link.max_spins) {
        atomicCAS(&link.words[0], 0u, 1u + (unsigned)p);
        complete = false;
        break;
      }
      __nanosleep(64);
      got = load_packet(slot);
    }
    const float x = __uint_as_float((unsigned)got);
    acc = p == 0 ? x : peer_combine(op, acc, x);
  }
  link.words[1] = seq;
  return complete ? acc : v;
}
#endif

// Host side (runtime.cu): an entry point called between arm and disarm hands the link (a device
// pointer) to the first launch of the kind it was armed FOR: the single-output segmented reduction
// of a full reduce, or the streaming cross-entropy kernel (which divides the exchanged sum by
// global_count). A launch of the other kind never takes it: the row-loss reduction behind the
// cross-entropy fallback kernels would otherwise exchange a sum and divide it by the LOCAL row
// count. disarm tells whether a launch took the link.
enum PeerConsumer { kPeerFullReduce = 0, kPeerCrossEntropy = 1 };
void arm_peer_link(const PeerLink *device_link, PeerConsumer consumer, float global_count);
bool take_peer_link(PeerConsumer consumer, const PeerLink **out, float *global_count); // true once per armed link
bool disarm_peer_link();                                        // returns whether a launch took it

} // namespace pb
