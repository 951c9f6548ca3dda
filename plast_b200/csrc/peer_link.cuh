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
// Polls allowed per wait. Once a wait of this group has run out (the status word is set) every
// later wait gives up after a few polls: a peer that is gone stays gone, and a step that would
// otherwise spend a second per packet finishes at once with its local values and the status set.
__device__ __forceinline__ unsigned peer_spin_limit(const PeerLink &link) {
  return *(volatile unsigned int *)&link.words[0] != 0u ? 256u : link.max_spins;
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
  const unsigned spin_limit = peer_spin_limit(link);
  for (int p = 0; p < link.world && complete; ++p) {
    const unsigned long long *slot = mine + (size_t)p * PLAST_B200_PEER_MAX_FLOATS;
    unsigned long long got = load_packet(slot);
    unsigned spins = 0;
    while ((unsigned)(got >> 32) != seq) {
      if (++spins > spin_limit) {
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

// The exchange of a STRIP of a multi-output reduction, run by the threads that hold the strip's
// final local values (one thread per VEC consecutive outputs, first output index `elem`): every
// value goes to slot [rank][elem + k] of every peer, then the world's packets for the same
// elements are polled and combined in rank order. All strips of the launch together form ONE call
// of the exchange sequence: every exchanging thread reads the sequence counter, which cannot move
// before peer_exchange_strip_done has been called for all `n_strips` strips of the grid.
template <int VEC>
__device__ __forceinline__ void peer_exchange_strip(const PeerLink &link, float (&v)[VEC], unsigned elem, int op) {
  unsigned seq = *(volatile unsigned int *)&link.words[1] + 1u;
  if (seq == 0u) seq = 2u;
  const size_t parity_base = (size_t)(seq & 1u) * link.world * PLAST_B200_PEER_MAX_FLOATS;
  for (int p = 0; p < link.world; ++p) {
    unsigned long long *dst = link.packets[p] + parity_base + (size_t)link.rank * PLAST_B200_PEER_MAX_FLOATS + elem;
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      store_packet(dst + k, ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v[k]));
  }
  // The VEC packets of one rank are requested together, rank after rank: a thread's chain of
  // dependent round trips is `world` long, as in the stand-alone exchange kernel, not world x VEC
  // (polled one packet at a time the fused column sum took 19 us at eight GPUs against 17 us for
  // reduce + exchange as two kernels).
  const unsigned long long *mine = link.packets[link.rank] + parity_base + elem;
  const unsigned spin_limit = peer_spin_limit(link);
  float acc[VEC];
  bool complete = true;
  for (int p = 0; p < link.world && complete; ++p) {
    const unsigned long long *slot = mine + (size_t)p * PLAST_B200_PEER_MAX_FLOATS;
    unsigned long long got[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) got[k] = load_packet(slot + k);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      unsigned spins = 0;
      while (complete && (unsigned)(got[k] >> 32) != seq) {
        if (++spins > spin_limit) {
          atomicCAS(&link.words[0], 0u, 1u + (unsigned)p);
          complete = false;
          break;
        }
        __nanosleep(64);
        got[k] = load_packet(slot + k);
      }
      const float x = __uint_as_float((unsigned)got[k]);
      acc[k] = p == 0 ? x : peer_combine(op, acc[k], x);
    }
  }
  if (complete) { // a give-up leaves the local values and raises the status word
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = acc[k];
  }
}
// One thread per strip, after every thread of the strip has returned from peer_exchange_strip
// (a barrier in between): the last strip of the grid advances the sequence counter.
__device__ __forceinline__ void peer_exchange_strip_done(const PeerLink &link, unsigned n_strips) {
  unsigned seq = *(volatile unsigned int *)&link.words[1] + 1u;
  if (seq == 0u) seq = 2u;
  __threadfence();
  if (atomicAdd(&link.words[2], 1u) == n_strips - 1) {
    link.words[2] = 0;
    link.words[1] = seq;
  }
}
#endif

// Host side (runtime.cu): an entry point called between arm and disarm hands the link (a device
// pointer) to the first launch of the kind it was armed FOR: the single-output segmented reduction
// of a full reduce, or the streaming cross-entropy kernel (which divides the exchanged sum by
// global_count). A launch of the other kind never takes it: the row-loss reduction behind the
// cross-entropy fallback kernels would otherwise exchange a sum and divide it by the LOCAL row
// count. disarm tells whether a launch took the link.
//
// kPeerEveryReduction is the bracket mode (plast_b200_peer_reduce_begin / _end): EVERY final
// reduction launched while it is armed is combined across the ranks, in launch order, fused into
// the kernel where the kernel shape allows it and by the stand-alone exchange kernel right behind
// the reduction otherwise; the link can be taken any number of times. Reductions that are internal
// steps (the first stage of a two-stage reduction, tie counts, per-row losses) suspend the link
// around themselves.
enum PeerConsumer { kPeerFullReduce = 0, kPeerCrossEntropy = 1, kPeerEveryReduction = 2 };
void arm_peer_link(const PeerLink *device_link, PeerConsumer consumer, float global_count);
bool take_peer_link(PeerConsumer consumer, const PeerLink **out, float *global_count); // true once per armed link
bool disarm_peer_link();                                        // returns whether a launch took it
bool peer_bracket_open();                // armed for kPeerEveryReduction and not suspended
const PeerLink *peer_bracket_take();     // the link of the open bracket; counts one exchange
int peer_bracket_exchanges();            // exchanges made since the bracket was armed
struct PeerSuspend {                     // scope guard: reductions inside are local steps
  PeerSuspend();
  ~PeerSuspend();
};
// peer.cu: one stand-alone exchange of n floats (n <= PLAST_B200_PEER_MAX_FLOATS) at `data` on the
// library stream, through the link in device memory; then dst (+)= data for a parked result.
void launch_peer_exchange(const PeerLink *device_link, float *data, unsigned n, int op);
void launch_add_parked(float *dst, const float *parked, unsigned n, bool accumulate);

} // namespace pb
