// Reduction engine: out[kept coords] (+)= reduce over the reduced dims of pro(in0 .. inN-1).
//
// One engine serves the axis / full reductions (sum, mean, max, min, argmax) and the
// broadcast-gradient reduce of the binary backward (a sum whose prologue computes the gradient
// term on the fly). The canonical plan (iter.h) is ordered by the streamed input's strides, so
// "dim 0" is the dim that is contiguous in memory; three kernel shapes cover every plan:
//
//   rows  dim 0 is reduced and is the only reduced dim: a (sub)warp per output walks its
//         contiguous run with 128-bit loads and combines with shuffles.
//   seg   dim 0 is reduced and either more reduced dims exist (N,H,W of an NCHW bias gradient)
//         or there are too few outputs to fill 148 SMs (a full reduction is the extreme case):
//         the reduction of one output is cut into segments; a CTA takes a chunk of segments;
//         chunks are combined by the last-arriving CTA (ticket counter) in a fixed order.
//   cols  dim 0 is kept: a CTA owns a 32*VEC-wide strip of outputs, its 8 warps stride over
//         the reduced dims (every load is a full coalesced row), partial strips are combined
//         in shared memory and, when the reduction is also split over CTAs, by ticket.
//
// No float atomics anywhere: results are bit-reproducible from run to run (the reference's
// atomicAdd / omp-atomic order is not, src/kernels/cuda/binary_ops.cu:85-89).
#pragma once

#include "common.cuh"
#include "ew_kernel_device.cuh" // pdl_wait / pdl_launch_dependents
#include "iter.h"
#include "peer_link.cuh"

#include <cooperative_groups.h>
#include <float.h>
#include <type_traits>
#include <string.h>

namespace pb {

constexpr int kRedThreads = 256;

// ---- combine operators ----------------------------------------------------------------------------
struct SumOp {
  using T = float;
  using Out = float;
  static constexpr bool kIndexed = false;
  static constexpr int kPeerOp = PLAST_B200_PEER_SUM; // combine of the cross-GPU exchange (-1: none)
  __device__ __forceinline__ static T identity() { return 0.0f; }
  __device__ __forceinline__ static T step(T acc, float v, unsigned) { return acc + v; }
  __device__ __forceinline__ static T combine(T a, T b) { return a + b; }
  __device__ __forceinline__ static T shfl_xor(T v, int m, int w) {
    return __shfl_xor_sync(0xffffffffu, v, m, w);
  }
  __device__ __forceinline__ static T load_cg(const T *p) { return __ldcg(p); }
  __device__ __forceinline__ static void store(Out *o, T v, bool acc, float div) {
    if (div > 0.0f) v = v / div;
    *o = acc ? *o + v : v;
  }
};
// src/kernels/cpu/reduce_ops.c:9-10, 273-278: start at -/+FLT_MAX, keep acc unless strictly beaten.
// For ordinary values `acc > v ? acc : v` and fmaxf(acc, v) are the same number, and fmaxf is one
// instruction instead of a compare and a select. They differ for NaN (the reference's result then
// depends on WHERE in its sequential walk the NaN sits, which no tree order can reproduce) and for
// the sign of a zero maximum (likewise position-dependent there); neither is part of the contract.
struct MaxOp {
  using T = float;
  using Out = float;
  static constexpr bool kIndexed = false;
  static constexpr int kPeerOp = PLAST_B200_PEER_MAX;
  __device__ __forceinline__ static T identity() { return -FLT_MAX; }
  __device__ __forceinline__ static T step(T acc, float v, unsigned) { return fmaxf(acc, v); }
  __device__ __forceinline__ static T combine(T a, T b) { return fmaxf(a, b); }
  __device__ __forceinline__ static T shfl_xor(T v, int m, int w) {
    return __shfl_xor_sync(0xffffffffu, v, m, w);
  }
  __device__ __forceinline__ static T load_cg(const T *p) { return __ldcg(p); }
  __device__ __forceinline__ static void store(Out *o, T v, bool, float) { *o = v; }
};
struct MinOp {
  using T = float;
  using Out = float;
  static constexpr bool kIndexed = false;
  static constexpr int kPeerOp = PLAST_B200_PEER_MIN;
  __device__ __forceinline__ static T identity() { return FLT_MAX; }
  __device__ __forceinline__ static T step(T acc, float v, unsigned) { return fminf(acc, v); }
  __device__ __forceinline__ static T combine(T a, T b) { return fminf(a, b); }
  __device__ __forceinline__ static T shfl_xor(T v, int m, int w) {
    return __shfl_xor_sync(0xffffffffu, v, m, w);
  }
  __device__ __forceinline__ static T load_cg(const T *p) { return __ldcg(p); }
  __device__ __forceinline__ static void store(Out *o, T v, bool, float) { *o = v; }
};
// Maximum with the position of its first occurrence (lowest index wins ties), any visiting order.
struct ArgMaxOp {
  struct T {
    float v;
    unsigned int i;
  };
  using Out = int;
  static constexpr bool kIndexed = true;
  static constexpr int kPeerOp = -1;
  __device__ __forceinline__ static T identity() { return T{-INFINITY, 0xffffffffu}; }
  // a thread visits its elements in increasing index order, so only a strictly greater value
  // replaces the running best
  __device__ __forceinline__ static T step(T acc, float v, unsigned i) {
    return (v > acc.v || acc.i == 0xffffffffu) ? T{v, i} : acc;
  }
  __device__ __forceinline__ static T combine(T a, T b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
  }
  __device__ __forceinline__ static T shfl_xor(T v, int m, int w) {
    T r;
    r.v = __shfl_xor_sync(0xffffffffu, v.v, m, w);
    r.i = __shfl_xor_sync(0xffffffffu, v.i, m, w);
    return r;
  }
  __device__ __forceinline__ static T load_cg(const T *p) {
    return T{__ldcg(&p->v), __ldcg(&p->i)};
  }
  __device__ __forceinline__ static void store(Out *o, T v, bool, float) { *o = (int)v.i; }
};
// Counts elements equal to a per-output target value (tie count of the max/min backward).
struct IdentityPro {
  __device__ __forceinline__ float operator()(const float *x) const { return x[0]; }
};

// ---- kernel parameters ------------------------------------------------------------------------------
// A sub-space is a list of dims (innermost first) with, per dim, its size and the element
// stride of the target and of every input.
template <int NIN> struct SubSpace {
  int n;
  u64 size[MAX_NDIM];
  u64 tstride[MAX_NDIM];
  u64 istride[NIN][MAX_NDIM];

  // Decodes a flat index into offsets (added to toff / ioff).
  __device__ __forceinline__ void offsets(u64 flat, u64 *toff, u64 *ioff) const {
#pragma unroll
    for (int d = 0; d < MAX_NDIM; ++d) {
      if (d >= n) break;
      u64 q, r;
      if (d == n - 1) {
        q = 0;
        r = flat;
      } else {
        q = flat / size[d];
        r = flat - q * size[d];
      }
      *toff += r * tstride[d];
#pragma unroll
      for (int a = 0; a < NIN; ++a) ioff[a] += r * istride[a][d];
      flat = q;
    }
  }
};

template <int NIN> struct RedParams {
  const float *in[NIN];
  void *out;
  SubSpace<NIN> kept;    // rows/seg: every kept dim; cols: kept dims other than dim 0
  SubSpace<NIN> red;     // rows/seg: reduced dims other than dim 0; cols: every reduced dim
  u64 n_kept;            // product of kept.size
  u64 n_red;             // product of red.size
  u64 len0;              // length of dim 0 in ITEMS (vectors of VEC elements)
  u64 tstride0;          // target stride along dim 0 (cols only)
  u64 istride0[NIN];     // per-ITEM input stride along dim 0 (0 = broadcast)
  unsigned vec_mask;     // bit a: input a is vector-loaded along dim 0
  int log_tx;            // threads per row-worker = 1 << log_tx
  u64 seg_len;           // seg: items per segment of dim 0
  u64 nsplit0;           // seg: segments per run of dim 0
  u64 nseg;              // seg: segments per output = nsplit0 * n_red
  u64 per_chunk;         // seg: segments per chunk; cols: reduced indices per chunk
  unsigned splits;       // chunks per output (tile); 1 = direct store
  bool accumulate;
  float post_div;
  unsigned int *counters;
  void *partials;
  const PeerLink *peer; // not NULL: the thread that holds the single final value exchanges it across GPUs
  unsigned cluster;     // cols: > 1 = the `splits` CTAs of a tile are one thread-block cluster and combine
                        // through distributed shared memory (no partials in global memory, no ticket)
  unsigned outers_per_cta; // cols: > 1 = the kept run along dim 0 is shorter than the strip and the lanes of
                        // a CTA cover this many consecutive outer kept indices (no split: splits == 1)
  bool strip_major;     // cols: consecutive CTAs take neighbouring strips of the same chunk of rows
  unsigned prefetch_batches; // cols: load batches ahead of which a row-worker asks L2 for its rows (0 = off)
  unsigned prefetch_until;   // cols: only the first so many batches of a chunk prefetch (0 = all of them)
  unsigned seg_prefetch;     // seg: trips ahead of which a row-worker asks L2 for its next segment (0 = off)
};

// The final value of a single-output reduction, combined across GPUs when a link is attached.
template <class Op>
__device__ __forceinline__ typename Op::T across_gpus(const PeerLink *link, typename Op::T v) {
  if constexpr (Op::kPeerOp >= 0) {
    if (link != nullptr) return peer_exchange_scalar(*link, v, Op::kPeerOp);
  }
  return v;
}

template <int VEC>
__device__ __forceinline__ void red_load(const float *p, bool vec, float *v) {
  if (VEC == 4 && vec) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if (VEC == 2 && vec) {
    const float2 t = __ldcs(reinterpret_cast<const float2 *>(p));
    v[0] = t.x; v[1] = t.y;
  } else {
    const float s = __ldg(p);
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = s;
  }
}

// Asks the memory system to bring [p, p + bytes) into L2 (p 16-byte aligned, bytes a multiple of
// 16); returns at once, nothing waits on it.
constexpr int kPrefetchAhead = 3;
__device__ __forceinline__ void prefetch_l2(const void *p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

template <class Op> __device__ __forceinline__ typename Op::T warp_reduce(typename Op::T v, int width) {
  for (int m = width >> 1; m > 0; m >>= 1) v = Op::combine(v, Op::shfl_xor(v, m, width));
  return v;
}

// All kRedThreads threads -> one value, valid in thread 0.
template <class Op> __device__ __forceinline__ typename Op::T block_reduce(typename Op::T v) {
  using T = typename Op::T;
  __shared__ T warp_vals[kRedThreads / 32];
  v = warp_reduce<Op>(v, 32);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_vals[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < kRedThreads / 32 ? warp_vals[lane] : Op::identity();
    v = warp_reduce<Op>(v, 8);
  }
  return v;
}

// Loads in flight per thread and input: 8 when one tensor is streamed, 4 with a prologue that
// reads several (registers).
template <int NIN> struct RedUnroll { static constexpr int value = NIN == 1 ? 8 : 4; };

// Accumulates items [begin, end) of one contiguous run, thread tx of width tx_n. Each trip issues
// up to kRedUnroll loads per input before the first use (predicated at the ragged end, so every
// thread of the row-worker makes the same number of trips).
// idx_base: flat reduced index of element 0 of the run (argmax only).
// NS: number of LEADING inputs that vary along the run. NS == NIN decides per input at run time
// (any mix); NS < NIN states at compile time that inputs [NS, NIN) are constant along the run
// (per-channel scale / bias of a gradient prologue), so they take one register each instead of a
// whole load batch.
template <class Op, class Pro, int NIN, int VEC, int NS>
__device__ __forceinline__ void accumulate_run(const RedParams<NIN> &p, const Pro &pro,
                                               const u64 *ioff, u64 begin, u64 end, unsigned tx,
                                               unsigned tx_n, unsigned idx_base, typename Op::T *acc) {
  // Pointers to item `begin` of the run; inside the run a 32-bit item index suffices (the host
  // never plans runs of 2^31 items or more). With VEC > 1 an input is either vector-loaded
  // (consecutive items are consecutive vectors) or constant along the run.
  constexpr bool kStatic = NS < NIN;
  constexpr int NV = kStatic ? NS : NIN; // inputs that get load slots
  const float *base[NIN];
  float fixed[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) {
    base[a] = p.in[a] + ioff[a] + begin * p.istride0[a];
    const bool is_fixed = kStatic ? a >= NS : p.istride0[a] == 0;
    fixed[a] = is_fixed ? __ldg(base[a]) : 0.0f;
  }
  const unsigned n = (unsigned)(end - begin);
  idx_base += (unsigned)begin * VEC;
  constexpr int kRedUnroll = RedUnroll<NV>::value * (VEC == 1 ? 2 : 1); // scalar items: more of them in flight
  auto load_item = [&](int a, unsigned i, float *v) {
    if (!kStatic && p.istride0[a] == 0) return;
    if (VEC == 4) {
      const float4 t = __ldcs(reinterpret_cast<const float4 *>(base[a]) + i);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if (VEC == 2) {
      const float2 t = __ldcs(reinterpret_cast<const float2 *>(base[a]) + i);
      v[0] = t.x; v[1] = t.y;
    } else {
      v[0] = __ldg(base[a] + (u64)i * p.istride0[a]);
    }
  };
  auto consume = [&](const float (*v)[VEC], unsigned i) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float x[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        const bool is_fixed = kStatic ? a >= NS : p.istride0[a] == 0;
        x[a] = is_fixed ? fixed[a] : v[a < NV ? a : 0][k];
      }
      acc[k] = Op::step(acc[k], pro(x), idx_base + i * VEC + k);
    }
  };
  // Every trip issues up to kRedUnroll loads per input before the first use; the ragged last trip
  // is predicated, so it is still one batch (not a chain of single dependent loads).
  for (unsigned b = tx; b < n + tx; b += kRedUnroll * tx_n) {
    float v[kRedUnroll][NV][VEC];
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) {
      const unsigned i = b + u * tx_n;
      if (i < n) {
#pragma unroll
        for (int a = 0; a < NV; ++a) load_item(a, i, v[u][a]);
      }
    }
#pragma unroll
    for (int u = 0; u < kRedUnroll; ++u) {
      const unsigned i = b + u * tx_n;
      if (i < n) consume(v[u], i);
    }
  }
}

// ---- rows: one (sub)warp per output -----------------------------------------------------------------
template <class Op, class Pro, int NIN, int VEC, int NS = NIN>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_kernel(RedParams<NIN> p, Pro pro) {
  using T = typename Op::T;
  pdl_wait();
  pdl_launch_dependents();
  const unsigned tx_n = 1u << p.log_tx;
  const unsigned tx = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> p.log_tx;
  const unsigned ty_n = kRedThreads >> p.log_tx;
  for (u64 row = (u64)blockIdx.x * ty_n + ty; row < p.n_kept; row += (u64)gridDim.x * ty_n) {
    u64 toff = 0, ioff[NIN];
#pragma unroll
    for (int a = 0; a < NIN; ++a) ioff[a] = 0;
    p.kept.offsets(row, &toff, ioff);
    T acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = Op::identity();
    accumulate_run<Op, Pro, NIN, VEC, NS>(p, pro, ioff, 0, p.len0, tx, tx_n, 0, acc);
    T r = acc[0];
#pragma unroll
    for (int k = 1; k < VEC; ++k) r = Op::combine(r, acc[k]);
    r = warp_reduce<Op>(r, (int)tx_n);
    if (tx == 0) Op::store((typename Op::Out *)p.out + toff, r, p.accumulate, p.post_div);
  }
}

// ---- tiny rows: one THREAD per output ------------------------------------------------------------------
// Dense rows of at most 48 elements (argmax over ten classes, the sum of a [N, 4] tensor) leave most
// lanes of a per-row thread group idle. A CTA moves 256 whole rows into shared memory with coalesced
// loads (odd row stride there: conflict-free afterwards) and every thread walks its own row left to
// right, which is also the reference's order of accumulation (src/kernels/cpu/reduce_ops.c:24-87).
constexpr int kTinyRowCols = 48; // measured against a slice of a warp per row: ahead up to 48 elements, behind at 64
template <class Op>
__global__ void __launch_bounds__(kRedThreads)
reduce_tiny_rows_kernel(const float *__restrict__ x, typename Op::Out *out, u64 rows, unsigned cols, unsigned div_magic,
                        bool accumulate, float post_div) {
  extern __shared__ float tiny_rows_tile[]; // kRedThreads rows of (cols | 1) floats
  pdl_wait();
  pdl_launch_dependents();
  const unsigned stride = cols | 1u;
  const u64 row0 = (u64)blockIdx.x * kRedThreads;
  const unsigned n_rows = (unsigned)(rows - row0 < (u64)kRedThreads ? rows - row0 : (u64)kRedThreads);
  const unsigned n = n_rows * cols;
  const float *xs = x + row0 * cols;
  for (unsigned i = threadIdx.x; i < n; i += kRedThreads) {
    const unsigned r = (unsigned)(((u64)i * div_magic) >> 21); // i / cols for i < 2^15, cols <= 64
    tiny_rows_tile[r * stride + (i - r * cols)] = __ldcs(xs + i);
  }
  __syncthreads();
  if (threadIdx.x < n_rows) {
    const float *mine = tiny_rows_tile + threadIdx.x * stride;
    typename Op::T acc = Op::identity();
    for (unsigned c = 0; c < cols; ++c) acc = Op::step(acc, mine[c], c);
    Op::store(out + row0 + threadIdx.x, acc, accumulate, post_div);
  }
}

// Last-arriving CTA of a tile: returns true in every thread of that CTA.
__device__ __forceinline__ bool take_ticket(unsigned int *counter, unsigned splits) {
  __shared__ bool is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(counter, 1u);
    is_last = (t == splits - 1);
    if (is_last) *counter = 0; // ready for the next launch
  }
  __syncthreads();
  if (is_last) __threadfence();
  return is_last;
}

// ---- seg: CTA per (output, chunk of segments) ---------------------------------------------------------
template <class Op, class Pro, int NIN, int VEC, int NS = NIN>
__global__ void __launch_bounds__(kRedThreads) reduce_seg_kernel(RedParams<NIN> p, Pro pro) {
  using T = typename Op::T;
  pdl_wait();
  pdl_launch_dependents();
  const u64 out_idx = blockIdx.x / p.splits;
  const unsigned chunk = blockIdx.x % p.splits;
  const unsigned tx_n = 1u << p.log_tx;
  const unsigned tx = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> p.log_tx;
  const unsigned ty_n = kRedThreads >> p.log_tx;

  u64 toff = 0, base[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) base[a] = 0;
  p.kept.offsets(out_idx, &toff, base);

  T acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = Op::identity();

  const u64 seg_begin = (u64)chunk * p.per_chunk;
  u64 seg_end = seg_begin + p.per_chunk;
  if (seg_end > p.nseg) seg_end = p.nseg;
  // Locates segment `seg`: input offsets of its run and the item range inside the run. The two
  // common shapes need no 64-bit division: one run cut into pieces (a full reduce), or whole
  // runs as segments (N,H,W of a channel gradient).
  auto locate = [&](u64 seg, u64 *ioff, u64 *begin, u64 *end, u64 *outer_out) {
    u64 outer, piece;
    if (p.n_red == 1) {
      outer = 0;
      piece = seg;
    } else if (p.nsplit0 == 1) {
      outer = seg;
      piece = 0;
    } else {
      outer = seg / p.nsplit0;
      piece = seg - outer * p.nsplit0;
    }
    u64 dummy = 0;
#pragma unroll
    for (int a = 0; a < NIN; ++a) ioff[a] = base[a];
    p.red.offsets(outer, &dummy, ioff);
    *begin = piece * p.seg_len;
    *end = *begin + p.seg_len;
    if (*end > p.len0) *end = p.len0;
    *outer_out = outer;
  };
  for (u64 seg = seg_begin + ty; seg < seg_end; seg += ty_n) {
    // Pull a segment this row-worker reads kPrefetchAhead trips from now into L2 with one bulk
    // prefetch per input, so DRAM stays busy beyond what the registers can keep in flight.
    if (VEC == 4 && tx == 0) {
      const u64 ahead = seg + (u64)p.seg_prefetch * ty_n;
      if (p.seg_prefetch != 0 && ahead < seg_end) {
        u64 poff[NIN], pb, pe, po;
        locate(ahead, poff, &pb, &pe, &po);
#pragma unroll
        for (int a = 0; a < NIN; ++a)
          if ((p.vec_mask >> a) & 1u)
            prefetch_l2(p.in[a] + poff[a] + pb * VEC, (unsigned)((pe - pb) * VEC * sizeof(float)));
      }
    }
    u64 ioff[NIN], begin, end, outer;
    locate(seg, ioff, &begin, &end, &outer);
    accumulate_run<Op, Pro, NIN, VEC, NS>(p, pro, ioff, begin, end, tx, tx_n,
                                      (unsigned)(outer * p.len0 * VEC), acc);
  }
  T r = acc[0];
#pragma unroll
  for (int k = 1; k < VEC; ++k) r = Op::combine(r, acc[k]);
  r = block_reduce<Op>(r);

  if (p.splits == 1) {
    if (threadIdx.x == 0)
      Op::store((typename Op::Out *)p.out + toff, across_gpus<Op>(p.peer, r), p.accumulate, p.post_div);
    return;
  }
  T *partials = (T *)p.partials + out_idx * p.splits;
  if (threadIdx.x == 0) partials[chunk] = r;
  if (!take_ticket(p.counters + out_idx, p.splits)) return;
  // Fixed assignment of chunks to threads, then the block tree: the result does not depend on
  // which CTA arrived last. All 256 threads share the partials so nobody walks a long chain of
  // dependent L2 loads at the very end of the kernel.
  T v = Op::identity();
  for (unsigned c = threadIdx.x; c < p.splits; c += kRedThreads) v = Op::combine(v, Op::load_cg(partials + c));
  __syncthreads(); // block_reduce's scratch was used above
  v = block_reduce<Op>(v);
  if (threadIdx.x == 0)
    Op::store((typename Op::Out *)p.out + toff, across_gpus<Op>(p.peer, v), p.accumulate, p.post_div);
}

// ---- cols: CTA per (strip of 32*VEC outputs along dim 0, outer kept index, chunk of reduced) ---------
template <class Op, class Pro, int NIN, int VEC>
__global__ void __launch_bounds__(kRedThreads) reduce_cols_kernel(RedParams<NIN> p, Pro pro) {
  using T = typename Op::T;
  pdl_wait();
  pdl_launch_dependents();
  // tx_n lanes across dim 0 (a strip of tx_n * VEC outputs, one coalesced run per reduced index),
  // ty_n row-workers striding over the reduced indices. Wide strips (up to 256 lanes = 4 KiB per
  // row) keep every DRAM page access long; narrow ones serve small dim 0.
  const unsigned tx_n = 1u << p.log_tx;
  const unsigned lane = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> p.log_tx;
  const unsigned ty_n = kRedThreads >> p.log_tx;
  const u64 strips = (p.len0 + tx_n - 1) >> p.log_tx;
  // (outer kept, strip) and chunk of the reduced dim; either the chunks of a tile or the tiles of a
  // chunk are neighbours in launch order
  const unsigned n_tiles = gridDim.x / p.splits;
  const u64 tile = p.strip_major ? blockIdx.x % n_tiles : blockIdx.x / p.splits;
  const unsigned chunk = p.strip_major ? blockIdx.x / n_tiles : blockIdx.x % p.splits;
  u64 outer, strip, item;
  bool live;
  if (p.outers_per_cta > 1) {
    // short kept runs: lanes = (outer kept index, item of its run)
    const unsigned sub = lane / (unsigned)p.len0;
    outer = tile * p.outers_per_cta + sub;
    strip = 0;
    item = lane - sub * (unsigned)p.len0;
    live = sub < p.outers_per_cta && outer < p.n_kept;
    if (!live) outer = 0;
  } else {
    outer = tile / strips;
    strip = tile - outer * strips;
    item = (strip << p.log_tx) + lane;
    live = item < p.len0;
  }

  u64 toff = 0, base[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) base[a] = 0;
  p.kept.offsets(outer, &toff, base);
  toff += item * VEC * p.tstride0;
#pragma unroll
  for (int a = 0; a < NIN; ++a) base[a] += item * p.istride0[a];

  T acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = Op::identity();

  u64 r_begin = (u64)chunk * p.per_chunk;
  if (r_begin > p.n_red) r_begin = p.n_red; // a cluster keeps its size even when the last chunks are empty
  u64 r_end = r_begin + p.per_chunk;
  if (r_end > p.n_red) r_end = p.n_red;
  constexpr int kRedUnroll = VEC == 1 ? 8 : 4; // scalar items: twice the rows per batch for bytes in flight
  const unsigned n = (unsigned)(r_end - r_begin); // the host keeps a chunk below 2^31 indices
  if (live && p.red.n <= 1) {
    // One reduced dim (the usual case): walk it with pointer increments, no index decoding.
    const float *ptr[NIN];
    u64 step[NIN];
#pragma unroll
    for (int a = 0; a < NIN; ++a) {
      const u64 rs = p.red.n == 1 ? p.red.istride[a][0] : 0;
      ptr[a] = p.in[a] + base[a] + (r_begin + ty) * rs;
      step[a] = (u64)ty_n * rs;
    }
    // Full batches first (every load of the batch issued back to back, nothing predicated),
    // then the ragged rest one row at a time.
    auto load_row = [&](const float *q, int a, float *v) {
      if ((p.vec_mask >> a) & 1u) {
        if (VEC == 4) {
          const float4 t = __ldcs(reinterpret_cast<const float4 *>(q));
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else if (VEC == 2) {
          const float2 t = __ldcs(reinterpret_cast<const float2 *>(q));
          v[0] = t.x; v[1] = t.y;
        } else {
          v[0] = __ldg(q);
        }
      } else {
        const float sc = __ldg(q);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = sc;
      }
    };
    unsigned rb = ty;
    // bytes of one row of the strip (the last strip of a row may be narrower)
    const unsigned strip_bytes =
        (unsigned)((p.len0 - (strip << p.log_tx) < tx_n ? p.len0 - (strip << p.log_tx) : tx_n) * VEC * sizeof(float));
    for (; rb + (kRedUnroll - 1) * ty_n < n; rb += kRedUnroll * ty_n) {
      if (VEC == 4 && p.prefetch_batches != 0 && lane == 0 &&
          (p.prefetch_until == 0 || rb < p.prefetch_until * kRedUnroll * ty_n)) {
        // the rows this worker reads `prefetch_batches` batches from now, one bulk prefetch per row
        const unsigned ahead = p.prefetch_batches * kRedUnroll;
#pragma unroll
        for (int u = 0; u < kRedUnroll; ++u)
          if (rb + (ahead + u) * ty_n < n) {
#pragma unroll
            for (int a = 0; a < NIN; ++a)
              if ((p.vec_mask >> a) & 1u) prefetch_l2(ptr[a] + (u64)(ahead + u) * step[a], strip_bytes);
          }
      }
      float v[kRedUnroll][NIN][VEC];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u)
#pragma unroll
        for (int a = 0; a < NIN; ++a) load_row(ptr[a] + (u64)u * step[a], a, v[u][a]);
#pragma unroll
      for (int a = 0; a < NIN; ++a) ptr[a] += (u64)kRedUnroll * step[a];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u)
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          float x[NIN];
#pragma unroll
          for (int a = 0; a < NIN; ++a) x[a] = v[u][a][k];
          acc[k] = Op::step(acc[k], pro(x), (unsigned)r_begin + rb + u * ty_n);
        }
    }
    for (; rb < n; rb += ty_n) {
      float v[NIN][VEC];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        load_row(ptr[a], a, v[a]);
        ptr[a] += step[a];
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float x[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) x[a] = v[a][k];
        acc[k] = Op::step(acc[k], pro(x), (unsigned)r_begin + rb);
      }
    }
  } else if (live) {
    for (unsigned rb = ty; rb < n + ty; rb += kRedUnroll * ty_n) {
      float v[kRedUnroll][NIN][VEC];
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) {
        const unsigned r = rb + u * ty_n;
        if (r < n) {
          u64 ioff[NIN], dummy = 0;
#pragma unroll
          for (int a = 0; a < NIN; ++a) ioff[a] = base[a];
          p.red.offsets(r_begin + r, &dummy, ioff);
#pragma unroll
          for (int a = 0; a < NIN; ++a)
            red_load<VEC>(p.in[a] + ioff[a], (p.vec_mask >> a) & 1u, v[u][a]);
        }
      }
#pragma unroll
      for (int u = 0; u < kRedUnroll; ++u) {
        const unsigned r = rb + u * ty_n;
        if (r < n) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            float x[NIN];
#pragma unroll
            for (int a = 0; a < NIN; ++a) x[a] = v[u][a][k];
            acc[k] = Op::step(acc[k], pro(x), (unsigned)r_begin + r);
          }
        }
      }
    }
  }
  // Combine the row-workers in shared memory (worker t holds reduced indices = t (mod ty_n)) as a
  // tree in a fixed order: a narrow strip has up to 256 workers, too many for one thread to walk.
  // The result is valid in the threads of worker 0.
  __shared__ T strip_vals[kRedThreads * VEC];
  auto combine_workers = [&](T(&vals)[VEC]) {
    if (ty_n == 1) return;
#pragma unroll
    for (int k = 0; k < VEC; ++k) strip_vals[((ty * VEC + k) << p.log_tx) + lane] = vals[k];
    __syncthreads();
    for (unsigned s = ty_n >> 1; s > 0; s >>= 1) {
      if (ty < s) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const unsigned mine = ((ty * VEC + k) << p.log_tx) + lane, other = (((ty + s) * VEC + k) << p.log_tx) + lane;
          strip_vals[mine] = Op::combine(strip_vals[mine], strip_vals[other]);
        }
      }
      __syncthreads();
    }
    if (ty == 0) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) vals[k] = strip_vals[(k << p.log_tx) + lane];
    }
  };
  T r[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) r[k] = acc[k];
  combine_workers(r);
  typename Op::Out *out = (typename Op::Out *)p.out;
  // With a link attached (the host only does that for a single row of strips whose outputs are
  // contiguous, at most PLAST_B200_PEER_MAX_FLOATS of them) the threads that hold a strip's final
  // local values exchange them across the GPUs before they store: reduce and all-reduce are one
  // kernel. Every thread of the CTA reaches this point together (a CTA that is not the last of its
  // tile has returned as a whole).
  auto across_gpus_strip = [&](T(&vals)[VEC]) {
    if constexpr (Op::kPeerOp >= 0 && !Op::kIndexed) {
      if (p.peer != nullptr) {
        if (ty == 0 && live) peer_exchange_strip<VEC>(*p.peer, vals, (unsigned)(item * VEC), Op::kPeerOp);
        __syncthreads();
        if (threadIdx.x == 0) peer_exchange_strip_done(*p.peer, (unsigned)strips);
      }
    }
  };
  if (p.splits == 1) {
    across_gpus_strip(r);
    if (ty == 0 && live) {
#pragma unroll
      for (int k = 0; k < VEC; ++k)
        Op::store(out + toff + (u64)k * p.tstride0, r[k], p.accumulate, p.post_div);
    }
    return;
  }
  if (p.cluster > 1) {
    // The chunks of this tile are the CTAs of one cluster (rank = chunk): each leaves its strip in
    // its own shared memory, rank 0 reads the others over the SM-to-SM network in rank order and
    // finishes. Nobody touches global memory or an atomic in between.
    cooperative_groups::cluster_group cl = cooperative_groups::this_cluster();
    __syncthreads(); // worker 0 has read its strip out of the tree
    if (ty == 0) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) strip_vals[(k << p.log_tx) + lane] = r[k];
    }
    cl.sync();
    if (chunk == 0) {
      if (ty == 0 && live) {
        for (unsigned c = 1; c < p.splits; ++c) {
          const T *theirs = cl.map_shared_rank(strip_vals, c);
#pragma unroll
          for (int k = 0; k < VEC; ++k) r[k] = Op::combine(r[k], theirs[(k << p.log_tx) + lane]);
        }
      }
      across_gpus_strip(r);
      if (ty == 0 && live) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) Op::store(out + toff + (u64)k * p.tstride0, r[k], p.accumulate, p.post_div);
      }
    }
    cl.sync(); // the other ranks' shared memory stays alive until rank 0 has read it
    return;
  }
  T *partials = (T *)p.partials + tile * p.splits * ((u64)VEC << p.log_tx);
  if (ty == 0) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) partials[(((u64)chunk * VEC + k) << p.log_tx) + lane] = r[k];
  }
  if (!take_ticket(p.counters + tile, p.splits)) return;
  // Last CTA of the tile: row-worker t adds chunks t, t + ty_n, ... (independent loads), then the
  // workers are combined in shared memory as above. Fixed assignment -> reproducible result.
  T fin[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    fin[k] = Op::identity();
    if (live)
      for (unsigned c = ty; c < p.splits; c += ty_n)
        fin[k] = Op::combine(fin[k], Op::load_cg(partials + (((u64)c * VEC + k) << p.log_tx) + lane));
  }
  __syncthreads(); // the shared strip is reused
  combine_workers(fin);
  across_gpus_strip(fin);
  if (ty == 0 && live) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) Op::store(out + toff + (u64)k * p.tstride0, fin[k], p.accumulate, p.post_div);
  }
}

// ---- host side ----------------------------------------------------------------------------------------
enum RedKind { kRedRows = 0, kRedSeg = 1, kRedCols = 2 };

struct RedChoice {
  RedKind kind;
  int vec;
  u64 grid;
};

// Fills every field of RedParams that does not depend on NIN-typed pointers; returns false (with
// the error set) when the plan cannot run. Implemented in reduce.cu.
struct RedGeometry {
  RedKind kind;
  int vec;
  unsigned vec_mask;
  int log_tx;
  u64 len0_items, seg_len, nsplit0, nseg, per_chunk, n_kept, n_red, grid;
  unsigned splits;
  unsigned cluster; // cols: the splits of a tile form a cluster of this many CTAs (0 or 1: no cluster)
  unsigned outers_per_cta; // cols: outer kept indices covered by the lanes of one CTA (short kept runs)
  int kept_dims[MAX_NDIM], n_kept_dims; // plan dim indices in each sub-space
  int red_dims[MAX_NDIM], n_red_dims;
};
// Resident CTAs per SM of each kernel shape ([kind][vec 1,2,4]), from the occupancy calculator.
struct RedOccupancy {
  int ctas_per_sm[3][3];
};
bool plan_reduce_geometry(const IterPlan &plan, const void *const *in_ptrs, int nin,
                          size_t elem_bytes, bool indexed, const RedOccupancy &occ, RedGeometry *g);

template <class Op, class Pro, int NIN> const RedOccupancy &reduce_occupancy() {
  static RedOccupancy occ = [] {
    RedOccupancy o;
    auto q = [](auto kernel) {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kRedThreads, 0) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 4;
      }
      return n;
    };
    o.ctas_per_sm[kRedRows][0] = q(reduce_rows_kernel<Op, Pro, NIN, 1>);
    o.ctas_per_sm[kRedRows][1] = q(reduce_rows_kernel<Op, Pro, NIN, 2>);
    o.ctas_per_sm[kRedRows][2] = q(reduce_rows_kernel<Op, Pro, NIN, 4>);
    o.ctas_per_sm[kRedSeg][0] = q(reduce_seg_kernel<Op, Pro, NIN, 1>);
    o.ctas_per_sm[kRedSeg][1] = q(reduce_seg_kernel<Op, Pro, NIN, 2>);
    o.ctas_per_sm[kRedSeg][2] = q(reduce_seg_kernel<Op, Pro, NIN, 4>);
    o.ctas_per_sm[kRedCols][0] = q(reduce_cols_kernel<Op, Pro, NIN, 1>);
    o.ctas_per_sm[kRedCols][1] = q(reduce_cols_kernel<Op, Pro, NIN, 2>);
    o.ctas_per_sm[kRedCols][2] = q(reduce_cols_kernel<Op, Pro, NIN, 4>);
    return o;
  }();
  return occ;
}

// Bracket mode with nothing to reduce on THIS rank (an empty shard): the ranks that hold data make
// one call of the exchange sequence for this reduction, so this rank makes it too and contributes
// the identity; its output then receives what the others reduced. `values` holds n identities.
template <class Op> void exchange_for_empty_shard(float *dst, float *values, u64 n, bool accumulate) {
  if constexpr (Op::kPeerOp >= 0 && !Op::kIndexed) {
    if (n > kParkedFloats) {
      set_error(PLAST_B200_ERR_UNSUPPORTED, "a reduction inside plast_b200_peer_reduce_begin/_end has at most %llu outputs",
                (unsigned long long)kParkedFloats);
      return;
    }
    launch_peer_exchange(peer_bracket_take(), values, (unsigned)n, Op::kPeerOp);
    if (dst != values) launch_add_parked(dst, values, (unsigned)n, accumulate);
  }
}

template <class Op, class Pro, int NIN>
void launch_reduce(const IterPlan &plan, typename Op::Out *out, const float *const *ins,
                   const Pro &pro, const Op &, bool accumulate, float post_div) {
  if (plan.numel == 0) {
    if constexpr (Op::kPeerOp >= 0 && !Op::kIndexed) {
      if (peer_bracket_open()) {
        u64 n_out = 1;
        for (int d = 0; d < plan.ndim; ++d)
          if (!plan.reduced[d]) n_out *= plan.size[d];
        Workspace wsp;
        if (n_out == 0 || plan.max_offset[0] != n_out - 1 || !get_workspace(&wsp)) return;
        float ident = 0.0f;
        if (Op::kPeerOp == PLAST_B200_PEER_MAX) ident = -FLT_MAX;
        if (Op::kPeerOp == PLAST_B200_PEER_MIN) ident = FLT_MAX;
        unsigned int bits;
        memcpy(&bits, &ident, 4);
        fill32(wsp.parked, bits, n_out < kParkedFloats ? n_out : kParkedFloats);
        exchange_for_empty_shard<Op>((float *)out, wsp.parked, n_out, accumulate);
      }
    }
    return;
  }
  RedGeometry g;
  const void *ptrs[NIN];
  for (int a = 0; a < NIN; ++a) ptrs[a] = ins[a];
  if (!plan_reduce_geometry(plan, ptrs, NIN, sizeof(typename Op::T), Op::kIndexed,
                            reduce_occupancy<Op, Pro, NIN>(), &g))
    return;

  // Several reduced dims around long contiguous runs (N, H, W of an NCHW channel gradient) with
  // plenty of (kept x outer-reduced) combinations: reduce every run on its own with the rows
  // kernel (the fastest shape: a warp per run, no cross-CTA traffic) into a small scratch matrix
  // [outer reduced][kept], then reduce that matrix over the outer dims. Two launches, but the
  // second one touches kilobytes.
  if (g.kind == kRedSeg && g.n_red > 1 && !Op::kIndexed && g.len0_items * (u64)g.vec >= 256 &&
      g.n_kept * g.n_red >= 4096 && g.n_kept * g.n_red <= kPartialFloats / 4) {
    Workspace ws2;
    if (!get_workspace(&ws2)) return;
    float *scratch = ws2.partials + (kPartialFloats / 4) * 3; // last quarter: two-stage partials
    IterPlan first = plan;
    u64 sh2[MAX_NDIM], st2[2][MAX_NDIM];
    bool red2[MAX_NDIM];
    u64 kflat = 1, rflat = g.n_kept;
    for (int d = 1; d < plan.ndim; ++d) {
      const u64 sst = plan.reduced[d] ? rflat : kflat;
      (plan.reduced[d] ? rflat : kflat) *= plan.size[d];
      first.reduced[d] = false;
      first.stride[0][d] = sst;
      const int o = plan.ndim - 1 - d; // outermost first for make_plan
      sh2[o] = plan.size[d];
      st2[0][o] = plan.stride[0][d];
      st2[1][o] = sst;
      red2[o] = plan.reduced[d];
    }
    first.stride[0][0] = 0;
    first.max_offset[0] = g.n_kept * g.n_red - 1;
    {
      PeerSuspend local_step; // partial sums into scratch: only the second stage's result crosses GPUs
      launch_reduce<Op, Pro, NIN>(first, (typename Op::Out *)scratch, ins, pro, Op{}, false, 0.0f);
    }
    if (failed()) return;
    IterPlan second;
    make_plan(&second, sh2, (u64)(plan.ndim - 1), 2, st2, red2, 1);
    const float *ins2[1] = {scratch};
    launch_reduce<Op, IdentityPro, 1>(second, out, ins2, IdentityPro{}, Op{}, accumulate, post_div);
    return;
  }

  RedParams<NIN> p;
  for (int a = 0; a < NIN; ++a) p.in[a] = ins[a];
  p.out = out;
  p.kept.n = g.n_kept_dims;
  p.red.n = g.n_red_dims;
  for (int d = 0; d < MAX_NDIM; ++d) {
    const int kd = d < g.n_kept_dims ? g.kept_dims[d] : -1;
    const int rd = d < g.n_red_dims ? g.red_dims[d] : -1;
    p.kept.size[d] = kd >= 0 ? plan.size[kd] : 1;
    p.kept.tstride[d] = kd >= 0 ? plan.stride[0][kd] : 0;
    p.red.size[d] = rd >= 0 ? plan.size[rd] : 1;
    p.red.tstride[d] = 0;
    for (int a = 0; a < NIN; ++a) {
      p.kept.istride[a][d] = kd >= 0 ? plan.stride[a + 1][kd] : 0;
      p.red.istride[a][d] = rd >= 0 ? plan.stride[a + 1][rd] : 0;
    }
  }
  p.n_kept = g.n_kept;
  p.n_red = g.n_red;
  p.len0 = g.len0_items;
  p.tstride0 = plan.stride[0][0];
  for (int a = 0; a < NIN; ++a) p.istride0[a] = plan.stride[a + 1][0] * (u64)g.vec;
  p.vec_mask = g.vec_mask;
  p.log_tx = g.log_tx;
  p.seg_len = g.seg_len;
  p.nsplit0 = g.nsplit0;
  p.nseg = g.nseg;
  p.per_chunk = g.per_chunk;
  p.splits = g.splits;
  p.accumulate = accumulate;
  p.post_div = post_div;
  p.counters = nullptr;
  p.partials = nullptr;
  p.peer = nullptr;
  p.cluster = g.cluster;
  p.outers_per_cta = g.kind == kRedCols ? g.outers_per_cta : 1;
  p.strip_major = g.cluster <= 1 && tuned(kTuneColsTileMajor) > 0; // measured: the order of the CTAs makes no difference
  // Column sweep: every row-worker asks L2 for the rows of its NEXT load batch (one bulk prefetch
  // per 512-byte row piece) during the first 16 batches of its chunk. Measured on B200: 46.5 -> 40.5
  // us for the column sum of 8192 x 8192 issued back to back (part of a 268 MB tensor survives in
  // the 126 MB L2 from launch to launch, and prefetched lines survive better than streamed ones),
  // 49 -> 51 us (one timer tick) on cold data, neutral from 512 MiB up; prefetching through the
  // whole chunk costs 10 % at 1 GiB, prefetching further ahead gains nothing.
  // Only long sweeps prefetch: with a handful of batches per row-worker (small inputs, narrow
  // strips) the extra instructions cost more than they bring (config 1's grad_b: 5.3 -> 10 us).
  const u64 batches_per_worker = g.per_chunk / (((u64)kRedThreads >> g.log_tx) * 4);
  p.prefetch_batches = tuned(kTuneColsPrefetch) >= 0 ? (unsigned)tuned(kTuneColsPrefetch)
                                                     : (g.kind == kRedCols && g.log_tx >= 5 && batches_per_worker >= 16 &&
                                                                g.outers_per_cta <= 1 ? 1u : 0u);
  p.prefetch_until = tuned(kTuneColsPrefetchUntil) >= 0 ? (unsigned)tuned(kTuneColsPrefetchUntil) : 16u;
  p.seg_prefetch = tuned(kTuneSegPrefetch) >= 0 ? (unsigned)tuned(kTuneSegPrefetch) : (unsigned)kPrefetchAhead;
  // a pending cross-GPU exchange rides on the kernel whose last CTA holds THE final value
  if (Op::kPeerOp >= 0 && g.kind == kRedSeg && g.n_kept == 1 && !take_peer_link(kPeerFullReduce, &p.peer, nullptr))
    p.peer = nullptr;
  // Bracket mode: this reduction's result is combined across the ranks. Inside the kernel where one
  // thread (single output) or the strip owners (column reduce over one row of strips, contiguous
  // outputs) hold the final values; otherwise the local result is parked in scratch, exchanged by
  // the stand-alone kernel right behind this launch and then stored / accumulated at its place.
  // Either way it is exactly one call of the exchange sequence, at this point of the launch order.
  float *parked_for = nullptr;
  unsigned parked_n = 0;
  bool parked_accumulate = false;
  if constexpr (Op::kPeerOp >= 0 && !Op::kIndexed) {
    if (peer_bracket_open()) {
      u64 n_out = g.n_kept * (plan.reduced[0] ? 1 : plan.size[0]);
      if (post_div > 0.0f || n_out > kParkedFloats || plan.max_offset[0] != n_out - 1) {
        set_error(PLAST_B200_ERR_UNSUPPORTED,
                  "a reduction inside plast_b200_peer_reduce_begin/_end must be a sum, max or min (a mean divides by the "
                  "local count) onto at most %llu contiguous outputs", (unsigned long long)kParkedFloats);
        return;
      }
      const bool single = g.kind == kRedSeg && g.n_kept == 1;
      const bool strips_row = g.kind == kRedCols && g.n_kept == 1 && plan.stride[0][0] == 1;
      if (single || strips_row) {
        p.peer = peer_bracket_take();
      } else {
        Workspace wsp;
        if (!get_workspace(&wsp)) return;
        parked_for = (float *)out;
        parked_n = (unsigned)n_out;
        parked_accumulate = accumulate;
        p.out = wsp.parked;
        p.accumulate = false;
      }
    }
  }
  Workspace ws = {};
  if (g.splits > 1 && g.cluster <= 1) {
    if (!get_workspace(&ws)) return;
    p.counters = ws.counters;
    p.partials = ws.partials;
  }
  cudaStream_t s = stream();
  dim3 grid((unsigned)g.grid), block(kRedThreads);
#define PB_RED_LAUNCH(KERNEL)                                                                      \
  do {                                                                                             \
    if (g.vec == 4) launch_kc(g.cluster, KERNEL<Op, Pro, NIN, 4>, grid, block, 0, s, p, pro);      \
    else if (g.vec == 2) launch_kc(g.cluster, KERNEL<Op, Pro, NIN, 2>, grid, block, 0, s, p, pro); \
    else launch_kc(g.cluster, KERNEL<Op, Pro, NIN, 1>, grid, block, 0, s, p, pro);                 \
  } while (0)
  // float4 plans whose inputs are "the first m vary along the run, the rest are constant"
  // (m = 1 or 2 < NIN) get the kernel that knows this at compile time (fewer registers).
  int lead = 0;
  while (lead < NIN && ((g.vec_mask >> lead) & 1u)) ++lead;
  const bool prefix = g.vec == 4 && lead < NIN && g.vec_mask == ((1u << lead) - 1u) && (lead == 1 || lead == 2);
#define PB_RED_LAUNCH_NS(KERNEL)                                                                   \
  do {                                                                                             \
    if (prefix && lead == 1) launch_k(KERNEL<Op, Pro, NIN, 4, (NIN > 1 ? 1 : NIN)>, grid, block, 0, s, p, pro); \
    else if (prefix && lead == 2) launch_k(KERNEL<Op, Pro, NIN, 4, (NIN > 2 ? 2 : NIN)>, grid, block, 0, s, p, pro); \
    else PB_RED_LAUNCH(KERNEL);                                                                    \
  } while (0)
  // dense rows of at most 48 elements, one plain input, many of them: a thread per row
  bool tiny_rows = false;
  if constexpr (NIN == 1 && std::is_same<Pro, IdentityPro>::value) {
    const u64 tiny_max = tuned(kTuneTinyRowCols) >= 0 ? (u64)tuned(kTuneTinyRowCols) : (u64)kTinyRowCols;
    tiny_rows = g.kind == kRedRows && g.n_red == 1 && plan.size[0] <= tiny_max && plan.size[0] <= (u64)kTinyRowCols &&
                plan.stride[1][0] == 1 &&
                g.n_kept >= 4096 && g.n_kept < ((u64)1 << 39);
    u64 run = 1;
    for (int d = 0; tiny_rows && d < g.n_kept_dims; ++d) {
      const int kd = g.kept_dims[d];
      if (plan.stride[1][kd] != run * plan.size[0] || plan.stride[0][kd] != run) tiny_rows = false;
      run *= plan.size[kd];
    }
  }
  if (tiny_rows) {
    if constexpr (NIN == 1 && std::is_same<Pro, IdentityPro>::value) {
      static bool ready = false;
      if (!ready) {
        cudaFuncSetAttribute(reduce_tiny_rows_kernel<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(kRedThreads * (kTinyRowCols + 1) * sizeof(float)));
        ready = true;
      }
      const unsigned cols = (unsigned)plan.size[0];
      launch_k(reduce_tiny_rows_kernel<Op>, dim3((unsigned)((g.n_kept + kRedThreads - 1) / kRedThreads)), block,
               (size_t)kRedThreads * (cols | 1u) * sizeof(float), s, p.in[0], (typename Op::Out *)p.out, g.n_kept, cols,
               (unsigned)(((u64)1 << 21) / cols + 1), p.accumulate, p.post_div);
      note_kernel("reduce_tiny_rows");
    }
  } else if (g.kind == kRedRows) {
    PB_RED_LAUNCH_NS(reduce_rows_kernel);
    note_kernel(g.vec == 4 ? "reduce_rows_vec4" : (g.vec == 2 ? "reduce_rows_vec2" : "reduce_rows_scalar"));
  } else if (g.kind == kRedSeg) {
    PB_RED_LAUNCH_NS(reduce_seg_kernel);
    note_kernel(g.vec == 4 ? "reduce_seg_vec4" : (g.vec == 2 ? "reduce_seg_vec2" : "reduce_seg_scalar"));
  } else {
    PB_RED_LAUNCH(reduce_cols_kernel);
    note_kernel(g.vec == 4 ? "reduce_cols_vec4" : (g.vec == 2 ? "reduce_cols_vec2" : "reduce_cols_scalar"));
  }
#undef PB_RED_LAUNCH_NS
#undef PB_RED_LAUNCH
  count_launch();
  if (parked_for != nullptr) {
    launch_peer_exchange(peer_bracket_take(), (float *)p.out, parked_n, Op::kPeerOp);
    launch_add_parked(parked_for, (const float *)p.out, parked_n, parked_accumulate);
  }
}

} // namespace pb
