// Fused softmax / log_softmax / cross_entropy (forward and backward) along one axis.
//
// The reference builds these from primitives (plast/nn/functional.py:77-97, 312-333):
//   softmax      max -> sub -> exp -> sum -> div          5 kernels, ~7 passes over the data
//   log_softmax  max -> sub -> exp -> sum -> log -> sub   6 kernels
//   cross_entropy  log_softmax -> one-hot mul -> sum(dim=1) -> neg -> mean
// Here a row is read from HBM once, kept in registers, and written once. Each intermediate is
// rounded to fp32 exactly where the primitive chain rounds it (the library is built with
// -fmad=false), so only the order of the row sum differs from the reference.
//
// Two kernels per op:
//   fast     rows are contiguous along the axis, 16-byte aligned, cols % 4 == 0 and
//            cols <= 8192: TX threads per row (32..256), up to 8 float4 per thread.
//   generic  anything else (long rows, strided axis, odd sizes): one CTA per row, an online
//            running (max, sum) pair in a single read pass, then one more pass to write.
#include "common.cuh"
#include "iter.h"
#include "reduce_engine.cuh"

#include <cooperative_groups.h>
#include <float.h>

namespace pb {

enum SmMode { kSoftmax = 0, kLogSoftmax = 1, kCrossEntropy = 2 };

// exp for the softmax family. The contract for softmax / log-softmax / cross-entropy is a relative
// error of 1e-5 on the result (not 2 ulp per element as for exp_cuda_forward), and with 4096
// exponentials per 16 KiB row the instruction count of expf, not HBM, bounds a read-only kernel
// like cross-entropy. This version keeps ~3 ulp without expf's explicit range reduction:
//   t = x * log2(e) rounded; err = the rounding error of that product (one FMA, exact) plus the
//   low part of log2(e); exp(x) = 2^t * 2^err ~= ex2(t) * (1 + err * ln 2).
// Five instructions instead of about ten; ex2.approx itself is good to ~2 ulp over its range and
// returns 0 / denormals for very negative t like expf.
// Arguments here are x - max <= 0; they are clamped at -104 (exp underflows to 0 below -103.3)
// so that -FLT_MAX-sized differences cannot turn the error term into inf * 0.
__device__ __forceinline__ float exp_softmax(float x) {
  x = fmaxf(x, -104.0f);
  const float kLog2eHi = 1.4426950216293335f;    // fp32(log2 e)
  const float kLog2eLo = 1.9259629911266175e-8f; // log2 e - kLog2eHi
  const float t = x * kLog2eHi;
  float err = __fmaf_rn(x, kLog2eHi, -t);
  err = __fmaf_rn(x, kLog2eLo, err);
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(t));
  return __fmaf_rn(r * 0.6931471805599453f, err, r);
}

// exp(d) for d = x - max <= 0 where only the ROW SUM of the exponentials is wanted (log-softmax, the
// cross-entropy loss): a multiply and ex2.approx, ~1e-6 relative on the sum, i.e. ~1e-6 absolute on
// its logarithm, against a contract of 1e-5. Elementwise results (softmax itself, the backward
// passes) keep exp_softmax.
__device__ __forceinline__ float exp_for_sum(float d) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d * 1.4426950408889634f));
  return r;
}

constexpr int kSmThreads = 256;
constexpr int kSmMaxVpt = 8;

struct SmRows {
  SubSpace<2> outer;  // dims other than the axis: tstride = out, istride[0] = x, istride[1] = 2nd input
  u64 rows, cols;
  u64 x_axis_stride, y_axis_stride, z_axis_stride; // element strides along the axis
};

// Reduction over the TX threads of a row-worker (TX = 1 << log_tx, 1 <= TX <= 256).
// Every thread of the CTA must call it (it synchronises when TX > 32).
// SUB: TX < 32 is possible (rows that take a slice of a warp); kernels that never see it keep the
// constant-width, fully unrolled shuffle tree (the float4 kernel is issue-bound: a run-time width
// cost it 2 - 4 % on [65536, 4096]).
template <class Op, bool SUB = false>
__device__ __forceinline__ float row_reduce(float v, int log_tx, float *smem /* [8] */) {
  if (SUB && log_tx < 5) return warp_reduce<Op>(v, 1 << log_tx);
  v = warp_reduce<Op>(v, 32);
  if (log_tx > 5) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpr = 1 << (log_tx - 5); // warps per row-worker
    __syncthreads();                   // previous use of smem is over
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    const int first = (warp / wpr) * wpr;
    v = smem[first];
    for (int w = 1; w < wpr; ++w) v = Op::combine(v, smem[first + w]);
  }
  return v;
}

// ---- forward, fast path ---------------------------------------------------------------------------
// CE: `labels` int32 per row, per-CTA partial loss sums go through the ticket scheme.
// Rows shorter than 32 vectors take a power-of-two slice of a warp each (log_tx < 5), so that a warp
// reads several whole rows per instruction.
template <int MODE, int VPT, bool SUB = false>
__global__ void __launch_bounds__(kSmThreads, 4)
softmax_fast_kernel(const float *__restrict__ x, float *__restrict__ y, const int *__restrict__ labels,
                    SmRows g, int log_tx, float *row_loss) {
  __shared__ float red_smem[kSmThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int tx_n = 1 << log_tx;
  const int tx = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> log_tx;
  const int rows_per_cta = kSmThreads >> log_tx;
  const u64 nvec = g.cols >> 2;
  // Every thread of the CTA reaches both row_reduce calls (they synchronise when TX > 32).
  { // one group of rows per CTA (the grid covers every row)
    const u64 row = (u64)blockIdx.x * rows_per_cta + ty;
    const bool live = row < g.rows;
    u64 yoff = 0, ioff[2] = {0, 0};
    if (live) g.outer.offsets(row, &yoff, ioff);
    const float4 *xr = reinterpret_cast<const float4 *>(x + ioff[0]);

    float4 v[VPT];
    float m = -FLT_MAX; // src/kernels/cpu/reduce_ops.c:273
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const u64 j = (u64)tx + (u64)i * tx_n;
      if (live && j < nvec) v[i] = __ldcs(xr + j);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const u64 j = (u64)tx + (u64)i * tx_n;
      if (live && j < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
    m = row_reduce<MaxOp, SUB>(m, log_tx, red_smem);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const u64 j = (u64)tx + (u64)i * tx_n;
      if (live && j < nvec) {
        // sub, then exp: two separately rounded ops
        v[i].x = v[i].x - m; v[i].y = v[i].y - m; v[i].z = v[i].z - m; v[i].w = v[i].w - m;
        if (MODE == kSoftmax) {
          v[i].x = exp_softmax(v[i].x); v[i].y = exp_softmax(v[i].y); v[i].z = exp_softmax(v[i].z); v[i].w = exp_softmax(v[i].w);
          s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        } else {
          s += (exp_for_sum(v[i].x) + exp_for_sum(v[i].y)) + (exp_for_sum(v[i].z) + exp_for_sum(v[i].w));
        }
      }
    }
    s = row_reduce<SumOp, SUB>(s, log_tx, red_smem);

    if (MODE == kCrossEntropy) {
      // loss_row = -((x[label] - m) - log(s)); v[] still holds x - m, so the thread that loaded
      // the label's vector picks it from its registers (no second trip to memory).
      if (live) {
        const int label = labels[row];
        if (label >= 0 && (u64)label < g.cols) {
          const u64 jv = (u64)label >> 2;
          if ((int)(jv & (u64)(tx_n - 1)) == tx) {
            const int slot = (int)(jv >> log_tx), comp = label & 3;
            float sh = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
              if (i == slot) sh = comp == 0 ? v[i].x : (comp == 1 ? v[i].y : (comp == 2 ? v[i].z : v[i].w));
            row_loss[row] = -(sh - logf(s));
          }
        } else if (tx == 0) {
          row_loss[row] = 0.0f; // label outside [0, cols): contributes nothing
        }
      }
      return;
    }

    float4 *yr = reinterpret_cast<float4 *>(y + yoff);
    const float lse = (MODE == kLogSoftmax) ? logf(s) : 0.0f;
    // One correctly rounded reciprocal per row, then a multiply per element: within 1 ulp of the
    // recipe's exp_x / sum_exp (the exponentials themselves are ~3 ulp), and a tenth of the
    // instructions of a full-precision division per element.
    const float inv_s = 1.0f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const u64 j = (u64)tx + (u64)i * tx_n;
      if (live && j < nvec) {
        float4 r;
        if (MODE == kSoftmax) {
          r.x = v[i].x * inv_s; r.y = v[i].y * inv_s; r.z = v[i].z * inv_s; r.w = v[i].w * inv_s;
        } else {
          r.x = v[i].x - lse; r.y = v[i].y - lse; r.z = v[i].z - lse; r.w = v[i].w - lse;
        }
        __stcs(yr + j, r);
      }
    }
  }
}

// The same kernel for rows the float4 kernel above cannot take: a row length that is not a multiple
// of 4, or rows that do not start on a 16-byte boundary (up to 8192 elements).
// VEC = 4: every row is covered by the ALIGNED float4 vectors that overlap it; a row that starts
//   `phase` floats into its first vector has phase + cols elements to cover, the vectors that lie
//   wholly inside the row move as float4, and the (at most two) vectors that hang over an end of the
//   row are read and written element by element, so nothing outside the row is touched. The output
//   row must start at the same phase (same shape and strides, equally aligned bases).
// VEC = 1: scalar accesses throughout, for outputs whose phase differs.
// This form measured 4 % slower than the kernel above on [65536, 4096], which therefore keeps the
// aligned rows.
template <int MODE, int VPT, int VEC>
__global__ void __launch_bounds__(kSmThreads, 4)
softmax_fast_any_kernel(const float *__restrict__ x, float *__restrict__ y, const int *__restrict__ labels,
                    SmRows g, int log_tx, float *row_loss) {
  __shared__ float red_smem[kSmThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int tx_n = 1 << log_tx;
  const int tx = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> log_tx;
  const int rows_per_cta = kSmThreads >> log_tx;
  // Every thread of the CTA reaches both row_reduce calls (they synchronise when TX > 32).
  { // one group of rows per CTA (the grid covers every row)
    const u64 row = (u64)blockIdx.x * rows_per_cta + ty;
    const bool live = row < g.rows;
    u64 yoff = 0, ioff[2] = {0, 0};
    if (live) g.outer.offsets(row, &yoff, ioff);
    // element e of the covering vectors is element e - lo of the row; valid for lo <= e < hi
    const unsigned lo = VEC == 4 ? (unsigned)(((uintptr_t)(x + ioff[0]) >> 2) & 3) : 0;
    const unsigned hi = lo + (unsigned)g.cols;
    const unsigned nvec = (hi + VEC - 1) / VEC;
    const float *xr = x + ioff[0] - lo;
    auto whole = [&](unsigned j) { return VEC == 1 || (j * VEC >= lo && j * VEC + VEC <= hi); };
    auto valid = [&](unsigned j, int k) { return j * VEC + k >= lo && j * VEC + k < hi; };

    float v[VPT][VEC];
    float m = -FLT_MAX; // src/kernels/cpu/reduce_ops.c:273
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * tx_n;
      if (live && j < nvec) {
        if (VEC == 4 && whole(j)) {
          const float4 t = __ldcs(reinterpret_cast<const float4 *>(xr) + j);
          v[i][0] = t.x; v[i][1] = t.y; v[i][VEC > 2 ? 2 : 0] = t.z; v[i][VEC > 3 ? 3 : 0] = t.w;
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) v[i][k] = valid(j, k) ? __ldcs(xr + j * VEC + k) : -FLT_MAX;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * tx_n;
      if (live && j < nvec) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) m = fmaxf(m, v[i][k]); // the fill value of an overhang never wins
      }
    }
    m = row_reduce<MaxOp, true>(m, log_tx, red_smem);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * tx_n;
      if (live && j < nvec) {
        // sub, then exp: two separately rounded ops
        float e[VEC];
        const bool all = whole(j);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          v[i][k] = v[i][k] - m;
          e[k] = (all || valid(j, k)) ? exp_softmax(v[i][k]) : 0.0f;
          if (MODE == kSoftmax) v[i][k] = e[k];
        }
        s += VEC == 4 ? (e[0] + e[1]) + (e[VEC > 2 ? 2 : 0] + e[VEC > 3 ? 3 : 0]) : e[0];
      }
    }
    s = row_reduce<SumOp, true>(s, log_tx, red_smem);

    if (MODE == kCrossEntropy) {
      // loss_row = -((x[label] - m) - log(s)); v[] still holds x - m, so the thread that loaded
      // the label's vector picks it from its registers (no second trip to memory).
      if (live) {
        const int label = labels[row];
        if (label >= 0 && (u64)label < g.cols) {
          const unsigned at = (unsigned)label + lo;
          const unsigned jv = at / VEC;
          if ((int)(jv & (unsigned)(tx_n - 1)) == tx) {
            const int slot = (int)(jv >> log_tx), comp = (int)(at % VEC);
            float sh = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
              for (int k = 0; k < VEC; ++k)
                if (i == slot && k == comp) sh = v[i][k];
            row_loss[row] = -(sh - logf(s));
          }
        } else if (tx == 0) {
          row_loss[row] = 0.0f; // label outside [0, cols): contributes nothing
        }
      }
      return;
    }

    float *yr = y + yoff - lo;
    const float lse = (MODE == kLogSoftmax) ? logf(s) : 0.0f;
    // One correctly rounded reciprocal per row, then a multiply per element: within 1 ulp of the
    // recipe's exp_x / sum_exp (the exponentials themselves are ~3 ulp), and a tenth of the
    // instructions of a full-precision division per element.
    const float inv_s = 1.0f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * tx_n;
      if (live && j < nvec) {
        float r[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) r[k] = (MODE == kSoftmax) ? v[i][k] * inv_s : v[i][k] - lse;
        if (VEC == 4 && whole(j)) {
          __stcs(reinterpret_cast<float4 *>(yr) + j, make_float4(r[0], r[1], r[VEC > 2 ? 2 : 0], r[VEC > 3 ? 3 : 0]));
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k)
            if (valid(j, k)) __stcs(yr + j * VEC + k, r[k]);
        }
      }
    }
  }
}

// ---- forward, rows of 8193 ... 65536 elements: one thread-block cluster per row -------------------------
// The CTAs of a cluster (2, 4 or 8 x 256 threads) take consecutive slices of ONE row, each slice in
// registers as above, so the row is read once and written once. Every CTA reduces its slice to a
// pair (m_i, s_i = sum exp(x - m_i)), stores the pair into slot `rank` of EVERY CTA of the cluster
// (distributed shared memory), and after ONE cluster barrier reads all pairs from its own shared
// memory: m = max m_i, s = sum s_i * exp(m_i - m); its elements leave as exp(x - m_i) * (exp(m_i - m) / s)
// or (x - m_i) + ((m_i - m) - log s). Nobody reads a neighbour's memory after the barrier, so CTAs
// leave without a second one; the barrier that makes sure every CTA of the cluster is running
// before its memory is written is split (arrive at entry, wait right before the stores).
constexpr int kSmMaxCluster = 8;
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

template <int MODE>
__global__ void __launch_bounds__(kSmThreads, 4)
softmax_cluster_kernel(const float *__restrict__ x, float *__restrict__ y, SmRows g, unsigned cluster_n) {
  constexpr int VPT = kSmMaxVpt;
  __shared__ float red_smem[kSmThreads / 32];
  __shared__ float2 pairs[kSmMaxCluster]; // (m_i, s_i) of every CTA of the cluster, written by their owners
  cluster_arrive();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned rank = blockIdx.x % cluster_n; // cluster dims (cluster_n, 1, 1): rank in the cluster
  const u64 row = blockIdx.x / cluster_n;
  const u64 all_vec = g.cols >> 2;
  const u64 slice = (all_vec + cluster_n - 1) / cluster_n;
  const u64 first = (u64)rank * slice;
  const u64 nvec = first >= all_vec ? 0 : (all_vec - first < slice ? all_vec - first : slice);
  u64 yoff = 0, ioff[2] = {0, 0};
  g.outer.offsets(row, &yoff, ioff);
  const float4 *xr = reinterpret_cast<const float4 *>(x + ioff[0]) + first;
  float4 v[VPT];
  float m = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const u64 j = (u64)threadIdx.x + (u64)i * kSmThreads;
    if (j < nvec) v[i] = __ldcs(xr + j);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const u64 j = (u64)threadIdx.x + (u64)i * kSmThreads;
    if (j < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
  }
  m = row_reduce<MaxOp>(m, 8, red_smem);
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const u64 j = (u64)threadIdx.x + (u64)i * kSmThreads;
    if (j < nvec) {
      v[i].x = v[i].x - m; v[i].y = v[i].y - m; v[i].z = v[i].z - m; v[i].w = v[i].w - m;
      const float e0 = exp_softmax(v[i].x), e1 = exp_softmax(v[i].y), e2 = exp_softmax(v[i].z), e3 = exp_softmax(v[i].w);
      s += (e0 + e1) + (e2 + e3);
      if (MODE == kSoftmax) v[i] = make_float4(e0, e1, e2, e3);
    }
  }
  s = row_reduce<SumOp>(s, 8, red_smem);
  cluster_wait(); // every CTA of the cluster has started: its shared memory may be written
  if (threadIdx.x < cluster_n) {
    cooperative_groups::cluster_group cl = cooperative_groups::this_cluster();
    float2 *theirs = cl.map_shared_rank(pairs, threadIdx.x);
    theirs[rank] = make_float2(m, s);
  }
  cluster_arrive();
  cluster_wait();
  float gm = -FLT_MAX;
  for (unsigned c = 0; c < cluster_n; ++c) gm = fmaxf(gm, pairs[c].x);
  float gs = 0.0f;
  for (unsigned c = 0; c < cluster_n; ++c) gs += pairs[c].y * exp_softmax(pairs[c].x - gm);
  float4 *yr = reinterpret_cast<float4 *>(y + yoff) + first;
  // softmax: one factor per CTA; log-softmax: one offset per CTA
  const float k = (MODE == kSoftmax) ? exp_softmax(m - gm) * (1.0f / gs) : (m - gm) - logf(gs);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const u64 j = (u64)threadIdx.x + (u64)i * kSmThreads;
    if (j < nvec) {
      float4 r;
      if (MODE == kSoftmax) {
        r.x = v[i].x * k; r.y = v[i].y * k; r.z = v[i].z * k; r.w = v[i].w * k;
      } else {
        r.x = v[i].x + k; r.y = v[i].y + k; r.z = v[i].z + k; r.w = v[i].w + k;
      }
      __stcs(yr + j, r);
    }
  }
}

// ---- forward, tiny rows (<= 64 classes: a 10-way classifier head) ---------------------------------------
// Dense rows this short leave most lanes of any per-row thread group idle. Here a CTA moves 256
// whole rows between global and shared memory with fully coalesced accesses (row stride in shared
// memory made odd: conflict-free for the next step), and every THREAD owns one row there: max, the
// exponentials and their sum, the results written back in place, no shuffles.
constexpr int kTinyCols = 64;
template <int MODE>
__global__ void __launch_bounds__(kSmThreads)
softmax_tiny_rows_kernel(const float *__restrict__ x, float *__restrict__ y, const int *__restrict__ labels,
                         u64 rows, unsigned cols, unsigned div_magic, float *row_loss) {
  extern __shared__ float tile[]; // kSmThreads rows of (cols | 1) floats
  pdl_wait();
  pdl_launch_dependents();
  const unsigned stride = cols | 1u;
  const u64 row0 = (u64)blockIdx.x * kSmThreads;
  const unsigned n_rows = (unsigned)(rows - row0 < (u64)kSmThreads ? rows - row0 : (u64)kSmThreads);
  const unsigned n = n_rows * cols;
  const float *xs = x + row0 * cols;
  for (unsigned i = threadIdx.x; i < n; i += kSmThreads) {
    const unsigned r = (unsigned)(((u64)i * div_magic) >> 21); // i / cols for i < 2^15, cols <= 64
    tile[r * stride + (i - r * cols)] = __ldcs(xs + i);
  }
  __syncthreads();
  if (threadIdx.x < n_rows) {
    float *mine = tile + threadIdx.x * stride;
    float m = -FLT_MAX; // src/kernels/cpu/reduce_ops.c:273
    for (unsigned c = 0; c < cols; ++c) m = fmaxf(m, mine[c]);
    float sum = 0.0f;
    for (unsigned c = 0; c < cols; ++c) {
      const float sh = mine[c] - m; // sub, then exp: two separately rounded ops
      const float e = exp_softmax(sh);
      sum += e;
      mine[c] = (MODE == kSoftmax) ? e : sh;
    }
    if (MODE == kCrossEntropy) {
      const int label = labels[row0 + threadIdx.x];
      row_loss[row0 + threadIdx.x] = (label >= 0 && (unsigned)label < cols) ? -(mine[label] - logf(sum)) : 0.0f;
    } else if (MODE == kSoftmax) {
      const float inv_s = 1.0f / sum; // as in the fast kernel: one reciprocal per row
      for (unsigned c = 0; c < cols; ++c) mine[c] *= inv_s;
    } else {
      const float lse = logf(sum);
      for (unsigned c = 0; c < cols; ++c) mine[c] -= lse;
    }
  }
  if (MODE == kCrossEntropy) return;
  __syncthreads();
  float *ys = y + row0 * cols;
  for (unsigned i = threadIdx.x; i < n; i += kSmThreads) {
    const unsigned r = (unsigned)(((u64)i * div_magic) >> 21);
    __stcs(ys + i, tile[r * stride + (i - r * cols)]);
  }
}

// ---- forward, generic path: online (max, sum) ---------------------------------------------------------
struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  // sum of exp(x - m) re-based onto the larger maximum
  if (a.m >= b.m) return MaxSum{a.m, a.s + b.s * exp_softmax(b.m - a.m)};
  return MaxSum{b.m, b.s + a.s * exp_softmax(a.m - b.m)};
}
__device__ __forceinline__ MaxSum ms_block_reduce(MaxSum v) {
  __shared__ MaxSum sm[kSmThreads / 32];
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = ms_combine(v, t);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  v = sm[0];
  for (int w = 1; w < kSmThreads / 32; ++w) v = ms_combine(v, sm[w]);
  return v; // valid in every thread
}

template <int MODE>
__global__ void __launch_bounds__(kSmThreads)
softmax_generic_kernel(const float *x, float *y, const int *labels, SmRows g, float *row_loss) {
  pdl_wait();
  pdl_launch_dependents();
  for (u64 row = blockIdx.x; row < g.rows; row += gridDim.x) {
    u64 yoff = 0, ioff[2] = {0, 0};
    g.outer.offsets(row, &yoff, ioff);
    const float *xr = x + ioff[0];
    float *yr = y + yoff;
    // Rows that are contiguous along the axis (any length, any alignment: a 50257-wide vocabulary)
    // are walked as a scalar head up to the first 16-byte boundary, a float4 body and a scalar tail;
    // the output row must share the input row's alignment phase to be written as float4 too.
    const bool unit = g.x_axis_stride == 1 && (MODE == kCrossEntropy || g.y_axis_stride == 1);
    const bool vec = unit && (MODE == kCrossEntropy || (((uintptr_t)xr ^ (uintptr_t)yr) & 15) == 0);
    u64 head = 0, nvec = 0;
    if (vec) {
      head = ((16 - ((uintptr_t)xr & 15)) & 15) / sizeof(float);
      if (head > g.cols) head = g.cols;
      nvec = (g.cols - head) >> 2;
    }
    const u64 tail_begin = head + (nvec << 2); // [0, head) and [tail_begin, cols) are scalar
    MaxSum acc{-FLT_MAX, 0.0f};
    auto take = [&](float xv) {
      if (xv > acc.m) {
        acc.s = acc.s * exp_softmax(acc.m - xv) + 1.0f;
        acc.m = xv;
      } else {
        acc.s += exp_softmax(xv - acc.m);
      }
    };
    if (vec) {
      const float4 *xb = reinterpret_cast<const float4 *>(xr + head);
      // batches of four float4 per thread: all loads first, one re-basing per batch
      for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec) v[u] = __ldg(xb + j0 + (u64)u * kSmThreads);
        float bm = -FLT_MAX;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec) bm = fmaxf(bm, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
        if (bm > acc.m) {
          acc.s *= exp_softmax(acc.m - bm);
          acc.m = bm;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec)
            acc.s += (exp_softmax(v[u].x - acc.m) + exp_softmax(v[u].y - acc.m)) +
                     (exp_softmax(v[u].z - acc.m) + exp_softmax(v[u].w - acc.m));
      }
      const u64 loose = head + (g.cols - tail_begin);
      if (threadIdx.x < loose) take(xr[threadIdx.x < head ? threadIdx.x : tail_begin + (threadIdx.x - head)]);
    } else {
      for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads) take(xr[j * g.x_axis_stride]);
    }
    acc = ms_block_reduce(acc);
    if (MODE == kCrossEntropy) {
      if (threadIdx.x == 0) {
        const int label = labels[row];
        float loss = 0.0f;
        if (label >= 0 && (u64)label < g.cols) {
          const float sh = xr[(u64)label * g.x_axis_stride] - acc.m;
          loss = -(sh - logf(acc.s));
        }
        row_loss[row] = loss;
      }
      continue;
    }
    const float lse = (MODE == kLogSoftmax) ? logf(acc.s) : 0.0f;
    auto finish = [&](float xv) {
      const float sh = xv - acc.m;
      return (MODE == kSoftmax) ? exp_softmax(sh) / acc.s : sh - lse;
    };
    if (vec) {
      // the row was just read by this CTA: the second pass finds it in L2
      const float4 *xb = reinterpret_cast<const float4 *>(xr + head);
      float4 *yb = reinterpret_cast<float4 *>(yr + head);
      for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec) v[u] = __ldcs(xb + j0 + (u64)u * kSmThreads);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec)
            __stcs(yb + j0 + (u64)u * kSmThreads, make_float4(finish(v[u].x), finish(v[u].y), finish(v[u].z), finish(v[u].w)));
      }
      const u64 loose = head + (g.cols - tail_begin);
      if (threadIdx.x < loose) {
        const u64 j = threadIdx.x < head ? threadIdx.x : tail_begin + (threadIdx.x - head);
        yr[j] = finish(xr[j]);
      }
    } else {
      for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads)
        yr[j * g.y_axis_stride] = finish(xr[j * g.x_axis_stride]);
    }
  }
}

// ---- cross entropy, streaming rows ------------------------------------------------------------------
// Cross entropy needs only max, sum(exp(x - max)) and x[label] of a row, so the row does not have
// to stay on chip: a warp streams it once with eight float4 loads in flight per lane and keeps a
// running (max, sum) pair per lane, re-based whenever a batch raises the maximum. With no row held
// in registers, 48+ warps fit per SM, which is what a read-only kernel needs to cover HBM latency
// (the register-resident kernel above tops out near 4.4 TB/s on [65536, 4096]).
constexpr int kCeBatch = 4; // float4 per lane per batch; two batches alternate
constexpr float kLog2e = 1.4426950408889634f;
// 2^(x * log2(e) - m2) with m2 = max * log2(e): exp(x - max) for the running sum. The argument is
// clamped at -150 (2^-150 is 0 in fp32) so a -FLT_MAX start value cannot overflow the product.
__device__ __forceinline__ float exp2_sum_term(float x, float m2) {
  float t = __fmaf_rn(fmaxf(x, -1.0e30f), kLog2e, -m2);
  t = fmaxf(t, -150.0f);
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
// The same term without the clamps, for callers that keep m2 finite: x = -inf or -FLT_MAX gives
// 2^(-inf) = 0, never inf - inf.
__device__ __forceinline__ float exp2_term_fast(float x, float m2) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fmaf_rn(x, kLog2e, -m2)));
  return r;
}
__global__ void __launch_bounds__(kSmThreads)
cross_entropy_rows_kernel(const float *__restrict__ x, const int *__restrict__ labels, SmRows g,
                          float *__restrict__ mean_out, unsigned int *counter, float *partials, const PeerLink *peer,
                          float global_count) {
  pdl_wait();
  pdl_launch_dependents();
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float warp_loss = 0.0f; // lane 0: sum of the losses of this warp's rows
  const unsigned warps_per_cta = kSmThreads / 32;
  const unsigned nvec = (unsigned)(g.cols >> 2);
  // The label and the logit it selects are two dependent loads; fetched at the end of a row they
  // would leave the warp idle for two memory latencies per row (~15 % of a 16 KiB row's time). The
  // label of the NEXT row is therefore requested while this row streams, and the selected logit at
  // the top of its row, so both have arrived long before they are used.
  const u64 row_step = (u64)gridDim.x * warps_per_cta;
  u64 row = (u64)blockIdx.x * warps_per_cta + warp;
  int label_next = row < g.rows ? __ldg(labels + row) : 0;
  for (; row < g.rows; row += row_step) {
    const int label = label_next;
    if (row + row_step < g.rows) label_next = __ldg(labels + row + row_step);
    u64 yoff = 0, ioff[2] = {0, 0};
    g.outer.offsets(row, &yoff, ioff);
    const float4 *xr = reinterpret_cast<const float4 *>(x + ioff[0]);
    const bool label_ok = label >= 0 && (u64)label < g.cols;
    const float x_label = label_ok ? __ldg(x + ioff[0] + label) : 0.0f;
    MaxSum acc{-FLT_MAX, 0.0f};
    // start of this warp's next row, for the prefetch below
    const float4 *xr_next = nullptr;
    if (row + row_step < g.rows) {
      u64 yoff2 = 0, ioff2[2] = {0, 0};
      g.outer.offsets(row + row_step, &yoff2, ioff2);
      xr_next = reinterpret_cast<const float4 *>(x + ioff2[0]);
    }
    // Two batches of kCeBatch float4 per lane alternate: while one is summed the loads of the next
    // are already in flight, and L2 is asked for the batch after that (lanes 0-15 take one
    // 128-byte line each of its 2 KiB; past the end of the row it is the head of the next row).
    const unsigned batch_vecs = kCeBatch * 32;
    const unsigned nvec_padded = (nvec + batch_vecs - 1) / batch_vecs * batch_vecs;
    auto load_batch = [&](float4(&v)[kCeBatch], unsigned b) {
#pragma unroll
      for (int u = 0; u < kCeBatch; ++u)
        if (b + u * 32 < nvec) v[u] = __ldcs(xr + b + u * 32);
    };
    auto prefetch_batch = [&](unsigned first) { // first: float4 index where that batch starts
      if (lane >= 16) return;
      const unsigned t = first + lane * 8;
      const float4 *pf = nullptr;
      if (t < nvec) pf = xr + t;
      else if (xr_next && t >= nvec_padded && t - nvec_padded < nvec) pf = xr_next + (t - nvec_padded);
      if (pf) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf));
    };
    auto sum_batch = [&](const float4(&v)[kCeBatch], unsigned b) {
      float bm = -FLT_MAX;
#pragma unroll
      for (int u = 0; u < kCeBatch; ++u)
        if (b + u * 32 < nvec) bm = fmaxf(bm, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
      if (bm > acc.m) {
        acc.s *= exp2_sum_term(acc.m, bm * kLog2e);
        acc.m = bm;
      }
      // Only the SUM of the exponentials is needed (its log enters the loss), and terms far below
      // the maximum do not move it, so each term is one FMA + ex2.approx: 2^(x log2e - m log2e).
      // Its relative error grows with |x - m| (about |x - m| * 1e-7) exactly where the term is
      // negligible; the sum stays within 1e-6 of the accurate one. m2 is kept finite so that a row
      // of -inf cannot produce inf - inf.
      const float m2 = fmaxf(acc.m * kLog2e, -3.0e38f);
#pragma unroll
      for (int u = 0; u < kCeBatch; ++u)
        if (b + u * 32 < nvec)
          acc.s += (exp2_term_fast(v[u].x, m2) + exp2_term_fast(v[u].y, m2)) +
                   (exp2_term_fast(v[u].z, m2) + exp2_term_fast(v[u].w, m2));
    };
    float4 va[kCeBatch], vb[kCeBatch];
    unsigned b = lane; // b - lane is the same in every lane, so the branches below are uniform
    load_batch(va, b);
    while (true) {
      const unsigned b1 = b + batch_vecs;
      const bool more1 = b1 - lane < nvec;
      if (more1) load_batch(vb, b1);
      prefetch_batch(b1 - lane + batch_vecs);
      sum_batch(va, b);
      if (!more1) break;
      const unsigned b2 = b1 + batch_vecs;
      const bool more2 = b2 - lane < nvec;
      if (more2) load_batch(va, b2);
      prefetch_batch(b2 - lane + batch_vecs);
      sum_batch(vb, b1);
      if (!more2) break;
      b = b2;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxSum t;
      t.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
      t.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
      acc = ms_combine(acc, t);
    }
    if (lane == 0 && label_ok) {
      const float sh = x_label - acc.m;
      warp_loss += -(sh - logf(acc.s));
    }
  }
  // mean over all rows: one partial per CTA, combined by the last CTA to arrive (fixed order)
  const float part = block_reduce<SumOp>(warp_loss);
  if (threadIdx.x == 0) partials[blockIdx.x] = part;
  if (!take_ticket(counter, gridDim.x)) return;
  float tot = 0.0f;
  for (unsigned c = threadIdx.x; c < gridDim.x; c += kSmThreads) tot += __ldcg(partials + c);
  __syncthreads();
  tot = block_reduce<SumOp>(tot);
  if (threadIdx.x == 0) {
    // Row-sharded logits: the loss SUMS of all ranks are exchanged right here (one thread, after
    // the grid has retired) and divided by the global row count: never a mean of means.
    if (peer != nullptr) mean_out[0] = peer_exchange_scalar(*peer, tot, PLAST_B200_PEER_SUM) / global_count;
    else mean_out[0] = tot / (float)g.rows; // src/kernels/cpu/reduce_ops.c:13
  }
}

// ---- backward ---------------------------------------------------------------------------------------
// One CTA per row, strided scalar access (rows are re-read from L2 for the second pass).
//   softmax      dx += y * (dy - sum(dy * y))
//   log_softmax  dx += dy - exp(y) * sum(dy)
//   cross_entropy (mean)  dlogits += (softmax(x) - onehot(label)) * dout / rows
template <int MODE>
__global__ void __launch_bounds__(kSmThreads, 2)
softmax_backward_kernel(const float *y_or_x, const float *dy, float *dx, const int *labels, SmRows g) {
  pdl_wait();
  pdl_launch_dependents();
  for (u64 row = blockIdx.x; row < g.rows; row += gridDim.x) {
    u64 doff = 0, ioff[2] = {0, 0};
    g.outer.offsets(row, &doff, ioff);
    const float *a = y_or_x + ioff[0]; // y (softmax / log_softmax) or logits x (cross entropy)
    float *dxr = dx + doff;
    const float *dyr = dy + ioff[1];
    // Long rows (a 32000 ... 128256-wide vocabulary) whose three tensors are contiguous along the axis
    // and 16-byte aligned are walked as float4 in batches of four loads per thread; the second pass
    // finds the row in L2.
    const bool vec = (g.cols & 3) == 0 && g.x_axis_stride == 1 && g.y_axis_stride == 1 &&
                     (MODE == kCrossEntropy || g.z_axis_stride == 1) &&
                     ((((uintptr_t)a | (uintptr_t)dxr | (MODE == kCrossEntropy ? 0 : (uintptr_t)dyr)) & 15) == 0);
    const u64 nvec = g.cols >> 2;
    if (MODE == kCrossEntropy) {
      MaxSum acc{-FLT_MAX, 0.0f};
      if (vec) {
        const float4 *xb = reinterpret_cast<const float4 *>(a);
        for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + (u64)u * kSmThreads < nvec) v[u] = __ldg(xb + j0 + (u64)u * kSmThreads);
          float bm = -FLT_MAX;
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + (u64)u * kSmThreads < nvec) bm = fmaxf(bm, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
          if (bm > acc.m) {
            acc.s *= exp_softmax(acc.m - bm);
            acc.m = bm;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + (u64)u * kSmThreads < nvec)
              acc.s += (exp_softmax(v[u].x - acc.m) + exp_softmax(v[u].y - acc.m)) +
                       (exp_softmax(v[u].z - acc.m) + exp_softmax(v[u].w - acc.m));
        }
      } else {
        for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads) {
          const float xv = a[j * g.x_axis_stride];
          if (xv > acc.m) {
            acc.s = acc.s * exp_softmax(acc.m - xv) + 1.0f;
            acc.m = xv;
          } else {
            acc.s += exp_softmax(xv - acc.m);
          }
        }
      }
      acc = ms_block_reduce(acc);
      const float gscale = dy[0] / (float)g.rows;
      const int label = labels[row];
      if (vec) {
        const float4 *xb = reinterpret_cast<const float4 *>(a);
        float4 *db = reinterpret_cast<float4 *>(dxr);
        const float inv_s = 1.0f / acc.s;
        for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
          float4 v[4], o[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + (u64)u * kSmThreads < nvec) {
              v[u] = __ldcs(xb + j0 + (u64)u * kSmThreads);
              o[u] = __ldcs(db + j0 + (u64)u * kSmThreads);
            }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const u64 j = j0 + (u64)u * kSmThreads;
            if (j < nvec) {
              const long e0 = (long)(j << 2);
              o[u].x += (exp_softmax(v[u].x - acc.m) * inv_s - (label == e0 ? 1.0f : 0.0f)) * gscale;
              o[u].y += (exp_softmax(v[u].y - acc.m) * inv_s - (label == e0 + 1 ? 1.0f : 0.0f)) * gscale;
              o[u].z += (exp_softmax(v[u].z - acc.m) * inv_s - (label == e0 + 2 ? 1.0f : 0.0f)) * gscale;
              o[u].w += (exp_softmax(v[u].w - acc.m) * inv_s - (label == e0 + 3 ? 1.0f : 0.0f)) * gscale;
              __stcs(db + j, o[u]);
            }
          }
        }
      } else {
        for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads) {
          const float p = exp_softmax(a[j * g.x_axis_stride] - acc.m) / acc.s;
          const float t = ((u64)label == j) ? 1.0f : 0.0f;
          dxr[j * g.y_axis_stride] += (p - t) * gscale;
        }
      }
      continue;
    }
    float part = 0.0f;
    if (vec) {
      const float4 *yb = reinterpret_cast<const float4 *>(a), *gb = reinterpret_cast<const float4 *>(dyr);
      for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
        float4 v[4], d[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec) {
            d[u] = __ldg(gb + j0 + (u64)u * kSmThreads);
            if (MODE == kSoftmax) v[u] = __ldg(yb + j0 + (u64)u * kSmThreads);
          }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec)
            part += (MODE == kSoftmax) ? (d[u].x * v[u].x + d[u].y * v[u].y) + (d[u].z * v[u].z + d[u].w * v[u].w)
                                       : (d[u].x + d[u].y) + (d[u].z + d[u].w);
      }
    } else {
      for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads) {
        const float d = dyr[j * g.z_axis_stride];
        part += (MODE == kSoftmax) ? d * a[j * g.x_axis_stride] : d;
      }
    }
    __syncthreads();
    float tot = block_reduce<SumOp>(part);
    __shared__ float bcast;
    if (threadIdx.x == 0) bcast = tot;
    __syncthreads();
    tot = bcast;
    if (vec) {
      const float4 *yb = reinterpret_cast<const float4 *>(a), *gb = reinterpret_cast<const float4 *>(dyr);
      float4 *db = reinterpret_cast<float4 *>(dxr);
      for (u64 j0 = threadIdx.x; j0 < nvec; j0 += 4 * kSmThreads) {
        float4 v[4], d[4], o[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + (u64)u * kSmThreads < nvec) {
            v[u] = __ldcs(yb + j0 + (u64)u * kSmThreads);
            d[u] = __ldcs(gb + j0 + (u64)u * kSmThreads);
            o[u] = __ldcs(db + j0 + (u64)u * kSmThreads);
          }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const u64 j = j0 + (u64)u * kSmThreads;
          if (j < nvec) {
            if (MODE == kSoftmax) {
              o[u].x += v[u].x * (d[u].x - tot); o[u].y += v[u].y * (d[u].y - tot);
              o[u].z += v[u].z * (d[u].z - tot); o[u].w += v[u].w * (d[u].w - tot);
            } else {
              o[u].x += d[u].x - exp_softmax(v[u].x) * tot; o[u].y += d[u].y - exp_softmax(v[u].y) * tot;
              o[u].z += d[u].z - exp_softmax(v[u].z) * tot; o[u].w += d[u].w - exp_softmax(v[u].w) * tot;
            }
            __stcs(db + j, o[u]);
          }
        }
      }
    } else {
      for (u64 j = threadIdx.x; j < g.cols; j += kSmThreads) {
        const float d = dyr[j * g.z_axis_stride];
        const float yv = a[j * g.x_axis_stride];
        const float gr = (MODE == kSoftmax) ? yv * (d - tot) : d - exp_softmax(yv) * tot;
        dxr[j * g.y_axis_stride] += gr;
      }
    }
  }
}

// ---- host ---------------------------------------------------------------------------------------------
// Describes "rows along `axis`" of tensors that share x's shape. t = tensor written / indexed
// by tstride (output or dx), x = first input, z = optional second input (dy).
static bool make_rows(const char *name, const Tensor *x, const Tensor *t, const Tensor *z, u64 axis,
                      SmRows *g) {
  if (x->ndim == 0 || axis >= x->ndim) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: axis %llu out of range for %llu dims", name,
              (unsigned long long)axis, (unsigned long long)x->ndim);
    return false;
  }
  g->cols = x->shape[axis];
  g->rows = 1;
  g->x_axis_stride = x->strides[axis];
  g->y_axis_stride = t ? t->strides[axis] : 0;
  g->z_axis_stride = z ? z->strides[axis] : 0;
  int n = 0;
  for (u64 d = x->ndim; d-- > 0;) { // innermost first
    if (d == axis || x->shape[d] == 1) continue;
    g->outer.size[n] = x->shape[d];
    g->outer.tstride[n] = t ? t->strides[d] : 0;
    g->outer.istride[0][n] = x->strides[d];
    g->outer.istride[1][n] = z ? z->strides[d] : 0;
    g->rows *= x->shape[d];
    ++n;
  }
  g->outer.n = n;
  for (int d = n; d < MAX_NDIM; ++d) {
    g->outer.size[d] = 1;
    g->outer.tstride[d] = g->outer.istride[0][d] = g->outer.istride[1][d] = 0;
  }
  return true;
}

static bool fast_ok(const SmRows &g, const void *x, const void *y, bool writes_rows, unsigned max_cluster = 1) {
  if (g.cols == 0 || (g.cols & 3) || g.cols > (u64)kSmThreads * 4 * kSmMaxVpt * max_cluster) return false;
  if (g.x_axis_stride != 1 || ((uintptr_t)x & 15)) return false;
  if (writes_rows && (g.y_axis_stride != 1 || ((uintptr_t)y & 15))) return false;
  for (int d = 0; d < g.outer.n; ++d) {
    if (g.outer.istride[0][d] & 3) return false;
    if (writes_rows && (g.outer.tstride[d] & 3)) return false;
  }
  return true;
}
// The same kernel with scalar accesses: any row length up to 2048 along a unit-stride axis.
static bool fast_scalar_ok(const SmRows &g, bool writes_rows) {
  if (g.cols == 0 || g.cols > (u64)kSmThreads * kSmMaxVpt) return false;
  return g.x_axis_stride == 1 && (!writes_rows || g.y_axis_stride == 1);
}
// Rows of any length up to 8188 and any alignment, as aligned float4 vectors with ragged ends: the
// output rows must start at the same phase of a 16-byte vector as the input rows.
static bool fast_ragged_ok(const SmRows &g, const void *x, const void *y, bool writes_rows) {
  if (g.cols < 8 || g.cols + 6 > (u64)kSmThreads * 4 * kSmMaxVpt || g.x_axis_stride != 1) return false;
  if (!writes_rows) return true;
  if (g.y_axis_stride != 1 || ((((uintptr_t)x ^ (uintptr_t)y) >> 2) & 3) != 0) return false;
  for (int d = 0; d < g.outer.n; ++d)
    if ((g.outer.istride[0][d] - g.outer.tstride[d]) & 3) return false;
  return true;
}

template <int MODE>
static void softmax_family_forward(const char *name, const Tensor **inputs, Tensor *output,
                                   KernelParams params) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name)) return;
  const Tensor *x = inputs[0];
  if (x->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", name, (int)x->dtype);
    return;
  }
  const int *labels = nullptr;
  u64 axis = params.dim;
  if (MODE == kCrossEntropy) {
    if (!check_tensor(inputs[1], name)) return;
    if (inputs[1]->dtype != INT32) {
      set_error(PLAST_B200_ERR_DTYPE, "%s: labels must be INT32 class indices", name);
      return;
    }
    if (x->ndim != 2 || inputs[1]->ndim != 1 || inputs[1]->shape[0] != x->shape[0] ||
        inputs[1]->strides[0] != 1) {
      set_error(PLAST_B200_ERR_SHAPE, "%s: expects logits [N,C] and contiguous labels [N]", name);
      return;
    }
    labels = (const int *)inputs[1]->data;
    axis = 1; // plast/nn/functional.py:322
  }
  SmRows g;
  if (!make_rows(name, x, MODE == kCrossEntropy ? nullptr : output, nullptr, axis, &g)) return;
  if (g.rows == 0 || g.cols == 0) return;
  cudaStream_t s = stream();
  // softmax / log-softmax rows of up to 8 x 8192 elements: a cluster of up to eight CTAs per row
  const bool fast_vec = fast_ok(g, x->data, output->data, MODE != kCrossEntropy, MODE == kCrossEntropy ? 1 : 8);
  unsigned cluster_n = 1;
  if (fast_vec)
    while ((u64)kSmThreads * 4 * kSmMaxVpt * cluster_n < g.cols) cluster_n *= 2;
  // rows of at most 64 elements lying densely one after another, in x and in the output
  // (from 33 elements on only where the float4 kernel does not apply: it is faster at 64)
  bool tiny = g.cols <= (u64)(fast_vec ? 32 : kTinyCols) && g.x_axis_stride == 1 && (MODE == kCrossEntropy || g.y_axis_stride == 1);
  {
    u64 run = g.cols;
    for (int d = 0; tiny && d < g.outer.n; ++d) {
      if (g.outer.istride[0][d] != run || (MODE != kCrossEntropy && g.outer.tstride[d] != run)) tiny = false;
      run *= g.outer.size[d];
    }
  }
  const bool fast_ragged = !fast_vec && fast_ragged_ok(g, x->data, output->data, MODE != kCrossEntropy);
  const bool fast = fast_vec || fast_ragged || fast_scalar_ok(g, MODE != kCrossEntropy);
  // the streaming cross-entropy kernel takes rows of any length (float4 layout permitting)
  SmRows any_len = g;
  any_len.cols = g.cols > 4 ? 4 : g.cols;
  const bool fast_ok_any_cols = MODE == kCrossEntropy && (g.cols & 3) == 0 && g.cols < ((u64)1 << 33) &&
                                fast_ok(any_len, x->data, output->data, false);
  u64 grid;
  int log_tx = 5, vpt = 1;
  if (tiny) {
    grid = (g.rows + kSmThreads - 1) / kSmThreads;
  } else if (fast) {
    const u64 nvec = fast_vec ? ((g.cols >> 2) + cluster_n - 1) / cluster_n : (fast_ragged ? (g.cols + 6) >> 2 : g.cols);
    // Threads per row: the smallest power of two with <= 8 vectors per thread (eight loads in flight),
    // but at least 128 bytes per load instruction and row (8 float4 lanes, 32 scalar lanes) where the
    // row is that long: short rows take a slice of a warp each.
    log_tx = 0;
    while (((u64)kSmMaxVpt << log_tx) < nvec) ++log_tx;
    const int min_log_tx = (fast_vec || fast_ragged) ? 3 : 5;
    while (log_tx < min_log_tx && ((u64)1 << log_tx) < nvec) ++log_tx;
    if (cluster_n > 1) log_tx = 8; // the whole CTA on its slice of the row
    vpt = (int)((nvec + ((u64)1 << log_tx) - 1) >> log_tx);
    const u64 rows_per_cta = (u64)kSmThreads >> log_tx;
    grid = (g.rows + rows_per_cta - 1) / rows_per_cta; // one trip per CTA: many small CTAs balance best
    if (cluster_n > 1) grid = g.rows * cluster_n;
  } else {
    grid = g.rows;
    const u64 cap = (u64)sm_count() * 16;
    if (grid > cap) grid = cap;
  }
  // cross entropy: per-row losses go to scratch, then one full reduce takes their mean
  float *row_loss = nullptr;
  if (MODE == kCrossEntropy) {
    Workspace ws;
    if (!get_workspace(&ws)) return;
    if (g.rows > kPartialFloats / 2) {
      set_error(PLAST_B200_ERR_LIMIT, "%s: %llu rows exceed the per-row loss scratch (%llu)", name,
                (unsigned long long)g.rows, (unsigned long long)(kPartialFloats / 2));
      return;
    }
    row_loss = ws.partials + kPartialFloats / 2; // second half: never used by split partials
  }
  if (grid > 0x7fffffffull) {
    set_error(PLAST_B200_ERR_LIMIT, "%s: too many rows", name);
    return;
  }
  float *y = (float *)output->data;
  const float *xd = (const float *)x->data;
  if (MODE == kCrossEntropy && fast_ok_any_cols) {
    // one resident wave of CTAs that stride over the rows; a single launch yields the mean
    u64 ce_grid = (g.rows + kSmThreads / 32 - 1) / (kSmThreads / 32);
    static int ce_ctas_per_sm = 0; // resident CTAs per SM of this kernel
    if (ce_ctas_per_sm == 0) {
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ce_ctas_per_sm, cross_entropy_rows_kernel,
                                                        kSmThreads, 0) != cudaSuccess || ce_ctas_per_sm <= 0) {
        cudaGetLastError();
        ce_ctas_per_sm = 4;
      }
    }
    const u64 ce_cap = (u64)sm_count() * (u64)ce_ctas_per_sm;
    if (ce_grid > ce_cap) ce_grid = ce_cap;
    Workspace ws;
    if (!get_workspace(&ws)) return;
    const PeerLink *link = nullptr;
    float global_count = 0.0f;
    if (!take_peer_link(kPeerCrossEntropy, &link, &global_count)) link = nullptr;
    launch_k(cross_entropy_rows_kernel, dim3((unsigned)ce_grid), dim3(kSmThreads), 0, s, xd, labels, g, y, ws.counters,
             ws.partials, link, global_count);
    count_launch();
    note_kernel("cross_entropy_rows");
    end_call();
    return;
  } else if (tiny) {
    static bool ready = false;
    if (!ready) {
      cudaFuncSetAttribute(softmax_tiny_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)(kSmThreads * (kTinyCols + 1) * sizeof(float)));
      ready = true;
    }
    launch_k(softmax_tiny_rows_kernel<MODE>, dim3((unsigned)grid), dim3(kSmThreads),
             (size_t)kSmThreads * (g.cols | 1) * sizeof(float), s, xd, y, labels, g.rows, (unsigned)g.cols,
             (unsigned)(((u64)1 << 21) / g.cols + 1), row_loss);
  } else if (fast && cluster_n > 1) {
    if constexpr (MODE != kCrossEntropy)
      launch_kc(cluster_n, softmax_cluster_kernel<MODE>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, g, cluster_n);
  } else if (fast) {
    int v = 1;
    while (v < vpt) v <<= 1;
#define PB_SM_LAUNCH(VPT)                                                                                      \
  do {                                                                                                        \
    if (fast_vec && log_tx < 5) launch_k(softmax_fast_kernel<MODE, VPT, true>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, labels, g, log_tx, row_loss); \
    else if (fast_vec) launch_k(softmax_fast_kernel<MODE, VPT>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, labels, g, log_tx, row_loss); \
    else if (fast_ragged) launch_k(softmax_fast_any_kernel<MODE, VPT, 4>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, labels, g, log_tx, row_loss); \
    else launch_k(softmax_fast_any_kernel<MODE, VPT, 1>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, labels, g, log_tx, row_loss); \
  } while (0)
    switch (v) {
    case 1: PB_SM_LAUNCH(1); break;
    case 2: PB_SM_LAUNCH(2); break;
    case 4: PB_SM_LAUNCH(4); break;
    default: PB_SM_LAUNCH(8); break;
    }
#undef PB_SM_LAUNCH
  } else {
    launch_k(softmax_generic_kernel<MODE>, dim3((unsigned)grid), dim3(kSmThreads), 0, s, xd, y, labels, g, row_loss);
  }
  count_launch();
  if (MODE == kCrossEntropy) {
    // mean = sum(loss) / rows (plast/nn/functional.py:391-396, src/kernels/cpu/reduce_ops.c:13)
    const u64 shape[1] = {g.rows};
    u64 st[2][MAX_NDIM] = {};
    st[1][0] = 1;
    const bool red[1] = {true};
    IterPlan plan;
    make_plan(&plan, shape, 1, 2, st, red, 1);
    plan.reduced[0] = true;
    const float *ins[1] = {row_loss};
    PeerSuspend local_step; // a mean over THIS rank's rows; sharded callers use plast_b200_peer_cross_entropy_mean
    launch_reduce<SumOp, IdentityPro, 1>(plan, y, ins, IdentityPro{}, SumOp{}, false, (float)g.rows);
  }
  if (!failed())
    note_kernel((MODE == kCrossEntropy && fast_ok_any_cols) ? "cross_entropy_rows" :
                tiny ? (MODE == kSoftmax ? "softmax_tiny_rows" : (MODE == kLogSoftmax ? "log_softmax_tiny_rows" : "cross_entropy_tiny_rows")) :
                (fast && cluster_n > 1) ? (MODE == kSoftmax ? "softmax_fast_cluster" : "log_softmax_fast_cluster") :
                fast ? (MODE == kSoftmax ? "softmax_fast" : (MODE == kLogSoftmax ? "log_softmax_fast" : "cross_entropy_fast"))
                     : (MODE == kSoftmax ? "softmax_online" : (MODE == kLogSoftmax ? "log_softmax_online" : "cross_entropy_online")));
  end_call();
}

// ---- backward, fast path --------------------------------------------------------------------------------
// Rows contiguous along the axis in all three tensors, 16-byte aligned, cols % 4 == 0, cols <= 4096:
// the row of y (or of the logits), of dy and of dx in registers, TX threads per row as in the
// forward kernel; one read of each, one write of dx (backward ACCUMULATES into dx).
//   softmax       dx += y * (dy - sum(y * dy))
//   log_softmax   dx += dy - exp(y) * sum(dy)
//   cross_entropy dx += (softmax(x) - onehot(label)) * dloss / rows
// The dx row is requested together with the others (at most four vectors of each per thread).
template <int MODE, int VPT>
__global__ void __launch_bounds__(kSmThreads, 2)
softmax_backward_fast_kernel(const float *__restrict__ a, const float *__restrict__ dy, float *__restrict__ dx,
                             const int *__restrict__ labels, SmRows g, int log_tx) {
  __shared__ float red_smem[kSmThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  constexpr bool kEarlyDx = VPT <= 4;
  const int tx_n = 1 << log_tx;
  const int tx = threadIdx.x & (tx_n - 1), ty = threadIdx.x >> log_tx;
  const int rows_per_cta = kSmThreads >> log_tx;
  const unsigned nvec = (unsigned)(g.cols >> 2); // at most 1024: 32-bit index math in the loops
  const u64 row = (u64)blockIdx.x * rows_per_cta + ty;
  const bool live = row < g.rows;
  u64 doff = 0, ioff[2] = {0, 0};
  if (live) g.outer.offsets(row, &doff, ioff);
  const float4 *ar = reinterpret_cast<const float4 *>(a + ioff[0]);
  const float4 *dyr = reinterpret_cast<const float4 *>(dy + ioff[1]);
  float4 *dxr = reinterpret_cast<float4 *>(dx + doff);
  float4 va[VPT], vd[VPT], vx[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const unsigned j = (unsigned)tx + (unsigned)i * (unsigned)tx_n;
    if (live && j < nvec) {
      va[i] = __ldcs(ar + j);
      if (MODE != kCrossEntropy) vd[i] = __ldcs(dyr + j);
      if (kEarlyDx) vx[i] = __ldcs(dxr + j);
    }
  }
  float k0 = 0.0f, k1 = 0.0f; // per-row constants of the last pass
  if (MODE == kCrossEntropy) {
    float m = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * (unsigned)tx_n;
      if (live && j < nvec) m = fmaxf(m, fmaxf(fmaxf(va[i].x, va[i].y), fmaxf(va[i].z, va[i].w)));
    }
    m = row_reduce<MaxOp, true>(m, log_tx, red_smem);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * (unsigned)tx_n;
      if (live && j < nvec) {
        va[i].x = exp_softmax(va[i].x - m); va[i].y = exp_softmax(va[i].y - m);
        va[i].z = exp_softmax(va[i].z - m); va[i].w = exp_softmax(va[i].w - m);
        sum += (va[i].x + va[i].y) + (va[i].z + va[i].w);
      }
    }
    sum = row_reduce<SumOp, true>(sum, log_tx, red_smem);
    k0 = 1.0f / sum;
    k1 = dy[0] / (float)g.rows;
  } else {
    float part = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const unsigned j = (unsigned)tx + (unsigned)i * (unsigned)tx_n;
      if (live && j < nvec) {
        if (MODE == kSoftmax) part += (vd[i].x * va[i].x + vd[i].y * va[i].y) + (vd[i].z * va[i].z + vd[i].w * va[i].w);
        else part += (vd[i].x + vd[i].y) + (vd[i].z + vd[i].w);
      }
    }
    k0 = row_reduce<SumOp, true>(part, log_tx, red_smem);
  }
  // cross-entropy: every element gets softmax * dloss / rows; the one-hot term is subtracted by the
  // single thread that holds the label's vector (a compare per element would double the instruction
  // count of this pass)
  const int label = (MODE == kCrossEntropy && live) ? labels[row] : -1;
  const float kk = k0 * k1;
  const unsigned label_vec = label >= 0 ? (unsigned)label >> 2 : 0xffffffffu;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const unsigned j = (unsigned)tx + (unsigned)i * (unsigned)tx_n;
    if (live && j < nvec) {
      float4 gr;
      if (MODE == kSoftmax) {
        gr.x = va[i].x * (vd[i].x - k0); gr.y = va[i].y * (vd[i].y - k0);
        gr.z = va[i].z * (vd[i].z - k0); gr.w = va[i].w * (vd[i].w - k0);
      } else if (MODE == kLogSoftmax) {
        gr.x = vd[i].x - exp_softmax(va[i].x) * k0; gr.y = vd[i].y - exp_softmax(va[i].y) * k0;
        gr.z = vd[i].z - exp_softmax(va[i].z) * k0; gr.w = vd[i].w - exp_softmax(va[i].w) * k0;
      } else {
        gr.x = va[i].x * kk; gr.y = va[i].y * kk; gr.z = va[i].z * kk; gr.w = va[i].w * kk;
        if (j == label_vec) {
          const int comp = label & 3;
          if (comp == 0) gr.x -= k1;
          else if (comp == 1) gr.y -= k1;
          else if (comp == 2) gr.z -= k1;
          else gr.w -= k1;
        }
      }
      const float4 old = kEarlyDx ? vx[i] : __ldcs(dxr + j);
      __stcs(dxr + j, make_float4(old.x + gr.x, old.y + gr.y, old.z + gr.z, old.w + gr.w));
    }
  }
}

// ---- backward, tiny rows (<= 32 classes, dense): one THREAD per row -------------------------------------
// The classifier-head case again (10 classes x a batch): a CTA per row would run two block
// reductions for ten elements. Here every thread walks its own row three times straight from
// global memory; the rows of a warp are neighbours, so its loads share cache lines.
template <int MODE>
__global__ void __launch_bounds__(kSmThreads)
softmax_backward_tiny_kernel(const float *__restrict__ a, const float *__restrict__ dy, float *__restrict__ dx,
                             const int *__restrict__ labels, u64 rows, unsigned cols) {
  pdl_wait();
  pdl_launch_dependents();
  const u64 row = (u64)blockIdx.x * kSmThreads + threadIdx.x;
  if (row >= rows) return;
  const float *ar = a + row * cols;
  float *dxr = dx + row * cols;
  if (MODE == kCrossEntropy) {
    float m = -FLT_MAX;
    for (unsigned c = 0; c < cols; ++c) m = fmaxf(m, ar[c]);
    float sum = 0.0f;
    for (unsigned c = 0; c < cols; ++c) sum += exp_softmax(ar[c] - m);
    const float gscale = dy[0] / (float)rows;
    const int label = labels[row];
    for (unsigned c = 0; c < cols; ++c) {
      const float p = exp_softmax(ar[c] - m) / sum;
      dxr[c] += (p - ((int)c == label ? 1.0f : 0.0f)) * gscale;
    }
    return;
  }
  const float *dyr = dy + row * cols;
  float tot = 0.0f;
  for (unsigned c = 0; c < cols; ++c) tot += (MODE == kSoftmax) ? dyr[c] * ar[c] : dyr[c];
  for (unsigned c = 0; c < cols; ++c) {
    const float d = dyr[c], yv = ar[c];
    dxr[c] += (MODE == kSoftmax) ? yv * (d - tot) : d - exp_softmax(yv) * tot;
  }
}

template <int MODE>
static void softmax_family_backward(const char *name, Tensor **inputs, const Tensor *output,
                                    KernelParams params) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name)) return;
  const Tensor *x = inputs[0];
  if (x->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", name, (int)x->dtype);
    return;
  }
  if (!x->requires_grad) return;
  if (!x->grad || !x->grad->data || !output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: missing grad tensor", name);
    return;
  }
  SmRows g;
  const int *labels = nullptr;
  const float *a = nullptr;
  if (MODE == kCrossEntropy) {
    if (!check_tensor(inputs[1], name)) return;
    if (inputs[1]->dtype != INT32 || x->ndim != 2 || inputs[1]->ndim != 1 ||
        inputs[1]->shape[0] != x->shape[0] || inputs[1]->strides[0] != 1) {
      set_error(PLAST_B200_ERR_SHAPE, "%s: expects logits [N,C] and contiguous INT32 labels [N]", name);
      return;
    }
    labels = (const int *)inputs[1]->data;
    if (!make_rows(name, x, x->grad, nullptr, 1, &g)) return;
    a = (const float *)x->data;
  } else {
    // rows of y (the forward result), dy and dx, all shaped like x
    if (!make_rows(name, output, x->grad, output->grad, params.dim, &g)) return;
    a = (const float *)output->data;
  }
  if (g.rows == 0 || g.cols == 0) return;
  const float *dyp = (const float *)output->grad->data;
  float *dxp = (float *)x->grad->data;
  // every row contiguous and 16-byte aligned in y (or x), dy and dx: the register-resident kernel
  // (up to four vectors per thread: rows of 4097 ... 8192 elements measured faster in the long-row
  // kernel, 6.6 against 4.9 TB/s, where eight vectors per thread leave no registers for dx)
  bool fast = (g.cols & 3) == 0 && g.cols <= (u64)kSmThreads * 4 * 4 && g.x_axis_stride == 1 &&
              g.y_axis_stride == 1 && (MODE == kCrossEntropy || g.z_axis_stride == 1) &&
              (((uintptr_t)a | (uintptr_t)dxp | (MODE == kCrossEntropy ? 0 : (uintptr_t)dyp)) & 15) == 0;
  for (int d = 0; fast && d < g.outer.n; ++d)
    if ((g.outer.istride[0][d] | g.outer.tstride[d] | (MODE == kCrossEntropy ? 0 : g.outer.istride[1][d])) & 3) fast = false;
  // dense rows of at most 32 elements that the float4 kernel does not take: a thread per row
  bool tiny = !fast && g.cols <= 32 && g.rows >= 64 && g.x_axis_stride == 1 && g.y_axis_stride == 1 &&
              (MODE == kCrossEntropy || g.z_axis_stride == 1);
  {
    u64 run = g.cols;
    for (int d = 0; tiny && d < g.outer.n; ++d) {
      if (g.outer.istride[0][d] != run || g.outer.tstride[d] != run ||
          (MODE != kCrossEntropy && g.outer.istride[1][d] != run))
        tiny = false;
      run *= g.outer.size[d];
    }
  }
  if (tiny) {
    const u64 grid = (g.rows + kSmThreads - 1) / kSmThreads;
    if (grid > 0x7fffffffull) {
      set_error(PLAST_B200_ERR_LIMIT, "%s: too many rows", name);
      return;
    }
    launch_k(softmax_backward_tiny_kernel<MODE>, dim3((unsigned)grid), dim3(kSmThreads), 0, stream(), a, dyp, dxp, labels,
             g.rows, (unsigned)g.cols);
    count_launch();
    note_kernel("softmax_backward_tiny_rows");
    end_call();
    return;
  }
  if (fast) {
    const u64 nvec = g.cols >> 2;
    int log_tx = 0;
    while (((u64)4 << log_tx) < nvec) ++log_tx; // smallest TX with <= 4 vectors per thread
    while (log_tx < 3 && ((u64)1 << log_tx) < nvec) ++log_tx;
    const int vpt = (int)((nvec + ((u64)1 << log_tx) - 1) >> log_tx);
    const u64 rows_per_cta = (u64)kSmThreads >> log_tx;
    const u64 grid = (g.rows + rows_per_cta - 1) / rows_per_cta;
    if (grid > 0x7fffffffull) {
      set_error(PLAST_B200_ERR_LIMIT, "%s: too many rows", name);
      return;
    }
    int v = 1;
    while (v < vpt) v <<= 1;
    switch (v) {
    case 1: launch_k(softmax_backward_fast_kernel<MODE, 1>, dim3((unsigned)grid), dim3(kSmThreads), 0, stream(), a, dyp, dxp, labels, g, log_tx); break;
    case 2: launch_k(softmax_backward_fast_kernel<MODE, 2>, dim3((unsigned)grid), dim3(kSmThreads), 0, stream(), a, dyp, dxp, labels, g, log_tx); break;
    default: launch_k(softmax_backward_fast_kernel<MODE, 4>, dim3((unsigned)grid), dim3(kSmThreads), 0, stream(), a, dyp, dxp, labels, g, log_tx); break;
    }
    count_launch();
    note_kernel("softmax_backward_fast");
    end_call();
    return;
  }
  u64 grid = g.rows;
  const u64 cap = (u64)sm_count() * 16;
  if (grid > cap) grid = cap;
  launch_k(softmax_backward_kernel<MODE>, dim3((unsigned)grid), dim3(kSmThreads), 0, stream(), a, dyp, dxp, labels, g);
  count_launch();
  note_kernel("softmax_backward");
  end_call();
}

} // namespace pb

using namespace pb;

extern "C" {
void softmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  softmax_family_forward<kSoftmax>("softmax", inputs, output, params);
}
void log_softmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  softmax_family_forward<kLogSoftmax>("log_softmax", inputs, output, params);
}
void cross_entropy_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  softmax_family_forward<kCrossEntropy>("cross_entropy", inputs, output, params);
}
void softmax_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  softmax_family_backward<kSoftmax>("softmax", inputs, output, params);
}
void log_softmax_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  softmax_family_backward<kLogSoftmax>("log_softmax", inputs, output, params);
}
void cross_entropy_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  softmax_family_backward<kCrossEntropy>("cross_entropy", inputs, output, params);
}
}
