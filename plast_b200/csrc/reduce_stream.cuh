// Streamed variants of the segmented and the column reduction: the same work split and the same
// epilogues as reduce_seg_kernel / reduce_cols_kernel, but the input reaches the SM through
// bulk asynchronous copies (cp.async.bulk, the 1-D form of TMA) into a ring of shared-memory
// stages, completion tracked by mbarriers. The bytes in flight per SM are then set by shared
// memory (3 CTAs x 3 stages x 16 KiB), not by how many loads the register file can hold, which
// is what a read-only kernel needs to keep HBM3e busy.
//
// Used when every streamed input is 16-byte aligned with a contiguous dim 0 (VEC == 4); other
// layouts take the register-staged kernels.
//
// Every wait on an mbarrier is bounded: a CTA that gives up raises a flag the host can read,
// stops issuing copies and leaves through the normal barriers, so the launch always ends.
#pragma once

#include "reduce_engine.cuh"

namespace pb {

constexpr int kStreamStages = 4;
constexpr int kStreamStageItems = 1024;                  // float4 per stage, all streamed inputs together
constexpr size_t kStreamSmemBytes = (size_t)kStreamStages * kStreamStageItems * sizeof(float4);
constexpr unsigned kStreamWaitLimit = 1u << 22;           // try_wait rounds before giving up

__device__ __forceinline__ unsigned smem_addr(const void *p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(ok)
               : "r"(smem_addr(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// Global -> shared bulk copy; src and dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, unsigned bytes,
                                              unsigned long long *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

template <int NIN> struct StreamParams {
  int slot[NIN];        // position of input a among the streamed inputs, -1 = not streamed
  int n_streamed;
  unsigned tile_items;  // float4 per streamed input per stage
  unsigned rows_per_tile; // cols: rows of the strip per tile
  unsigned int *gave_up; // host-visible flag
};

// ---- seg: CTA per (output, chunk of segments); one segment = one tile ----------------------------------
template <class Op, class Pro, int NIN>
__global__ void __launch_bounds__(kRedThreads)
reduce_seg_stream_kernel(RedParams<NIN> p, StreamParams<NIN> sp, Pro pro) {
  using T = typename Op::T;
  extern __shared__ __align__(128) unsigned char stream_smem[];
  float4 *stage_buf = reinterpret_cast<float4 *>(stream_smem);
  __shared__ unsigned long long full_bar[kStreamStages];
  __shared__ volatile int abort_flag;

  const u64 out_idx = blockIdx.x / p.splits;
  const unsigned chunk = blockIdx.x % p.splits;
  const unsigned tid = threadIdx.x;
  u64 toff = 0, base[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) base[a] = 0;
  p.kept.offsets(out_idx, &toff, base);

  if (tid == 0) {
    for (int s = 0; s < kStreamStages; ++s) mbar_init(&full_bar[s], 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Chunks are interleaved: chunk c takes segments c, c + splits, c + 2 splits, ... so that at any
  // moment all CTAs of the grid read neighbouring segments and the DRAM access front stays linear
  // (blocked chunks would be hundreds of distant streams fighting over the same banks).
  const unsigned n_tiles = p.nseg > chunk ? (unsigned)((p.nseg - chunk + p.splits - 1) / p.splits) : 0u;

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
  // thread 0 queues the copies of tile t into its stage
  auto issue = [&](unsigned t) {
    u64 ioff[NIN], b, e, o;
    locate((u64)chunk + (u64)t * p.splits, ioff, &b, &e, &o);
    const unsigned s = t % kStreamStages;
    const unsigned bytes = (unsigned)(e - b) * (unsigned)sizeof(float4);
    mbar_arrive_expect_tx(&full_bar[s], bytes * (unsigned)sp.n_streamed);
#pragma unroll
    for (int a = 0; a < NIN; ++a)
      if (sp.slot[a] >= 0)
        bulk_copy_g2s(stage_buf + ((size_t)s * sp.n_streamed + sp.slot[a]) * sp.tile_items,
                      p.in[a] + ioff[a] + b * 4, bytes, &full_bar[s]);
  };

  if (tid == 0)
    for (unsigned t = 0; t < n_tiles && t < (unsigned)kStreamStages; ++t) issue(t);

  T acc[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[k] = Op::identity();

  for (unsigned t = 0; t < n_tiles; ++t) {
    const unsigned s = t % kStreamStages, parity = (t / kStreamStages) & 1u;
    u64 ioff[NIN], b, e, outer;
    locate((u64)chunk + (u64)t * p.splits, ioff, &b, &e, &outer);
    float fixed[NIN];
#pragma unroll
    for (int a = 0; a < NIN; ++a) fixed[a] = sp.slot[a] < 0 ? __ldg(p.in[a] + ioff[a]) : 0.0f;
    unsigned tries = 0;
    while (!mbar_try_wait(&full_bar[s], parity)) {
      if (++tries > kStreamWaitLimit) {
        abort_flag = 1;
        break;
      }
    }
    const unsigned n = (unsigned)(e - b);
    const unsigned idx_base = (unsigned)(outer * p.len0 * 4 + b * 4);
    if (!abort_flag) {
      for (unsigned i = tid; i < n; i += kRedThreads) {
        float4 v[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a)
          if (sp.slot[a] >= 0)
            v[a] = stage_buf[((size_t)s * sp.n_streamed + sp.slot[a]) * sp.tile_items + i];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float x[NIN];
#pragma unroll
          for (int a = 0; a < NIN; ++a)
            x[a] = sp.slot[a] >= 0 ? (k == 0 ? v[a].x : (k == 1 ? v[a].y : (k == 2 ? v[a].z : v[a].w)))
                                   : fixed[a];
          acc[k] = Op::step(acc[k], pro(x), idx_base + i * 4 + k);
        }
      }
    }
    __syncthreads(); // every thread is done with stage s (and has seen abort_flag)
    if (abort_flag) break;
    if (tid == 0 && t + kStreamStages < n_tiles) issue(t + kStreamStages);
  }
  if (abort_flag) {
    if (tid == 0) *sp.gave_up = 1u;
    return; // no thread passes another barrier after this point
  }

  T r = acc[0];
#pragma unroll
  for (int k = 1; k < 4; ++k) r = Op::combine(r, acc[k]);
  r = block_reduce<Op>(r);
  if (p.splits == 1) {
    if (tid == 0) Op::store((typename Op::Out *)p.out + toff, r, p.accumulate, p.post_div);
    return;
  }
  T *partials = (T *)p.partials + out_idx * p.splits;
  if (tid == 0) partials[chunk] = r;
  if (!take_ticket(p.counters + out_idx, p.splits)) return;
  T v = Op::identity();
  if (tid < 32) {
    for (unsigned c = tid; c < p.splits; c += 32) v = Op::combine(v, Op::load_cg(partials + c));
    v = warp_reduce<Op>(v, 32);
    if (tid == 0) Op::store((typename Op::Out *)p.out + toff, v, p.accumulate, p.post_div);
  }
}

// ---- cols: CTA per (strip, outer kept, chunk of rows); a tile = rows_per_tile rows of the strip --------
// Only plans with one reduced dim take this kernel.
template <class Op, class Pro, int NIN>
__global__ void __launch_bounds__(kRedThreads)
reduce_cols_stream_kernel(RedParams<NIN> p, StreamParams<NIN> sp, Pro pro) {
  using T = typename Op::T;
  extern __shared__ __align__(128) unsigned char stream_smem[];
  float4 *stage_buf = reinterpret_cast<float4 *>(stream_smem);
  __shared__ unsigned long long full_bar[kStreamStages];
  __shared__ volatile int abort_flag;

  const unsigned tid = threadIdx.x;
  const unsigned tx_n = 1u << p.log_tx;
  const unsigned lane = tid & (tx_n - 1), ty = tid >> p.log_tx;
  const unsigned ty_n = kRedThreads >> p.log_tx;
  const u64 strips = (p.len0 + tx_n - 1) >> p.log_tx;
  const u64 tile_id = blockIdx.x / p.splits;
  const unsigned chunk = blockIdx.x % p.splits;
  const u64 outer = tile_id / strips;
  const u64 strip = tile_id - outer * strips;
  const u64 item0 = strip << p.log_tx;
  const unsigned strip_items = (unsigned)(p.len0 - item0 < tx_n ? p.len0 - item0 : tx_n);
  const bool live = lane < strip_items;

  u64 toff = 0, base[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) base[a] = 0;
  p.kept.offsets(outer, &toff, base);
  toff += (item0 + lane) * 4 * p.tstride0;
  u64 rstride[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) {
    base[a] += item0 * p.istride0[a]; // first item of the strip (per-item stride is 4 or 0)
    rstride[a] = p.red.n == 1 ? p.red.istride[a][0] : 0;
  }

  if (tid == 0) {
    for (int s = 0; s < kStreamStages; ++s) mbar_init(&full_bar[s], 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Row tiles are interleaved over the chunks (chunk c takes tiles c, c + splits, ...): all CTAs
  // then work on neighbouring rows and the DRAM access front sweeps the matrix once.
  const unsigned R = sp.rows_per_tile;
  const u64 row_tiles = (p.n_red + R - 1) / R;
  const unsigned n_tiles = row_tiles > chunk ? (unsigned)((row_tiles - chunk + p.splits - 1) / p.splits) : 0u;
  const unsigned row_bytes = strip_items * (unsigned)sizeof(float4);

  // warp 0 queues tile t: one copy per row and streamed input
  auto issue = [&](unsigned t) {
    const unsigned s = t % kStreamStages;
    const u64 first = ((u64)chunk + (u64)t * p.splits) * R;
    const unsigned rows = (unsigned)(p.n_red - first < R ? p.n_red - first : R);
    if (tid == 0) mbar_arrive_expect_tx(&full_bar[s], rows * row_bytes * (unsigned)sp.n_streamed);
    __syncwarp();
    for (unsigned r = tid; r < rows; r += 32) {
#pragma unroll
      for (int a = 0; a < NIN; ++a)
        if (sp.slot[a] >= 0)
          bulk_copy_g2s(stage_buf + ((size_t)s * sp.n_streamed + sp.slot[a]) * sp.tile_items +
                            ((size_t)r << p.log_tx),
                        p.in[a] + base[a] + (first + r) * rstride[a], row_bytes, &full_bar[s]);
    }
  };

  if (tid < 32)
    for (unsigned t = 0; t < n_tiles && t < (unsigned)kStreamStages; ++t) issue(t);

  T acc[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[k] = Op::identity();

  for (unsigned t = 0; t < n_tiles; ++t) {
    const unsigned s = t % kStreamStages, parity = (t / kStreamStages) & 1u;
    const u64 first = ((u64)chunk + (u64)t * p.splits) * R;
    const unsigned rows = (unsigned)(p.n_red - first < R ? p.n_red - first : R);
    unsigned tries = 0;
    while (!mbar_try_wait(&full_bar[s], parity)) {
      if (++tries > kStreamWaitLimit) {
        abort_flag = 1;
        break;
      }
    }
    if (!abort_flag && live) {
      for (unsigned r = ty; r < rows; r += ty_n) {
        float4 v[NIN];
        float scalar[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
          if (sp.slot[a] >= 0)
            v[a] = stage_buf[((size_t)s * sp.n_streamed + sp.slot[a]) * sp.tile_items +
                             ((size_t)r << p.log_tx) + lane];
          else
            scalar[a] = __ldg(p.in[a] + base[a] + (first + r) * rstride[a]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float x[NIN];
#pragma unroll
          for (int a = 0; a < NIN; ++a)
            x[a] = sp.slot[a] >= 0 ? (k == 0 ? v[a].x : (k == 1 ? v[a].y : (k == 2 ? v[a].z : v[a].w)))
                                   : scalar[a];
          acc[k] = Op::step(acc[k], pro(x), (unsigned)(first + r));
        }
      }
    }
    __syncthreads();
    if (abort_flag) break;
    if (tid < 32 && t + kStreamStages < n_tiles) issue(t + kStreamStages);
  }
  if (abort_flag) {
    if (tid == 0) *sp.gave_up = 1u;
    return;
  }

  // Same epilogue as reduce_cols_kernel: combine the row-workers, then the chunks by ticket.
  __shared__ T strip_vals[kRedThreads * 4];
  T r[4];
  if (ty_n > 1) {
#pragma unroll
    for (int k = 0; k < 4; ++k) strip_vals[((ty * 4 + k) << p.log_tx) + lane] = acc[k];
    __syncthreads();
    if (ty == 0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        r[k] = strip_vals[(k << p.log_tx) + lane];
        for (unsigned w = 1; w < ty_n; ++w)
          r[k] = Op::combine(r[k], strip_vals[((w * 4 + k) << p.log_tx) + lane]);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) r[k] = acc[k];
  }
  typename Op::Out *out = (typename Op::Out *)p.out;
  if (p.splits == 1) {
    if (ty == 0 && live) {
#pragma unroll
      for (int k = 0; k < 4; ++k) Op::store(out + toff + (u64)k * p.tstride0, r[k], p.accumulate, p.post_div);
    }
    return;
  }
  T *partials = (T *)p.partials + tile_id * p.splits * ((u64)4 << p.log_tx);
  if (ty == 0) {
#pragma unroll
    for (int k = 0; k < 4; ++k) partials[(((u64)chunk * 4 + k) << p.log_tx) + lane] = r[k];
  }
  if (!take_ticket(p.counters + tile_id, p.splits)) return;
  if (ty == 0 && live) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      T v = Op::identity();
      for (unsigned c = 0; c < p.splits; ++c)
        v = Op::combine(v, Op::load_cg(partials + (((u64)c * 4 + k) << p.log_tx) + lane));
      Op::store(out + toff + (u64)k * p.tstride0, v, p.accumulate, p.post_div);
    }
  }
}

} // namespace pb
