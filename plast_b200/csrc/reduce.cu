// Reduction geometry + entry points of sum / mean / max / min (forward, backward) and argmax.
#include "ew_engine.cuh"
#include "functors.cuh"
#include "reduce_engine.cuh"

#include <stdlib.h>
#include <string.h>
#include <type_traits>

namespace pb {

static u64 ceil_div(u64 a, u64 b) { return (a + b - 1) / b; }
static int log2_ceil(u64 v) {
  int l = 0;
  while (((u64)1 << l) < v) ++l;
  return l;
}

bool plan_reduce_geometry(const IterPlan &plan, const void *const *in_ptrs, int nin,
                          size_t elem_bytes, bool indexed, const RedOccupancy &occ, RedGeometry *g) {
  // Vector width along dim 0 (same rule as the elementwise engine, inputs only).
  g->vec = 1;
  g->vec_mask = 0;
  const int cand[2] = {4, 2};
  for (int ci = 0; ci < 2; ++ci) {
    const int vec = cand[ci];
    bool ok = plan.size[0] % (u64)vec == 0;
    unsigned mask = 0;
    bool any_vec = false;
    for (int a = 0; ok && a < nin; ++a) {
      const u64 s0 = plan.stride[a + 1][0];
      if (s0 == 0) continue;
      if (s0 != 1) { ok = false; break; }
      if (((uintptr_t)in_ptrs[a]) % (sizeof(float) * vec) != 0) { ok = false; break; }
      for (int d = 1; d < plan.ndim; ++d)
        if (plan.stride[a + 1][d] % (u64)vec != 0) { ok = false; break; }
      mask |= 1u << a;
      any_vec = true;
    }
    if (ok && any_vec) {
      g->vec = vec;
      g->vec_mask = mask;
      break;
    }
  }
  const u64 vec = (u64)g->vec;
  g->len0_items = plan.size[0] / vec;
  g->n_kept_dims = g->n_red_dims = 0;
  g->n_kept = g->n_red = 1;
  const bool dim0_reduced = plan.reduced[0];
  int n_reduced_total = 0;
  for (int d = 0; d < plan.ndim; ++d) n_reduced_total += plan.reduced[d] ? 1 : 0;
  if (indexed && n_reduced_total > 1) {
    set_error(PLAST_B200_ERR_UNSUPPORTED,
              "argmax over more than one non-mergeable axis (a non-contiguous full reduce)");
    return false;
  }
  for (int d = 1; d < plan.ndim; ++d) {
    if (plan.reduced[d]) {
      g->red_dims[g->n_red_dims++] = d;
      g->n_red *= plan.size[d];
    } else {
      g->kept_dims[g->n_kept_dims++] = d;
      g->n_kept *= plan.size[d];
    }
  }
  const u64 sms = (u64)sm_count();
  // One resident wave: every CTA of a split reduction gets the same share of the work, so more
  // CTAs than fit at once would only add a second, partly empty wave.
  const int vi = g->vec == 4 ? 2 : (g->vec == 2 ? 1 : 0);
  const u64 target_ctas = sms * (u64)occ.ctas_per_sm[dim0_reduced ? kRedSeg : kRedCols][vi];
  g->splits = 1;
  g->cluster = 0;
  g->outers_per_cta = 1;
  g->seg_len = g->nsplit0 = g->nseg = g->per_chunk = 0;
  g->log_tx = 5;

  if (dim0_reduced) {
    if (indexed && plan.size[0] * (g->n_red) > 0xffffffffull) {
      set_error(PLAST_B200_ERR_LIMIT, "argmax over more than 2^32 elements");
      return false;
    }
    // Lanes per row: about eight items per lane (eight loads in flight), at least eight lanes (a
    // 128-byte piece per load instruction and row), at most a warp. A lane per item left rows of
    // 65 ... 512 elements with one or two loads in flight per lane ([262144, 256]: 3.3 TB/s).
    // (scalar items come in batches of sixteen)
    int log_tx = log2_ceil(ceil_div(g->len0_items, g->vec == 1 ? 16 : 8));
    if (log_tx < 3) log_tx = 3;
    if (log_tx > log2_ceil(g->len0_items)) log_tx = log2_ceil(g->len0_items);
    if (log_tx > 5) log_tx = 5;
    const u64 warps = g->n_kept * ((u64)1 << log_tx) / 32;
    if (g->n_red == 1 && (warps >= sms * 16 || g->len0_items <= 256)) {
      g->kind = kRedRows;
      g->log_tx = log_tx;
      const u64 rows_per_cta = (u64)kRedThreads >> log_tx;
      u64 blocks = ceil_div(g->n_kept, rows_per_cta);
      const u64 cap = sms * 64; // grid-stride beyond this (a CTA per group of rows measured 15 % slower for short rows)
      g->grid = blocks < cap ? blocks : cap;
      return true;
    }
    g->kind = kRedSeg;
    const u64 seg_cap = (u64)kRedThreads * (nin == 1 ? 8 : 4) * (g->vec == 1 ? 2 : 1); // one full load batch
    if (g->len0_items <= seg_cap) {
      // whole runs as segments: a row-worker of ~1/16 of the run's items walks it in several
      // full load batches; the other row-workers of the CTA take the next runs
      g->nsplit0 = 1;
      g->seg_len = g->len0_items;
      g->log_tx = log2_ceil(ceil_div(g->len0_items, 16));
      if (g->log_tx < 5 && g->len0_items >= 32) g->log_tx = 5;
      if (g->log_tx > 8) g->log_tx = 8;
    } else {
      // one trip of the load batch per segment
      g->seg_len = seg_cap;
      g->nsplit0 = ceil_div(g->len0_items, g->seg_len);
      g->log_tx = 8;
      if (tuned(kTuneSegLogTx) >= 5 && tuned(kTuneSegLogTx) <= 8) g->log_tx = (int)tuned(kTuneSegLogTx);
    }
    g->nseg = g->nsplit0 * g->n_red;
    const u64 ty_n = (u64)kRedThreads >> g->log_tx;
    // a chunk should give every row-worker >= 2 segments and move >= ~64 KiB
    u64 min_per = ty_n * 2;
    const u64 seg_bytes = g->seg_len * vec * sizeof(float);
    if (min_per * seg_bytes < (64u << 10)) min_per = ceil_div(64u << 10, seg_bytes);
    u64 splits = ceil_div(target_ctas, g->n_kept);
    const u64 max_splits = g->nseg / min_per > 0 ? g->nseg / min_per : 1;
    if (splits > max_splits) splits = max_splits;
    if (splits > 1 && (g->n_kept > kCounters ||
                       g->n_kept * splits * elem_bytes > kPartialFloats / 2 * sizeof(float)))
      splits = 1;
    g->per_chunk = ceil_div(g->nseg, splits);
    g->splits = (unsigned)ceil_div(g->nseg, g->per_chunk);
    g->grid = g->n_kept * g->splits;
  } else {
    if (indexed && g->n_red > 0xffffffffull) {
      set_error(PLAST_B200_ERR_LIMIT, "argmax over more than 2^32 elements");
      return false;
    }
    g->kind = kRedCols;
    // A CTA sweeps a strip of tx_n lanes (x VEC outputs) with 256 / tx_n row-workers; the reduced
    // dim is cut into `splits` chunks so that ONE resident wave of equally loaded CTAs covers the
    // tensor (CTAs beyond the wave would run as a second, mostly empty one). Strip width: the widest
    // of 8 / 16 / 32 lanes that still leaves 64 strips, i.e. FEW chunks per strip. Measured on B200
    // (graph replay, float4 lanes): 8192 x 8192 46 us with 8 lanes, 40 with 32, 49 / 62 / 113 with
    // 64 / 128 / 256; but with few columns 32 lanes leave a handful of strips cut into hundreds of
    // chunks each, and narrower strips win by far: 65536 x 256 46.6 -> 13.6 us, 262144 x 128
    // 95 -> 30, 32768 x 512 29.7 -> 13.5, 8192 x 1024 18.0 -> 8.2, 4096 x 4096 13.8 -> 10.2 (16 lanes).
    u64 ctas_per_sm = (u64)occ.ctas_per_sm[kRedCols][vi] < 4 ? (u64)occ.ctas_per_sm[kRedCols][vi] : 4;
    if (tuned(kTuneColsCtasPerSm) > 0) ctas_per_sm = (u64)tuned(kTuneColsCtasPerSm);
    const u64 wave = sms * ctas_per_sm;
    // a chunk gives every row-worker at least this many full load batches of four rows
    u64 min_batches = 2; // (one batch per row-worker, i.e. twice the CTAs, measured slower even at 4 MiB)
    if (tuned(kTuneColsMinBatches) > 0) min_batches = (u64)tuned(kTuneColsMinBatches);
    double best_fill = -1.0;
    // (lanes of narrower items, when the layout does not allow float4, are scaled up to the same
    // bytes per row: 32 ... 128 scalar lanes)
    const int wider = g->vec == 4 ? 0 : (g->vec == 2 ? 1 : 2);
    int forced_ltx = 3 + wider;
    for (int ltx = 5 + wider; ltx > 3 + wider; --ltx)
      if (g->n_kept * ceil_div(g->len0_items, (u64)1 << ltx) >= 64) {
        forced_ltx = ltx;
        break;
      }
    // A SHORT reduced dim (a [4096, 16, 1024] sum over the middle axis) cannot feed many row-workers:
    // widen the strip instead until every worker has at least 16 indices (four load batches) or the
    // strip covers the whole kept run; with 16 indices that is one thread per output vector and no
    // tree at all (268 MB: 186 us with eight workers of two rows each).
    // A kept run shorter than that strip ([65536, 16, 64] over the middle axis) shares the CTA with
    // the runs of the next outer indices: lanes = (outer index, item).
    while (forced_ltx < 8 && ((u64)kRedThreads >> forced_ltx) * 16 > g->n_red &&
           ((u64)1 << forced_ltx) < g->len0_items * g->n_kept)
      ++forced_ltx;
    u64 cluster = 0;      // forced cluster size (tuning hook)
    bool auto_cluster = true;
    u64 in_bytes = 0;
    for (int a = 0; a < nin; ++a) in_bytes += (plan.max_offset[a + 1] + 1) * sizeof(float);
    {
      // Inputs that fit L2 with a short reduced dim (the bias gradient of a 1024 x 1024 layer) are
      // bound by the latencies of a split reduction: partial store, fence, ticket, second pass.
      // Narrow strips (2+ lanes of float4, the other threads of the CTA as row-workers) give the
      // same number of CTAs without a split: every CTA reduces its columns over ALL rows in at most
      // four load batches per thread and stores the result itself.
      if (in_bytes <= ((u64)32 << 20) && g->n_red_dims <= 1) {
        for (int ltx = 1; ltx < 5; ++ltx) {
          const u64 tx_n = (u64)1 << ltx, ty_n = (u64)kRedThreads >> ltx;
          const u64 tiles = g->n_kept * ceil_div(g->len0_items, tx_n);
          if (tiles <= 2 * sms && tiles * 4 >= sms && ceil_div(g->n_red, ty_n) <= 16) {
            forced_ltx = ltx;
            break;
          }
        }
      }
    }
    if (tuned(kTuneColsLogTx) >= 0 && tuned(kTuneColsLogTx) <= 8) forced_ltx = (int)tuned(kTuneColsLogTx);
    if (tuned(kTuneColsCluster) >= 0) {
      cluster = tuned(kTuneColsCluster) <= 8 ? (u64)tuned(kTuneColsCluster) : 8;
      auto_cluster = false;
    }
    for (int ltx = forced_ltx; ltx <= forced_ltx; ++ltx) {
      const u64 tx_n = (u64)1 << ltx, ty_n = (u64)kRedThreads >> ltx;
      u64 outers = 1;
      if (g->n_kept > 1 && tx_n >= 2 * g->len0_items && g->len0_items <= 0xffffu) {
        outers = tx_n / g->len0_items;
        if (outers > g->n_kept) outers = g->n_kept;
      }
      g->outers_per_cta = (unsigned)outers;
      const u64 strips = outers > 1 ? 1 : ceil_div(g->len0_items, tx_n);
      const u64 tiles = outers > 1 ? ceil_div(g->n_kept, outers) : g->n_kept * strips;
      u64 splits = wave / tiles > 0 ? wave / tiles : 1;
      if (outers > 1) splits = 1;
      const u64 min_per = ty_n * 4 * min_batches;
      const u64 max_splits = g->n_red / min_per > 0 ? g->n_red / min_per : 1;
      if (splits > max_splits) splits = max_splits;
      if (splits > 1 && (tiles > kCounters || tiles * splits * tx_n * vec * elem_bytes >
                                                  kPartialFloats / 2 * sizeof(float)))
        splits = 1;
      u64 per_chunk = ceil_div(g->n_red, splits);
      splits = ceil_div(g->n_red, per_chunk);
      // A tile cut into few chunks combines them as ONE thread-block cluster through distributed
      // shared memory: no partials in global memory, no fence, no ticket, no second pass. Measured
      // against the ticket with the same strips: 8192 x 8192 38.4 against 40.5 us (eight chunks
      // instead of nine), 1024 x 8192 7.6 against 12.8 us. A tile that needs more than ~8 chunks to
      // fill the GPU keeps the ticket (4096 x 4096: 18 chunks, 14.3 us; as a cluster of 8, 16.5 us).
      // Up to 64 MiB eight chunks per strip also beat a wave-filling ticket split when that still
      // gives ~1.5 CTAs per SM (8192 x 1024: 32 strips x 8 = 256 CTAs 8.2 us, x 18 with a ticket 10.0).
      if (auto_cluster && splits >= 2 &&
          (splits <= 10 || (tiles * 16 >= 3 * sms && in_bytes <= ((u64)64 << 20))))
        cluster = splits < 8 ? splits : 8;
      if (cluster > 1 && g->n_red >= cluster && outers <= 1) {
        // exactly `cluster` chunks (trailing ones may be empty)
        splits = cluster;
        per_chunk = ceil_div(g->n_red, splits);
        g->cluster = (unsigned)cluster;
      }
      const u64 ctas = tiles * splits;
      const double fill = (double)ctas / (double)(ceil_div(ctas, wave) * wave) *
                          ((double)g->len0_items / (double)(strips * tx_n));
      if (fill > best_fill + 0.015) {
        best_fill = fill;
        g->log_tx = ltx;
        g->per_chunk = per_chunk;
        g->splits = (unsigned)splits;
        g->grid = ctas;
      }
    }
  }
  if (g->grid == 0 || g->grid > 0x7fffffffull) {
    set_error(PLAST_B200_ERR_LIMIT, "reduction needs %llu blocks", (unsigned long long)g->grid);
    return false;
  }
  return true;
}

// ---- forward ---------------------------------------------------------------------------------------
// Shape the CPU path writes into the output of an axis reduce (src/kernels/cpu/cpu_utils.c:121-154).
static void reduced_shape(const Tensor *a, u64 dim, bool keepdim, u64 *shape, u64 *ndim, u64 *strides) {
  u64 nd = 0;
  if (keepdim) {
    for (u64 i = 0; i < a->ndim; ++i) shape[i] = (i == dim) ? 1 : a->shape[i];
    nd = a->ndim;
  } else {
    for (u64 i = 0; i < a->ndim; ++i)
      if (i != dim) shape[nd++] = a->shape[i];
    if (nd == 0) {
      shape[0] = 1;
      nd = 1;
    }
  }
  *ndim = nd;
  u64 s = 1;
  for (u64 i = nd; i-- > 0;) {
    strides[i] = s;
    s *= shape[i];
  }
}

// Strides of the reduced tensor `c` seen from a's dims (0 on the reduced dim).
static void out_strides_in_a_dims(const Tensor *a, u64 dim, bool keepdim, const u64 *c_strides,
                                  u64 *st) {
  for (u64 j = 0; j < a->ndim; ++j) {
    if (j == dim) st[j] = 0;
    else if (keepdim) st[j] = c_strides[j];
    else st[j] = c_strides[j < dim ? j : j - 1];
  }
  // when every dim is reduced away the output is the single element at offset 0
}

static bool reduce_common_checks(const char *name, const Tensor *a, const Tensor *output, u64 dim) {
  if (a->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", name, (int)a->dtype);
    return false;
  }
  if (dim != PLAST_FULL_REDUCE && dim >= a->ndim) {
    set_error(PLAST_B200_ERR_SHAPE, "%s: axis %llu out of range for %llu dims", name,
              (unsigned long long)dim, (unsigned long long)a->ndim);
    return false;
  }
  (void)output;
  return true;
}

// Builds the plan of reducing `a` over `dim` (or everything) into a target indexed by tst[].
static void reduce_plan(IterPlan *plan, const Tensor *a, u64 dim, const u64 *target_strides) {
  u64 st[2][MAX_NDIM] = {};
  bool red[MAX_NDIM] = {};
  for (u64 j = 0; j < a->ndim; ++j) {
    st[0][j] = target_strides ? target_strides[j] : 0;
    st[1][j] = a->strides[j];
    red[j] = (dim == PLAST_FULL_REDUCE) || (j == dim);
  }
  make_plan(plan, a->shape, a->ndim, 2, st, red, 1);
  if (a->ndim == 0 || plan->ndim == 1) {
    // single element, or fully merged: make sure a lone dim of a full reduce is marked reduced
    if (dim == PLAST_FULL_REDUCE) plan->reduced[0] = true;
  }
}

// True when walking the tensor in logical row-major order walks memory front to back.
static bool row_major_dense(const Tensor *t) {
  u64 expect = 1;
  for (u64 d = t->ndim; d-- > 0;) {
    if (t->shape[d] == 1) continue;
    if (t->strides[d] != expect) return false;
    expect *= t->shape[d];
  }
  return true;
}

template <class Op>
static void reduce_forward(const char *name, const Tensor **inputs, Tensor *output,
                           KernelParams params, bool mean) {
  begin_call();
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name)) return;
  const Tensor *a = inputs[0];
  const u64 dim = params.dim;
  if (!reduce_common_checks(name, a, output, dim)) return;
  u64 tst[MAX_NDIM] = {};
  u64 count = 0;
  if (dim == PLAST_FULL_REDUCE) {
    count = numel(a);
  } else {
    const bool keepdim = params.keepdim != 0;
    reduced_shape(a, dim, keepdim, output->shape, &output->ndim, output->strides);
    out_strides_in_a_dims(a, dim, keepdim, output->strides, tst);
    count = a->shape[dim];
  }
  if (numel(a) == 0) {
    // Nothing to reduce: every output holds the start value of the CPU loop
    // (src/kernels/cpu/reduce_ops.c:26,53: 0 for sum, -/+FLT_MAX for max / min; mean is 0 / 0).
    u64 n_out = 1;
    if (dim != PLAST_FULL_REDUCE) {
      n_out = 1;
      for (u64 j = 0; j < output->ndim; ++j) n_out *= output->shape[j];
    }
    float start = 0.0f;
    if (std::is_same<Op, MaxOp>::value) start = -FLT_MAX;
    if (std::is_same<Op, MinOp>::value) start = FLT_MAX;
    if (mean) start = nanf("");
    unsigned int bits;
    memcpy(&bits, &start, 4);
    if (std::is_same<Op, ArgMaxOp>::value) bits = 0;
    fill32(output->data, bits, n_out);
    // an empty shard inside the cross-GPU bracket still takes part in the exchange (with the
    // start value just written as its contribution)
    if (!mean && peer_bracket_open()) exchange_for_empty_shard<Op>((float *)output->data, (float *)output->data, n_out, false);
    end_call();
    return;
  }
  if (std::is_same<Op, ArgMaxOp>::value && dim == PLAST_FULL_REDUCE && !row_major_dense(a)) {
    // The flat index of a full argmax counts elements in the view's logical row-major order
    // (cpu_utils.c:121-154 walks coordinates), which is not the order a permuted or expanded
    // view lies in memory. Gather the view into a stream-ordered scratch copy and reduce that.
    void *packed = nullptr;
    PB_CUDA(scratch_alloc_async(&packed, numel(a) * sizeof(float)));
    plast_b200_pack(a, packed);
    if (!failed()) {
      Tensor dense = *a;
      dense.data = packed;
      u64 s = 1;
      for (u64 d = a->ndim; d-- > 0;) {
        dense.strides[d] = s;
        s *= a->shape[d];
      }
      IterPlan plan;
      reduce_plan(&plan, &dense, dim, tst);
      const float *ins[1] = {(const float *)packed};
      launch_reduce<Op, IdentityPro, 1>(plan, (typename Op::Out *)output->data, ins, IdentityPro{}, Op{},
                                        false, 0.0f);
    }
    cudaFreeAsync(packed, stream());
    if (!failed()) note_kernel("argmax_of_packed_view");
    end_call();
    return;
  }
  IterPlan plan;
  reduce_plan(&plan, a, dim, tst);
  const float *ins[1] = {(const float *)a->data};
  launch_reduce<Op, IdentityPro, 1>(plan, (typename Op::Out *)output->data, ins, IdentityPro{}, Op{},
                                    false, mean ? (float)count : 0.0f);
  end_call();
}

// ---- backward ----------------------------------------------------------------------------------------
// sum / mean: da[coords] += g[out coords] (/ n): src/kernels/cpu/reduce_ops.c:90-154.
struct AddGrad { // x = {g, old}
  __device__ __forceinline__ float operator()(const float *x) const { return x[1] + x[0]; }
};
struct AddGradScaled { // mean: grad / n first, then accumulate
  float n;
  __device__ __forceinline__ float operator()(const float *x) const { return x[1] + x[0] / n; }
};
// max / min: da[i] += g / ties where a[i] equals the extreme (reduce_ops.c:157-262).
struct EqualsPro { // x = {a, extreme}
  __device__ __forceinline__ float operator()(const float *x) const { return x[0] == x[1] ? 1.0f : 0.0f; }
};
struct TieGrad { // x = {a, extreme, g, ties, old}
  __device__ __forceinline__ float operator()(const float *x) const {
    return x[0] == x[1] ? x[4] + x[2] / x[3] : x[4];
  }
};

static bool backward_checks(const char *name, Tensor **inputs, const Tensor *output) {
  if (!inputs || !check_tensor(inputs[0], name) || !check_tensor(output, name, false)) return false;
  const Tensor *a = inputs[0];
  if (a->dtype != FLOAT32) {
    set_error(PLAST_B200_ERR_DTYPE, "%s: unsupported dtype %d", name, (int)a->dtype);
    return false;
  }
  if (!a->requires_grad) return false; // nothing to do (reduce_ops.c:134)
  if (!a->grad || !a->grad->data || !output->grad || !output->grad->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: missing grad tensor", name);
    return false;
  }
  return true;
}

static void sum_mean_backward(const char *name, Tensor **inputs, const Tensor *output,
                              KernelParams params, bool mean) {
  begin_call();
  if (!backward_checks(name, inputs, output)) return;
  const Tensor *a = inputs[0];
  const u64 dim = params.dim;
  if (!reduce_common_checks(name, a, output, dim)) return;
  u64 st[3][MAX_NDIM] = {};
  u64 gst[MAX_NDIM] = {};
  u64 count = numel(a);
  if (dim != PLAST_FULL_REDUCE) {
    out_strides_in_a_dims(a, dim, params.keepdim != 0, output->strides, gst);
    count = a->shape[dim];
  }
  for (u64 j = 0; j < a->ndim; ++j) {
    st[0][j] = a->grad->strides[j];
    st[1][j] = gst[j];
    st[2][j] = a->grad->strides[j];
  }
  IterPlan plan;
  make_plan(&plan, a->shape, a->ndim, 3, st, nullptr, 0);
  const float *ins[2] = {(const float *)output->grad->data, (const float *)a->grad->data};
  if (mean) launch_ew<AddGradScaled, 2>(plan, (float *)a->grad->data, ins, AddGradScaled{(float)count});
  else launch_ew<AddGrad, 2>(plan, (float *)a->grad->data, ins, AddGrad{});
  end_call();
}

static void max_min_backward(const char *name, Tensor **inputs, const Tensor *output,
                             KernelParams params) {
  begin_call();
  if (!backward_checks(name, inputs, output)) return;
  const Tensor *a = inputs[0];
  const u64 dim = params.dim;
  if (!reduce_common_checks(name, a, output, dim)) return;
  if (!output->data) {
    set_error(PLAST_B200_ERR_NULL, "%s: output data is NULL", name);
    return;
  }
  u64 cst[MAX_NDIM] = {};
  u64 n_out = 1;
  if (dim != PLAST_FULL_REDUCE) {
    out_strides_in_a_dims(a, dim, params.keepdim != 0, output->strides, cst);
    n_out = numel(a) / (a->shape[dim] ? a->shape[dim] : 1);
  }
  Workspace ws;
  if (!get_workspace(&ws)) return;
  if (n_out > kPartialFloats / 2) {
    set_error(PLAST_B200_ERR_LIMIT, "%s backward: %llu outputs exceed the tie-count scratch (%llu)",
              name, (unsigned long long)n_out, (unsigned long long)(kPartialFloats / 2));
    return;
  }
  float *ties = ws.partials + kPartialFloats / 2; // second half: never used by split partials
  // 1) ties[out] = number of elements equal to the extreme, laid out like the output
  {
    u64 st[3][MAX_NDIM] = {};
    bool red[MAX_NDIM] = {};
    for (u64 j = 0; j < a->ndim; ++j) {
      st[0][j] = cst[j];
      st[1][j] = a->strides[j];
      st[2][j] = cst[j];
      red[j] = (dim == PLAST_FULL_REDUCE) || (j == dim);
    }
    IterPlan plan;
    make_plan(&plan, a->shape, a->ndim, 3, st, red, 1);
    if (dim == PLAST_FULL_REDUCE) plan.reduced[0] = true;
    const float *ins[2] = {(const float *)a->data, (const float *)output->data};
    PeerSuspend local_step; // tie counts are scratch of this call, not a result that crosses GPUs
    launch_reduce<SumOp, EqualsPro, 2>(plan, ties, ins, EqualsPro{}, SumOp{}, false, 0.0f);
    if (failed()) return;
  }
  // 2) da += g / ties where equal
  {
    u64 st[6][MAX_NDIM] = {};
    for (u64 j = 0; j < a->ndim; ++j) {
      st[0][j] = a->grad->strides[j];
      st[1][j] = a->strides[j];
      st[2][j] = cst[j];
      st[3][j] = cst[j];
      st[4][j] = cst[j];
      st[5][j] = a->grad->strides[j];
    }
    IterPlan plan;
    make_plan(&plan, a->shape, a->ndim, 6, st, nullptr, 0);
    const float *ins[5] = {(const float *)a->data, (const float *)output->data,
                           (const float *)output->grad->data, ties, (const float *)a->grad->data};
    launch_ew<TieGrad, 5>(plan, (float *)a->grad->data, ins, TieGrad{});
  }
  end_call();
}

} // namespace pb

using namespace pb;

extern "C" {

void sum_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  reduce_forward<SumOp>("sum", inputs, output, params, false);
}
void mean_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  reduce_forward<SumOp>("mean", inputs, output, params, true);
}
void max_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  reduce_forward<MaxOp>("max", inputs, output, params, false);
}
void min_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  reduce_forward<MinOp>("min", inputs, output, params, false);
}
void argmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params) {
  reduce_forward<ArgMaxOp>("argmax", inputs, output, params, false);
}
void sum_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  sum_mean_backward("sum", inputs, output, params, false);
}
void mean_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  sum_mean_backward("mean", inputs, output, params, true);
}
void max_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  max_min_backward("max", inputs, output, params);
}
void min_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params) {
  max_min_backward("min", inputs, output, params);
}

} // extern "C"
