// Elementwise engine: one templated kernel family that evaluates out = f(in0 .. inN-1) over a
// canonical iteration space (iter.h). Bound by HBM bandwidth, so everything here is about
// bytes in flight and coalescing:
//   * items are 16-byte (float4) or 8-byte (float2) vectors along the innermost dim whenever
//     every operand is either contiguous or broadcast along it and the pointers allow it
//     (arena allocations are only 8-byte aligned, src/core/tensor.c:66 -> float2 path);
//   * every thread issues all loads of its kUnroll items before the first use, streaming
//     (evict-first) for operands that are read once, default-cached for broadcast operands;
//   * outer coordinates come from one multiply-shift division per dim (no 64-bit div/mod per
//     element as in src/kernels/cuda/binary_ops.cu:41-54), or none at all for 1-D plans.
#pragma once

#include "common.cuh"
#include "iter.h"

#include "ew_kernel_device.cuh"
#include <type_traits>

namespace pb {

struct FastDivU32 {
  uint32_t magic, shift;
};
FastDivU32 make_fast_div(uint32_t d);

// Chosen launch geometry, for tests and profiling.
struct EwChoice {
  int vec;
  bool one_d;
  bool idx64;
};

EwChoice choose_ew(const IterPlan &plan, const void *const *ptrs, int nargs, u64 *n_items,
                   uint32_t *vec_mask);


template <int NARGS, typename index_t>
void fill_offset_calc(OffsetCalc<NARGS, index_t> *oc, const IterPlan &plan, int vec) {
  oc->ndim = plan.ndim;
  for (int d = 0; d < MAX_NDIM; ++d) {
    u64 sz = d < plan.ndim ? plan.size[d] : 1;
    if (d == 0) sz /= (u64)vec;
    oc->size[d] = (index_t)sz;
    FastDivU32 fd = make_fast_div((uint32_t)(sz > 0x7fffffffull ? 1 : (sz == 0 ? 1 : sz)));
    oc->magic[d] = fd.magic;
    oc->shift[d] = fd.shift;
    for (int a = 0; a < NARGS; ++a) {
      u64 s = d < plan.ndim ? plan.stride[a][d] : 0;
      if (d == 0) s *= (u64)vec;
      oc->stride[a][d] = (index_t)s;
    }
  }
}

// Launches f over the plan. ptrs[0] = output, ptrs[1..NIN] = inputs (device pointers).
template <class F, int NIN>
void launch_ew_one(const IterPlan &plan, float *out, const float *const *ins, const F &f) {
  if (plan.numel == 0) return;
  const void *ptrs[NIN + 1];
  ptrs[0] = out;
  for (int a = 0; a < NIN; ++a) ptrs[a + 1] = ins[a];
  u64 n_items = 0;
  uint32_t vec_mask = 0;
  EwChoice c = choose_ew(plan, ptrs, NIN + 1, &n_items, &vec_mask);
  InPtrs<NIN> ip;
  for (int a = 0; a < NIN; ++a) ip.p[a] = ins[a];
  const u64 per_block = (u64)kEwThreads * kEwUnroll;
  const u64 blocks = (n_items + per_block - 1) / per_block;
  if (blocks > 0x7fffffffull) {
    set_error(PLAST_B200_ERR_LIMIT, "elementwise launch needs %llu blocks", (unsigned long long)blocks);
    return;
  }
  dim3 grid((unsigned)blocks), block(kEwThreads);
  cudaStream_t s = stream();
#define PB_EW_LAUNCH(VEC, IDX, ONED)                                                               \
  do {                                                                                             \
    OffsetCalc<NIN + 1, IDX> oc;                                                                   \
    fill_offset_calc(&oc, plan, VEC);                                                              \
    launch_k(ew_kernel<F, NIN, VEC, IDX, ONED>, grid, block, 0, s, f, out, ip, oc, (IDX)n_items,  \
             vec_mask);                                                                            \
  } while (0)
#define PB_EW_BY_VEC(IDX, ONED)                                                                    \
  do {                                                                                             \
    if (c.vec == 4) PB_EW_LAUNCH(4, IDX, ONED);                                                    \
    else if (c.vec == 2) PB_EW_LAUNCH(2, IDX, ONED);                                               \
    else PB_EW_LAUNCH(1, IDX, ONED);                                                               \
  } while (0)
  // compile-time operand masks for the two shapes that matter: one streamed operand (the first
  // or the second) and per-row / constant operands beside it
  bool launched = false;
  if constexpr (NIN >= 2) {
    if (c.vec == 4 && !c.idx64 && (vec_mask == 1u || vec_mask == 2u)) {
      OffsetCalc<NIN + 1, uint32_t> oc;
      fill_offset_calc(&oc, plan, 4);
#define PB_EW_MASKED(ONED, CMASK)                                                                  \
  launch_k(ew_kernel<F, NIN, 4, uint32_t, ONED, CMASK>, grid, block, 0, s, f, out, ip, oc, (uint32_t)n_items, vec_mask)
      if (vec_mask == 1u) {
        if (c.one_d) PB_EW_MASKED(true, 1u); else PB_EW_MASKED(false, 1u);
      } else {
        if (c.one_d) PB_EW_MASKED(true, 2u); else PB_EW_MASKED(false, 2u);
      }
#undef PB_EW_MASKED
      launched = true;
    }
  }
  if (launched) {
  } else if (c.idx64) {
    if (c.one_d) PB_EW_BY_VEC(uint64_t, true);
    else PB_EW_BY_VEC(uint64_t, false);
  } else {
    if (c.one_d) PB_EW_BY_VEC(uint32_t, true);
    else PB_EW_BY_VEC(uint32_t, false);
  }
#undef PB_EW_BY_VEC
#undef PB_EW_LAUNCH
  count_launch();
  static const char *names[3][2] = {{"ew_scalar_nd", "ew_scalar_1d"},
                                    {"ew_vec2_nd", "ew_vec2_1d"},
                                    {"ew_vec4_nd", "ew_vec4_1d"}};
  note_kernel(names[c.vec == 4 ? 2 : (c.vec == 2 ? 1 : 0)][c.one_d ? 1 : 0]);
}

// ---- transposed operands: shared-memory tile transpose ------------------------------------------------
// When the output is contiguous along dim 0 but some input is contiguous along another dim dT
// (a transposed view: x.T + y, pack(x.T), the transpose gradient), reading that input along dim 0
// would touch one 32-byte sector per element. Instead a CTA owns a 32 x 32 tile of (dim 0, dT):
// transposed inputs are loaded with threads running along dT (coalesced), parked in shared memory
// [32][33] (the pad avoids bank conflicts) and read back with threads running along dim 0, where
// the other inputs and the output are coalesced.
constexpr int kTileDim = 32;
constexpr int kTileRows = 8; // threads per tile column; each thread handles 32 / 8 = 4 rows

template <int NIN> struct TiledParams {
  const float *in[NIN];
  float *out;
  u64 n0, nT;             // extents of dim 0 and dT
  u64 s0[NIN + 1], sT[NIN + 1]; // element strides of out (index 0) and inputs along dim 0 / dT
  int n_outer;            // remaining dims, flattened into blockIdx.z
  u64 outer_size[MAX_NDIM];
  u64 outer_stride[NIN + 1][MAX_NDIM];
  unsigned tmask;         // bit a: input a is contiguous along dT (goes through shared memory)
  u64 tiles0;             // tiles along dim 0 (blockIdx.x = tile0 + tiles0 * tileT)
};

template <class F, int NIN>
__global__ void __launch_bounds__(kTileDim * kTileRows) ew_tiled_kernel(F f, TiledParams<NIN> p) {
  __shared__ float tile[NIN][kTileDim][kTileDim + 1];
  pdl_wait();
  pdl_launch_dependents();
  const u64 t0 = blockIdx.x % p.tiles0, tT = blockIdx.x / p.tiles0;
  u64 off[NIN + 1];
#pragma unroll
  for (int a = 0; a <= NIN; ++a) off[a] = 0;
  u64 rest = blockIdx.y;
  for (int d = 0; d < p.n_outer; ++d) {
    const u64 q = rest / p.outer_size[d], r = rest - q * p.outer_size[d];
#pragma unroll
    for (int a = 0; a <= NIN; ++a) off[a] += r * p.outer_stride[a][d];
    rest = q;
  }
  const unsigned tx = threadIdx.x, ty = threadIdx.y;
  // phase 1: transposed inputs, threads along dT
#pragma unroll
  for (int a = 0; a < NIN; ++a) {
    if (!((p.tmask >> a) & 1u)) continue;
    const u64 cT = tT * kTileDim + tx;
#pragma unroll
    for (int j = 0; j < kTileDim; j += kTileRows) {
      const u64 c0 = t0 * kTileDim + ty + j;
      if (cT < p.nT && c0 < p.n0)
        tile[a][ty + j][tx] = p.in[a][off[a + 1] + c0 * p.s0[a + 1] + cT * p.sT[a + 1]];
    }
  }
  __syncthreads();
  // phase 2: threads along dim 0
  const u64 c0 = t0 * kTileDim + tx;
#pragma unroll
  for (int j = 0; j < kTileDim; j += kTileRows) {
    const u64 cT = tT * kTileDim + ty + j;
    if (c0 < p.n0 && cT < p.nT) {
      float x[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a)
        x[a] = ((p.tmask >> a) & 1u) ? tile[a][tx][ty + j]
                                     : p.in[a][off[a + 1] + c0 * p.s0[a + 1] + cT * p.sT[a + 1]];
      p.out[off[0] + c0 * p.s0[0] + cT * p.sT[0]] = f(x);
    }
  }
}

// Picks dT (>= 1) when the plan fits the tiled kernel; returns -1 otherwise.
int choose_tiled_dim(const IterPlan &plan, int nargs, unsigned *tmask);

// 64 x 64 tiles moved as float4 in both directions (extents, strides and pointers permitting):
// four 16-byte loads in flight per thread and input instead of four 4-byte ones.
constexpr int kTile4 = 64;
template <class F, int NIN>
__global__ void __launch_bounds__(256) ew_tiled4_kernel(F f, TiledParams<NIN> p) {
  extern __shared__ float tile4_smem[]; // [NIN][64][65]
  pdl_wait();
  pdl_launch_dependents();
  const u64 t0 = blockIdx.x % p.tiles0, tT = blockIdx.x / p.tiles0;
  u64 off[NIN + 1];
#pragma unroll
  for (int a = 0; a <= NIN; ++a) off[a] = 0;
  u64 rest = blockIdx.y;
  for (int d = 0; d < p.n_outer; ++d) {
    const u64 q = rest / p.outer_size[d], r = rest - q * p.outer_size[d];
#pragma unroll
    for (int a = 0; a <= NIN; ++a) off[a] += r * p.outer_stride[a][d];
    rest = q;
  }
  const unsigned q4 = threadIdx.x & 15, row = threadIdx.x >> 4; // 16 float4 across, 16 rows per pass
  // Every load of the tile is issued before anything waits: the transposed inputs as float4 along dT
  // (rows along dim 0), the others as float4 along dim 0 (rows along dT), 4 x NIN vectors in flight
  // per thread and ONE trip to memory per tile instead of one per phase.
  const u64 c0v = t0 * kTile4 + q4 * 4; // phase-2 position of this thread along dim 0
  float4 v[4][NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) {
    if ((p.tmask >> a) & 1u) {
      const u64 cT = tT * kTile4 + q4 * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const u64 c0 = t0 * kTile4 + row + j * 16;
        if (cT < p.nT && c0 < p.n0)
          v[j][a] = __ldcs(reinterpret_cast<const float4 *>(p.in[a] + off[a + 1] + c0 * p.s0[a + 1] + cT));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const u64 cT = tT * kTile4 + row + j * 16;
        if (c0v < p.n0 && cT < p.nT) {
          const float *q = p.in[a] + off[a + 1] + c0v * p.s0[a + 1] + cT * p.sT[a + 1];
          if (p.s0[a + 1] == 1) {
            v[j][a] = __ldcs(reinterpret_cast<const float4 *>(q));
          } else { // broadcast along dim 0
            const float sc = __ldg(q);
            v[j][a] = make_float4(sc, sc, sc, sc);
          }
        }
      }
    }
  }
  // phase 1: park the transposed inputs in shared memory, [dim 0][dT] with a one-float pad
#pragma unroll
  for (int a = 0; a < NIN; ++a) {
    if (!((p.tmask >> a) & 1u)) continue;
    float *tl = tile4_smem + (size_t)a * kTile4 * (kTile4 + 1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float *dst = tl + (row + j * 16) * (kTile4 + 1) + q4 * 4;
      dst[0] = v[j][a].x; dst[1] = v[j][a].y; dst[2] = v[j][a].z; dst[3] = v[j][a].w;
    }
  }
  __syncthreads();
  // phase 2: float4 along dim 0, rows along dT
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const u64 cT = tT * kTile4 + row + j * 16;
    if (c0v < p.n0 && cT < p.nT) {
      float r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float x[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
          if ((p.tmask >> a) & 1u) {
            x[a] = tile4_smem[(size_t)a * kTile4 * (kTile4 + 1) + (q4 * 4 + k) * (kTile4 + 1) + row + j * 16];
          } else {
            const float4 d = v[j][a];
            x[a] = k == 0 ? d.x : (k == 1 ? d.y : (k == 2 ? d.z : d.w));
          }
        }
        r[k] = f(x);
      }
      __stcs(reinterpret_cast<float4 *>(p.out + off[0] + c0v + cT * p.sT[0]), make_float4(r[0], r[1], r[2], r[3]));
    }
  }
}

template <class F, int NIN>
bool launch_ew_tiled(const IterPlan &plan, float *out, const float *const *ins, const F &f) {
  unsigned tmask = 0;
  const int dT = choose_tiled_dim(plan, NIN + 1, &tmask);
  if (dT < 0) return false;
  TiledParams<NIN> p;
  for (int a = 0; a < NIN; ++a) p.in[a] = ins[a];
  p.out = out;
  p.n0 = plan.size[0];
  p.nT = plan.size[dT];
  p.tmask = tmask;
  p.n_outer = 0;
  u64 outer = 1;
  for (int d = 1; d < plan.ndim; ++d) {
    if (d == dT) continue;
    p.outer_size[p.n_outer] = plan.size[d];
    for (int a = 0; a <= NIN; ++a) p.outer_stride[a][p.n_outer] = plan.stride[a][d];
    outer *= plan.size[d];
    ++p.n_outer;
  }
  for (int d = p.n_outer; d < MAX_NDIM; ++d) {
    p.outer_size[d] = 1;
    for (int a = 0; a <= NIN; ++a) p.outer_stride[a][d] = 0;
  }
  for (int a = 0; a <= NIN; ++a) {
    p.s0[a] = plan.stride[a][0];
    p.sT[a] = plan.stride[a][dT];
  }
  if (outer > 65535) return false; // grid limit: the generic path takes it
  // float4 both ways needs 4-divisible extents, 16-byte aligned bases and 4-divisible strides
  bool vec4 = (p.n0 % 4 == 0) && (p.nT % 4 == 0) && (((uintptr_t)out) % 16 == 0);
  for (int a = 0; vec4 && a < NIN; ++a) vec4 = ((uintptr_t)ins[a]) % 16 == 0;
  for (int a = 0; vec4 && a <= NIN; ++a) {
    const bool t = a > 0 && ((tmask >> (a - 1)) & 1u);
    // along the arg's own contiguous dim the stride is 1; every other stride must keep alignment
    if ((t ? p.s0[a] : p.sT[a]) % 4 != 0) vec4 = false;
    for (int d = 0; d < p.n_outer; ++d)
      if (p.outer_stride[a][d] % 4 != 0) vec4 = false;
  }
  const size_t smem4 = (size_t)NIN * kTile4 * (kTile4 + 1) * sizeof(float);
  if (vec4 && smem4 <= 99 * 1024) {
    p.tiles0 = (p.n0 + kTile4 - 1) / kTile4;
    const u64 tilesT = (p.nT + kTile4 - 1) / kTile4;
    if (p.tiles0 * tilesT <= 0x7fffffffull) {
      static bool ready = false;
      if (!ready) {
        cudaFuncSetAttribute(ew_tiled4_kernel<F, NIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
        ready = true;
      }
      dim3 grid((unsigned)(p.tiles0 * tilesT), (unsigned)outer);
      launch_k(ew_tiled4_kernel<F, NIN>, grid, dim3(256), smem4, stream(), f, p);
      count_launch();
      note_kernel("ew_tiled_transpose");
      return true;
    }
  }
  p.tiles0 = (p.n0 + kTileDim - 1) / kTileDim;
  const u64 tilesT = (p.nT + kTileDim - 1) / kTileDim;
  if (p.tiles0 * tilesT > 0x7fffffffull) return false;
  dim3 grid((unsigned)(p.tiles0 * tilesT), (unsigned)outer), block(kTileDim, kTileRows);
  launch_k(ew_tiled_kernel<F, NIN>, grid, block, 0, stream(), f, p);
  count_launch();
  note_kernel("ew_tiled_transpose");
  return true;
}

// ---- inputs contiguous along two DIFFERENT dims, neither of them the output's -------------------------
// x.transpose(0, 2) + y.transpose(1, 2) on 3-D tensors: one 2-D tile can only turn one of the two
// dims. A 3-D tile of 32 (output's dim 0) x 16 (dA) x 16 (dB) elements turns both: an input that is
// contiguous along dA (or dB) is read as float4 along that dim, 64 bytes per tile row, parked in
// shared memory and read back along dim 0; the output (and any input laid out like it) moves as
// float4 along dim 0. Every byte crosses DRAM once.
// Tile shape: D0 along the output's dim 0, DX along dA and dB. 8 x 32 x 32 reads whole 128-byte lines
// of the turned inputs and writes 32-byte pieces of output lines (the L2 merges those before they
// reach DRAM); 32 x 16 x 16 reads 64-byte pieces and writes whole lines.
template <int D0, int DX, int NT> struct Tile3 {
  static constexpr int kLanes = DX / 4;                    // float4 lanes along an input's own dim
  static constexpr int kStageH = NT / (kLanes * D0);      // staging: tile rows of the other dim per trip
  static constexpr int kStageTrips = DX / kStageH;
  static constexpr int kQ0 = D0 / 4;                       // float4 along dim 0 in the output pass
  static constexpr int kOutH = NT / (kQ0 * DX);
  static constexpr int kOutTrips = DX / kOutH;
  // element (jA, jB, i0) lives at jB * kPlane + jA * kRow + i0; both strides are chosen so that the
  // four scalar stores of a staged float4 land in distinct banks across a warp
  static constexpr int kRow = D0 + 1;
  static constexpr int kWant = (32 / kLanes) / 4;          // kPlane = kWant (mod 8)
  static constexpr int kPlane = DX * kRow + ((kWant - (DX * kRow) % 8) % 8 + 8) % 8;
  static constexpr int kFloats = DX * kPlane;              // per staged input
  static_assert(kStageTrips * NT * 4 == D0 * DX * DX && kOutTrips * NT * 4 == D0 * DX * DX, "whole tile per pass");
};

template <int NIN> struct Tiled3Params {
  const float *in[NIN];
  float *out;
  u64 n0, nA, nB;
  u64 s0[NIN + 1], sA[NIN + 1], sB[NIN + 1]; // element strides of out (index 0) and the inputs
  int cls[NIN];           // 0: read directly along dim 0 (unit stride or broadcast), 1: unit stride along dA, 2: along dB
  int slot[NIN];          // shared-memory slot of a staged input
  int n_outer;
  u64 outer_size[MAX_NDIM];
  u64 outer_stride[NIN + 1][MAX_NDIM];
  // blockIdx.x = tile0 + tiles0 * (tileA + tilesA * tileB). Dealing the tiles out in groups of
  // neighbours along the three dims instead (so that resident CTAs complete whole output lines and
  // whole rows of the turned inputs together) measured no different on B200.
  unsigned tiles0, tilesA;
};

template <class F, int NIN, int D0, int DX, int NT>
__global__ void __launch_bounds__(NT, 2) ew_tiled3_kernel(F f, Tiled3Params<NIN> p) {
  using T = Tile3<D0, DX, NT>;
  extern __shared__ float tile3_smem[]; // [staged inputs][jB][jA][i0], padded
  pdl_wait();
  pdl_launch_dependents();
  const unsigned t0 = blockIdx.x % p.tiles0, tAB = blockIdx.x / p.tiles0;
  const unsigned tA = tAB % p.tilesA, tB = tAB / p.tilesA;
  u64 off[NIN + 1];
#pragma unroll
  for (int a = 0; a <= NIN; ++a) off[a] = 0;
  u64 rest = blockIdx.y;
  for (int d = 0; d < p.n_outer; ++d) {
    const u64 q = rest / p.outer_size[d], r = rest - q * p.outer_size[d];
#pragma unroll
    for (int a = 0; a <= NIN; ++a) off[a] += r * p.outer_stride[a][d];
    rest = q;
  }
  const u64 c0 = (u64)t0 * D0, cA = (u64)tA * DX, cB = (u64)tB * DX; // tile origin
  // A tile that lies wholly inside the tensor (all of them, for extents that are multiples of the tile)
  // runs without per-access bounds checks.
  auto run = [&](auto full_tile) {
    constexpr bool FULL = decltype(full_tile)::value;
    // staging pass: thread = (sq: float4 lane along the input's own dim, si: along dim 0, sh), a few
    // trips over the remaining dim; every load is issued before the first store to shared memory
    const unsigned sq = threadIdx.x % T::kLanes, si = (threadIdx.x / T::kLanes) % D0, sh = threadIdx.x / (T::kLanes * D0);
    float4 v[NIN][T::kStageTrips];
  #pragma unroll
    for (int a = 0; a < NIN; ++a) {
      if (p.cls[a] == 0) continue;
      const bool alongA = p.cls[a] == 1;
      const u64 own = (alongA ? cA : cB) + sq * 4, own_n = alongA ? p.nA : p.nB;
      const u64 oth0 = alongA ? cB : cA, oth_n = alongA ? p.nB : p.nA, oth_s = alongA ? p.sB[a + 1] : p.sA[a + 1];
      const float *base = p.in[a] + off[a + 1] + (c0 + si) * p.s0[a + 1] + own;
  #pragma unroll
      for (int j = 0; j < T::kStageTrips; ++j) {
        const u64 oth = oth0 + sh + T::kStageH * j;
        if (FULL || (c0 + si < p.n0 && own < own_n && oth < oth_n))
          v[a][j] = __ldcs(reinterpret_cast<const float4 *>(base + oth * oth_s));
      }
    }
  #pragma unroll
    for (int a = 0; a < NIN; ++a) {
      if (p.cls[a] == 0) continue;
      const bool alongA = p.cls[a] == 1;
      float *tl = tile3_smem + (size_t)p.slot[a] * T::kFloats + si;
  #pragma unroll
      for (int j = 0; j < T::kStageTrips; ++j) {
        const unsigned oth = sh + T::kStageH * j;
        const unsigned at = alongA ? oth * T::kPlane + (sq * 4) * T::kRow : (sq * 4) * T::kPlane + oth * T::kRow;
        const unsigned step = alongA ? T::kRow : T::kPlane;
        tl[at] = v[a][j].x; tl[at + step] = v[a][j].y; tl[at + 2 * step] = v[a][j].z; tl[at + 3 * step] = v[a][j].w;
      }
    }
    __syncthreads();
    // output pass: thread = (q4: float4 along dim 0, jA, oh), a few trips over jB
    const unsigned q4 = threadIdx.x % T::kQ0, jA = (threadIdx.x / T::kQ0) % DX, oh = threadIdx.x / (T::kQ0 * DX);
    const u64 i0 = c0 + q4 * 4;
    if (!FULL && (i0 >= p.n0 || cA + jA >= p.nA)) return;
  #pragma unroll
    for (int j = 0; j < T::kOutTrips; ++j) {
      const unsigned jB = oh + T::kOutH * j;
      if (!FULL && cB + jB >= p.nB) continue;
      float x[4][NIN];
  #pragma unroll
      for (int a = 0; a < NIN; ++a) {
        if (p.cls[a] == 0) {
          const float *q = p.in[a] + off[a + 1] + i0 * p.s0[a + 1] + (cA + jA) * p.sA[a + 1] + (cB + jB) * p.sB[a + 1];
          if (p.s0[a + 1] == 1) {
            const float4 d = __ldcs(reinterpret_cast<const float4 *>(q));
            x[0][a] = d.x; x[1][a] = d.y; x[2][a] = d.z; x[3][a] = d.w;
          } else { // broadcast along dim 0
            const float sc = __ldg(q);
            x[0][a] = x[1][a] = x[2][a] = x[3][a] = sc;
          }
        } else {
          const float *tl = tile3_smem + (size_t)p.slot[a] * T::kFloats + jB * T::kPlane + jA * T::kRow + q4 * 4;
          x[0][a] = tl[0]; x[1][a] = tl[1]; x[2][a] = tl[2]; x[3][a] = tl[3];
        }
      }
      __stcs(reinterpret_cast<float4 *>(p.out + off[0] + i0 + (cA + jA) * p.sA[0] + (cB + jB) * p.sB[0]),
             make_float4(f(x[0]), f(x[1]), f(x[2]), f(x[3])));
    }
  };
  if (c0 + D0 <= p.n0 && cA + DX <= p.nA && cB + DX <= p.nB) run(std::true_type{});
  else run(std::false_type{});
}

// The same turn with 8 x 32 x 32 tiles staged by cp.async: every thread sends four 16-byte pieces per
// turned input straight from global to shared memory (no registers in between, no scalar scatter),
// rows kept as they lie in memory; the turn happens when the output pass reads shared memory along
// dim 0. Row stride 36 floats and plane stride 292 keep every piece 16-byte aligned and make the
// reads of BOTH kinds of input conflict-free when a warp covers 2 float4 (dim 0) x 4 (dA) x 4 (dB):
// bank = 16 * q4 + jA + 4 * jB for an input that runs along dA, 16 * q4 + jB + 4 * jA along dB.
struct Tile3Async {
  static constexpr int kD0 = 8, kDX = 32, kThreads = 512;
  static constexpr int kRow = kDX + 4;            // floats between rows (dim 0) of one plane
  static constexpr int kPlane = kD0 * kRow + 4;   // floats between planes (the input's other dim)
  static constexpr int kFloats = kDX * kPlane;    // per staged input
};

__device__ __forceinline__ void cp_async_16(float *smem_dst, const float *src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <class F, int NIN>
__global__ void __launch_bounds__(Tile3Async::kThreads, 3) ew_tiled3_async_kernel(F f, Tiled3Params<NIN> p) {
  using T = Tile3Async;
  extern __shared__ __align__(16) float tile3a_smem[]; // [staged inputs][other dim][dim 0][own dim], padded
  pdl_wait();
  pdl_launch_dependents();
  const unsigned t0 = blockIdx.x % p.tiles0, tAB = blockIdx.x / p.tiles0;
  const unsigned tA = tAB % p.tilesA, tB = tAB / p.tilesA;
  u64 off[NIN + 1];
#pragma unroll
  for (int a = 0; a <= NIN; ++a) off[a] = 0;
  u64 rest = blockIdx.y;
  for (int d = 0; d < p.n_outer; ++d) {
    const u64 q = rest / p.outer_size[d], r = rest - q * p.outer_size[d];
#pragma unroll
    for (int a = 0; a <= NIN; ++a) off[a] += r * p.outer_stride[a][d];
    rest = q;
  }
  const u64 c0 = (u64)t0 * T::kD0, cA = (u64)tA * T::kDX, cB = (u64)tB * T::kDX; // tile origin
  auto run = [&](auto full_tile) {
    constexpr bool FULL = decltype(full_tile)::value;
    // staging: thread = (sq: 16-byte piece along the input's own dim, si: row along dim 0, sh), four
    // trips over the input's other dim
    const unsigned sq = threadIdx.x & 7, si = (threadIdx.x >> 3) & 7, sh = threadIdx.x >> 6;
#pragma unroll
    for (int a = 0; a < NIN; ++a) {
      if (p.cls[a] == 0) continue;
      const bool alongA = p.cls[a] == 1;
      const u64 own = (alongA ? cA : cB) + sq * 4, own_n = alongA ? p.nA : p.nB;
      const u64 oth0 = (alongA ? cB : cA) + sh, oth_n = alongA ? p.nB : p.nA, oth_s = alongA ? p.sB[a + 1] : p.sA[a + 1];
      const float *src = p.in[a] + off[a + 1] + (c0 + si) * p.s0[a + 1] + own + oth0 * oth_s;
      float *dst = tile3a_smem + (size_t)p.slot[a] * T::kFloats + sh * T::kPlane + si * T::kRow + sq * 4;
      const bool mine = FULL || (c0 + si < p.n0 && own < own_n);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (mine && (FULL || oth0 + 8 * j < oth_n)) cp_async_16(dst + j * 8 * T::kPlane, src);
        src += 8 * oth_s;
      }
    }
    cp_async_wait_all();
    __syncthreads();
    // output pass: a warp covers 2 float4 along dim 0 x 4 along dA x 4 along dB; 16 warps, four trips
    const unsigned q4 = threadIdx.x & 1, jAl = (threadIdx.x >> 1) & 3, jBl = (threadIdx.x >> 3) & 3, w = threadIdx.x >> 5;
    const u64 i0 = c0 + q4 * 4;
    if (!FULL && i0 >= p.n0) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned pair = w + 16 * j;
      const unsigned jA = (pair & 7) * 4 + jAl, jB = (pair >> 3) * 4 + jBl;
      if (!FULL && (cA + jA >= p.nA || cB + jB >= p.nB)) continue;
      float x[4][NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        if (p.cls[a] == 0) {
          const float *q = p.in[a] + off[a + 1] + i0 * p.s0[a + 1] + (cA + jA) * p.sA[a + 1] + (cB + jB) * p.sB[a + 1];
          if (p.s0[a + 1] == 1) {
            const float4 d = __ldcs(reinterpret_cast<const float4 *>(q));
            x[0][a] = d.x; x[1][a] = d.y; x[2][a] = d.z; x[3][a] = d.w;
          } else { // broadcast along dim 0
            const float sc = __ldg(q);
            x[0][a] = x[1][a] = x[2][a] = x[3][a] = sc;
          }
        } else {
          const bool alongA = p.cls[a] == 1;
          const float *tl = tile3a_smem + (size_t)p.slot[a] * T::kFloats + (alongA ? jB : jA) * T::kPlane +
                            (q4 * 4) * T::kRow + (alongA ? jA : jB);
          x[0][a] = tl[0]; x[1][a] = tl[T::kRow]; x[2][a] = tl[2 * T::kRow]; x[3][a] = tl[3 * T::kRow];
        }
      }
      __stcs(reinterpret_cast<float4 *>(p.out + off[0] + i0 + (cA + jA) * p.sA[0] + (cB + jB) * p.sB[0]),
             make_float4(f(x[0]), f(x[1]), f(x[2]), f(x[3])));
    }
  };
  if (c0 + T::kD0 <= p.n0 && cA + T::kDX <= p.nA && cB + T::kDX <= p.nB) run(std::true_type{});
  else run(std::false_type{});
}

// Runs the plan through the 3-D tile kernel when exactly two different unit-stride dims other than
// dim 0 occur among the inputs and everything can move as float4; false = not applicable.
template <class F, int NIN>
bool launch_ew_tiled3(const IterPlan &plan, float *out, const float *const *ins, const F &f) {
  if (plan.ndim < 3 || plan.stride[0][0] != 1 || plan.size[0] % 4 != 0 || ((uintptr_t)out) % 16 != 0) return false;
  Tiled3Params<NIN> p;
  int dA = -1, dB = -1, staged = 0;
  for (int a = 0; a < NIN; ++a) {
    p.cls[a] = 0;
    p.slot[a] = 0;
    if (plan.stride[a + 1][0] <= 1) continue;
    int mine = -1;
    for (int d = 1; d < plan.ndim; ++d)
      if (plan.stride[a + 1][d] == 1 && plan.size[d] > 1) mine = d;
    if (mine < 0) return false;
    if (dA < 0 || mine == dA) {
      dA = mine;
      p.cls[a] = 1;
    } else if (dB < 0 || mine == dB) {
      dB = mine;
      p.cls[a] = 2;
    } else {
      return false;
    }
    p.slot[a] = staged++;
  }
  if (dA < 0 || dB < 0) return false; // one turned dim: the 2-D tile kernel's case
  if (plan.size[dA] % 4 != 0 || plan.size[dB] % 4 != 0 || plan.size[dA] < 8 || plan.size[dB] < 8) return false;
  p.out = out;
  p.n0 = plan.size[0];
  p.nA = plan.size[dA];
  p.nB = plan.size[dB];
  p.n_outer = 0;
  u64 outer = 1;
  for (int d = 1; d < plan.ndim; ++d) {
    if (d == dA || d == dB) continue;
    p.outer_size[p.n_outer] = plan.size[d];
    for (int a = 0; a <= NIN; ++a) p.outer_stride[a][p.n_outer] = plan.stride[a][d];
    outer *= plan.size[d];
    ++p.n_outer;
  }
  for (int d = p.n_outer; d < MAX_NDIM; ++d) {
    p.outer_size[d] = 1;
    for (int a = 0; a <= NIN; ++a) p.outer_stride[a][d] = 0;
  }
  if (outer > 65535) return false;
  for (int a = 0; a <= NIN; ++a) {
    p.s0[a] = plan.stride[a][0];
    p.sA[a] = plan.stride[a][dA];
    p.sB[a] = plan.stride[a][dB];
    // float4 along the argument's own unit-stride dim: every other stride keeps 16-byte alignment
    const int cls = a == 0 ? 0 : p.cls[a - 1];
    if (cls == 0 && p.s0[a] == 0) continue; // broadcast along dim 0: scalar loads
    if (a > 0 && ((uintptr_t)ins[a - 1]) % 16 != 0) return false;
    if (cls != 0 && p.s0[a] % 4 != 0) return false;
    if (cls != 1 && p.sA[a] % 4 != 0) return false;
    if (cls != 2 && p.sB[a] % 4 != 0) return false;
    for (int d = 0; d < p.n_outer; ++d)
      if (p.outer_stride[a][d] % 4 != 0) return false;
  }
  for (int a = 0; a < NIN; ++a) p.in[a] = ins[a];
  const bool wide_reads = tuned(kTuneTile3Shape) != 1 && p.nA >= 32 && p.nB >= 32;
  const u64 d0 = wide_reads ? 8 : 32, dx = wide_reads ? 32 : 16;
  const u64 tiles0 = (p.n0 + d0 - 1) / d0, tilesA = (p.nA + dx - 1) / dx, tilesB = (p.nB + dx - 1) / dx;
  if (tiles0 > 0xfffffful || tilesA > 0xfffffful || tilesB > 0xfffffful) return false;
  p.tiles0 = (unsigned)tiles0;
  p.tilesA = (unsigned)tilesA;
  const u64 tiles = tiles0 * tilesA * tilesB;
  if (tiles > 0x7fffffffull) return false;
  const dim3 grid((unsigned)tiles, (unsigned)outer);
  // 512 threads with four float4 per thread and input (64 registers, two CTAs per SM) measured 3 %
  // faster than 256 threads with eight (122 registers, two CTAs of half the size).
  auto go = [&](auto kernel, size_t floats_per_input) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(NIN * floats_per_input * sizeof(float)));
    launch_k(kernel, grid, dim3(512), (size_t)staged * floats_per_input * sizeof(float), stream(), f, p);
  };
  if (wide_reads) go(ew_tiled3_async_kernel<F, NIN>, Tile3Async::kFloats);
  else go(ew_tiled3_kernel<F, NIN, 32, 16, 512>, Tile3<32, 16, 512>::kFloats);
  count_launch();
  note_kernel("ew_tiled_transpose_two_dims");
  return true;
}

// Inputs that are contiguous along two DIFFERENT dims other than the output's (x.transpose(0, 2) +
// y.transpose(1, 2) on 3-D tensors): one tile transpose can only turn one of those dims. The inputs
// that do not share the first such dim are gathered, each by one pass of the tile kernel, into
// stream-ordered scratch laid out like the output; the op then reads the scratch. That costs 8 more
// bytes per element and gathered input; reading such an input in place would touch a 32-byte
// sector for every 4-byte element. Returns the number of inputs replaced (0: nothing to do or not
// applicable), fills `plan2` / `ins2` and the scratch pointers to free after the launch.
struct EwCopy {
  __device__ __forceinline__ float operator()(const float *x) const { return x[0]; }
};
template <class F, int NIN> bool launch_ew_tiled(const IterPlan &plan, float *out, const float *const *ins, const F &f);
template <int NIN>
int gather_second_transposed_inputs(const IterPlan &plan, const float *const *ins, IterPlan *plan2,
                                    const float **ins2, void **scratch) {
  if (plan.ndim < 3 || plan.stride[0][0] != 1) return 0;
  int unit_dim[NIN], first = -1, n_other = 0;
  for (int a = 0; a < NIN; ++a) {
    unit_dim[a] = -1;
    if (plan.stride[a + 1][0] <= 1) continue;
    bool expands = false;
    for (int d = 0; d < plan.ndim; ++d) {
      if (plan.stride[a + 1][d] == 0) expands = true;
      if (d >= 1 && plan.stride[a + 1][d] == 1 && plan.size[d] > 1) unit_dim[a] = d;
    }
    if (expands) unit_dim[a] = -1; // a broadcasting view would be blown up by the gather
    if (unit_dim[a] < 0) continue;
    if (first < 0) first = unit_dim[a];
    else if (unit_dim[a] != first) ++n_other;
  }
  if (n_other == 0) return 0;
  *plan2 = plan;
  u64 dense[MAX_NDIM], run = 1;
  for (int d = 0; d < plan.ndim; ++d) {
    dense[d] = run;
    run *= plan.size[d];
  }
  int replaced = 0;
  for (int a = 0; a < NIN; ++a) {
    ins2[a] = ins[a];
    if (unit_dim[a] < 0 || unit_dim[a] == first) continue;
    void *buf = nullptr;
    if (scratch_alloc_async(&buf, plan.numel * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      continue; // no scratch: this input stays where it is, the generic kernel reads it in place
    }
    IterPlan copy;
    copy.ndim = plan.ndim;
    copy.nargs = 2;
    copy.numel = plan.numel;
    for (int d = 0; d < plan.ndim; ++d) {
      copy.size[d] = plan.size[d];
      copy.stride[0][d] = dense[d];
      copy.stride[1][d] = plan.stride[a + 1][d];
    }
    copy.max_offset[0] = plan.numel - 1;
    copy.max_offset[1] = plan.max_offset[a + 1];
    const float *src[1] = {ins[a]};
    if (!launch_ew_tiled<EwCopy, 1>(copy, (float *)buf, src, EwCopy{})) launch_ew_one<EwCopy, 1>(copy, (float *)buf, src, EwCopy{});
    for (int d = 0; d < plan.ndim; ++d) plan2->stride[a + 1][d] = dense[d];
    plan2->max_offset[a + 1] = plan.numel - 1;
    ins2[a] = (const float *)buf;
    scratch[replaced++] = buf;
  }
  return replaced;
}

// Public entry: 1-D plans whose length is not a multiple of 4 run as a vector body plus a
// <= 3 element tail, so an odd element count does not force the whole tensor onto scalar loads.
template <class F, int NIN>
void launch_ew(const IterPlan &plan, float *out, const float *const *ins, const F &f) {
  if (plan.ndim == 1 && plan.size[0] >= 8 && (plan.size[0] & 3) != 0 && plan.stride[0][0] == 1) {
    bool ok = true;
    for (int a = 1; a <= NIN; ++a) ok = ok && plan.stride[a][0] <= 1;
    if (ok) {
      const u64 body_n = plan.size[0] & ~(u64)3;
      IterPlan body = plan, tail = plan;
      body.size[0] = body_n;
      body.numel = body_n;
      tail.size[0] = plan.size[0] - body_n;
      tail.numel = tail.size[0];
      const float *tins[NIN];
      for (int a = 0; a <= NIN; ++a) {
        body.max_offset[a] = (body_n - 1) * plan.stride[a][0];
        tail.max_offset[a] = (tail.size[0] - 1) * plan.stride[a][0];
        if (a > 0) tins[a - 1] = ins[a - 1] + body_n * plan.stride[a][0];
      }
      launch_ew_one<F, NIN>(body, out, ins, f);
      launch_ew_one<F, NIN>(tail, out + body_n, tins, f);
      return;
    }
  }
  if (plan.numel != 0 && launch_ew_tiled<F, NIN>(plan, out, ins, f)) return;
  if (plan.numel != 0 && launch_ew_tiled3<F, NIN>(plan, out, ins, f)) return;
  if (plan.numel != 0) {
    IterPlan plan2;
    const float *ins2[NIN];
    void *scratch[NIN];
    const int replaced = gather_second_transposed_inputs<NIN>(plan, ins, &plan2, ins2, scratch);
    if (replaced > 0) {
      if (!failed() && !launch_ew_tiled<F, NIN>(plan2, out, ins2, f)) launch_ew_one<F, NIN>(plan2, out, ins2, f);
      for (int i = 0; i < replaced; ++i) cudaFreeAsync(scratch[i], stream());
      if (!failed()) note_kernel("ew_gather_then_tiled_transpose");
      return;
    }
  }
  launch_ew_one<F, NIN>(plan, out, ins, f);
}

} // namespace pb
