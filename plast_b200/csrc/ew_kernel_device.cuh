// Device side of the elementwise engine: the kernel template and what it needs, with no host
// includes, so the same text is compiled ahead of time (through ew_engine.cuh) and at run time by
// NVRTC for fused chains (chain_jit.cpp embeds this file as a string).
#pragma once

#ifdef __CUDACC_RTC__
typedef unsigned int uint32_t;
typedef unsigned long long uint64_t;
typedef unsigned long long u64;
#ifndef MAX_NDIM
#define MAX_NDIM 8
#endif
#endif

namespace pb {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

// Programmatic dependent launch: pdl_wait() returns once the grid this one depends on has completed
// and its memory is visible (at once for a plain launch); pdl_launch_dependents() lets the next
// grid in the stream become resident early (it waits the same way before touching memory).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <int VEC> struct VecOf;
template <> struct VecOf<4> { using type = float4; };
template <> struct VecOf<2> { using type = float2; };
template <> struct VecOf<1> { using type = float; };

// Bulk traffic is streaming (evict-first): tensors are read and written once per kernel. A policy
// switched per launch by working-set size (default caching for tensors that fit L2) was measured:
// no gain on 4 MiB tensors in a stream or a graph, and the extra predicated instructions cost the
// compute-heaviest fused chain 4 % at 1 GiB, so there is none.
template <int VEC> __device__ __forceinline__ void load_stream(const float *p, float *v);
template <> __device__ __forceinline__ void load_stream<4>(const float *p, float *v) {
  float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load_stream<2>(const float *p, float *v) {
  float2 t = __ldcs(reinterpret_cast<const float2 *>(p));
  v[0] = t.x; v[1] = t.y;
}
template <> __device__ __forceinline__ void load_stream<1>(const float *p, float *v) { v[0] = *p; }

template <int VEC> __device__ __forceinline__ void store_stream(float *p, const float *v);
template <> __device__ __forceinline__ void store_stream<4>(float *p, const float *v) {
  __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
}
template <> __device__ __forceinline__ void store_stream<2>(float *p, const float *v) {
  __stcs(reinterpret_cast<float2 *>(p), make_float2(v[0], v[1]));
}
template <> __device__ __forceinline__ void store_stream<1>(float *p, const float *v) { *p = v[0]; }

// Offsets of one item for NARGS operands. index_t = uint32_t when every count and offset fits
// in 31 bits (multiply-shift division), uint64_t otherwise (hardware-emulated division).
template <int NARGS, typename index_t> struct OffsetCalc {
  int ndim;
  index_t size[MAX_NDIM];   // size[0] counted in items
  uint32_t magic[MAX_NDIM]; // uint32_t path: q = (umulhi(n, magic) + n) >> shift, n < 2^31
  uint32_t shift[MAX_NDIM];
  index_t stride[NARGS][MAX_NDIM]; // elements per step; stride[.][0] is per ITEM

  __device__ __forceinline__ void get(index_t item, index_t *off) const {
#pragma unroll
    for (int a = 0; a < NARGS; ++a) off[a] = 0;
#pragma unroll
    for (int d = 0; d < MAX_NDIM; ++d) {
      if (d >= ndim) break;
      index_t q, r;
      if (d == ndim - 1) { // outermost: no wrap
        q = 0;
        r = item;
      } else if (sizeof(index_t) == 4) {
        q = (index_t)((__umulhi((uint32_t)item, magic[d]) + (uint32_t)item) >> shift[d]);
        r = item - q * size[d];
      } else {
        q = item / size[d];
        r = item - q * size[d];
      }
#pragma unroll
      for (int a = 0; a < NARGS; ++a) off[a] += r * stride[a][d];
      item = q;
    }
  }
};

template <int NIN> struct InPtrs { const float *p[NIN]; };

// vec_mask bit a set: input a is contiguous along dim 0 (vector load); clear: broadcast along
// dim 0 (one scalar load, replicated). Only meaningful for VEC > 1.
// CMASK != 0 fixes the mask at compile time: the replicated copies of a broadcast operand are then
// one register instead of VEC (a [N,C,H,W] tensor times a per-channel scale plus a bias keeps 24
// fewer registers per thread), which is worth a CTA more per SM.
template <class F, int NIN, int VEC, typename index_t, bool ONE_D, uint32_t CMASK = 0>
__global__ void __launch_bounds__(kEwThreads)
ew_kernel(F f, float *out, InPtrs<NIN> in, OffsetCalc<NIN + 1, index_t> oc, index_t n_items,
          uint32_t vec_mask_arg) {
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t vec_mask = CMASK ? CMASK : vec_mask_arg;
  const index_t tile = (index_t)blockIdx.x * (kEwThreads * kEwUnroll) + threadIdx.x;
  float v[kEwUnroll][NIN][VEC];
  index_t out_off[kEwUnroll];
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const index_t item = tile + (index_t)u * kEwThreads;
    if (item < n_items) {
      index_t off[NIN + 1];
      if (ONE_D) {
#pragma unroll
        for (int a = 0; a <= NIN; ++a) off[a] = item * oc.stride[a][0];
      } else {
        oc.get(item, off);
      }
      out_off[u] = off[0];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        const float *p = in.p[a] + off[a + 1];
        if (VEC == 1) {
          v[u][a][0] = *p;
        } else if (vec_mask & (1u << a)) {
          load_stream<VEC>(p, v[u][a]);
        } else {
          const float s = __ldg(p);
#pragma unroll
          for (int k = 0; k < VEC; ++k) v[u][a][k] = s;
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const index_t item = tile + (index_t)u * kEwThreads;
    if (item < n_items) {
      float r[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float x[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) x[a] = v[u][a][k];
        r[k] = f(x);
      }
      store_stream<VEC>(out + out_off[u], r);
    }
  }
}

} // namespace pb
