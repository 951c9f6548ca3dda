// Scalar functors shared by the elementwise engine, the reduce prologues and the chain kernel.
// The library is compiled with -fmad=false: every * and + below rounds on its own, which is
// what a sequence of separate plast ops does (each op writes fp32 to memory). Transcendentals
// are the accurate CUDA math functions, never the __expf-style intrinsics that
// src/kernels/cuda/unary_ops.cu:197-210 uses.
#pragma once

#include <cuda_runtime.h>
#include <math.h>

namespace pb {

// ---- binary forward: src/kernels/cpu/binary_ops.c:18-60 -----------------------------------------
struct AddF { __device__ __forceinline__ float operator()(const float *x) const { return x[0] + x[1]; } };
struct SubF { __device__ __forceinline__ float operator()(const float *x) const { return x[0] - x[1]; } };
struct MulF { __device__ __forceinline__ float operator()(const float *x) const { return x[0] * x[1]; } };
struct DivF { __device__ __forceinline__ float operator()(const float *x) const { return x[0] / x[1]; } };

// ---- binary backward terms: value added to an operand's gradient ----------------------------------
// x = {g} / {g, p} / {g, p, q}; which tensors p and q are is chosen by the caller.
struct GradPass { __device__ __forceinline__ float operator()(const float *x) const { return x[0]; } };
struct GradNeg { __device__ __forceinline__ float operator()(const float *x) const { return -x[0]; } };
struct GradMul { __device__ __forceinline__ float operator()(const float *x) const { return x[0] * x[1]; } };
struct GradDiv { __device__ __forceinline__ float operator()(const float *x) const { return x[0] / x[1]; } };
struct GradDivB { // -(g) * a / (b * b), x = {g, a, b}
  __device__ __forceinline__ float operator()(const float *x) const {
    return -x[0] * x[1] / (x[2] * x[2]);
  }
};

// ---- unary forward: src/kernels/cpu/unary_ops.c:9-31 ---------------------------------------------
struct AbsF { __device__ __forceinline__ float operator()(const float *x) const { return fabsf(x[0]); } };
struct NegF { __device__ __forceinline__ float operator()(const float *x) const { return -x[0]; } };
struct ExpF { __device__ __forceinline__ float operator()(const float *x) const { return expf(x[0]); } };
struct LogF { __device__ __forceinline__ float operator()(const float *x) const { return logf(x[0]); } };
struct SinF { __device__ __forceinline__ float operator()(const float *x) const { return sinf(x[0]); } };
struct CosF { __device__ __forceinline__ float operator()(const float *x) const { return cosf(x[0]); } };
// CUDA's tanf may be 4 ulp off; the contract is <= 2 ulp of glibc's tanf, so tan is evaluated in
// double and rounded once (<= 1 ulp of the correctly rounded value).
__device__ __forceinline__ float tan_accurate(float x) { return (float)tan((double)x); }
struct TanF { __device__ __forceinline__ float operator()(const float *x) const { return tan_accurate(x[0]); } };
struct LeakyReluF {
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    return x[0] > 0.0f ? x[0] : x[0] * alpha;
  }
};

// ---- unary backward: x = {g, a, old}; out = old + g * f'(a) ---------------------------------------
struct AbsB {
  __device__ __forceinline__ float operator()(const float *x) const {
    const float m = x[1] > 0.0f ? 1.0f : (x[1] < 0.0f ? -1.0f : 0.0f);
    return x[2] + x[0] * m;
  }
};
struct NegB { __device__ __forceinline__ float operator()(const float *x) const { return x[2] - x[0]; } };
struct ExpB { __device__ __forceinline__ float operator()(const float *x) const { return x[2] + x[0] * expf(x[1]); } };
struct LogB { __device__ __forceinline__ float operator()(const float *x) const { return x[2] + x[0] * (1.0f / x[1]); } };
struct SinB { __device__ __forceinline__ float operator()(const float *x) const { return x[2] + x[0] * cosf(x[1]); } };
struct CosB { __device__ __forceinline__ float operator()(const float *x) const { return x[2] + x[0] * (-sinf(x[1])); } };
struct TanB {
  __device__ __forceinline__ float operator()(const float *x) const {
    const float t = tan_accurate(x[1]);
    return x[2] + x[0] * (1.0f + t * t);
  }
};
struct LeakyReluB {
  float alpha;
  __device__ __forceinline__ float operator()(const float *x) const {
    return x[2] + x[0] * (x[1] > 0.0f ? 1.0f : alpha);
  }
};

} // namespace pb
