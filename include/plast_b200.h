/*
 * plast_b200.h — C ABI of libplast_b200.so: sm_100a kernels behind plast's kernel entry points.
 *
 * Every `<op>_cuda_forward/backward` symbol below has the signature the plast op table binds
 * (ForwardKernel / BackwardKernel, include/core/op.h:5-6) and is called the same way:
 * Tensor structs, their shape[] and strides[] arrays live in HOST memory; `data` (and
 * `grad->data`) point to DEVICE memory of the current CUDA device. Strides are in elements.
 * Forward overwrites output->data. Backward ACCUMULATES (+=) into inputs[i]->grad->data for
 * every input with requires_grad set, reading output->grad->data.
 *
 * All launches go to the stream set with plast_b200_set_stream (default: the legacy default
 * stream, which is what the reference uses). Entry points return void like the reference's;
 * the outcome of the last call on this host thread is readable with plast_b200_last_error().
 * A failed call prints one line on stderr (the reference's behaviour) and launches nothing.
 *
 * Struct layouts restate include/core/definitions.h:17-23 and include/core/tensor.h:8-30 of the
 * reference; define PLAST_B200_USE_REFERENCE_TYPES and put the reference's include/ on the
 * include path to compile against its own headers instead.
 */
#ifndef PLAST_B200_H
#define PLAST_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef PLAST_B200_USE_REFERENCE_TYPES
#include "core/definitions.h"
#include "core/tensor.h"
#else

#ifndef MAX_NDIM
#define MAX_NDIM 8
#endif

typedef uint64_t u64;
typedef int32_t i32;

/* include/core/definitions.h:19-23 — 24 bytes: dim@0 keepdim@8 fval@16 */
typedef struct {
  u64 dim;     /* reduce axis; PLAST_FULL_REDUCE (= MAX_NDIM + 1) reduces every axis */
  u64 keepdim; /* 0/1 */
  float fval;  /* leaky-relu slope */
} KernelParams;

/* include/core/tensor.h:8 */
typedef enum DTYPE { INT32, FLOAT32 } DTYPE;
/* include/core/arena.h:17 */
typedef enum DEVICE { CPU, CUDA } DEVICE;

struct Node;

/* include/core/tensor.h:20-30 — 176 bytes:
 * grad@0 creator@8 data@16 shape@24 strides@88 ndim@152 dtype@160 device@164 requires_grad@168 */
typedef struct Tensor {
  struct Tensor *grad;
  struct Node *creator;
  void *data;
  u64 shape[MAX_NDIM];
  u64 strides[MAX_NDIM];
  u64 ndim;
  DTYPE dtype;
  DEVICE device;
  bool requires_grad;
} Tensor;

#endif /* PLAST_B200_USE_REFERENCE_TYPES */

/* params.dim value that means "reduce all axes" (plast/tensor.py:601, reduce_ops.c:69). */
#define PLAST_FULL_REDUCE ((u64)(MAX_NDIM + 1))

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------
 * Binary elementwise, NumPy broadcasting (right-aligned; size-1 dims read offset 0).
 * Replaces include/kernels/ops/binary.h:19-29 (src/kernels/cuda/binary_ops.cu:94-141);
 * semantics follow the CPU path include/kernels/kernel_macros.h:191-325.
 * inputs = {a, b}. Backward of a broadcast operand is the broadcast-gradient reduce: the
 * gradient is summed over the broadcast axes (deterministic tree order, no float atomics) and
 * then added to the operand's grad buffer.
 * ------------------------------------------------------------------------------------------ */
void add_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void add_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void sub_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void sub_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void mul_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void mul_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void div_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void div_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);

/* ------------------------------------------------------------------------------------------
 * Unary elementwise. Replaces include/kernels/ops/unary.h:23-33
 * (src/kernels/cuda/unary_ops.cu); semantics follow src/kernels/cpu/unary_ops.c.
 * Transcendentals are the accurate (not fast-math) versions. leaky_relu uses params.fval as
 * the slope: x > 0 ? x : x * slope (so slope 0 gives -0.0 for negative x, as the CPU path).
 * ------------------------------------------------------------------------------------------ */
void abs_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void abs_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void cos_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void cos_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void sin_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void sin_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void tan_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void tan_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void exp_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void exp_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void log_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void log_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void neg_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void neg_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);

/* ------------------------------------------------------------------------------------------
 * Reductions over one axis (params.dim, params.keepdim) or over everything
 * (params.dim == PLAST_FULL_REDUCE, result shape [1]).
 * Replaces include/kernels/ops/reduce.h:19-29 (src/kernels/cuda/reduce_ops.cu:338-514);
 * semantics follow src/kernels/cpu/reduce_ops.c:24-278: the axis forward rewrites
 * output->shape/ndim/strides like the CPU path (reduce_ops.c:80-81); mean divides the fp32
 * sum by the count; max/min start from -/+FLT_MAX and compare with > / <; max/min backward
 * splits the gradient evenly among tied elements (reduce_ops.c:166-177).
 * ------------------------------------------------------------------------------------------ */
void sum_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void sum_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void mean_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void mean_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void max_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void max_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void min_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void min_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);

/* argmax over one axis (or everything): output dtype INT32, lowest index on ties. The reference
 * op table (include/core/ops.def:1-28) has no ARGMAX; this entry point keeps the ForwardKernel
 * signature so it can be added to the table unchanged. The index counts along params.dim (for a
 * full reduce: the row-major linear index of the view). */
void argmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);

/* Column sum for callers that must not allocate device memory. No counterpart in the reference:
 * this is an addition of this library. It computes what sum_cuda_forward computes for
 * params.dim == 0 on a contiguous 2-D FLOAT32 tensor [rows, cols] (the shape of a bias /
 * broadcast gradient), but keeps its split partials in a fixed ~1 MiB array inside the library
 * image instead of the cudaMalloc'ed workspace, and calls no allocating routine at all. Use it
 * from code that has given all device memory to its own arena, or that must never trigger the
 * allocator's device-wide synchronisation.
 * Limits: cols <= 16384 and rows < 2^31, else PLAST_B200_ERR_LIMIT and nothing is launched;
 * any other layout / axis gives PLAST_B200_ERR_UNSUPPORTED. All calls on a device share the array
 * (it keeps the previous call's contents; what must start at zero is cleared per call): calls
 * whose kernels overlap on the GPU race, so issue them on one stream. The first call on each
 * device looks up the array's device address; make that call before any stream capture. Under
 * CUDA's default lazy module loading that first call is also when the driver claims the array's
 * memory on the device: make it BEFORE handing the rest of device memory to an arena (or set
 * CUDA_MODULE_LOADING=EAGER); no later call asks the driver for memory. */
void sum_axis0_noalloc_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);

/* ------------------------------------------------------------------------------------------
 * Fused recipes. Each equals the op sequence the reference builds from primitives, with the
 * same per-op fp32 rounding (no FMA contraction across ops), in one pass over the data.
 * ------------------------------------------------------------------------------------------ */
/* softmax / log_softmax along params.dim: plast/nn/functional.py:77-97
 * (max -> sub -> exp -> sum -> div / log -> sub). inputs = {x}. */
void softmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void softmax_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
void log_softmax_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void log_softmax_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
/* cross_entropy: plast/nn/functional.py:312-333 with reduction="mean". inputs = {logits [N,C]
 * FLOAT32, labels [N] INT32 class indices}; output = [1] mean loss. The reference turns labels
 * into a host-side one-hot matrix; here the label indexes the row directly. */
void cross_entropy_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void cross_entropy_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
/* sigmoid: plast/nn/functional.py:42-47 (neg -> exp -> +1 -> 1/.). inputs = {x}. */
void sigmoid_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void sigmoid_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
/* scale_bias_leaky_relu: leaky_relu(x * scale + bias) as mul -> add -> leaky_relu
 * (include/kernels/kernel_macros.h:191-242, src/kernels/cpu/unary_ops.c:218-232).
 * inputs = {x, scale, bias}; scale and bias broadcast against x. Backward computes
 * g = dout * (y > 0 ? 1 : slope) once and accumulates dx += g * scale,
 * dscale += sum_bcast(g * x), dbias += sum_bcast(g). */
void scale_bias_leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void scale_bias_leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);
/* add_leaky_relu: leaky_relu(a + b) as add -> leaky_relu. inputs = {a, b}. */
void add_leaky_relu_cuda_forward(const Tensor **inputs, Tensor *output, KernelParams params);
void add_leaky_relu_cuda_backward(Tensor **inputs, const Tensor *output, KernelParams params);

/* Forward of the graph `C = leaky_relu(A + b); s = sum(C, last axis)` in one pass over A: both
 * results are written (the ForwardKernel signature has one output, hence the explicit arguments).
 * b holds one row ([cols] or [1, cols]) or has A's shape. C is bit-identical to add -> leaky_relu;
 * s is a tree sum of C's rows (the reference adds left to right). Layouts the one-pass kernel does
 * not take (views, cols % 4 != 0, unaligned) run as add_leaky_relu followed by sum. */
void plast_b200_add_leaky_relu_row_sum(const Tensor *a, const Tensor *b, Tensor *c, Tensor *s, float slope);

/* ------------------------------------------------------------------------------------------
 * Fused elementwise chain: what the scheduler's chain fusion issues for a maximal subgraph of
 * same-shape / broadcast elementwise nodes (the reference scheduler runs such a chain node by
 * node, src/scheduler/scheduler.c:16-52, src/core/graph.c:57-60; its fusion pass only knows
 * matmul/conv patterns, src/scheduler/fusion.c:28-90).
 * The program is a list of steps over a small register file; register r < n_inputs is preloaded
 * with inputs[r] (broadcast against the output shape); each step writes register
 * n_inputs + step_index; the last step's register is stored to output. Every step rounds to
 * fp32 exactly like the standalone op. A program is compiled at run time on first use (NVRTC,
 * cached per program structure; the scalar constants are arguments) and runs at the speed of a
 * hand-written fused kernel; without libnvrtc / libcuda an in-kernel interpreter is used
 * (PLAST_B200_CHAIN_JIT=0 forces it).
 * ------------------------------------------------------------------------------------------ */
typedef enum PlastChainOpcode {
  PLAST_CHAIN_ADD = 0,
  PLAST_CHAIN_SUB,
  PLAST_CHAIN_MUL,
  PLAST_CHAIN_DIV,
  PLAST_CHAIN_NEG,
  PLAST_CHAIN_ABS,
  PLAST_CHAIN_EXP,
  PLAST_CHAIN_LOG,
  PLAST_CHAIN_SIN,
  PLAST_CHAIN_COS,
  PLAST_CHAIN_TAN,
  PLAST_CHAIN_LEAKY_RELU, /* slope = fval */
  PLAST_CHAIN_ADD_SCALAR, /* reg[a] + fval   (0-dim operand on the right) */
  PLAST_CHAIN_RSUB_SCALAR, /* fval - reg[a] */
  PLAST_CHAIN_MUL_SCALAR, /* reg[a] * fval */
  PLAST_CHAIN_RDIV_SCALAR /* fval / reg[a]  (0-dim operand on the left) */
} PlastChainOpcode;

typedef struct PlastChainStep {
  i32 opcode; /* PlastChainOpcode */
  i32 a;      /* first operand register */
  i32 b;      /* second operand register (binary opcodes) */
  float fval; /* scalar operand / slope */
} PlastChainStep;

#define PLAST_CHAIN_MAX_INPUTS 8
#define PLAST_CHAIN_MAX_STEPS 24

void plast_b200_chain_forward(const Tensor **inputs, int n_inputs, Tensor *output,
                              const PlastChainStep *steps, int n_steps);

/* Backward of the chain: for every input with requires_grad, inputs[i]->grad += d(output)/d(input i)
 * applied to output->grad, summed over the dims input i broadcasts. The chain's intermediate values
 * are recomputed from the inputs inside the kernel (nothing was saved by the forward), and every
 * gradient contribution is applied in the order and with the rounding of the node-by-node backward,
 * so an input of the output's shape receives the same bits as nine separate backward launches
 * would give it. Needs the run-time compiler (PLAST_B200_ERR_UNSUPPORTED without libnvrtc /
 * libcuda). */
void plast_b200_chain_backward(Tensor **inputs, int n_inputs, const Tensor *output,
                               const PlastChainStep *steps, int n_steps);

/* 1 when chains can be compiled at run time (libnvrtc and libcuda found, PLAST_B200_CHAIN_JIT not
 * set to 0): then the forward runs as a compiled kernel and the backward exists; 0 = the forward
 * falls back to the in-kernel interpreter and plast_b200_chain_backward reports UNSUPPORTED. */
int plast_b200_chain_jit_available(void);

/* The same chain on HOST buffers (what a caller pays when its data starts and ends on the host,
 * the reference's numpy -> tensor -> op -> numpy() round trip, src/python/bindings.cpp:93,144):
 * host_inputs[i] holds input_elems[i] floats, either n or 1 (a constant); host_output receives n
 * floats. The work is cut into 32 MiB chunks that are copied in, computed and copied out on three
 * streams at once (three staging slots on the device, kept until plast_b200_release_workspace),
 * so both directions of the link stay busy; pass pinned memory, pageable memory serialises the
 * copies. Everything is queued behind the work already on the library stream and is complete
 * when that stream is: synchronise it before reading host_output. */
void plast_b200_chain_forward_host(const float *const *host_inputs, const u64 *input_elems, int n_inputs,
                                   float *host_output, u64 n, const PlastChainStep *steps, int n_steps);

/* ------------------------------------------------------------------------------------------
 * Symbols the reference's other translation units link against.
 * ------------------------------------------------------------------------------------------ */
/* include/kernels/cuda/cuda_tensor_init.h:9-11 (called from src/core/tensor.c:88,107,118,149) */
void zeros_cuda(Tensor *t, u64 num_elements);
void ones_cuda(Tensor *t, u64 num_elements);
void set_ones_grad_cuda(Tensor *t);
/* include/optimizers/zero_grad.h:11 */
void zero_grad_cuda(Tensor *t);
/* declared in src/kernels/cpu/shape_ops.c:8-11: da += dout for view-like ops, and the
 * transposed accumulate (da[coords] += dout[coords with axis1/axis2 swapped]).
 * shape/stride arrays are host pointers. */
void reshape_backward_cuda(float *da, const float *dout, u64 num_elements);
void transpose_backward_cuda(float *da, const float *dout, const u64 *a_shape,
                             const u64 *da_strides, const u64 *dout_strides, u64 ndim, u64 axis1,
                             u64 axis2, u64 num_elements);
/* include/core/arena_cuda.h:9-14 (called from src/core/arena.c and src/python/bindings.cpp) */
void *arena_alloc_cuda(u64 size);
void arena_free_cuda(void *ptr);
void arena_memset_cuda(void *ptr, int value, u64 size);
/* Fill policy of arena_memset_cuda for the calling thread (no counterpart in the reference).
 * The reference's arena zero-fills every allocation (src/core/arena.c:94-102): the output of a
 * forward op is written twice (4 extra bytes per element of HBM traffic on top of the op's own
 * 8 - 12) and a gradient twin is zeroed twice (src/core/tensor.c:82-90 calls zeros_cuda after the
 * arena's fill). With PLAST_B200_ARENA_SKIP_FILL, arena_memset_cuda(ptr, 0, size) returns without
 * touching memory; zeros_cuda / ones_cuda / zero_grad_cuda still fill, so gradients start at zero,
 * filled once. The caller sets it around allocations whose first use overwrites them completely
 * (every forward entry point of this library does) and restores PLAST_B200_ARENA_FILL afterwards;
 * the default is the reference's behaviour. plast_b200_arena_fill_stats reports the bytes filled and
 * the bytes skipped since the library was loaded. */
#define PLAST_B200_ARENA_FILL 0
#define PLAST_B200_ARENA_SKIP_FILL 1
void plast_b200_arena_fill_policy(int policy);
void plast_b200_arena_fill_stats(u64 *filled_bytes, u64 *skipped_bytes);
void arena_memcpy_h2d_cuda(void *dest, const void *src, u64 size);
void arena_memcpy_d2h_cuda(void *dest, const void *src, u64 size);
void arena_memcpy_d2d_cuda(void *dest, const void *src, u64 size);
/* Strided view -> contiguous copy: the gather behind include/kernels/pack.h:17-23
 * (src/kernels/cuda/cuda_pack.cu:29-96). dst is caller-allocated, numel(t) elements. The
 * C++-linkage cuda_tensor_pack_init/release wrappers are exported by the same library. */
void plast_b200_pack(const Tensor *t, void *dst);

/* Backward pieces of the reference's fused GEMM / conv epilogues (matmul_relu, matmul_bias_relu,
 * conv_relu), which stay the reference's own kernels but spend their backward in these two
 * bandwidth-bound steps. plast_b200_relu_grad_modulate replaces launch_relu_grad_modulate_cuda
 * (src/kernels/cuda/matmul_relu.cu:137-150) without the launch dims:
 * dc[i] = dout[i] * (out_data[i] > 0 ? 1 : alpha). plast_b200_bias_grad_reduce replaces the
 * cudaMemset + bias_grad_reduce_kernel pair (matmul_bias_relu.cu:143-151, 219-223): dbias[c] =
 * sum over rows of the contiguous [num_elements / cols, cols] matrix dc_mod (overwrites dbias;
 * deterministic, no float atomics). plast_b200_bias_grad_masked does both in one pass over dout
 * and out_data, so the dc_mod buffer is not needed for the bias gradient. */
void plast_b200_relu_grad_modulate(const float *dout, const float *out_data, float *dc, u64 num_elements,
                                   float alpha);
void plast_b200_bias_grad_reduce(const float *dc_mod, float *dbias, u64 num_elements, u64 cols);
void plast_b200_bias_grad_masked(const float *dout, const float *out_data, float *dbias, u64 num_elements,
                                 u64 cols, float alpha);

/* ------------------------------------------------------------------------------------------
 * Library control (no counterpart in the reference).
 * ------------------------------------------------------------------------------------------ */
typedef enum PlastB200Error {
  PLAST_B200_OK = 0,
  PLAST_B200_ERR_DTYPE = 1,     /* unsupported dtype (the reference prints and continues) */
  PLAST_B200_ERR_SHAPE = 2,     /* shapes not broadcastable / bad axis / ndim > MAX_NDIM */
  PLAST_B200_ERR_NULL = 3,      /* missing tensor, data or grad pointer */
  PLAST_B200_ERR_CUDA = 4,      /* a CUDA runtime call failed */
  PLAST_B200_ERR_UNSUPPORTED = 5, /* valid request this build has no kernel for */
  PLAST_B200_ERR_LIMIT = 6      /* size beyond a stated maximum */
} PlastB200Error;

int plast_b200_last_error(void);
const char *plast_b200_last_error_message(void);
void plast_b200_clear_error(void);
/* Stream for all following launches from any thread (a cudaStream_t; NULL = legacy default). */
void plast_b200_set_stream(void *cuda_stream);
void *plast_b200_get_stream(void);
/* 1: cudaDeviceSynchronize after every entry point like the reference does
 * (src/kernels/cuda/binary_ops.cu:113); 0 (default): asynchronous. */
void plast_b200_set_sync(int on);
/* Number of kernels this library has launched since load (all threads). */
u64 plast_b200_launch_count(void);
/* Name of the kernel family chosen by the last entry-point call on this thread
 * (e.g. "ew_vec4", "reduce_row"); for tests and profiling. */
const char *plast_b200_last_kernel(void);
/* Frees the per-device scratch the reductions keep between calls. */
void plast_b200_release_workspace(void);
const char *plast_b200_version(void);
/* Test hooks of the chain compiler (no GPU needed): the CUDA C++ functor generated for a program
 * (returns its length, copies at most capacity - 1 characters; -1 = malformed program), and a trial
 * compile of the whole kernel with NVRTC for sm_100a (0 = compiled, -2 = libnvrtc not available,
 * other = the NVRTC error, log on stderr). Bit i of scalar_mask marks input i as a one-element
 * constant, which the compiler reads once per thread through a pointer (at run time it finds
 * these itself: inputs that broadcast along every dim of the output). */
int plast_b200_chain_source(const PlastChainStep *steps, int n_steps, int n_inputs, unsigned scalar_mask,
                            char *buf, size_t capacity);
int plast_b200_chain_try_compile(const PlastChainStep *steps, int n_steps, int n_inputs,
                                 unsigned scalar_mask);
/* The same two hooks for the backward functor of input `wrt` (accumulate != 0: the kernel's last
 * operand is the input's current gradient and the functor returns the updated one). */
int plast_b200_chain_backward_source(const PlastChainStep *steps, int n_steps, int n_inputs,
                                     unsigned scalar_mask, int wrt, int accumulate, char *buf, size_t capacity);
int plast_b200_chain_backward_try_compile(const PlastChainStep *steps, int n_steps, int n_inputs,
                                          unsigned scalar_mask, int wrt, int accumulate);
/* Tuning hook: overrides one launch-geometry choice of the reductions for the whole process
 * (key 0: log2 of the lanes across a strip of the column reduce, 1: resident CTAs per SM the
 * column reduce plans for, 2: load batches per row-worker below which a column reduce is not split
 * further, 3: resident CTAs per SM the segmented reduce plans for, 4: longest dense row that the
 * thread-per-row reduction takes (0 = never; at most 48), 5: order of the column reduce's
 * CTAs, 6 / 7: L2 prefetch distance of the column sweep in load batches and the number of batches
 * per chunk that prefetch, 8: prefetch distance of the segmented reduce in trips, 9: log2 of the
 * threads that share a segment, 10: CTAs per thread-block cluster when the chunks of a column
 * reduce combine through distributed shared memory instead of a ticket in global memory, 0 or 1 =
 * never, 11: 1 = the 3-D tile kernel for inputs turned along two different dims uses 32 x 16 x 16
 * tiles instead of 8 x 32 x 32); a negative value restores the built-in choice. Results do not
 * depend on the geometry beyond the order of additions. */
void plast_b200_tune(int key, long value);
/* Test hook: runs the host-side iteration planner (drop size-1 dims, order by the strides of
 * argument `sort_arg`, merge dims every argument walks as one run) on caller-supplied metadata.
 * strides / out_strides are [nargs][MAX_NDIM] row-major, outermost dim first on input; the
 * result lists the innermost dim first. Returns the planned ndim, or -1 on bad arguments.
 * Needs no GPU. */
int plast_b200_plan_debug(const u64 *shape, u64 ndim, int nargs, const u64 *strides,
                          const unsigned char *reduced, int sort_arg, u64 *out_size,
                          u64 *out_strides, unsigned char *out_reduced);

#ifdef __cplusplus
}
#endif

#endif /* PLAST_B200_H */
