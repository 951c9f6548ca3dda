// Host-side iteration planner ("tensor iterator"). Plain C++, no CUDA: it turns the
// (shape, strides) of an output and its operands into a canonical iteration space that the
// kernels receive BY VALUE — the Tensor structs and their shape/stride arrays live in host
// memory (plast/_internal.py:14,23 allocates them from a CPU arena), so nothing on the device
// may dereference them.
//
// Canonical form: size-1 dims dropped, dims ordered by a chosen operand's stride, adjacent dims
// merged when every operand walks them as one run (and, for reductions, when both are kept or
// both reduced). Dim 0 is the INNERMOST (fastest varying) dim.
#pragma once

#include "plast_b200.h"

#include <stdint.h>

namespace pb {

constexpr int kMaxArgs = 11; // output + up to 10 operands (the widest fused chain's backward)
static_assert(PLAST_CHAIN_MAX_INPUTS + 3 <= kMaxArgs, "a chain's operands must fit the planner");

struct IterPlan {
  int ndim = 0;  // >= 1 after planning (a single element plans as one dim of size 1)
  int nargs = 0; // arg 0 is the output of an elementwise op / the streamed input of a reduce
  u64 size[MAX_NDIM] = {};
  u64 stride[kMaxArgs][MAX_NDIM] = {}; // elements; 0 = broadcast along that dim
  bool reduced[MAX_NDIM] = {};         // reductions only: dim is summed away
  u64 numel = 0;
  u64 max_offset[kMaxArgs] = {}; // largest element offset each arg touches
};

// Strides of `t` aligned to an output of `out_ndim` dims (NumPy rules, right-aligned):
// missing leading dims and size-1 dims get stride 0 (include/kernels/kernel_macros.h:156-168).
// Returns false when t's shape does not broadcast to out_shape.
bool broadcast_strides(const Tensor *t, const u64 *out_shape, u64 out_ndim, u64 *strides_out);

// Builds the canonical plan. `strides[a][d]` are per-arg strides aligned to `shape` (outermost
// first, as in a Tensor). `sort_arg` is the arg whose strides order the dims (descending, so its
// memory order becomes the iteration order); `reduced` may be NULL.
void make_plan(IterPlan *plan, const u64 *shape, u64 ndim, int nargs,
               const u64 (*strides)[MAX_NDIM], const bool *reduced, int sort_arg);

// True when the dims of arg `a` tile a dense block of memory exactly once (some permutation of
// a contiguous layout, no gaps, no overlap).
bool is_dense(const IterPlan *plan, int a);

} // namespace pb
