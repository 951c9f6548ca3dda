// target.grad (+)= term(in0 .. inN-1), where the target operand may broadcast against the
// iteration shape. Dims the operand broadcasts over (size 1, missing, or stride 0) collapse onto
// one gradient address, so they are summed first (the broadcast-gradient reduce of
// include/kernels/kernel_macros.h:273-300) and the sum is then added to the gradient buffer;
// without broadcast dims this is a plain elementwise accumulate.
#pragma once

#include "ew_engine.cuh"
#include "reduce_engine.cuh"

namespace pb {

template <class Term, int NIN> struct AccumulateTerm { // x = {in0..inN-1, old}
  Term t;
  __device__ __forceinline__ float operator()(const float *x) const { return x[NIN] + t(x); }
};

// shape/ndim: iteration space (the upstream gradient's shape). target_strides: the operand's
// strides aligned to that shape (0 where it broadcasts). in_strides[a]: aligned input strides.
template <class Term, int NIN>
void accumulate_grad(const u64 *shape, u64 ndim, float *target, const u64 *target_strides,
                     const u64 (*in_strides)[MAX_NDIM], const float *const *ins, const Term &term) {
  bool reduced[MAX_NDIM] = {};
  bool any_reduced = false;
  for (u64 d = 0; d < ndim; ++d) {
    reduced[d] = (target_strides[d] == 0 && shape[d] > 1);
    any_reduced = any_reduced || reduced[d];
  }
  u64 st[NIN + 2][MAX_NDIM] = {};
  for (u64 d = 0; d < ndim; ++d) {
    st[0][d] = target_strides[d];
    for (int a = 0; a < NIN; ++a) st[a + 1][d] = in_strides[a][d];
    st[NIN + 1][d] = target_strides[d];
  }
  IterPlan plan;
  if (!any_reduced) {
    make_plan(&plan, shape, ndim, NIN + 2, st, nullptr, 0);
    const float *all[NIN + 1];
    for (int a = 0; a < NIN; ++a) all[a] = ins[a];
    all[NIN] = target;
    launch_ew<AccumulateTerm<Term, NIN>, NIN + 1>(plan, target, all, AccumulateTerm<Term, NIN>{term});
  } else {
    make_plan(&plan, shape, ndim, NIN + 1, st, reduced, 1);
    launch_reduce<SumOp, Term, NIN>(plan, target, ins, term, SumOp{}, /*accumulate=*/true, 0.0f);
  }
}

} // namespace pb
