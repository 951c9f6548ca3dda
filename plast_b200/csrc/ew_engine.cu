// Host-side geometry choice for the elementwise engine.
#include "ew_engine.cuh"

namespace pb {

FastDivU32 make_fast_div(uint32_t d) {
  // For 1 <= d < 2^31 and n < 2^31: n / d == (umulhi(n, magic) + n) >> shift.
  FastDivU32 r;
  uint32_t s = 0;
  while (s < 32 && (1ull << s) < (unsigned long long)d) ++s;
  unsigned long long one = 1;
  r.magic = (uint32_t)(((one << 32) * ((one << s) - d)) / d + 1);
  r.shift = s;
  return r;
}

EwChoice choose_ew(const IterPlan &plan, const void *const *ptrs, int nargs, u64 *n_items,
                   uint32_t *vec_mask) {
  EwChoice c;
  c.vec = 1;
  c.one_d = (plan.ndim == 1);
  *vec_mask = 0;
  const int cand[2] = {4, 2};
  for (int ci = 0; ci < 2; ++ci) {
    const int vec = cand[ci];
    bool ok = plan.size[0] % (u64)vec == 0 && plan.stride[0][0] == 1;
    uint32_t mask = 0;
    for (int a = 0; ok && a < nargs; ++a) {
      const u64 s0 = plan.stride[a][0];
      if (s0 == 0) continue; // broadcast along dim 0: scalar load
      if (s0 != 1) { ok = false; break; }
      if (((uintptr_t)ptrs[a]) % (sizeof(float) * vec) != 0) { ok = false; break; }
      for (int d = 1; d < plan.ndim; ++d)
        if (plan.stride[a][d] % (u64)vec != 0) { ok = false; break; }
      if (a > 0) mask |= 1u << (a - 1);
    }
    if (ok) {
      c.vec = vec;
      *vec_mask = mask;
      break;
    }
  }
  *n_items = plan.numel / (u64)c.vec;
  c.idx64 = *n_items > 0x7fffffffull;
  for (int a = 0; a < nargs; ++a)
    if (plan.max_offset[a] > 0xffffffffull) c.idx64 = true;
  for (int d = 0; d < plan.ndim; ++d)
    if (plan.size[d] > 0x7fffffffull * (d == 0 ? (u64)c.vec : 1)) c.idx64 = true;
  return c;
}

int choose_tiled_dim(const IterPlan &plan, int nargs, unsigned *tmask) {
  *tmask = 0;
  if (plan.ndim < 2 || plan.stride[0][0] != 1) return -1; // output must run along dim 0
  int dT = -1;
  unsigned mask = 0;
  for (int a = 1; a < nargs; ++a) {
    const u64 s0 = plan.stride[a][0];
    if (s0 <= 1) continue; // contiguous or broadcast along dim 0: read directly
    int mine = -1;
    for (int d = 1; d < plan.ndim; ++d)
      if (plan.stride[a][d] == 1 && plan.size[d] > 1) mine = d;
    if (mine < 0 || (dT >= 0 && mine != dT)) return -1; // strided with no unit-stride dim, or two different ones
    dT = mine;
    mask |= 1u << (a - 1);
  }
  if (dT < 0) return -1;
  if (plan.size[0] < 8 || plan.size[dT] < 8) return -1; // tiny extents: the generic kernel is fine
  *tmask = mask;
  return dT;
}

} // namespace pb
