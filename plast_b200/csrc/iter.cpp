#include "iter.h"

namespace pb {

bool broadcast_strides(const Tensor *t, const u64 *out_shape, u64 out_ndim, u64 *strides_out) {
  if (t->ndim > out_ndim) return false;
  u64 shift = out_ndim - t->ndim;
  for (u64 d = 0; d < out_ndim; ++d) {
    if (d < shift) {
      strides_out[d] = 0;
      continue;
    }
    u64 j = d - shift;
    if (t->shape[j] == 1) {
      strides_out[d] = 0;
    } else if (t->shape[j] == out_shape[d]) {
      strides_out[d] = t->strides[j];
    } else {
      return false;
    }
  }
  return true;
}

void make_plan(IterPlan *plan, const u64 *shape, u64 ndim, int nargs,
               const u64 (*strides)[MAX_NDIM], const bool *reduced, int sort_arg) {
  // Work outermost-first, then flip at the end.
  u64 sz[MAX_NDIM];
  u64 st[kMaxArgs][MAX_NDIM];
  bool rd[MAX_NDIM];
  int n = 0;
  u64 total = 1;
  for (u64 d = 0; d < ndim; ++d) {
    total *= shape[d];
    if (shape[d] == 1) continue; // size-1 dims never move a pointer
    sz[n] = shape[d];
    for (int a = 0; a < nargs; ++a) st[a][n] = strides[a][d];
    rd[n] = reduced ? reduced[d] : false;
    ++n;
  }
  // Stable insertion sort: descending stride of sort_arg.
  for (int i = 1; i < n; ++i) {
    for (int j = i; j > 0 && st[sort_arg][j - 1] < st[sort_arg][j]; --j) {
      u64 t = sz[j]; sz[j] = sz[j - 1]; sz[j - 1] = t;
      bool b = rd[j]; rd[j] = rd[j - 1]; rd[j - 1] = b;
      for (int a = 0; a < nargs; ++a) {
        u64 s = st[a][j]; st[a][j] = st[a][j - 1]; st[a][j - 1] = s;
      }
    }
  }
  // Merge dim i into dim i+1 when every arg walks them as one run.
  int m = 0; // number of dims kept so far; dim m-1 is the current innermost candidate
  for (int i = 0; i < n; ++i) {
    if (m > 0) {
      bool ok = (rd[m - 1] == rd[i]);
      for (int a = 0; ok && a < nargs; ++a) ok = (st[a][m - 1] == st[a][i] * sz[i]);
      if (ok) {
        sz[m - 1] *= sz[i];
        for (int a = 0; a < nargs; ++a) st[a][m - 1] = st[a][i];
        continue;
      }
    }
    sz[m] = sz[i];
    rd[m] = rd[i];
    for (int a = 0; a < nargs; ++a) st[a][m] = st[a][i];
    ++m;
  }
  if (m == 0) { // a single element (or an empty tensor: numel 0)
    sz[0] = total == 0 ? 0 : 1;
    rd[0] = reduced ? true : false;
    if (reduced) {
      // a reduce over size-1 dims only: keep it "reduced" iff any original dim was
      bool any = false;
      for (u64 d = 0; d < ndim; ++d) any = any || reduced[d];
      rd[0] = any;
    }
    for (int a = 0; a < nargs; ++a) st[a][0] = 0;
    m = 1;
  }
  plan->ndim = m;
  plan->nargs = nargs;
  plan->numel = total;
  for (int a = 0; a < nargs; ++a) plan->max_offset[a] = 0;
  for (int d = 0; d < m; ++d) {
    int s = m - 1 - d; // flip: innermost first
    plan->size[d] = sz[s];
    plan->reduced[d] = rd[s];
    for (int a = 0; a < nargs; ++a) {
      plan->stride[a][d] = st[a][s];
      if (sz[s] > 0) plan->max_offset[a] += (sz[s] - 1) * st[a][s];
    }
  }
  for (int d = m; d < MAX_NDIM; ++d) {
    plan->size[d] = 1;
    plan->reduced[d] = false;
    for (int a = 0; a < nargs; ++a) plan->stride[a][d] = 0;
  }
}

bool is_dense(const IterPlan *plan, int a) {
  // Sort this arg's (stride, size) pairs ascending and check stride[i] == prod(size[<i]).
  u64 sz[MAX_NDIM], st[MAX_NDIM];
  int n = plan->ndim;
  for (int d = 0; d < n; ++d) {
    sz[d] = plan->size[d];
    st[d] = plan->stride[a][d];
  }
  for (int i = 1; i < n; ++i)
    for (int j = i; j > 0 && st[j - 1] > st[j]; --j) {
      u64 t = sz[j]; sz[j] = sz[j - 1]; sz[j - 1] = t;
      t = st[j]; st[j] = st[j - 1]; st[j - 1] = t;
    }
  u64 expect = 1;
  for (int d = 0; d < n; ++d) {
    if (sz[d] == 1) continue;
    if (st[d] != expect) return false;
    expect *= sz[d];
  }
  return true;
}

} // namespace pb

// Test hook (declared in include/plast_b200.h): runs the planner on caller-supplied metadata.
extern "C" int plast_b200_plan_debug(const u64 *shape, u64 ndim, int nargs, const u64 *strides,
                                     const unsigned char *reduced, int sort_arg, u64 *out_size,
                                     u64 *out_strides, unsigned char *out_reduced) {
  if (!shape || !strides || !out_size || !out_strides || ndim > MAX_NDIM || nargs < 1 ||
      nargs > pb::kMaxArgs || sort_arg < 0 || sort_arg >= nargs)
    return -1;
  u64 st[pb::kMaxArgs][MAX_NDIM] = {};
  bool red[MAX_NDIM] = {};
  for (int a = 0; a < nargs; ++a)
    for (u64 d = 0; d < ndim; ++d) st[a][d] = strides[(u64)a * MAX_NDIM + d];
  if (reduced)
    for (u64 d = 0; d < ndim; ++d) red[d] = reduced[d] != 0;
  pb::IterPlan plan;
  pb::make_plan(&plan, shape, ndim, nargs, st, reduced ? red : nullptr, sort_arg);
  for (int d = 0; d < MAX_NDIM; ++d) {
    out_size[d] = plan.size[d];
    if (out_reduced) out_reduced[d] = plan.reduced[d] ? 1 : 0;
    for (int a = 0; a < nargs; ++a) out_strides[(u64)a * MAX_NDIM + d] = plan.stride[a][d];
  }
  return plan.ndim;
}
