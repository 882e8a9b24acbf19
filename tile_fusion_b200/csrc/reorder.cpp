// Reordered layouts of the reference's executors, and a bandwidth-reducing ordering.
//
//   * tf_schedule_unfused_csr    the rows of the second wave of a schedule as a CSR of their own, in
//                                schedule order (createUnfusedData,
//                                fusion/example/SpMM_SpMM_SP_Demo_Utils.h:600-636);
//   * tf_schedule_reordered_adj  all rows of A in the order the schedule visits them as second-loop rows,
//                                with the old row of every new row and the re-based per-partition pointers
//                                (createReorderedAdj, fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:618-653);
//   * tf_rcm_order / tf_permute_csr   reverse Cuthill-McKee on the symmetrised pattern and P A P^T.  The
//                                reference reorders with METIS (get_reorderd_matrix, fusion/src/Fusion_Utils.cpp:181-203,
//                                compiled only with METIS); the purpose is the same -- pull a row's columns next to
//                                the row, which is what both the reference's fusion criterion and the gather tiles
//                                of this library feed on.
#include <algorithm>
#include <cstdlib>
#include <numeric>
#include <queue>
#include <vector>

#include "tf_internal.h"

namespace {

using tf::fail;

template <class T>
T *dup(const std::vector<T> &v) {
  T *b = (T *)malloc(sizeof(T) * std::max<size_t>(v.size(), 1));
  if (b && !v.empty()) std::copy(v.begin(), v.end(), b);
  return b;
}

}  // namespace

extern "C" {

// Arrays are malloc'd (tf_free): uf_ap[n_rows + 1], uf_ai / uf_ax[uf_ap[n_rows]].
int tf_schedule_unfused_csr(const tf_schedule *s, int m, const int *ap, const int *ai, const float *ax, int **uf_ap, int **uf_ai,
                            float **uf_ax, int *n_rows) {
  if (!s || !ap || !ai || !ax || !uf_ap || !uf_ai || !uf_ax || !n_rows) return fail(TF_ERR_ARG, "tf_schedule_unfused_csr: null argument");
  if (!s->has_ker || s->n1 < 2) return fail(TF_ERR_ARG, "tf_schedule_unfused_csr: needs a two-wave schedule with ker_begin");
  std::vector<int> p(1, 0), ci;
  std::vector<float> x;
  for (int l1 = s->ptr1[1]; l1 < s->ptr1[2]; ++l1)
    for (int i1 = s->ker[2 * l1]; i1 < s->ker[2 * l1 + 1]; ++i1) {
      const int row = s->id[i1];
      if (row < 0 || row >= m) return fail(TF_ERR_ARG, "tf_schedule_unfused_csr: schedule row out of range");
      for (int j = ap[row]; j < ap[row + 1]; ++j) { ci.push_back(ai[j]); x.push_back(ax[j]); }
      p.push_back((int)ci.size());
    }
  *uf_ap = dup(p); *uf_ai = dup(ci); *uf_ax = dup(x); *n_rows = (int)p.size() - 1;
  if (!*uf_ap || !*uf_ai || !*uf_ax) return fail(TF_ERR_NOMEM, "tf_schedule_unfused_csr: out of memory");
  return TF_OK;
}

// Arrays are malloc'd (tf_free): r_ap[m + 1], r_ai / r_ax[nnz], l2_ptr[m] (old row of every new row),
// new_mix[2 * (partitions + 1)].
int tf_schedule_reordered_adj(const tf_schedule *s, int m, const int *ap, const int *ai, const float *ax, int **r_ap, int **r_ai,
                              float **r_ax, int **l2_ptr, int **new_mix, int *n_mix) {
  if (!s || !ap || !ai || !ax || !r_ap || !r_ai || !r_ax || !l2_ptr || !new_mix || !n_mix)
    return fail(TF_ERR_ARG, "tf_schedule_reordered_adj: null argument");
  if (!s->has_ker || s->n1 < 1) return fail(TF_ERR_ARG, "tf_schedule_reordered_adj: needs a schedule with ker_begin");
  const int levels = 2;
  const int n_parts = s->n1 >= 2 ? s->ptr1[2] : s->ptr1[1];
  std::vector<int> p((size_t)m + 1, 0), ci((size_t)ap[m]), l2((size_t)m, 0), mix(2 * ((size_t)n_parts + 1), 0);
  std::vector<float> x((size_t)ap[m]);
  int nnz = 0, rows = 0;
  for (int l1 = 0; l1 < levels && l1 < s->n1; ++l1)
    for (int p1 = s->ptr1[l1]; p1 < s->ptr1[l1 + 1]; ++p1) {
      const int kb = s->ker[2 * p1], ke = s->ker[2 * p1 + 1];
      mix[2 * ((size_t)p1 + 1)] = kb - rows;
      for (int i1 = kb; i1 < ke; ++i1) {
        const int row = s->id[i1];
        if (row < 0 || row >= m || rows >= m) return fail(TF_ERR_ARG, "tf_schedule_reordered_adj: schedule does not list every row once");
        l2[rows] = row;
        for (int j = ap[row]; j < ap[row + 1]; ++j) { x[nnz] = ax[j]; ci[nnz] = ai[j]; ++nnz; }
        p[++rows] = nnz;
      }
      mix[2 * ((size_t)p1 + 1) + 1] = rows;
    }
  *r_ap = dup(p); *r_ai = dup(ci); *r_ax = dup(x); *l2_ptr = dup(l2); *new_mix = dup(mix); *n_mix = (int)mix.size();
  if (!*r_ap || !*r_ai || !*r_ax || !*l2_ptr || !*new_mix) return fail(TF_ERR_NOMEM, "tf_schedule_reordered_adj: out of memory");
  return TF_OK;
}

// perm[new] = old.  Reverse Cuthill-McKee over the pattern of A + A^T, every component started from a vertex of
// lowest degree, neighbours visited by increasing degree (ties by index: the order is deterministic).
int tf_rcm_order(int m, const int *ap, const int *ai, int *perm) {
  if (!ap || !ai || !perm || m <= 0) return fail(TF_ERR_ARG, "tf_rcm_order: bad argument");
  std::vector<int> deg((size_t)m, 0);
  for (int r = 0; r < m; ++r)
    for (int j = ap[r]; j < ap[r + 1]; ++j) {
      const int c = ai[j];
      if (c < 0 || c >= m) return fail(TF_ERR_ARG, "tf_rcm_order: needs a square matrix");
      if (c != r) { ++deg[r]; ++deg[c]; }
    }
  std::vector<long long> sp((size_t)m + 1, 0);
  for (int r = 0; r < m; ++r) sp[r + 1] = sp[r] + deg[r];
  std::vector<int> adj((size_t)sp[m]), fill((size_t)m, 0);
  for (int r = 0; r < m; ++r)
    for (int j = ap[r]; j < ap[r + 1]; ++j) {
      const int c = ai[j];
      if (c == r) continue;
      adj[sp[r] + fill[r]++] = c;
      adj[sp[c] + fill[c]++] = r;
    }
  // (entries present in both triangles appear twice in a list; harmless for the traversal)
  std::vector<int> order;
  order.reserve(m);
  std::vector<char> seen((size_t)m, 0);
  std::vector<int> by_deg((size_t)m);
  std::iota(by_deg.begin(), by_deg.end(), 0);
  std::stable_sort(by_deg.begin(), by_deg.end(), [&](int a, int b) { return deg[a] < deg[b]; });
  std::vector<int> nb;
  for (int start : by_deg) {
    if (seen[start]) continue;
    seen[start] = 1;
    size_t head = order.size();
    order.push_back(start);
    while (head < order.size()) {
      const int v = order[head++];
      nb.clear();
      for (long long q = sp[v]; q < sp[v + 1]; ++q)
        if (!seen[adj[q]]) { seen[adj[q]] = 1; nb.push_back(adj[q]); }
      std::sort(nb.begin(), nb.end(), [&](int a, int b) { return deg[a] != deg[b] ? deg[a] < deg[b] : a < b; });
      order.insert(order.end(), nb.begin(), nb.end());
    }
  }
  for (int i = 0; i < m; ++i) perm[i] = order[(size_t)m - 1 - i];
  return TF_OK;
}

// B = P A P^T with perm[new] = old: row `new` of B is row perm[new] of A with every column c replaced by its new
// index.  Columns of B are sorted.  out arrays are caller-allocated: b_ap[m + 1], b_ai / b_ax[ap[m]].
int tf_permute_csr(int m, const int *ap, const int *ai, const float *ax, const int *perm, int *b_ap, int *b_ai, float *b_ax) {
  if (!ap || !ai || !ax || !perm || !b_ap || !b_ai || !b_ax || m <= 0) return fail(TF_ERR_ARG, "tf_permute_csr: bad argument");
  std::vector<int> inv((size_t)m, -1);
  for (int i = 0; i < m; ++i) {
    if (perm[i] < 0 || perm[i] >= m || inv[perm[i]] != -1) return fail(TF_ERR_ARG, "tf_permute_csr: perm is not a permutation");
    inv[perm[i]] = i;
  }
  std::vector<std::pair<int, float>> row;
  b_ap[0] = 0;
  for (int i = 0; i < m; ++i) {
    const int old = perm[i];
    row.clear();
    for (int j = ap[old]; j < ap[old + 1]; ++j) {
      if (ai[j] < 0 || ai[j] >= m) return fail(TF_ERR_ARG, "tf_permute_csr: needs a square matrix");
      row.emplace_back(inv[ai[j]], ax[j]);
    }
    std::sort(row.begin(), row.end(), [](const std::pair<int, float> &a, const std::pair<int, float> &b) { return a.first < b.first; });
    int q = b_ap[i];
    for (const auto &e : row) { b_ai[q] = e.first; b_ax[q] = e.second; ++q; }
    b_ap[i + 1] = q;
  }
  return TF_OK;
}

}  // extern "C"
