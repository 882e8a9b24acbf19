// Host planner: turns the sparsity patterns of a chain into the ticket-ordered
// item list the persistent executor walks.
//
// Rows of the intermediate T = (first operator) * C are produced in row blocks
// and rows of D = A * T are consumed in row blocks.  A consumer block may run
// once every producer block that covers its column window is complete.  Items
// are handed to CTAs in list order, so the list is a topological order of that
// dependence: a consumer is listed `slack` blocks after the last producer it
// needs, which gives that producer time to finish before the consumer's ticket
// comes up.  When every consumer window (plus slack) fits in `ring_bytes`, the
// intermediate is a ring of that many rows -- small enough to stay in L2, so T
// never travels to HBM -- and a producer additionally waits until the consumers
// that still read the rows it is about to overwrite have finished.
#include <algorithm>
#include <climits>
#include <cstdlib>

#include "tf_internal.h"

namespace tf {

namespace {

// consecutive row blocks with at most `rows` rows and `max_nnz` nonzeros (a heavier row stands alone)
std::vector<int> split_rows(int m, const int *ap, int rows, int max_nnz) {
  std::vector<int> b{0};
  int r = 0;
  while (r < m) {
    int e = r + 1;
    if (ap) {
      long long nnz = ap[r + 1] - ap[r];
      while (e < m && e - r < rows && nnz + (ap[e + 1] - ap[e]) <= max_nnz) { nnz += ap[e + 1] - ap[e]; ++e; }
    } else {
      e = std::min(m, r + rows);
    }
    b.push_back(e);
    r = e;
  }
  return b;
}

inline int block_of(const std::vector<int> &bounds, int row) {
  return (int)(std::upper_bound(bounds.begin(), bounds.end(), row) - bounds.begin()) - 1;
}

}  // namespace

int build_stream_plan(const PlanParams &pp, const int *first_ap, const int * /*first_ai*/, const int *sec_ap,
                      const int *sec_ai, HostPlan &out) {
  const int m = pp.m;
  const int rb = pp.rows_per_block;
  out.prod_rows = split_rows(m, pp.producer_is_gemm ? nullptr : first_ap, rb, pp.max_block_nnz);
  out.cons_rows = split_rows(m, sec_ap, rb, pp.max_block_nnz);
  const int np = (int)out.prod_rows.size() - 1, nc = (int)out.cons_rows.size() - 1;

  // column window of every consumer block, local columns only (columns >= m are halo rows)
  std::vector<int> cmin(nc, INT_MAX), cmax(nc, -1);
  std::vector<char> halo(nc, 0);
  for (int c = 0; c < nc; ++c)
    for (int r = out.cons_rows[c]; r < out.cons_rows[c + 1]; ++r)
      for (int j = sec_ap[r]; j < sec_ap[r + 1]; ++j) {
        const int col = sec_ai[j];
        if (col >= m) { halo[c] = 1; continue; }
        cmin[c] = std::min(cmin[c], col);
        cmax[c] = std::max(cmax[c], col);
      }
  // monotone closure so that one contiguous watermark per side expresses every dependence
  std::vector<int> emax(nc), emin(nc);
  for (int c = 0, run = -1; c < nc; ++c) { run = std::max(run, cmax[c]); emax[c] = run; }
  for (int c = nc - 1, run = INT_MAX; c >= 0; --c) { run = std::min(run, cmin[c]); emin[c] = run; }
  std::vector<int> need(nc);  // producer blocks that must be complete
  for (int c = 0; c < nc; ++c) need[c] = emax[c] < 0 ? 0 : block_of(out.prod_rows, emax[c]) + 1;

  int slack = pp.slack_blocks >= 0 ? pp.slack_blocks : std::max(1, pp.max_ctas / 2);
  slack = std::min(slack, np);
  int max_block = 1;
  for (int p = 0; p < np; ++p) max_block = std::max(max_block, out.prod_rows[p + 1] - out.prod_rows[p]);

  // widest live window in rows: from the lowest row any not-yet-finished consumer still reads to the
  // highest row produced when that consumer's ticket comes up
  long long span = 0;
  for (int c = 0; c < nc; ++c) {
    if (emax[c] < 0) continue;
    const int hi_block = std::min(np, need[c] + slack);
    const long long hi_row = out.prod_rows[hi_block];
    const long long lo_row = std::min<long long>(emin[c] == INT_MAX ? hi_row : emin[c], hi_row);
    span = std::max(span, hi_row - lo_row);
  }
  const bool multi = pp.halo_rows > 0 || !pp.boundary_rows.empty();
  long long ring_rows = 0;
  if (pp.ring_bytes > 0 && !multi) {
    // producers run up to `slack` blocks past the window before they have to wait
    long long want = span + (long long)(slack + 2) * max_block;
    want = (want + 7) / 8 * 8;
    if (want * pp.n_cols * 4LL <= pp.ring_bytes && want < m) ring_rows = want;
  }
  out.ring_rows = ring_rows;
  out.inter_rows = ring_rows ? ring_rows : (long long)m + pp.halo_rows;

  // consumers a producer must see finished before it may overwrite its ring slot
  auto cons_before = [&](int p) -> int {
    if (!ring_rows) return 0;
    const long long x = (long long)out.prod_rows[p + 1] - 1 - ring_rows;  // highest old row in the slot
    if (x < 0) return 0;
    // consumers c with emin[c] <= x still read rows at or below x; emin is non-decreasing
    int lo = 0, hi = nc;
    while (lo < hi) { int mid = (lo + hi) / 2; if (emin[mid] <= x) lo = mid + 1; else hi = mid; }
    return lo;
  };

  out.items.clear();
  out.phase_begin[0] = 0;
  out.phase_begin[1] = 0;  // phase 0 (boundary rows) is a row-list kernel, not items
  int pi = 0, ci = 0;
  std::vector<int> late;  // consumers that read halo rows
  auto emit_cons = [&](int c) {
    Item it{};
    it.kind = ITEM_CONSUME; it.block = c;
    it.row_begin = out.cons_rows[c]; it.row_end = out.cons_rows[c + 1];
    it.need = need[c];
    it.base = 0;
    if (ring_rows && emin[c] != INT_MAX) it.base = (int)((emin[c] / ring_rows) * ring_rows);
    out.items.push_back(it);
  };
  while (pi < np || ci < nc) {
    while (ci < nc && halo[ci] && multi) { late.push_back(ci); ++ci; }
    if (ci >= nc && pi >= np) break;
    const bool cons_ready = ci < nc && pi >= std::min(np, need[ci] + slack);
    if (cons_ready) { emit_cons(ci); ++ci; continue; }
    if (pi < np) {
      const int cb = cons_before(pi);
      if (cb > ci) {
        // ring too small for this ordering: should not happen given how ring_rows was sized
        return fail(TF_ERR_UNSUPPORTED, "planner: ring dependence cycle (internal sizing error)");
      }
      Item it{};
      it.kind = ITEM_PRODUCE; it.block = pi;
      it.row_begin = out.prod_rows[pi]; it.row_end = out.prod_rows[pi + 1];
      it.need = cb;
      out.items.push_back(it);
      ++pi;
      continue;
    }
    // only consumers left and all producers are listed
    emit_cons(ci); ++ci;
  }
  out.phase_begin[2] = (int)out.items.size();
  for (int c : late) emit_cons(c);
  out.phase_begin[3] = (int)out.items.size();
  return TF_OK;
}

int build_single_pass_plan(const PlanParams &pp, const int *ap, HostPlan &out) {
  out.prod_rows.clear();
  out.cons_rows = split_rows(pp.m, ap, pp.rows_per_block, pp.max_block_nnz);
  const int nc = (int)out.cons_rows.size() - 1;
  out.items.clear();
  for (int c = 0; c < nc; ++c) {
    Item it{};
    it.kind = ITEM_SDDMM; it.block = c;
    it.row_begin = out.cons_rows[c]; it.row_end = out.cons_rows[c + 1];
    out.items.push_back(it);
  }
  out.phase_begin[0] = out.phase_begin[1] = 0;
  out.phase_begin[2] = out.phase_begin[3] = (int)out.items.size();
  out.ring_rows = 0;
  out.inter_rows = 0;
  return TF_OK;
}

}  // namespace tf

// Host-only view of the stream plan, for inspection and for tests that have no GPU.
extern "C" int tf_plan_preview(const tf_csr *A, const tf_csr *B, int producer_is_gemm, int n_cols,
                               const tf_plan_opts *o, int resident_ctas, int **items_out, long long *n_items,
                               long long info[8]) {
  if (!A || !items_out || !n_items || !info) return tf::fail(TF_ERR_ARG, "tf_plan_preview: null argument");
  tf::PlanParams pp;
  pp.m = A->m; pp.n_cols = n_cols;
  pp.producer_is_gemm = producer_is_gemm != 0;
  pp.rows_per_block = o && o->rows_per_block > 0 ? o->rows_per_block : (producer_is_gemm ? 64 : (n_cols >= 128 ? 64 : 128));
  pp.max_block_nnz = pp.rows_per_block * 32;
  pp.halo_rows = o ? o->halo_rows : 0;
  if (o && o->n_boundary > 0) pp.boundary_rows.assign(o->boundary_rows, o->boundary_rows + o->n_boundary);
  const int rb = o ? o->ring_bytes : 0;
  pp.ring_bytes = rb == 0 ? (48LL << 20) : (long long)rb;
  pp.max_ctas = resident_ctas;
  pp.slack_blocks = o ? o->slack_blocks : -1;
  if (o && o->mode == TF_MODE_UNFUSED) { pp.slack_blocks = 1 << 30; pp.ring_bytes = -1; }
  const tf_csr *F = producer_is_gemm ? nullptr : (B ? B : A);
  tf::HostPlan hp;
  int rc = tf::build_stream_plan(pp, F ? F->ap : nullptr, F ? F->ai : nullptr, A->ap, A->ai, hp);
  if (rc != TF_OK) return rc;
  int *buf = (int *)malloc(sizeof(int) * 8 * std::max<size_t>(hp.items.size(), 1));
  if (!buf) return tf::fail(TF_ERR_NOMEM, "tf_plan_preview: out of memory");
  for (size_t i = 0; i < hp.items.size(); ++i) {
    const tf::Item &it = hp.items[i];
    int *q = buf + 8 * i;
    q[0] = it.kind; q[1] = it.block; q[2] = it.row_begin; q[3] = it.row_end;
    q[4] = it.need; q[5] = it.base; q[6] = it.aux0; q[7] = it.aux1;
  }
  *items_out = buf;
  *n_items = (long long)hp.items.size();
  info[0] = (long long)hp.items.size();
  info[1] = (long long)hp.prod_rows.size() - 1;
  info[2] = (long long)hp.cons_rows.size() - 1;
  info[3] = hp.ring_rows;
  info[4] = hp.phase_begin[1]; info[5] = hp.phase_begin[2]; info[6] = hp.phase_begin[3];
  info[7] = hp.inter_rows;
  return TF_OK;
}

extern "C" void tf_free(void *p) { free(p); }
