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

// Units of the direct path: consecutive row blocks with at most `rows` rows and `max_nnz` nonzeros; a
// row of kHeavyRowNnz or more nonzeros stands alone; a row above kSegmentNnz is cut into segments.
std::vector<Unit> split_rows(int m, const int *ap, int rows, int max_nnz) {
  std::vector<Unit> u;
  int r = 0;
  while (r < m) {
    if (!ap) {
      const int e = std::min(m, r + rows);
      u.push_back(Unit{r, e, 0, 0, false});
      r = e;
      continue;
    }
    const int len = ap[r + 1] - ap[r];
    if (len > kSegmentNnz) {
      const int nseg = (len + kSegmentNnz - 1) / kSegmentNnz, per = (len + nseg - 1) / nseg;
      for (int s = 0; s < nseg; ++s)
        u.push_back(Unit{r, r + 1, ap[r] + s * per, std::min(ap[r + 1], ap[r] + (s + 1) * per), true});
      ++r;
      continue;
    }
    int e = r + 1;
    if (len < kHeavyRowNnz) {
      long long nnz = len;
      while (e < m && e - r < rows && ap[e + 1] - ap[e] < kHeavyRowNnz && nnz + (ap[e + 1] - ap[e]) <= max_nnz) {
        nnz += ap[e + 1] - ap[e];
        ++e;
      }
    }
    u.push_back(Unit{r, e, ap[r], ap[e], false});
    r = e;
  }
  return u;
}

inline int block_of(const std::vector<int> &bounds, int row) {
  return (int)(std::upper_bound(bounds.begin(), bounds.end(), row) - bounds.begin()) - 1;
}

}  // namespace

int build_stream_plan(const PlanParams &pp, const int *first_ap, const int *first_ai, const int *sec_ap,
                      const int *sec_ai, const Tiling *ptile, const Tiling *ctile, HostPlan &out) {
  const int m = pp.m;
  const int rb = pp.rows_per_block;
  const bool p_tiled = ptile && ptile->tiled, c_tiled = ctile && ctile->tiled;

  // ---- units: gather tiles where the operator is tiled, consecutive row blocks otherwise ----
  out.prod_units.clear();
  out.cons_units.clear();
  out.seg_t_rows.clear();
  out.seg_out_rows.clear();
  if (!p_tiled) out.prod_units = split_rows(m, pp.producer_is_gemm ? nullptr : first_ap, rb, pp.max_block_nnz);
  if (!c_tiled) out.cons_units = split_rows(m, sec_ap, rb, pp.max_block_nnz);
  const int np = p_tiled ? ptile->tiles() : (int)out.prod_units.size();
  const int nc = c_tiled ? ctile->tiles() : (int)out.cons_units.size();
  bool any_seg = false;
  for (const Unit &u : out.prod_units) if (u.seg) { any_seg = true; if (out.seg_t_rows.empty() || out.seg_t_rows.back() != u.r0) out.seg_t_rows.push_back(u.r0); }
  for (const Unit &u : out.cons_units) if (u.seg) { any_seg = true; if (out.seg_out_rows.empty() || out.seg_out_rows.back() != u.r0) out.seg_out_rows.push_back(u.r0); }
  out.n_prod = np;
  out.n_cons = nc;

  std::vector<int> prod_of_row((size_t)m, 0), pmin(np, INT_MAX), pmax(np, -1);
  for (int j = 0; j < np; ++j) {
    if (p_tiled) {
      for (int k = ptile->tile_row_ptr[j]; k < ptile->tile_row_ptr[j + 1]; ++k) {
        const int r = ptile->rows[k];
        prod_of_row[r] = j; pmin[j] = std::min(pmin[j], r); pmax[j] = std::max(pmax[j], r);
      }
    } else {
      // the last segment of a cut row stands for the row: waiting for it waits for every earlier unit
      for (int r = out.prod_units[j].r0; r < out.prod_units[j].r1; ++r) prod_of_row[r] = j;
      pmin[j] = out.prod_units[j].r0; pmax[j] = out.prod_units[j].r1 - 1;
    }
  }
  // what every consumer unit reads: lowest / highest local row, last producer unit, any halo row
  std::vector<int> cmin(nc, INT_MAX), cmax(nc, -1), need(nc, 0);
  std::vector<char> halo(nc, 0);
  auto see = [&](int c, int col) {
    if (col >= m) { halo[c] = 1; return; }
    cmin[c] = std::min(cmin[c], col);
    cmax[c] = std::max(cmax[c], col);
    need[c] = std::max(need[c], prod_of_row[col] + 1);
  };
  for (int c = 0; c < nc; ++c) {
    if (c_tiled) {
      for (int k = ctile->tile_halo_ptr[c]; k < ctile->tile_halo_ptr[c + 1]; ++k) see(c, ctile->halo[k]);
    } else {
      const Unit &u = out.cons_units[c];
      if (u.seg) { for (int j = u.p0; j < u.p1; ++j) see(c, sec_ai[j]); }
      else for (int r = u.r0; r < u.r1; ++r)
        for (int j = sec_ap[r]; j < sec_ap[r + 1]; ++j) see(c, sec_ai[j]);
    }
  }

  // every resident CTA holds the item it works on and the next ticket, about half of them producers
  // bounds used by the host pipeline that overlaps copies with execution
  std::vector<int> psrc_max(np, 0), cout_min(nc, 0);
  for (int j = 0; j < np; ++j) {
    int mx = 0;
    if (pp.producer_is_gemm) mx = pmax[j];
    else if (p_tiled) { for (int k = ptile->tile_halo_ptr[j]; k < ptile->tile_halo_ptr[j + 1]; ++k) mx = std::max(mx, ptile->halo[k]); }
    else {
      const Unit &u = out.prod_units[j];
      const int q0 = u.seg ? u.p0 : first_ap[u.r0], q1 = u.seg ? u.p1 : first_ap[u.r1];
      for (int q = q0; q < q1; ++q) mx = std::max(mx, first_ai[q]);
    }
    psrc_max[j] = mx;
  }
  for (int c = 0; c < nc; ++c) {
    int mn = INT_MAX;
    if (c_tiled) { for (int k = ctile->tile_row_ptr[c]; k < ctile->tile_row_ptr[c + 1]; ++k) mn = std::min(mn, ctile->rows[k]); }
    else mn = out.cons_units[c].r0;
    cout_min[c] = mn == INT_MAX ? 0 : mn;
  }

  int slack = pp.slack_blocks >= 0 ? pp.slack_blocks : std::max(1, pp.max_ctas + 8);
  slack = std::min(slack, np);
  const bool multi = pp.halo_rows > 0 || !pp.boundary_rows.empty();

  // ---- ticket order: a consumer is listed once `slack` producers beyond its last need are listed ----
  struct Entry { int is_cons, idx, cons_before; };
  std::vector<Entry> order;
  order.reserve((size_t)np + nc);
  std::vector<int> late;
  {
    int pi = 0, ci = 0;
    while (pi < np || ci < nc) {
      while (ci < nc && halo[ci] && multi) { late.push_back(ci); ++ci; }
      if (ci >= nc && pi >= np) break;
      if (ci < nc && pi >= std::min(np, need[ci] + slack)) { order.push_back({1, ci, ci}); ++ci; }
      else if (pi < np) { order.push_back({0, pi, ci}); ++pi; }
      else { order.push_back({1, ci, ci}); ++ci; }
    }
  }
  // lowest row still to be read by consumer c or any later one (halo consumers never read the ring)
  std::vector<int> sufmin((size_t)nc + 1, INT_MAX);
  for (int c = nc - 1; c >= 0; --c) sufmin[c] = std::min(sufmin[c + 1], (multi && halo[c]) ? INT_MAX : cmin[c]);

  // ---- ring: large enough that a producer never overwrites a row a listed-later consumer reads ----
  long long ring_rows = 0;
  if (pp.ring_bytes > 0 && !multi && !any_seg) {
    // A producer should find its slot free without waiting: count as finished only the consumers
    // listed at least `lag` tickets before it (about one ticket per resident CTA).
    const int lag = 2 * slack + 2;
    long long live = 0;
    for (size_t q = 0; q < order.size(); ++q) {
      const Entry &e = order[q];
      if (e.is_cons) continue;
      live = std::max<long long>(live, (long long)pmax[e.idx] - pmin[e.idx] + 1);
      const int done_before = q >= (size_t)lag ? order[q - lag].cons_before : 0;
      if (sufmin[done_before] != INT_MAX && sufmin[done_before] <= pmax[e.idx])
        live = std::max<long long>(live, (long long)pmax[e.idx] - sufmin[done_before] + 1);
    }
    for (int c = 0; c < nc; ++c)
      if (cmax[c] >= 0) live = std::max<long long>(live, (long long)cmax[c] - cmin[c] + 1);
    const long long want = (live + 1 + 7) / 8 * 8;
    if (want * pp.n_cols * 4LL <= pp.ring_bytes && want < m) ring_rows = want;
  }
  out.ring_rows = ring_rows;
  out.inter_rows = ring_rows ? ring_rows : (long long)m + pp.halo_rows;

  out.items.clear();
  out.phase_begin[0] = out.phase_begin[1] = 0;
  auto emit_cons = [&](int c) {
    Item it{};
    it.kind = c_tiled ? ITEM_CONSUME_TILED : ITEM_CONSUME;
    it.block = c;
    it.row_begin = c_tiled ? c : out.cons_units[c].r0;
    it.row_end = c_tiled ? c + 1 : out.cons_units[c].r1;
    it.need = need[c];
    it.base = (ring_rows && cmin[c] != INT_MAX) ? (int)((cmin[c] / ring_rows) * ring_rows) : 0;
    if (!c_tiled && out.cons_units[c].seg) {
      it.kind = ITEM_CONSUME_SEG; it.row_end = out.cons_units[c].p0; it.base = out.cons_units[c].p1;
    }
    it.aux1 = cout_min[c];  // lowest output row this unit writes
    out.items.push_back(it);
  };
  for (const Entry &e : order) {
    if (e.is_cons) { emit_cons(e.idx); continue; }
    const int j = e.idx;
    Item it{};
    it.kind = p_tiled ? ITEM_PRODUCE_TILED : ITEM_PRODUCE;
    it.block = j;
    it.row_begin = p_tiled ? j : out.prod_units[j].r0;
    it.row_end = p_tiled ? j + 1 : out.prod_units[j].r1;
    it.base = ring_rows ? (int)((pmin[j] / ring_rows) * ring_rows) : 0;
    if (!p_tiled && out.prod_units[j].seg) {
      it.kind = ITEM_PRODUCE_SEG; it.row_end = out.prod_units[j].p0; it.base = out.prod_units[j].p1;
    }
    it.aux0 = psrc_max[j];  // highest row of the producer's dense input this unit reads
    if (ring_rows) {
      // consumers that still read the rows this unit overwrites: those with sufmin <= pmax - ring
      const long long x = (long long)pmax[j] - ring_rows;
      int lo = 0, hi = nc;
      while (lo < hi) { const int mid = (lo + hi) / 2; if (sufmin[mid] <= x) lo = mid + 1; else hi = mid; }
      it.need = x < 0 ? 0 : lo;
      if (it.need > e.cons_before) return fail(TF_ERR_UNSUPPORTED, "planner: ring dependence cycle (internal sizing error)");
    }
    out.items.push_back(it);
  }
  out.phase_begin[2] = (int)out.items.size();
  for (int c : late) emit_cons(c);
  out.phase_begin[3] = (int)out.items.size();
  return TF_OK;
}

int build_single_pass_plan(const PlanParams &pp, const int *ap, HostPlan &out) {
  out.prod_units.clear();
  out.seg_t_rows.clear();
  out.seg_out_rows.clear();
  out.cons_units = split_rows(pp.m, ap, pp.rows_per_block, pp.max_block_nnz);
  const int nc = (int)out.cons_units.size();
  out.n_prod = 0;
  out.n_cons = nc;
  out.items.clear();
  for (int c = 0; c < nc; ++c) {
    Item it{};
    it.kind = ITEM_SDDMM; it.block = c;
    const Unit &u = out.cons_units[c];
    it.row_begin = u.r0; it.row_end = u.r1;
    if (u.seg) {
      it.kind = ITEM_SDDMM_SEG; it.row_end = u.p0; it.base = u.p1;
      if (out.seg_out_rows.empty() || out.seg_out_rows.back() != u.r0) out.seg_out_rows.push_back(u.r0);
    }
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
  tf::Tiling pt, ct;
  const int cap = (!o || o->tile_slots == 0) ? (producer_is_gemm ? tf::kDefaultTileSlots : tf::kDefaultTileSlotsSmall) : o->tile_slots;
  const int tile_rows = 512;
  if (cap > 0 && n_cols % 4 == 0 && !(o && o->mode == TF_MODE_SCHEDULE)) {
    if (F) tf::build_tiling(F->m, F->ap, F->ai, cap, (o && o->tile_max_bz > 0) ? o->tile_max_bz : tf::kDefaultTileMaxBz, tile_rows, pt);
    tf::build_tiling(A->m, A->ap, A->ai, cap, (o && o->tile_max_bz > 0) ? o->tile_max_bz : tf::kDefaultTileMaxBz, tile_rows, ct);
  }
  int rc = tf::build_stream_plan(pp, F ? F->ap : nullptr, F ? F->ai : nullptr, A->ap, A->ai, &pt, &ct, hp);
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
  info[1] = hp.n_prod;
  info[2] = hp.n_cons;
  info[3] = hp.ring_rows;
  info[4] = hp.phase_begin[1]; info[5] = hp.phase_begin[2]; info[6] = hp.phase_begin[3];
  info[7] = hp.inter_rows;
  return TF_OK;
}

extern "C" void tf_free(void *p) { free(p); }

// Host-only view of the gather tiles the library would build for an operator.
extern "C" int tf_tiling_preview(const tf_csr *A, int tile_slots, int tile_max_bz, int **row_ptr, int **rows,
                                 int **halo_ptr, int **halo, int *n_tiles, int info[4]) {
  if (!A || !row_ptr || !rows || !halo_ptr || !halo || !n_tiles || !info)
    return tf::fail(TF_ERR_ARG, "tf_tiling_preview: null argument");
  tf::Tiling t;
  const int cap = tile_slots == 0 ? tf::kDefaultTileSlotsSmall : tile_slots;
  if (cap > 0) tf::build_tiling(A->m, A->ap, A->ai, cap, tile_max_bz > 0 ? tile_max_bz : tf::kDefaultTileMaxBz, 512, t);
  *n_tiles = t.tiled ? t.tiles() : 0;
  info[0] = t.bx; info[1] = t.by; info[2] = t.bz; info[3] = (int)(t.reuse * 1000);
  auto dup = [](const std::vector<int> &v) {
    int *b = (int *)malloc(sizeof(int) * std::max<size_t>(v.size(), 1));
    if (b && !v.empty()) std::copy(v.begin(), v.end(), b);
    return b;
  };
  *row_ptr = dup(t.tile_row_ptr); *rows = dup(t.rows); *halo_ptr = dup(t.tile_halo_ptr); *halo = dup(t.halo);
  return TF_OK;
}
