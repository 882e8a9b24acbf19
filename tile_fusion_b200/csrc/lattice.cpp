// Lattice operators: recognising a CSR operator as a star stencil on a grid in natural order.
//
// The reference fuses a row of the second product into a tile when all of its columns fall inside the
// tile (Fusion_Inspector.h:713).  On a grid Laplacian in natural order the columns of a row are the row's
// own grid neighbours, so "columns inside the tile" is a statement about geometry: a tile that is an
// x-y rectangle marched along z holds, at any moment, every intermediate row its output rows name.  This
// file checks that an operator really has that structure -- every nonzero of row (x, y, z) names one of
// (x, y, z), (x+-1, y, z), (x, y+-1, z), (x, y, z+-1), never across a grid edge -- and rewrites it as
// per-row coefficient vectors in CSR (sorted-column) order, so that the executor adds the same products in
// the same order as the reference's row loop (SpMM_SpMM.cpp:211-248).  Rows are grouped into classes of
// equal coefficient vectors; the executor keeps the few distinct vectors on chip and reads one class byte
// per row.  Anything that does not fit (other offsets, too many classes, rows that are not whole planes)
// is declined and runs on the general CSR path.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

#include "tf_internal.h"

namespace tf {

namespace {

struct VecKey {
  uint32_t w[7];
  bool operator==(const VecKey &o) const { return std::memcmp(w, o.w, sizeof(w)) == 0; }
};
struct VecHash {
  size_t operator()(const VecKey &k) const {
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 7; ++i) { h ^= k.w[i]; h *= 0xBF58476D1CE4E5B9ull; h ^= h >> 29; }
    return (size_t)h;
  }
};

}  // namespace

int analyse_lattice_operator(int m, int ncols, const int *ap, const int *ai, const float *ax, int halo_rows,
                             LatticeOp &out) {
  out = LatticeOp();
  const Lattice L = detect_lattice(m, ap, ai);
  if (L.dims != 3 || L.nx < 2 || L.ny < 2 || L.nx % 2 != 0) return TF_OK;  // (the executor reads x in pairs)
  const long long plane = (long long)L.nx * L.ny;
  if (plane <= L.nx || m % plane != 0) return TF_OK;
  const int nx = L.nx, ny = L.ny, nz = (int)(m / plane);
  if (nz < 2) return TF_OK;
  const int local_cols = ncols - halo_rows;  // columns addressed as shifted lattice neighbours
  int ghost_lo = 0, ghost_hi = 0;
  bool halo_lo = false, halo_hi = false;
  if (halo_rows == 0) {
    if (L.shift < 0 || L.shift % plane != 0) return TF_OK;
    ghost_lo = (int)(L.shift / plane);
    const long long above = (long long)local_cols - L.shift - m;
    if (above < 0 || above % plane != 0) return TF_OK;
    ghost_hi = (int)(above / plane);
  } else {
    if (L.shift != 0 || local_cols != m) return TF_OK;
    // appended halo planes: the lower neighbour's plane first, then the upper neighbour's
    for (int r = 0; r < plane && !halo_lo; ++r)
      for (int j = ap[r]; j < ap[r + 1]; ++j)
        if (ai[j] >= m) { halo_lo = true; break; }
    for (long long r = m - plane; r < m && !halo_hi; ++r)
      for (int j = ap[r]; j < ap[r + 1]; ++j)
        if (ai[j] >= m) { halo_hi = true; break; }
    if ((long long)halo_rows != ((int)halo_lo + (int)halo_hi) * plane) return TF_OK;
    ghost_lo = halo_lo; ghost_hi = halo_hi;
  }

  std::unordered_map<VecKey, int, VecHash> ids;
  std::vector<VecKey> vecs;
  std::vector<long long> count;
  std::vector<uint8_t> cls((size_t)m);
  for (int z = 0, r = 0; z < nz; ++z)
    for (int y = 0; y < ny; ++y)
      for (int x = 0; x < nx; ++x, ++r) {
        VecKey k;
        std::memset(&k, 0, sizeof(k));
        unsigned seen = 0;
        for (int j = ap[r]; j < ap[r + 1]; ++j) {
          const int c = ai[j];
          int slot = -1;
          if (c >= local_cols) {  // appended halo row of the intermediate
            const long long h = c - local_cols;
            if (z == 0 && halo_lo && h == (long long)y * nx + x) slot = 0;
            else if (z == nz - 1 && halo_hi && h == (halo_lo ? plane : 0) + (long long)y * nx + x) slot = 6;
          } else {
            const long long d = (long long)c - L.shift - r;
            if (d == 0) slot = 3;
            else if (d == -1 && x > 0) slot = 2;
            else if (d == 1 && x < nx - 1) slot = 4;
            else if (d == -nx && y > 0) slot = 1;
            else if (d == nx && y < ny - 1) slot = 5;
            else if (d == -plane && (z > 0 || (halo_rows == 0 && ghost_lo > 0))) slot = 0;
            else if (d == plane && (z < nz - 1 || (halo_rows == 0 && ghost_hi > 0))) slot = 6;
          }
          if (slot < 0 || (seen >> slot & 1u)) return TF_OK;  // not a grid neighbour, or named twice
          seen |= 1u << slot;
          std::memcpy(&k.w[slot], &ax[j], 4);
        }
        auto it = ids.find(k);
        int id;
        if (it == ids.end()) {
          if ((int)vecs.size() >= kMarchMaxClasses) return TF_OK;
          id = (int)vecs.size();
          ids.emplace(k, id);
          vecs.push_back(k);
          count.push_back(0);
        } else id = it->second;
        ++count[id];
        cls[r] = (uint8_t)id;
      }

  // class 0 = the most frequent vector (the interior rows): the executor keeps it in registers
  const int nc = (int)vecs.size();
  std::vector<int> order(nc), rank(nc);
  for (int i = 0; i < nc; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return count[a] > count[b]; });
  for (int i = 0; i < nc; ++i) rank[order[i]] = i;
  out.dict.assign((size_t)(nc + 1) * 8, 0.f);
  for (int i = 0; i < nc; ++i) std::memcpy(&out.dict[(size_t)rank[i] * 8], vecs[i].w, 28);
  const int pnx = (nx + 1) / 2, pny = (ny + 1) / 2;
  out.patch_cls.assign((size_t)nz * pny * pnx, 0x01010101u * (uint32_t)nc);
  for (int z = 0, r = 0; z < nz; ++z)
    for (int y = 0; y < ny; ++y)
      for (int x = 0; x < nx; ++x, ++r) {
        uint32_t &w = out.patch_cls[((size_t)z * pny + (y >> 1)) * pnx + (x >> 1)];
        const int sh = 8 * (2 * (y & 1) + (x & 1));
        w = (w & ~(0xFFu << sh)) | ((uint32_t)rank[cls[r]] << sh);
      }
  out.nx = nx; out.ny = ny; out.nz = nz;
  out.ghost_lo = ghost_lo; out.ghost_hi = ghost_hi;
  out.n_classes = nc;
  out.ok = true;
  return TF_OK;
}

void build_march_items(int nx, int ny, int z_begin, int z_end, int n_cols, int tile_w, int tile_h, int chunk,
                       int ctas, int min_segments, std::vector<MarchItem> &out) {
  const int nzl = z_end - z_begin;
  if (nzl <= 0) return;
  ctas = std::max(1, ctas);
  min_segments = std::max(1, min_segments);
  const int tx = (nx + tile_w - 1) / tile_w, ty = (ny + tile_h - 1) / tile_h, nch = (n_cols + chunk - 1) / chunk;
  const long long columns = (long long)tx * ty * nch;
  // A piece of L planes costs L + 4 steps (two planes of lead-in for each of the two products), so whole columns
  // are the cheapest items; but the CTAs take items in rounds, and a last round that only a few CTAs work in
  // costs a whole column's time.  So: `full` rounds of whole columns (one column per CTA and round), then the
  // remaining columns cut into pieces whose number is a multiple of the CTA count.  (full, q) is chosen by the
  // step count of the slowest CTA, full * (nzl + 4) + q * (longest piece + 4).
  long long best_t = -1, best_full = 0, best_pieces = 0;
  const long long max_full = min_segments > 1 ? 0 : columns / ctas;
  for (long long full = max_full; full >= 0; --full) {
    const long long rest = columns - full * ctas;
    if (rest == 0) {
      const long long t = full * (nzl + 4);
      if (best_t < 0 || t < best_t) { best_t = t; best_full = full; best_pieces = 0; }
      continue;
    }
    for (long long q = 1; q <= 64; ++q) {
      const long long pieces = std::max(q * ctas, rest * min_segments);
      const long long per_col = std::min<long long>(pieces / rest, nzl);   // pieces of the least-cut column
      if (per_col < min_segments) continue;
      const long long longest = (nzl + per_col - 1) / per_col;
      if (per_col > 1 && longest < 8 && q > 1) break;
      const long long rounds = (std::min(pieces, rest * (long long)nzl) + ctas - 1) / ctas;
      const long long t = full * (nzl + 4) + rounds * (longest + 4);
      if (best_t < 0 || t < best_t) { best_t = t; best_full = full; best_pieces = pieces; }
    }
  }
  // whole columns first, in (tile, chunk) order: the chunks of a tile run side by side and share DRAM pages
  long long col = 0;
  auto item_of = [&](long long c, int zs, int ze) {
    const int ch = (int)(c % nch);
    const long long t = c / nch;
    out.push_back(MarchItem{(int)(t % tx) * tile_w, (int)(t / tx) * tile_h, zs, ze, ch * chunk, 0});
  };
  for (; col < best_full * ctas; ++col) item_of(col, z_begin, z_end);
  const long long rest = columns - col;
  if (rest <= 0) return;
  // the remainder: column r of it gets base or base + 1 pieces; pieces of one cut level are emitted together
  // (level by level), longest pieces first
  const long long base = std::max<long long>(1, std::min<long long>(best_pieces / rest, nzl));
  const long long extra = base < nzl ? std::max<long long>(0, std::min(best_pieces - base * rest, rest)) : 0;
  const long long levels = base + (extra > 0 ? 1 : 0);
  for (long long lv = 0; lv < levels; ++lv)
    for (long long r = 0; r < rest; ++r) {
      // the columns with one more piece are the last `extra` ones
      const long long n = base + (r >= rest - extra ? 1 : 0);
      if (lv >= n) continue;
      const int zs = z_begin + (int)((long long)nzl * lv / n), ze = z_begin + (int)((long long)nzl * (lv + 1) / n);
      if (ze > zs) item_of(col + r, zs, ze);
    }
}

}  // namespace tf

extern "C" int tf_lattice_preview(const tf_csr *A, int halo_rows, int n_cols, int ctas, int info[8], float **dict,
                                  unsigned **patch_cls, int **items, int *n_items) {
  if (!A || !info || !dict || !patch_cls || !items || !n_items)
    return tf::fail(TF_ERR_ARG, "tf_lattice_preview: null argument");
  int rc = tf::check_csr(A->m, A->n, A->ap, A->ai, false);
  if (rc != TF_OK) return rc;
  tf::LatticeOp op;
  rc = tf::analyse_lattice_operator(A->m, A->n, A->ap, A->ai, A->ax, halo_rows, op);
  if (rc != TF_OK) return rc;
  info[0] = op.ok; info[1] = op.nx; info[2] = op.ny; info[3] = op.nz;
  info[4] = op.ghost_lo; info[5] = op.ghost_hi; info[6] = op.n_classes; info[7] = 0;
  *dict = nullptr; *patch_cls = nullptr; *items = nullptr; *n_items = 0;
  if (!op.ok) return TF_OK;
  *dict = (float *)malloc(sizeof(float) * op.dict.size());
  *patch_cls = (unsigned *)malloc(sizeof(unsigned) * op.patch_cls.size());
  if (!*dict || !*patch_cls) return tf::fail(TF_ERR_NOMEM, "tf_lattice_preview: out of memory");
  std::copy(op.dict.begin(), op.dict.end(), *dict);
  std::copy(op.patch_cls.begin(), op.patch_cls.end(), *patch_cls);
  std::vector<tf::MarchItem> it;
  tf::build_march_items(op.nx, op.ny, 0, op.nz, n_cols, 16, 8, 16, ctas > 0 ? ctas : 296, 1, it);
  *n_items = (int)it.size();
  *items = (int *)malloc(sizeof(int) * 6 * std::max<size_t>(it.size(), 1));
  if (!*items) return tf::fail(TF_ERR_NOMEM, "tf_lattice_preview: out of memory");
  for (size_t i = 0; i < it.size(); ++i) {
    int *q = *items + 6 * i;
    q[0] = it[i].x0; q[1] = it[i].y0; q[2] = it[i].zs; q[3] = it[i].ze; q[4] = it[i].c0; q[5] = it[i].flags;
  }
  return TF_OK;
}
