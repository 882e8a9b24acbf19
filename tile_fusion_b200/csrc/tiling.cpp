// Gather tiles: groups of output rows whose source rows (the dense rows their nonzeros name) are
// staged once in shared memory and reused by every row of the group.
//
// The reference fuses a second-operation row into a tile only if all of its columns lie inside the
// tile's own contiguous row range (Fusion_Inspector.h:576,713,886), which leaves nothing fused on a
// naturally ordered 3-D grid.  Here a tile may be any set of rows.  When the pattern is a lattice --
// the dominant column offsets are 1, nx and nx*ny, as in grid Laplacians in natural order -- tiles
// are bx x by x bz bricks, so a staged row is reused by up to seven output rows; otherwise tiles are runs of
// consecutive rows grown against the slot budget, kept when a staged row is reused at least twice.
#include <algorithm>
#include <cstdint>
#include <unordered_map>

#include "tf_internal.h"

namespace tf {

Lattice detect_lattice(int m, const int *ap, const int *ai) {
  Lattice L;
  std::unordered_map<int, int> hist;
  // every 3rd row is enough to see the dominant offsets
  int sampled = 0;
  for (int r = 0; r < m; r += 3) {
    ++sampled;
    for (int j = ap[r]; j < ap[r + 1]; ++j) ++hist[ai[j] - r];
    if (hist.size() > 4096) return L;  // unstructured
  }
  // frequent offsets; the middle one is the operator's own diagonal (0 for a square operator, a
  // constant shift when the columns were renumbered, as for one rank's rows of a partitioned chain)
  std::vector<int> freq;
  for (auto &kv : hist)
    if (kv.second * 2 >= sampled) freq.push_back(kv.first);
  std::sort(freq.begin(), freq.end());
  if (freq.empty() || freq.size() % 2 == 0) return L;
  const int d0 = freq[freq.size() / 2];
  L.shift = d0;
  std::vector<int> pos;
  for (int f : freq)
    if (f > d0) pos.push_back(f - d0);
  if (pos.empty() || pos[0] != 1 || pos.size() > 3) return L;
  L.dims = (int)pos.size();
  if (L.dims >= 2) L.nx = pos[1];
  if (L.dims == 3) {
    if (pos[2] % pos[1] != 0) { L.dims = 2; }
    else L.ny = pos[2] / pos[1];
  }
  if (L.dims == 1) L.nx = m;
  return L;
}

namespace {

// Tiles for any pattern: consecutive rows are added to the open tile until the set of distinct columns they name
// would pass the slot budget (or the row cap).  The reference's second-wave packer grows its tiles the same way
// against a cache budget (Fusion_Inspector.h:762-786).  Banded patterns -- FEM matrices, graphs after a
// bandwidth-reducing ordering -- reuse a staged row several times; where they do not (reuse below 2 nonzeros
// per staged row) tiling is declined and the executor gathers straight from global memory.
void build_generic_tiling(int m, const int *ap, const int *ai, int slot_cap, int max_rows, Tiling &out) {
  out = Tiling();
  int max_col = m - 1;
  for (int j = 0; j < ap[m]; ++j) max_col = std::max(max_col, ai[j]);
  std::vector<int> stamp((size_t)max_col + 1, -1), where((size_t)max_col + 1, 0);
  out.tile_row_ptr.assign(1, 0);
  out.tile_halo_ptr.assign(1, 0);
  out.slot.assign((size_t)ap[m], 0);
  out.rows.reserve(m);
  const int row_cap = std::min(max_rows, kTileMaxRows);
  long long staged = 0;
  int tile_id = 0, r = 0;
  while (r < m) {
    const size_t h0 = out.halo.size();
    const int r_begin = r;
    while (r < m && r - r_begin < row_cap) {
      const size_t before = out.halo.size();
      for (int j = ap[r]; j < ap[r + 1]; ++j) {
        const int c = ai[j];
        if (stamp[c] != tile_id) { stamp[c] = tile_id; out.halo.push_back(c); }
      }
      if ((int)(out.halo.size() - h0) > slot_cap) {
        if (r == r_begin) { out = Tiling(); return; }  // a single row names more columns than a tile can stage
        for (size_t q = before; q < out.halo.size(); ++q) stamp[out.halo[q]] = -1;
        out.halo.resize(before);
        break;
      }
      ++r;
    }
    std::sort(out.halo.begin() + h0, out.halo.end());
    for (size_t q = h0; q < out.halo.size(); ++q) where[out.halo[q]] = (int)(q - h0);
    for (int i = r_begin; i < r; ++i) {
      out.rows.push_back(i);
      for (int j = ap[i]; j < ap[i + 1]; ++j) out.slot[j] = (uint16_t)where[ai[j]];
    }
    staged += (long long)(out.halo.size() - h0);
    out.tile_row_ptr.push_back((int)out.rows.size());
    out.tile_halo_ptr.push_back((int)out.halo.size());
    ++tile_id;
  }
  out.reuse = staged > 0 ? (double)ap[m] / (double)staged : 0.0;
  out.tiled = out.reuse >= 2.0;
  if (!out.tiled) out = Tiling();
}

}  // namespace

int build_tiling(int m, const int *ap, const int *ai, int slot_cap, int max_bz, int max_rows, Tiling &out) {
  out = Tiling();
  if (slot_cap < 64 || slot_cap > 65535) return TF_OK;
  const Lattice L = detect_lattice(m, ap, ai);
  if (L.dims == 0) { build_generic_tiling(m, ap, ai, slot_cap, max_rows, out); return TF_OK; }
  const int nx = L.nx;
  const int ny = L.dims >= 3 ? L.ny : (L.dims == 2 ? (m + nx - 1) / nx : 1);
  const int nz = L.dims >= 3 ? (int)(((long long)m + (long long)nx * ny - 1) / ((long long)nx * ny)) : 1;
  // brick search: fewest staged rows per output row within the slot budget
  static const int cand[] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 128};
  int bx = 0, by = 1, bz = 1;
  double best = 1e30;
  // enough tiles to keep every SM busy several times over
  const long long max_vol = std::min<long long>(std::min(max_rows, kTileMaxRows), std::max<long long>(64, (long long)m / 1200));
  for (int cx : cand) {
    if (cx < 4 || cx > nx) continue;
    for (int cy : cand) {
      if (cy > ny || (L.dims < 2 && cy > 1)) continue;
      for (int cz : cand) {
        if (cz > nz || cz > max_bz || (L.dims < 3 && cz > 1)) continue;
        const long long vol = (long long)cx * cy * cz;
        long long h = vol + 2LL * cy * cz;
        if (L.dims >= 2) h += 2LL * cx * cz;
        if (L.dims >= 3) h += 2LL * cx * cy;
        if (h > slot_cap || vol < 64 || vol > max_vol) continue;
        // ties go to the larger brick, then to the longer x extent (contiguous rows)
        const double ratio = (double)h / (double)vol - 1e-9 * (double)vol - 1e-12 * cx;
        if (ratio < best) { best = ratio; bx = cx; by = cy; bz = cz; }
      }
    }
  }
  if (bx == 0) { build_generic_tiling(m, ap, ai, slot_cap, max_rows, out); return TF_OK; }

  out.nx = nx; out.ny = ny; out.bx = bx; out.by = by; out.bz = bz;
  out.tile_row_ptr.assign(1, 0);
  out.tile_halo_ptr.assign(1, 0);
  out.slot.assign((size_t)ap[m], 0);
  out.rows.reserve(m);
  std::vector<int> stamp((size_t)std::max(m, 1), -1), where((size_t)std::max(m, 1), 0);
  // source rows may exceed m (halo columns of a partitioned operator): size the marks to the widest column
  int max_col = m - 1;
  for (int j = 0; j < ap[m]; ++j) max_col = std::max(max_col, ai[j]);
  stamp.assign((size_t)max_col + 1, -1);
  where.assign((size_t)max_col + 1, 0);

  std::vector<int> trows;
  int tile_id = 0;
  long long staged = 0;
  // emits one tile; splits it when irregular rows push it over the slot budget
  auto emit = [&](auto &&self, const int *rs, int n) -> void {
    if (n == 0) return;
    const size_t h0 = out.halo.size();
    for (int i = 0; i < n; ++i)
      for (int j = ap[rs[i]]; j < ap[rs[i] + 1]; ++j) {
        const int c = ai[j];
        if (stamp[c] != tile_id) { stamp[c] = tile_id; where[c] = (int)(out.halo.size() - h0); out.halo.push_back(c); }
      }
    if ((int)(out.halo.size() - h0) > slot_cap && n > 1) {
      out.halo.resize(h0);
      ++tile_id;  // invalidate the marks of the aborted attempt
      self(self, rs, n / 2);
      self(self, rs + n / 2, n - n / 2);
      return;
    }
    if ((int)(out.halo.size() - h0) > slot_cap) { out.tiled = false; out.failed = true; return; }
    // slots in source-row order: consecutive rows of a band then read consecutive slots
    std::sort(out.halo.begin() + h0, out.halo.end());
    for (size_t q = h0; q < out.halo.size(); ++q) where[out.halo[q]] = (int)(q - h0);
    for (int i = 0; i < n; ++i) {
      out.rows.push_back(rs[i]);
      for (int j = ap[rs[i]]; j < ap[rs[i] + 1]; ++j) out.slot[j] = (uint16_t)where[ai[j]];
    }
    staged += (long long)(out.halo.size() - h0);
    out.tile_row_ptr.push_back((int)out.rows.size());
    out.tile_halo_ptr.push_back((int)out.halo.size());
    ++tile_id;
  };
  for (int z0 = 0; z0 < nz && !out.failed; z0 += bz)
    for (int y0 = 0; y0 < ny && !out.failed; y0 += by)
      for (int x0 = 0; x0 < nx && !out.failed; x0 += bx) {
        trows.clear();
        for (int z = z0; z < std::min(nz, z0 + bz); ++z)
          for (int y = y0; y < std::min(ny, y0 + by); ++y) {
            const long long b = ((long long)z * ny + y) * nx;
            for (int x = x0; x < std::min(nx, x0 + bx); ++x)
              if (b + x < m) trows.push_back((int)(b + x));
          }
        emit(emit, trows.data(), (int)trows.size());
      }
  if (out.failed || (int)out.rows.size() != m) { build_generic_tiling(m, ap, ai, slot_cap, max_rows, out); return TF_OK; }
  out.reuse = staged > 0 ? (double)ap[m] / (double)staged : 0.0;
  out.tiled = out.reuse >= 2.0;  // below that, staging costs more than it saves
  if (!out.tiled) build_generic_tiling(m, ap, ai, slot_cap, max_rows, out);
  return TF_OK;
}

}  // namespace tf
