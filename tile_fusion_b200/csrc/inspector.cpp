// Host inspector: reproduces, bit for bit, the schedules of the reference's
// tile-fusion inspectors (paths inside the reference project):
//   fixed tiles      SparseFusionInspector::generateFusedScheduleForAllFused
//                    fusion/include/sparse-fusion/Fusion_Inspector.h:32-55 (+ SparseFusion.cpp:30-142,
//                    Fusion_Utils.cpp:316-388,510-548, MultiDimensionalSet.cpp:124-185)
//   variable tiles   InspectorForTileFusedCSRVariableTileSize, Fusion_Inspector.h:542, :676, :851
// The algorithms are re-implemented on flat arrays (an explicit split stack and
// epoch-stamped column marks instead of a linked list and std::set rebuilds), so a
// 2M-row matrix is inspected in well under a second; the arrays that come out are
// the same.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>

#include "tf_internal.h"

namespace tf {

static thread_local std::string g_err;
void set_error(const std::string &msg) { g_err = msg; }
int fail(int code, const std::string &msg) { g_err = msg; return code; }
const char *last_error_cstr() { return g_err.c_str(); }

int check_csr(int m, int ncols, const int *ap, const int *ai, bool need_sorted) {
  if (m < 0 || !ap) return fail(TF_ERR_ARG, "CSR: null row pointer or negative size");
  if (ap[0] != 0) return fail(TF_ERR_ARG, "CSR: Ap[0] must be 0");
  for (int i = 0; i < m; ++i) {
    if (ap[i + 1] < ap[i]) return fail(TF_ERR_ARG, "CSR: row pointers must be non-decreasing");
    for (int j = ap[i]; j < ap[i + 1]; ++j) {
      if (!ai) return fail(TF_ERR_ARG, "CSR: null column index array");
      if (ai[j] < 0 || ai[j] >= ncols) return fail(TF_ERR_ARG, "CSR: column index out of range");
      if (need_sorted && j > ap[i] && ai[j] <= ai[j - 1])
        return fail(TF_ERR_ARG, "CSR: columns must be sorted and unique within a row");
    }
  }
  return TF_OK;
}

namespace {

// 32-bit wrapping arithmetic: the reference's cost models are plain `int` expressions.
inline int32_t w32(int64_t x) { return (int32_t)(uint32_t)(uint64_t)x; }
inline int ws_spmm(int nnz, int uniq, int bcol, int tile, int fused, int ds) {
  int32_t s = w32((int64_t)nnz + w32((int64_t)uniq * bcol));
  s = w32((int64_t)s + w32((int64_t)tile * bcol));
  s = w32((int64_t)s + w32((int64_t)fused * bcol));
  s = w32((int64_t)s * ds);
  return w32((int64_t)s + w32((int64_t)nnz * 4));
}
inline int ws_gemm(int fnnz, int bcol, int ccol, int tile, int fused, int ds) {
  int32_t s = w32((int64_t)w32((int64_t)tile * ccol) + w32((int64_t)ccol * bcol));
  s = w32((int64_t)s + w32((int64_t)tile * bcol));
  s = w32((int64_t)s + w32((int64_t)fused * ccol));
  s = w32((int64_t)s + fnnz);
  s = w32((int64_t)s * ds);
  return w32((int64_t)s + w32((int64_t)fnnz * 4));
}

// Consecutive partition with unit weights: even = ceil(n/parts); trailing parts may be empty.
std::vector<int> split_even(int n, int parts) {
  std::vector<int> idx(parts + 1, 0);
  const double even = std::ceil((double)n / parts);
  int j = 0;
  for (int i = 0; i < parts; ++i) {
    double w = 0;
    while (w < even && j < n) { w += 1.0; ++j; }
    idx[i + 1] = j;
  }
  return idx;
}

void finish_stats(tf_schedule &s, const int *ap) {
  long long fused = 0, fnnz = 0;
  if (s.n1 > 0)
    for (int k = s.ptr2[s.ptr1[0]]; k < s.ptr2[s.ptr1[1]]; ++k)
      if (s.type[k] == 1) { ++fused; fnnz += ap[s.id[k] + 1] - ap[s.id[k]]; }
  s.stats[0] = (double)fused;
  s.stats[1] = (double)(int)fnnz;
  s.stats[4] = (double)s.ptr1[s.n1];
}

int inspect_fixed(int m, const int *ap, const int *ai, const tf_sched_params &p, tf_schedule &s) {
  if (p.iter_per_partition <= 0 || p.num_threads <= 0)
    return fail(TF_ERR_ARG, "fixed-tile inspector: iter_per_partition and num_threads must be positive");
  const int P = std::max(m / p.iter_per_partition, 2 * p.num_threads);
  const std::vector<int> part = split_even(m, P);
  std::vector<char> fused(m, 0);
  for (int q = 0; q < P; ++q) {
    const int lo = part[q], hi = part[q + 1];
    for (int r = lo; r < hi; ++r) {
      bool ok = true;
      for (int j = ap[r]; j < ap[r + 1] && ok; ++j) ok = ai[j] >= lo && ai[j] < hi;
      fused[r] = ok;
    }
  }
  std::vector<int> rest;
  for (int r = 0; r < m; ++r)
    if (!fused[r]) rest.push_back(r);
  const bool wave2 = !rest.empty();
  s.n1 = wave2 ? 2 : 1;
  s.has_ker = true;
  s.ptr1.assign(s.n1 + 1, 0);
  s.ptr2.assign(1, 0);
  s.id.reserve((size_t)2 * m);
  s.type.reserve((size_t)2 * m);
  for (int q = 0; q < P; ++q) {
    for (int r = part[q]; r < part[q + 1]; ++r) { s.id.push_back(r); s.type.push_back(0); }
    s.ker.push_back((int)s.id.size());
    for (int r = part[q]; r < part[q + 1]; ++r)
      if (fused[r]) { s.id.push_back(r); s.type.push_back(1); }
    s.ker.push_back((int)s.id.size());
    s.ptr2.push_back((int)s.id.size());
  }
  s.ptr1[1] = P;
  if (wave2) {
    const std::vector<int> rp = split_even((int)rest.size(), P);
    for (int q = 0; q < P; ++q) {
      s.ker.push_back((int)s.id.size());
      for (int k = rp[q]; k < rp[q + 1]; ++k) { s.id.push_back(rest[k]); s.type.push_back(1); }
      s.ker.push_back((int)s.id.size());
      s.ptr2.push_back((int)s.id.size());
    }
    s.ptr1[2] = 2 * P;
  }
  finish_stats(s, ap);
  return TF_OK;
}

struct Tile {
  int start, end;
  std::vector<int> fused;
};

int inspect_variable(int m, const int *ap, const int *ai, const tf_sched_params &p, tf_schedule &s) {
  const int kind = p.kind, ds = p.data_size, bcol = p.b_cols, ccol = p.c_cols, cache = p.tile_m;
  if (p.num_threads <= 0 || ds <= 0 || bcol <= 0 || (kind == TF_INSPECT_VT_GEMM && ccol <= 0))
    return fail(TF_ERR_ARG, "variable-tile inspector: threads, data_size and dense widths must be positive");
  for (int i = 0; i < m; ++i)
    if (ap[i + 1] == ap[i]) return fail(TF_ERR_ARG, "variable-tile inspector: empty row (the reference reads Ai[Ap[i]])");
  int min_max = 0, init;
  if (kind == TF_INSPECT_VT_SPMM) { min_max = m / (2 * p.num_threads); init = std::min(4096, min_max); }
  else if (kind == TF_INSPECT_VT_GEMM) init = std::min((cache / ds - bcol * ccol) / (bcol + ccol), m);
  else init = std::min(4096, m);
  if (init <= 0)
    return fail(TF_ERR_ARG, "variable-tile inspector: initial tile size is not positive "
                            "(too few rows per thread, or a cache budget below the dense operand)");
  const int extra = m % init, ntiles0 = m / init;
  const int per = (int)std::ceil(extra / (double)ntiles0);
  std::vector<Tile> initial(ntiles0);
  for (int i = 0, removed = 0; i < ntiles0; ++i) {
    int st = init * i + removed, en = st + init;
    if (extra > removed) { int ext = std::min(extra - removed, per); en += ext; removed += ext; }
    initial[i].start = st; initial[i].end = en;
  }
  std::vector<int> rest;
  auto inside = [&](int r, int lo, int hi) { return ai[ap[r]] >= lo && ai[ap[r + 1] - 1] < hi; };
  if (kind == TF_INSPECT_VT_SPMM_THREADS) {
    // every row is offered to every tile in order; the first tile containing its columns takes it
    for (int r = 0; r < m; ++r) {
      const int lo = ai[ap[r]], hi = ai[ap[r + 1] - 1];
      // tiles are consecutive and sorted: the tile holding `lo` is the only candidate
      auto it = std::upper_bound(initial.begin(), initial.end(), lo,
                                 [](int v, const Tile &t) { return v < t.end; });
      if (it != initial.end() && lo >= it->start && hi < it->end) it->fused.push_back(r);
      else rest.push_back(r);
    }
  } else {
    for (auto &t : initial)
      for (int r = t.start; r < t.end; ++r) (inside(r, t.start, t.end) ? t.fused : rest).push_back(r);
  }
  // shrink pass: depth-first, left half first, exactly the order of the reference's list walk
  std::vector<int> stamp(std::max(m, 1), 0);
  int epoch = 0;
  std::vector<Tile> done;
  done.reserve(initial.size());
  std::vector<Tile> stack;
  for (size_t ti = 0; ti < initial.size(); ++ti) {
    stack.clear();
    stack.push_back(std::move(initial[ti]));
    while (!stack.empty()) {
      Tile t = std::move(stack.back());
      stack.pop_back();
      const int ts = t.end - t.start;
      int ws;
      if (kind == TF_INSPECT_VT_GEMM) {
        int fnnz = 0;
        for (int r : t.fused) fnnz += ap[r + 1] - ap[r];
        ws = ws_gemm(fnnz, bcol, ccol, ts, (int)t.fused.size(), ds);
      } else {
        ++epoch;
        int uq = 0;
        for (int j = ap[t.start]; j < ap[t.end]; ++j)
          if (stamp[ai[j]] != epoch) { stamp[ai[j]] = epoch; ++uq; }
        ws = ws_spmm(ap[t.end] - ap[t.start], uq, bcol, ts, (int)t.fused.size(), ds);
      }
      if (ws > cache && ts > 1) {
        const int sep = ts / 2 + t.start;
        Tile a{t.start, sep, {}}, b{sep, t.end, {}};
        for (int r : t.fused) {
          if (ai[ap[r + 1] - 1] < sep) a.fused.push_back(r);
          else if (ai[ap[r]] >= sep) b.fused.push_back(r);
          else rest.push_back(r);
        }
        stack.push_back(std::move(b));
        stack.push_back(std::move(a));
      } else {
        done.push_back(std::move(t));
      }
    }
  }
  const int ntiles = (int)done.size();
  const int u = (int)rest.size();
  std::vector<int> ufptr;
  if (kind == TF_INSPECT_VT_SPMM_THREADS) {
    const int per_part = (int)std::ceil(u / float(p.num_threads));
    for (int q = 0; q <= p.num_threads; ++q) ufptr.push_back(std::min(q * per_part, u));
  } else {
    std::sort(rest.begin(), rest.end());
    int stride = 16, nnz = 0, uft = 0, size = 0, uq = 0;
    ++epoch;
    ufptr.push_back(0);
    while (uft < u) {
      if (stride == 0)
        return fail(TF_ERR_ARG, "variable-tile inspector: wave-2 stride reached 0 "
                                "(the reference does not terminate on this input; use fewer threads)");
      for (int ii = uft; ii < std::min(u, uft + stride); ++ii) {
        const int r = rest[ii];
        for (int j = ap[r]; j < ap[r + 1]; ++j)
          if (stamp[ai[j]] != epoch) { stamp[ai[j]] = epoch; ++uq; }
        nnz += ap[r + 1] - ap[r];
        ++size;
      }
      const int ws = ws_spmm(nnz, uq, bcol, size, 0, ds);
      const bool grow = kind == TF_INSPECT_VT_SPMM ? ((ws < cache || size == 1) && size + stride < min_max)
                                                   : (ws < cache || size <= 16);
      if (grow) uft += stride;
      else {
        ufptr.push_back(uft);
        nnz = 0; uq = 0; ++epoch;
        if (size <= stride) stride /= 2;
        if (size >= 3 * stride) stride *= 2;
        size = 0;
      }
    }
    ufptr.push_back(u);
  }
  const int nuf = (int)ufptr.size() - 1;
  s.n1 = 2;
  s.has_ker = kind != TF_INSPECT_VT_SPMM_THREADS;
  s.ptr1 = {0, ntiles, ntiles + nuf};
  s.ptr2.assign(1, 0);
  s.id.reserve((size_t)2 * m);
  s.type.reserve((size_t)2 * m);
  double acc = 0;
  for (const Tile &t : done) {
    for (int r = t.start; r < t.end; ++r) { s.id.push_back(r); s.type.push_back(0); }
    if (s.has_ker) s.ker.push_back((int)s.id.size());
    for (int r : t.fused) { s.id.push_back(r); s.type.push_back(1); }
    if (s.has_ker) s.ker.push_back((int)s.id.size());
    s.ptr2.push_back((int)s.id.size());
    acc += t.end - t.start;
  }
  {  // tile-size mean / std in float, as extractTilesSizeData does (Fusion_Inspector.h:1034-1050)
    const float average = (float)(acc / ntiles);
    float var = 0;
    for (const Tile &t : done) var += ((t.end - t.start) - average) * ((t.end - t.start) - average);
    var /= ntiles;
    s.stats[2] = average;
    s.stats[3] = (float)std::sqrt(var);
  }
  for (int q = 0; q < nuf; ++q) {
    if (s.has_ker) s.ker.push_back((int)s.id.size());
    for (int k = ufptr[q]; k < ufptr[q + 1]; ++k) { s.id.push_back(rest[k]); s.type.push_back(1); }
    if (s.has_ker) s.ker.push_back((int)s.id.size());
    s.ptr2.push_back((int)s.id.size());
  }
  finish_stats(s, ap);
  return TF_OK;
}

}  // namespace
}  // namespace tf

extern "C" {

const char *tf_last_error(void) { return tf::last_error_cstr(); }
const char *tf_version(void) { return "tile_fusion_b200 0.1 (sm_100a)"; }

int tf_inspect(int m, const int *Ap, const int *Ai, const tf_sched_params *p, tf_schedule **out) {
  if (!Ap || !Ai || !p || !out) return tf::fail(TF_ERR_ARG, "tf_inspect: null argument");
  if (m <= 0) return tf::fail(TF_ERR_ARG, "tf_inspect: matrix must have at least one row");
  const bool variable = p->kind != TF_INSPECT_FIXED;
  if (p->kind < TF_INSPECT_FIXED || p->kind > TF_INSPECT_VT_SPMM_THREADS)
    return tf::fail(TF_ERR_ARG, "tf_inspect: unknown inspector kind");
  // the variable-tile inspectors test only the first and last column of a row: sorted columns required
  int rc = tf::check_csr(m, m, Ap, Ai, variable);
  if (rc != TF_OK) return rc;
  tf_schedule *s = new tf_schedule();
  rc = variable ? tf::inspect_variable(m, Ap, Ai, *p, *s) : tf::inspect_fixed(m, Ap, Ai, *p, *s);
  if (rc != TF_OK) { delete s; return rc; }
  *out = s;
  return TF_OK;
}

int tf_schedule_dims(const tf_schedule *s, int *n1, int *n_parts, int *n_ids, int *has_ker) {
  if (!s) return tf::fail(TF_ERR_ARG, "tf_schedule_dims: null schedule");
  if (n1) *n1 = s->n1;
  if (n_parts) *n_parts = s->ptr1[s->n1];
  if (n_ids) *n_ids = (int)s->id.size();
  if (has_ker) *has_ker = s->has_ker;
  return TF_OK;
}

int tf_schedule_arrays(const tf_schedule *s, const int **ptr1, const int **ptr2, const int **id,
                       const int **type, const int **ker_begin) {
  if (!s) return tf::fail(TF_ERR_ARG, "tf_schedule_arrays: null schedule");
  if (ptr1) *ptr1 = s->ptr1.data();
  if (ptr2) *ptr2 = s->ptr2.data();
  if (id) *id = s->id.data();
  if (type) *type = s->type.data();
  if (ker_begin) *ker_begin = s->has_ker ? s->ker.data() : nullptr;
  return TF_OK;
}

int tf_schedule_stats(const tf_schedule *s, double stats[5]) {
  if (!s || !stats) return tf::fail(TF_ERR_ARG, "tf_schedule_stats: null argument");
  std::memcpy(stats, s->stats, sizeof(double) * 5);
  return TF_OK;
}

static int validate_schedule(const tf_schedule &s) {
  if (s.n1 < 1 || s.n1 > 2) return tf::fail(TF_ERR_ARG, "schedule: one or two levels expected");
  if ((int)s.ptr1.size() != s.n1 + 1 || s.ptr1[0] != 0) return tf::fail(TF_ERR_ARG, "schedule: bad ptr1");
  for (int l = 0; l < s.n1; ++l)
    if (s.ptr1[l + 1] < s.ptr1[l]) return tf::fail(TF_ERR_ARG, "schedule: ptr1 must be non-decreasing");
  const int np = s.ptr1[s.n1];
  if ((int)s.ptr2.size() != np + 1 || s.ptr2[0] != 0) return tf::fail(TF_ERR_ARG, "schedule: bad ptr2");
  for (int w = 0; w < np; ++w)
    if (s.ptr2[w + 1] < s.ptr2[w]) return tf::fail(TF_ERR_ARG, "schedule: ptr2 must be non-decreasing");
  if ((int)s.id.size() != s.ptr2[np] || s.type.size() != s.id.size())
    return tf::fail(TF_ERR_ARG, "schedule: id/type length must equal ptr2[n_parts]");
  if (s.has_ker) {
    if ((int)s.ker.size() != 2 * np) return tf::fail(TF_ERR_ARG, "schedule: ker_begin must hold 2 entries per partition");
    for (int w = 0; w < np; ++w)
      if (s.ker[2 * w] < s.ptr2[w] || s.ker[2 * w + 1] < s.ker[2 * w] || s.ker[2 * w + 1] != s.ptr2[w + 1])
        return tf::fail(TF_ERR_ARG, "schedule: ker_begin inconsistent with ptr2");
  }
  return TF_OK;
}

int tf_schedule_from_arrays(int n1, const int *ptr1, const int *ptr2, const int *id, const int *type,
                            const int *ker_begin, tf_schedule **out) {
  if (!ptr1 || !ptr2 || !out || n1 < 1 || n1 > 2) return tf::fail(TF_ERR_ARG, "tf_schedule_from_arrays: bad argument");
  tf_schedule *s = new tf_schedule();
  s->n1 = n1;
  s->ptr1.assign(ptr1, ptr1 + n1 + 1);
  const int np = ptr1[n1];
  if (np < 0) { delete s; return tf::fail(TF_ERR_ARG, "tf_schedule_from_arrays: negative partition count"); }
  s->ptr2.assign(ptr2, ptr2 + np + 1);
  const int ni = ptr2[np];
  if (ni < 0 || (ni > 0 && (!id || !type))) { delete s; return tf::fail(TF_ERR_ARG, "tf_schedule_from_arrays: bad id/type"); }
  s->id.assign(id, id + ni);
  s->type.assign(type, type + ni);
  s->has_ker = ker_begin != nullptr;
  if (ker_begin) s->ker.assign(ker_begin, ker_begin + 2 * (size_t)np);
  int rc = validate_schedule(*s);
  if (rc != TF_OK) { delete s; return rc; }
  s->stats[4] = np;
  long long fused = 0;
  for (int k = s->ptr2[s->ptr1[0]]; k < s->ptr2[s->ptr1[1]]; ++k) fused += s->type[k] == 1;
  s->stats[0] = (double)fused;
  *out = s;
  return TF_OK;
}

// image: magic, n1, n_parts, n_ids, has_ker, stats (5 doubles as 10 ints), ptr1, ptr2, id, type, ker
static const int kMagic = 0x54463031;  // "TF01"

int tf_schedule_serialized_size(const tf_schedule *s, size_t *n_ints) {
  if (!s || !n_ints) return tf::fail(TF_ERR_ARG, "tf_schedule_serialized_size: null argument");
  *n_ints = 5 + 10 + s->ptr1.size() + s->ptr2.size() + 2 * s->id.size() + s->ker.size();
  return TF_OK;
}

int tf_schedule_serialize(const tf_schedule *s, int *buf, size_t n_ints) {
  size_t need = 0;
  if (!s || !buf) return tf::fail(TF_ERR_ARG, "tf_schedule_serialize: null argument");
  tf_schedule_serialized_size(s, &need);
  if (n_ints < need) return tf::fail(TF_ERR_ARG, "tf_schedule_serialize: buffer too small");
  int *q = buf;
  *q++ = kMagic; *q++ = s->n1; *q++ = s->ptr1[s->n1]; *q++ = (int)s->id.size(); *q++ = s->has_ker;
  std::memcpy(q, s->stats, sizeof(double) * 5); q += 10;
  auto put = [&](const std::vector<int> &v) { if (!v.empty()) std::memcpy(q, v.data(), v.size() * sizeof(int)); q += v.size(); };
  put(s->ptr1); put(s->ptr2); put(s->id); put(s->type); put(s->ker);
  return TF_OK;
}

int tf_schedule_deserialize(const int *buf, size_t n_ints, tf_schedule **out) {
  if (!buf || !out || n_ints < 15 || buf[0] != kMagic) return tf::fail(TF_ERR_ARG, "tf_schedule_deserialize: not a schedule image");
  const int n1 = buf[1], np = buf[2], ni = buf[3], hk = buf[4];
  if (n1 < 1 || n1 > 2 || np < 0 || ni < 0) return tf::fail(TF_ERR_ARG, "tf_schedule_deserialize: corrupt header");
  const size_t need = 15 + (size_t)(n1 + 1) + (size_t)(np + 1) + 2 * (size_t)ni + (hk ? 2 * (size_t)np : 0);
  if (n_ints < need) return tf::fail(TF_ERR_ARG, "tf_schedule_deserialize: truncated image");
  tf_schedule *s = new tf_schedule();
  s->n1 = n1; s->has_ker = hk != 0;
  std::memcpy(s->stats, buf + 5, sizeof(double) * 5);
  const int *q = buf + 15;
  s->ptr1.assign(q, q + n1 + 1); q += n1 + 1;
  s->ptr2.assign(q, q + np + 1); q += np + 1;
  s->id.assign(q, q + ni); q += ni;
  s->type.assign(q, q + ni); q += ni;
  if (hk) s->ker.assign(q, q + 2 * (size_t)np);
  if (s->ptr1[n1] != np) { delete s; return tf::fail(TF_ERR_ARG, "tf_schedule_deserialize: inconsistent image"); }
  int rc = validate_schedule(*s);
  if (rc != TF_OK) { delete s; return rc; }
  *out = s;
  return TF_OK;
}

void tf_schedule_free(tf_schedule *s) { delete s; }

}  // extern "C"
