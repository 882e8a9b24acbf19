// Matrix ingestion: the two file formats the reference's experiment drivers read
// (get_matrix_from_parameter, fusion/src/Fusion_Utils.cpp:252-272):
//   *.mtx   Matrix Market, coordinate format (real / integer / pattern; general / symmetric / skew-symmetric),
//           and the dense "array" format the GCN demos read their feature matrices from (:274-283);
//   *.smtx  the DLMC text format (readSparseMatrix, ibid. :205-250): "rows, cols, nnz", the row pointers, the
//           column indices; every value 1.
// The result is CSR with int32 indices, fp32 values and sorted columns (what every executor here takes);
// duplicate entries of a Matrix Market file are added up.  The reference exits the process on a file it cannot
// open; here every failure is an error code with a message.
#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "tf_internal.h"

namespace {

using tf::fail;

std::string lower(std::string s) {
  for (char &c : s) c = (char)std::tolower((unsigned char)c);
  return s;
}

struct Triplets {
  long long m = 0, n = 0;
  std::vector<int> r, c;
  std::vector<float> v;
};

// rows sorted, columns sorted inside a row, duplicates summed
int to_csr(const Triplets &t, int **ap_out, int **ai_out, float **ax_out, long long *nnz_out) {
  const size_t nz = t.r.size();
  std::vector<size_t> order(nz);
  for (size_t i = 0; i < nz; ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) {
    return t.r[a] != t.r[b] ? t.r[a] < t.r[b] : (t.c[a] != t.c[b] ? t.c[a] < t.c[b] : a < b);
  });
  std::vector<int> ap((size_t)t.m + 1, 0), ai;
  std::vector<float> ax;
  ai.reserve(nz); ax.reserve(nz);
  int last_r = -1, last_c = -1;
  for (size_t q = 0; q < nz; ++q) {
    const size_t i = order[q];
    if (t.r[i] == last_r && t.c[i] == last_c) { ax.back() += t.v[i]; continue; }
    ai.push_back(t.c[i]); ax.push_back(t.v[i]);
    ++ap[(size_t)t.r[i] + 1];
    last_r = t.r[i]; last_c = t.c[i];
  }
  for (long long i = 0; i < t.m; ++i) ap[i + 1] += ap[i];
  int *p = (int *)malloc(sizeof(int) * ap.size());
  int *ci = (int *)malloc(sizeof(int) * std::max<size_t>(ai.size(), 1));
  float *x = (float *)malloc(sizeof(float) * std::max<size_t>(ax.size(), 1));
  if (!p || !ci || !x) { free(p); free(ci); free(x); return fail(TF_ERR_NOMEM, "matrix reader: out of memory"); }
  std::copy(ap.begin(), ap.end(), p);
  std::copy(ai.begin(), ai.end(), ci);
  std::copy(ax.begin(), ax.end(), x);
  *ap_out = p; *ai_out = ci; *ax_out = x; *nnz_out = (long long)ai.size();
  return TF_OK;
}

int read_mtx(std::ifstream &f, const std::string &path, bool expand_symmetric, Triplets &t) {
  std::string line;
  if (!std::getline(f, line)) return fail(TF_ERR_ARG, path + ": empty file");
  std::istringstream hdr(lower(line));
  std::string banner, object, format, field, symmetry;
  hdr >> banner >> object >> format >> field >> symmetry;
  if (banner != "%%matrixmarket" || object != "matrix") return fail(TF_ERR_ARG, path + ": not a Matrix Market matrix file");
  if (format != "coordinate") return fail(TF_ERR_UNSUPPORTED, path + ": sparse reader wants the coordinate format (array files: tf_read_dense_mtx)");
  if (field != "real" && field != "integer" && field != "pattern" && field != "double")
    return fail(TF_ERR_UNSUPPORTED, path + ": field '" + field + "' is not supported (real, integer, pattern)");
  if (symmetry != "general" && symmetry != "symmetric" && symmetry != "skew-symmetric")
    return fail(TF_ERR_UNSUPPORTED, path + ": symmetry '" + symmetry + "' is not supported");
  while (std::getline(f, line))
    if (!line.empty() && line[0] != '%') break;
  long long m = 0, n = 0, nz = 0;
  if (sscanf(line.c_str(), "%lld %lld %lld", &m, &n, &nz) != 3 || m <= 0 || n <= 0 || nz < 0)
    return fail(TF_ERR_ARG, path + ": bad size line");
  if (m > 0x7fffffffLL || n > 0x7fffffffLL) return fail(TF_ERR_UNSUPPORTED, path + ": dimensions above 2^31");
  t.m = m; t.n = n;
  const bool pattern = field == "pattern";
  const bool sym = symmetry != "general";
  const float mirror = symmetry == "skew-symmetric" ? -1.f : 1.f;
  t.r.reserve((size_t)nz * (sym && expand_symmetric ? 2 : 1));
  t.c.reserve(t.r.capacity()); t.v.reserve(t.r.capacity());
  for (long long q = 0; q < nz; ++q) {
    long long i, j;
    double v = 1.0;
    if (!(f >> i >> j)) return fail(TF_ERR_ARG, path + ": fewer entries than the size line announces");
    if (!pattern && !(f >> v)) return fail(TF_ERR_ARG, path + ": entry without a value");
    if (i < 1 || i > m || j < 1 || j > n) return fail(TF_ERR_ARG, path + ": index out of range (indices are 1-based)");
    t.r.push_back((int)(i - 1)); t.c.push_back((int)(j - 1)); t.v.push_back((float)v);
    if (sym && expand_symmetric && i != j) { t.r.push_back((int)(j - 1)); t.c.push_back((int)(i - 1)); t.v.push_back(mirror * (float)v); }
  }
  return TF_OK;
}

int read_smtx(std::ifstream &f, const std::string &path, Triplets &t) {
  std::string line;
  if (!std::getline(f, line)) return fail(TF_ERR_ARG, path + ": empty file");
  std::replace(line.begin(), line.end(), ',', ' ');
  long long m = 0, n = 0, nz = 0;
  if (sscanf(line.c_str(), "%lld %lld %lld", &m, &n, &nz) != 3 || m <= 0 || n <= 0 || nz < 0)
    return fail(TF_ERR_ARG, path + ": bad first line (rows, cols, nnz)");
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || nz > 0x7fffffffLL) return fail(TF_ERR_UNSUPPORTED, path + ": sizes above 2^31");
  std::vector<long long> p((size_t)m + 1);
  for (long long i = 0; i <= m; ++i)
    if (!(f >> p[i])) return fail(TF_ERR_ARG, path + ": row pointer line is short");
  if (p[0] != 0 || p[m] != nz) return fail(TF_ERR_ARG, path + ": row pointers do not span the nonzeros");
  t.m = m; t.n = n;
  t.r.resize((size_t)nz); t.c.resize((size_t)nz); t.v.assign((size_t)nz, 1.f);
  for (long long i = 0; i < m; ++i) {
    if (p[i + 1] < p[i]) return fail(TF_ERR_ARG, path + ": row pointers decrease");
    for (long long q = p[i]; q < p[i + 1]; ++q) t.r[q] = (int)i;
  }
  for (long long q = 0; q < nz; ++q) {
    long long j;
    if (!(f >> j)) return fail(TF_ERR_ARG, path + ": column index line is short");
    if (j < 0 || j >= n) return fail(TF_ERR_ARG, path + ": column index out of range");
    t.c[q] = (int)j;
  }
  return TF_OK;
}

}  // namespace

extern "C" int tf_read_matrix(const char *path, int expand_symmetric, int *m, int *n, long long *nnz, int **ap, int **ai,
                              float **ax) {
  if (!path || !m || !n || !nnz || !ap || !ai || !ax) return fail(TF_ERR_ARG, "tf_read_matrix: null argument");
  const std::string p(path);
  const size_t dot = p.find_last_of('.');
  const std::string ext = dot == std::string::npos ? "" : lower(p.substr(dot + 1));
  if (ext != "mtx" && ext != "smtx") return fail(TF_ERR_UNSUPPORTED, p + ": file extension is not supported (mtx, smtx)");
  std::ifstream f(p);
  if (!f.is_open()) return fail(TF_ERR_ARG, p + ": file could not be opened");
  Triplets t;
  int rc = ext == "mtx" ? read_mtx(f, p, expand_symmetric != 0, t) : read_smtx(f, p, t);
  if (rc != TF_OK) return rc;
  rc = to_csr(t, ap, ai, ax, nnz);
  if (rc != TF_OK) return rc;
  *m = (int)t.m; *n = (int)t.n;
  return TF_OK;
}

// Dense matrix from a Matrix Market "array" file (column-major in the file), returned row-major.
extern "C" int tf_read_dense_mtx(const char *path, int *rows, int *cols, float **data) {
  if (!path || !rows || !cols || !data) return fail(TF_ERR_ARG, "tf_read_dense_mtx: null argument");
  const std::string p(path);
  std::ifstream f(p);
  if (!f.is_open()) return fail(TF_ERR_ARG, p + ": file could not be opened");
  std::string line;
  if (!std::getline(f, line)) return fail(TF_ERR_ARG, p + ": empty file");
  std::istringstream hdr(lower(line));
  std::string banner, object, format;
  hdr >> banner >> object >> format;
  if (banner != "%%matrixmarket" || object != "matrix" || format != "array")
    return fail(TF_ERR_ARG, p + ": not a Matrix Market array file");
  while (std::getline(f, line))
    if (!line.empty() && line[0] != '%') break;
  long long m = 0, n = 0;
  if (sscanf(line.c_str(), "%lld %lld", &m, &n) != 2 || m <= 0 || n <= 0 || m * n > 0x7fffffffLL)
    return fail(TF_ERR_ARG, p + ": bad size line");
  float *d = (float *)malloc(sizeof(float) * (size_t)(m * n));
  if (!d) return fail(TF_ERR_NOMEM, "tf_read_dense_mtx: out of memory");
  for (long long j = 0; j < n; ++j)
    for (long long i = 0; i < m; ++i) {
      double v;
      if (!(f >> v)) { free(d); return fail(TF_ERR_ARG, p + ": fewer values than the size line announces"); }
      d[i * n + j] = (float)v;
    }
  *rows = (int)m; *cols = (int)n; *data = d;
  return TF_OK;
}
