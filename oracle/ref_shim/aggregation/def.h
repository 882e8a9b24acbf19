// Stand-in for the un-vendored sympiler/aggregation "def.h": only the plain
// sparse/dense containers the fusion sources touch.  Written for the oracle
// build (test infrastructure); field order follows the mirrored layout in the
// reference's fusion/gcn/GCN_Def.h:12-22.
#ifndef ORACLE_SHIM_AGGREGATION_DEF_H
#define ORACLE_SHIM_AGGREGATION_DEF_H
#include <cstddef>
#include <cstdlib>
#ifndef NULLPNTR
#define NULLPNTR nullptr
#endif
namespace sym_lib {
struct CSC {
  size_t m, n, nnz;
  int stype;
  bool is_pattern, pre_alloc;
  int *p, *i;
  double *x;
  CSC(size_t M, size_t N, size_t NNZ)
      : m(M), n(N), nnz(NNZ), stype(0), is_pattern(false), pre_alloc(false) {
    p = N > 0 ? new int[N + 1]() : nullptr;
    i = NNZ > 0 ? new int[NNZ]() : nullptr;
    x = NNZ > 0 ? new double[NNZ]() : nullptr;
  }
  CSC(size_t M, size_t N, size_t NNZ, int *Ap, int *Ai, double *Ax)
      : m(M), n(N), nnz(NNZ), stype(0), is_pattern(false), pre_alloc(true),
        p(Ap), i(Ai), x(Ax) {}
  ~CSC() {
    if (!pre_alloc) { delete[] p; delete[] i; delete[] x; }
  }
};
struct CSR {
  size_t m, n, nnz;
  int stype;
  bool is_pattern, pre_alloc;
  int *p, *i;
  double *x;
  CSR(size_t M, size_t N, size_t NNZ)
      : m(M), n(N), nnz(NNZ), stype(0), is_pattern(false), pre_alloc(false) {
    p = M > 0 ? new int[M + 1]() : nullptr;
    i = NNZ > 0 ? new int[NNZ]() : nullptr;
    x = NNZ > 0 ? new double[NNZ]() : nullptr;
  }
  CSR(size_t M, size_t N, size_t NNZ, int *Ap, int *Ai, double *Ax)
      : m(M), n(N), nnz(NNZ), stype(0), is_pattern(false), pre_alloc(true),
        p(Ap), i(Ai), x(Ax) {}
  ~CSR() {
    if (!pre_alloc) { delete[] p; delete[] i; delete[] x; }
  }
};
struct Dense {
  size_t row, col, lda;
  double *a;
  Dense(size_t M, size_t N, size_t L) : row(M), col(N), lda(L) {
    a = new double[M * N]();
  }
  ~Dense() { delete[] a; }
};
} // namespace sym_lib
#endif
