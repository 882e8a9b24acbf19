// Stand-in for sympiler/aggregation "sparse_utilities.h": the fixed-tile
// inspector only needs diagonal(); the rest of the library is never reached.
#ifndef ORACLE_SHIM_SPARSE_UTILITIES_H
#define ORACLE_SHIM_SPARSE_UTILITIES_H
#include "aggregation/def.h"
#include <cstdio>
#include <cstdlib>
namespace sym_lib {
inline CSC *diagonal(int N, double V) {
  CSC *d = new CSC(N, N, N);
  for (int i = 0; i < N; ++i) { d->p[i] = i; d->i[i] = i; d->x[i] = V; }
  d->p[N] = N;
  return d;
}
[[noreturn]] inline void oracle_shim_unreachable(const char *what) {
  std::fprintf(stderr, "oracle shim: %s is not part of the fused hot path\n", what);
  std::abort();
}
inline CSC *csr_to_csc(CSR *) { oracle_shim_unreachable("csr_to_csc"); }
inline CSC *make_full(CSC *) { oracle_shim_unreachable("make_full"); }
inline CSC *random_square_sparse(size_t, double) { oracle_shim_unreachable("random_square_sparse"); }
} // namespace sym_lib
#endif
