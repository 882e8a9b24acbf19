// Stand-in: matrix-market readers are not used by the oracle (inputs are generated).
#ifndef ORACLE_SHIM_SPARSE_IO_H
#define ORACLE_SHIM_SPARSE_IO_H
#include "aggregation/sparse_utilities.h"
#include <fstream>
namespace sym_lib {
inline void read_mtx_csc_real(std::ifstream &, CSC *&, bool) { oracle_shim_unreachable("read_mtx_csc_real"); }
inline void read_mtx_array_real(std::ifstream &, Dense *&) { oracle_shim_unreachable("read_mtx_array_real"); }
} // namespace sym_lib
#endif
