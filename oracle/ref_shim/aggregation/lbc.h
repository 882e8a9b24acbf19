// Stand-in: LBC level-set coarsening is only taken for non-diagonal DAGs
// (Fusion_Utils.cpp:493), which the fused SpMM/GeMM chains never build.
#ifndef ORACLE_SHIM_LBC_H
#define ORACLE_SHIM_LBC_H
#include "aggregation/sparse_utilities.h"
namespace sym_lib {
inline int get_coarse_levelSet_DAG_CSC_tree(size_t, int *, int *, int, int &, int *&, int &,
                                            int *&, int *&, int, int, int, double *) {
  oracle_shim_unreachable("get_coarse_levelSet_DAG_CSC_tree");
}
} // namespace sym_lib
#endif
