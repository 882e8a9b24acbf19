// TEST INFRASTRUCTURE ONLY.  C-ABI wrapper around the *unmodified* reference
// sources of SwiftWare-Lab/tile-fusion, compiled where they lie (see
// oracle/Makefile, target `ref`).  Nothing of the reference is copied here:
// this file only calls into it.  The product library never links or loads the
// resulting oracle/_ref/libtf_ref.so; tests, the golden-vector generator and
// bench.py's CPU-baseline leg do.
//
// Wrapped reference entry points (paths inside the reference project):
//   I1  SparseFusionInspector::generateFusedScheduleForAllFused
//         fusion/include/sparse-fusion/Fusion_Inspector.h:32
//   I4  InspectorForTileFusedCSRVariableTileSize::generateVariableTileSizeSchedule        :542
//   I2  ...::generateVariableTileSizeScheduleForBothWavefronts                            :676
//   I3  ...::generateVariableTileSizeScheduleGeMMSpMM                                     :851
//   E1  swiftware::sparse::spmmCsrSpmmCsrFused<float>          fusion/src/SpMM_SpMM.cpp:211
//   E2  swiftware::sparse::spmmCsrSpmmCsrFusedVectorized2_32SP fusion/src/SpMM_SpMM_vectorized.cpp:876
//   E4  swiftware::sparse::spmmCsrParallel<float>              fusion/src/SpMM_SpMM.cpp:37
//   E3  forwardForOneLayerFusedParallelSeparatedVectorizedSP   fusion/gcn/GCN_Layer_MKL_Forward_Utils.h:218
//       forwardForOneLayerFusedParallelSeparatedSP (scalar, transposed weight)            :182
//       forwardForOneLayerWithMKLGeMMAndSpMMSPVectorized (unfused)                        :1138
//   E2' swiftware::sparse::spmmCsrSpmmCsrFusedVectorized2_32Avx512SP (built only with AVX-512F)
//         fusion/src/SpMM_SpMM_vectorized.cpp:221
//   E6  GnnTensorSpInputs::normalizeAdjacencyMatrix
//         fusion/gcn/SingleLayer/GCN_Single_Layer_SP_Demo_Utils.h:40-53 -- the header itself needs the
//         un-vendored benchmark framework, so the Makefile cuts exactly this member function out of it
//         (into _ref/normalize_adjacency.inc) and it is compiled here inside a struct that has the three
//         fields it touches
//   createUnfusedData (fusion/example/SpMM_SpMM_SP_Demo_Utils.h:600-636) and createReorderedAdj
//         (GCN_Single_Layer_SP_Demo_Utils.h:618-653): the reordered layouts of the bench classes, cut out the same way
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#define MKL 1
#include "sparse-fusion/Fusion_Inspector.h"
#include "sparse-fusion/SpMM_SpMM.h"
#include "sparse-fusion/SpMM_SpMM_vectorized.h"
#include "GCN_Layer_MKL_Forward_Utils.h"

// ---------------------------------------------------------------------------
// cblas_sgemm for the reference GeMM tile: forwards to a Fortran sgemm_ given
// at run time (MKL inside libtorch_cpu.so, handed over by the Python side), or
// falls back to a plain triple loop.  Row-major C = A*B is column-major
// C^T = B^T * A^T.
// ---------------------------------------------------------------------------
typedef void (*sgemm_fn)(const char *, const char *, const int *, const int *, const int *,
                         const float *, const float *, const int *, const float *, const int *,
                         const float *, float *, const int *);
static sgemm_fn g_sgemm = nullptr;
typedef int (*mkl_local_threads_fn)(int);

extern "C" void tf_ref_set_sgemm(void *fn) { g_sgemm = (sgemm_fn)fn; }
extern "C" int tf_ref_has_sgemm() { return g_sgemm != nullptr; }

extern "C" void cblas_sgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N,
                            int K, float alpha, const float *A, int lda, const float *B, int ldb,
                            float beta, float *C, int ldc) {
  if (layout != CblasRowMajor) { std::fprintf(stderr, "tf_ref: only row-major sgemm\n"); std::abort(); }
  if (M <= 0 || N <= 0) return;
  if (g_sgemm) {
    // column-major: C^T (N x M) = op(B)^T (N x K) * op(A)^T (K x M)
    const char opB = (tb == CblasNoTrans) ? 'N' : 'T';
    const char opA = (ta == CblasNoTrans) ? 'N' : 'T';
    g_sgemm(&opB, &opA, &N, &M, &K, &alpha, B, &ldb, A, &lda, &beta, C, &ldc);
    return;
  }
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        float a = (ta == CblasNoTrans) ? A[(size_t)i * lda + k] : A[(size_t)k * lda + i];
        float b = (tb == CblasNoTrans) ? B[(size_t)k * ldb + j] : B[(size_t)j * ldb + k];
        acc += a * b;
      }
      C[(size_t)i * ldc + j] = alpha * acc + (beta == 0.f ? 0.f : beta * C[(size_t)i * ldc + j]);
    }
}
extern "C" void cblas_dgemm(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, double,
                            const double *, int, const double *, int, double, double *, int) {
  std::fprintf(stderr, "tf_ref: cblas_dgemm is outside the fp32 hot path\n"); std::abort();
}
extern "C" void cblas_sgemv(CBLAS_LAYOUT, CBLAS_TRANSPOSE, int, int, float, const float *, int,
                            const float *, int, float, float *, int) {
  std::fprintf(stderr, "tf_ref: cblas_sgemv is outside the hot path\n"); std::abort();
}
extern "C" void cblas_dgemv(CBLAS_LAYOUT, CBLAS_TRANSPOSE, int, int, double, const double *, int,
                            const double *, int, double, double *, int) {
  std::fprintf(stderr, "tf_ref: cblas_dgemv is outside the hot path\n"); std::abort();
}
extern "C" int mkl_sparse_s_mm(sparse_operation_t, float, sparse_matrix_t, struct matrix_descr,
                               sparse_layout_t, const float *, int, int, float, float *, int) {
  std::fprintf(stderr, "tf_ref: mkl_sparse_s_mm not wired\n"); std::abort();
}
extern "C" int mkl_sparse_d_mm(sparse_operation_t, double, sparse_matrix_t, struct matrix_descr,
                               sparse_layout_t, const double *, int, int, double, double *, int) {
  std::fprintf(stderr, "tf_ref: mkl_sparse_d_mm not wired\n"); std::abort();
}
extern "C" void mkl_set_num_threads(int) {}

// ---------------------------------------------------------------------------
// Schedules
// ---------------------------------------------------------------------------
struct RefSched {
  sym_lib::MultiDimensionalSet *s;
  double stats[8]; // fused nodes, fused nnz, tile mean, tile std, num partitions
};

static sym_lib::ScheduleParameters make_sp(int threads, int ipp, int tile_m) {
  sym_lib::ScheduleParameters sp;
  sp._num_threads = threads;
  sp._num_w_partition = threads;
  sp.IterPerPartition = ipp;
  sp.TileM = tile_m;
  sp.TileN = 32;
  sp.SeedPartitioningParallelism = sym_lib::CONSECUTIVE;
  return sp;
}

static double stat_or(Stats &st, const char *k, double d) {
  auto it = st.OtherStats.find(k);
  return (it == st.OtherStats.end() || it->second.empty()) ? d : it->second[0];
}

// kind: 1 = I1 fixed tiles (uses ipp), 2 = I2 SpMM-SpMM variable tiles (bcol, tile_m),
//       3 = I3 GeMM-SpMM variable tiles (bcol, ccol, tile_m), 4 = I4 (bcol, tile_m)
extern "C" void *tf_ref_inspect(int kind, int m, int nnz, int *Ap, int *Ai, int threads, int ipp,
                                int tile_m, int bcol, int ccol, int data_size) {
  Stats st;
  sym_lib::ScheduleParameters sp = make_sp(threads, ipp, tile_m);
  sym_lib::CSR a((size_t)m, (size_t)m, (size_t)nnz, Ap, Ai, nullptr);
  RefSched *r = new RefSched();
  std::memset(r->stats, 0, sizeof(r->stats));
  if (kind == 1) {
    st.OtherStats["PackingType"] = {(double)sym_lib::Separated};
    SparseFusionInspector insp(sp, &st);
    r->s = insp.generateFusedScheduleForAllFused(&a);
    r->stats[0] = r->s->getNumberOfFusedNodes();
    r->stats[1] = r->s->getFusedNnzNum(&a);
  } else {
    InspectorForTileFusedCSRVariableTileSize insp(sp, &st);
    if (kind == 2) r->s = insp.generateVariableTileSizeScheduleForBothWavefronts(&a, bcol, data_size);
    else if (kind == 3) r->s = insp.generateVariableTileSizeScheduleGeMMSpMM(&a, bcol, ccol, data_size);
    else r->s = insp.generateVariableTileSizeSchedule(&a, bcol, data_size);
    r->stats[0] = stat_or(st, kind == 3 ? "FusedIterations" : "Number of Fused Nodes", 0);
    r->stats[1] = kind == 3 ? (double)r->s->getFusedNnzNum(&a) : stat_or(st, "Number of Fused nnz", 0);
    r->stats[2] = stat_or(st, "Tile Size Mean", 0);
    r->stats[3] = stat_or(st, "Tile Size STD", 0);
  }
  r->stats[4] = r->s->ptr1_[r->s->n1_];
  return r;
}

extern "C" void tf_ref_sched_dims(void *h, int *n1, int *n_parts, int *n_ids, int *has_ker) {
  RefSched *r = (RefSched *)h;
  *n1 = r->s->n1_;
  *n_parts = r->s->ptr1_[r->s->n1_];
  *n_ids = r->s->ptr2_[*n_parts];
  *has_ker = r->s->ker_begin_ != nullptr;
}
extern "C" void tf_ref_sched_copy(void *h, int *ptr1, int *ptr2, int *id, int *type, int *ker,
                                  double *stats) {
  RefSched *r = (RefSched *)h;
  int n1 = r->s->n1_, np = r->s->ptr1_[n1], ni = r->s->ptr2_[np];
  std::memcpy(ptr1, r->s->ptr1_, sizeof(int) * (n1 + 1));
  std::memcpy(ptr2, r->s->ptr2_, sizeof(int) * (np + 1));
  std::memcpy(id, r->s->id_, sizeof(int) * ni);
  std::memcpy(type, r->s->type_, sizeof(int) * ni);
  if (ker && r->s->ker_begin_) std::memcpy(ker, r->s->ker_begin_, sizeof(int) * 2 * np);
  if (stats) std::memcpy(stats, r->stats, sizeof(r->stats));
}
extern "C" void tf_ref_sched_free(void *h) {
  RefSched *r = (RefSched *)h;
  delete r->s;
  delete r;
}

// ---------------------------------------------------------------------------
// Executors.  D and the intermediate must be zeroed by the caller exactly as
// the reference's bench classes do before each run.
// ---------------------------------------------------------------------------
extern "C" void tf_ref_spmm_csr(int m, int n, const int *Ap, const int *Ai, const float *Ax,
                                const float *Bx, float *Cx, int threads) {
  if (threads <= 1) swiftware::sparse::spmmCsrSequential<float>(m, n, m, Ap, Ai, Ax, Bx, Cx);
  else swiftware::sparse::spmmCsrParallel<float>(m, n, m, Ap, Ai, Ax, Bx, Cx, threads);
}

extern "C" int tf_ref_has_avx512() {
#ifdef __AVX512F__
  return 1;
#else
  return 0;
#endif
}

// variant 0 = scalar E1, 1 = AVX2 E2 (needs n % 32 == 0), 2 = AVX-512 (needs n % 32 == 0 and a build with AVX-512F)
extern "C" void tf_ref_spmm_spmm_fused(int variant, int m, int n, const int *Ap, const int *Ai,
                                       const float *Ax, const int *Bp, const int *Bi, const float *Bx,
                                       const float *Cx, float *Dx, float *ACx, int level_no,
                                       const int *level_ptr, const int *par_ptr, const int *partition,
                                       const int *par_type, int threads) {
  if (variant == 0)
    swiftware::sparse::spmmCsrSpmmCsrFused<float>(m, n, m, m, Ap, Ai, Ax, Bp, Bi, Bx, Cx, Dx, ACx,
                                                  level_no, level_ptr, par_ptr, partition, par_type,
                                                  threads);
#ifdef __AVX512F__
  else if (variant == 2)
    swiftware::sparse::spmmCsrSpmmCsrFusedVectorized2_32Avx512SP(m, n, m, m, Ap, Ai, Ax, Bp, Bi, Bx, Cx,
                                                                 Dx, ACx, level_no, level_ptr, par_ptr,
                                                                 partition, par_type, threads);
#endif
  else
    swiftware::sparse::spmmCsrSpmmCsrFusedVectorized2_32SP(m, n, m, m, Ap, Ai, Ax, Bp, Bi, Bx, Cx, Dx,
                                                           ACx, level_no, level_ptr, par_ptr, partition,
                                                           par_type, threads);
}

// variant 0 = scalar (weight stored [N x K], CblasTrans), 1 = AVX2 (weight [K x N], n % 32 == 0)
extern "C" void tf_ref_gemm_spmm_fused(int variant, int m, int *Ap, int *Ai, float *Ax, int k, int n,
                                       float *feat, float *weight, float *out, float *inter,
                                       int threads, int level_no, const int *level_ptr,
                                       const int *par_ptr, const int *mix_ptr, const int *partition) {
  if (variant == 0)
    forwardForOneLayerFusedParallelSeparatedSP(m, Ap, Ai, Ax, k, n, feat, weight, out, inter, threads,
                                               level_no, level_ptr, par_ptr, mix_ptr, partition);
  else
    forwardForOneLayerFusedParallelSeparatedVectorizedSP(m, Ap, Ai, Ax, k, n, feat, weight, out, inter,
                                                         threads, level_no, level_ptr, par_ptr, mix_ptr,
                                                         partition);
}

// unfused: full sgemm then AVX2 SpMM (n % 32 == 0), weight [K x N]
extern "C" void tf_ref_gemm_spmm_unfused(int m, int *Ap, int *Ai, float *Ax, int k, int n, float *feat,
                                         float *weight, float *out, float *inter, int threads) {
  forwardForOneLayerWithMKLGeMMAndSpMMSPVectorized(m, Ap, Ai, Ax, feat, k, weight, n, out, inter,
                                                   threads);
}

// ---------------------------------------------------------------------------
// Adjacency normalisation of the GCN demos: values / sqrt(deg_i * deg_j), deg = row length.
// ---------------------------------------------------------------------------
#if __has_include("_ref/normalize_adjacency.inc")
namespace {
struct RefNormalize {
  int *Degrees;
  size_t NumOfNodes;
  sym_lib::CSR *AdjacencyMatrix;
#include "_ref/normalize_adjacency.inc"
};
}  // namespace
// ax: the values as doubles (the reference's CSR holds doubles; its demos convert to float afterwards)
extern "C" int tf_ref_normalize_adjacency(int n, int *ap, int *ai, double *ax) {
  sym_lib::CSR a((size_t)n, (size_t)n, (size_t)ap[n], ap, ai, ax);
  RefNormalize r;
  r.Degrees = nullptr;
  r.NumOfNodes = (size_t)n;
  r.AdjacencyMatrix = &a;
  r.normalizeAdjacencyMatrix();
  delete[] r.Degrees;
  return 1;
}
#else
extern "C" int tf_ref_normalize_adjacency(int, int *, int *, double *) { return 0; }
#endif

// ---------------------------------------------------------------------------
// Reordered layouts of the bench classes (member functions cut out of their headers by the Makefile).
// ---------------------------------------------------------------------------
#if __has_include("_ref/create_unfused_data.inc") && __has_include("_ref/create_reordered_adj.inc")
namespace {
struct RefUnfusedData {
  struct In { sym_lib::CSR *ACsr; } in_, *InTensor = &in_;
  float *AValues = nullptr;
  int *UFAp = nullptr, *UFAi = nullptr;
  float *UFAx = nullptr;
#include "_ref/create_unfused_data.inc"
};
struct RefReorderedAdj {
  struct In { sym_lib::CSR *AdjacencyMatrix; float *AMValues; } in_, *InTensor = &in_;
  int *Ap = nullptr, *Ai = nullptr, *L2Ptr = nullptr, *NewMixPtr = nullptr;
  float *Ax = nullptr;
#include "_ref/create_reordered_adj.inc"
};
}  // namespace
// h: a schedule made by tf_ref_inspect.  Outputs are caller-allocated (uf arrays: at most m + 1 / nnz entries).
extern "C" int tf_ref_create_unfused_data(void *h, int m, int *ap, int *ai, float *ax, int *uf_ap, int *uf_ai, float *uf_ax) {
  RefSched *r = (RefSched *)h;
  sym_lib::CSR a((size_t)m, (size_t)m, (size_t)ap[m], ap, ai, nullptr);
  RefUnfusedData u;
  u.in_.ACsr = &a;
  u.AValues = ax;
  u.createUnfusedData(r->s->ptr1_, r->s->ker_begin_, r->s->id_);
  int rows = 0;
  for (int l1 = r->s->ptr1_[1]; l1 < r->s->ptr1_[2]; ++l1) rows += r->s->ker_begin_[2 * l1 + 1] - r->s->ker_begin_[2 * l1];
  for (int i = 0; i <= rows; ++i) uf_ap[i] = u.UFAp[i];
  for (int j = 0; j < u.UFAp[rows]; ++j) { uf_ai[j] = u.UFAi[j]; uf_ax[j] = u.UFAx[j]; }
  delete[] u.UFAp; delete[] u.UFAi; delete[] u.UFAx;
  return rows;
}
extern "C" int tf_ref_create_reordered_adj(void *h, int m, int *ap, int *ai, float *ax, int *r_ap, int *r_ai, float *r_ax,
                                           int *l2_ptr, int *new_mix) {
  RefSched *r = (RefSched *)h;
  sym_lib::CSR a((size_t)m, (size_t)m, (size_t)ap[m], ap, ai, nullptr);
  RefReorderedAdj u;
  u.in_.AdjacencyMatrix = &a;
  u.in_.AMValues = ax;
  u.createReorderedAdj(r->s->ptr1_, r->s->ker_begin_, r->s->id_);
  const int n_mix = (r->s->ptr1_[2] + 1) * 2;
  for (int i = 0; i <= m; ++i) r_ap[i] = u.Ap[i];
  for (int j = 0; j < ap[m]; ++j) { r_ai[j] = u.Ai[j]; r_ax[j] = u.Ax[j]; }
  for (int i = 0; i < m; ++i) l2_ptr[i] = u.L2Ptr[i];
  for (int i = 0; i < n_mix; ++i) new_mix[i] = u.NewMixPtr[i];
  delete[] u.Ap; delete[] u.Ai; delete[] u.Ax; delete[] u.L2Ptr; delete[] u.NewMixPtr;
  return n_mix;
}
#else
extern "C" int tf_ref_create_unfused_data(void *, int, int *, int *, float *, int *, int *, float *) { return -1; }
extern "C" int tf_ref_create_reordered_adj(void *, int, int *, int *, float *, int *, int *, float *, int *, int *) { return -1; }
#endif
