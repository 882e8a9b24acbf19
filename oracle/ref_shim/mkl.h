// Stand-in for Intel MKL's "mkl.h": the CBLAS enums and the prototypes the
// GeMM-SpMM executors name.  cblas_sgemm is implemented in ref_driver.cpp on
// top of the Fortran sgemm_ exported by libtorch_cpu.so (MKL inside torch) or
// a plain loop when that is not linked.
#ifndef ORACLE_SHIM_MKL_H
#define ORACLE_SHIM_MKL_H
extern "C" {
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int M, int N, int K, float alpha,
                 const float *A, int lda, const float *B, int ldb, float beta, float *C, int ldc);
void cblas_dgemm(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int M, int N, int K, double alpha,
                 const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc);
void cblas_sgemv(CBLAS_LAYOUT, CBLAS_TRANSPOSE, int M, int N, float alpha, const float *A, int lda,
                 const float *X, int incX, float beta, float *Y, int incY);
void cblas_dgemv(CBLAS_LAYOUT, CBLAS_TRANSPOSE, int M, int N, double alpha, const double *A, int lda,
                 const double *X, int incX, double beta, double *Y, int incY);
typedef void *sparse_matrix_t;
typedef enum { SPARSE_OPERATION_NON_TRANSPOSE = 10 } sparse_operation_t;
typedef enum { SPARSE_MATRIX_TYPE_GENERAL = 20 } sparse_matrix_type_t;
typedef enum { SPARSE_LAYOUT_ROW_MAJOR = 101 } sparse_layout_t;
struct matrix_descr { sparse_matrix_type_t type; int mode; int diag; };
int mkl_sparse_s_mm(sparse_operation_t, float alpha, sparse_matrix_t, struct matrix_descr, sparse_layout_t,
                    const float *B, int cols, int ldb, float beta, float *C, int ldc);
int mkl_sparse_d_mm(sparse_operation_t, double alpha, sparse_matrix_t, struct matrix_descr, sparse_layout_t,
                    const double *B, int cols, int ldb, double beta, double *C, int ldc);
void mkl_set_num_threads(int);
}
#endif
