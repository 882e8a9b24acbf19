// Host side and stand-alone kernels of the tensor-core dense producer (see gemm_tc.cuh).
#include "gemm_tc.cuh"

#include <string>

#include "gemm_tc_host.h"
#include "tf_internal.h"

namespace tfk {

static_assert(kTcRowsHost == kTcRows, "host and device tile heights differ");

// Wt_hi / Wt_lo [N][K] (K contiguous) from W [K][N], or from W [N][K] when w_transposed.
__global__ void split_weight_kernel(const float *__restrict__ W, int w_transposed, int K, int N,
                                    float *__restrict__ hi, float *__restrict__ lo) {
  const long long total = (long long)K * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i / K), k = (int)(i % K);
    const float w = w_transposed ? W[i] : W[(size_t)k * N + n];
    const float h = tf32_round(w);
    hi[i] = h;
    lo[i] = w - h;
  }
}

// T = B * W for all 128-row tiles, one CTA per tile (grid-stride).
__global__ void __launch_bounds__(256, 2)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmWhi,
               const __grid_constant__ CUtensorMap tmWlo, int m, int K, int N, float *T, int *error, int wait_limit) {
  extern __shared__ char dyn[];
  __shared__ TcShared s;
  char *smem = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~(uintptr_t)1023);
  tc_begin(s);
  unsigned phase = 0;
  auto dst_row = [&](int r) -> float * { return T + (size_t)r * N; };
  for (int r0 = blockIdx.x * kTcRows; r0 < m; r0 += gridDim.x * kTcRows) {
    if (!tc_gemm_rows<256>(&tmA, &tmWhi, &tmWlo, r0, min(m, r0 + kTcRows), K, N, dst_row, smem, s, phase, wait_limit)) {
      if (threadIdx.x == 0) atomicExch(error, 1);
      break;
    }
  }
  tc_end(s);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

bool tc_supported(int K, int N) { return K >= 4 && K % 4 == 0 && N >= 16 && N % 16 == 0 && N <= kTcMaxN; }

// fp32 row-major [rows][K] tensor, box = 32 columns (128 bytes) x box_rows, 128-byte swizzle, zero fill
int tc_make_map(CUtensorMap *out, const float *base, long long rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return tf::fail(TF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return tf::fail(TF_ERR_ARG, "tensor-core producer: operand must be 16-byte aligned");
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)kTcKSlice, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return tf::fail(TF_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return TF_OK;
}

cudaError_t tc_split_weight(const float *W, int w_transposed, int K, int N, float *hi, float *lo, cudaStream_t s) {
  const long long total = (long long)K * N;
  const int grid = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  split_weight_kernel<<<grid, 256, 0, s>>>(W, w_transposed, K, N, hi, lo);
  return cudaGetLastError();
}

cudaError_t tc_launch_gemm(const CUtensorMap &a, const CUtensorMap &whi, const CUtensorMap &wlo, int m, int K, int N,
                           float *T, int *error, int wait_limit, int sm_count, cudaStream_t s) {
  const size_t smem = (size_t)tc_smem_bytes(N);
  cudaError_t e = cudaFuncSetAttribute((const void *)tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int tiles = (m + kTcRows - 1) / kTcRows;
  const int grid = std::max(1, std::min(tiles, sm_count * 2));
  tc_gemm_kernel<<<grid, 256, smem, s>>>(a, whi, wlo, m, K, N, T, error, wait_limit);
  return cudaGetLastError();
}

}  // namespace tfk

// T = B * W on device pointers with the tensor-core producer alone (test and profiling entry).
extern "C" int tf_gemm_tc_dev(const float *B, const float *W, int w_transposed, int m, int K, int N, float *T,
                              void *stream) {
  if (!B || !W || !T) return tf::fail(TF_ERR_ARG, "tf_gemm_tc_dev: null argument");
  if (m <= 0 || !tfk::tc_supported(K, N))
    return tf::fail(TF_ERR_UNSUPPORTED, "tf_gemm_tc_dev: needs K % 4 == 0, N % 16 == 0, N <= 256");
  cudaStream_t s = (cudaStream_t)stream;
  float *hi = nullptr, *lo = nullptr;
  int *err = nullptr;
  cudaError_t e = cudaMalloc(&hi, (size_t)K * N * 4);
  if (e == cudaSuccess) e = cudaMalloc(&lo, (size_t)K * N * 4);
  if (e == cudaSuccess) e = cudaMalloc(&err, 4);
  if (e == cudaSuccess) e = cudaMemsetAsync(err, 0, 4, s);
  int rc = TF_OK;
  if (e != cudaSuccess) rc = tf::fail(TF_ERR_NOMEM, std::string("tf_gemm_tc_dev: ") + cudaGetErrorString(e));
  CUtensorMap ma, mh, ml;
  if (rc == TF_OK) rc = tfk::tc_make_map(&ma, B, m, K, tfk::kTcRows);
  if (rc == TF_OK) rc = tfk::tc_make_map(&mh, hi, N, K, N);
  if (rc == TF_OK) rc = tfk::tc_make_map(&ml, lo, N, K, N);
  if (rc == TF_OK) {
    e = tfk::tc_split_weight(W, w_transposed, K, N, hi, lo, s);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = tfk::tc_launch_gemm(ma, mh, ml, m, K, N, T, err, 1 << 20, sms, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    int h_err = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&h_err, err, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = tf::fail(TF_ERR_CUDA, std::string("tf_gemm_tc_dev: ") + cudaGetErrorString(e));
    else if (h_err) rc = tf::fail(TF_ERR_TIMEOUT, "tf_gemm_tc_dev: a bounded wait on a copy or on the tensor core ran out");
  }
  cudaFree(hi); cudaFree(lo); cudaFree(err);
  return rc;
}
