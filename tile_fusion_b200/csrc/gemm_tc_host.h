// Host-callable pieces of the tensor-core dense producer (gemm_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace tfk {
bool tc_supported(int K, int N);
int tc_make_map(CUtensorMap *out, const float *base, long long rows, int K, int box_rows);
cudaError_t tc_split_weight(const float *W, int w_transposed, int K, int N, float *hi, float *lo, cudaStream_t s);
cudaError_t tc_launch_gemm(const CUtensorMap &a, const CUtensorMap &whi, const CUtensorMap &wlo, int m, int K, int N,
                           float *T, int *error, int wait_limit, int sm_count, cudaStream_t s);
}  // namespace tfk
