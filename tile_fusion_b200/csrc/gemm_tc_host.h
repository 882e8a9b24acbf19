// Host-callable pieces of the tensor-core dense producer (gemm_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace tfk {
constexpr int kTcRowsHost = 128;  // rows per tensor-core tile (= kTcRows)
// dynamic shared memory of one K slice for width n: B hi/lo (2 x 16 KB), W hi/lo (2 x n x 128 B), alignment slack
inline int tc_smem_bytes_host(int n) { return 2 * 128 * 128 + 2 * n * 128 + 1024; }
bool tc_supported(int K, int N);
int tc_make_map(CUtensorMap *out, const float *base, long long rows, int K, int box_rows);
cudaError_t tc_split_weight(const float *W, int w_transposed, int K, int N, float *hi, float *lo, cudaStream_t s);
cudaError_t tc_launch_gemm(const CUtensorMap &a, const CUtensorMap &whi, const CUtensorMap &wlo, int m, int K, int N,
                           float *T, int *error, int wait_limit, int sm_count, cudaStream_t s);
}  // namespace tfk
