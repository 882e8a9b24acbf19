// SpMM-SpMM for callers that must not allocate: the intermediate lives in a fixed device array
// that is part of the library image.  See tf_spmm_spmm_noalloc in include/tile_fusion_b200.h.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "launch.h"
#include "tf_internal.h"

namespace {

// 4 Mi floats = 16 MiB per GPU that loads the library, held until the process exits.
constexpr long long kScratchFloats = 4LL << 20;
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, once per device.
constexpr int kMaxDevices = 64;
float *g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

int scratch_for_current_device(float **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return tf::fail(TF_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return tf::fail(TF_ERR_UNSUPPORTED, "tf_spmm_spmm_noalloc: device index above 63");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    float *p = nullptr;
    e = cudaGetSymbolAddress((void **)&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return tf::fail(TF_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return TF_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" long long tf_noalloc_max_floats(void) { return kScratchFloats; }

extern "C" int tf_spmm_spmm_noalloc(const int *Ap, const int *Ai, const float *Ax, int m, const float *C,
                                    int n_cols, float *D, void *stream) {
  if (!Ap || !Ai || !Ax || !C || !D) return tf::fail(TF_ERR_ARG, "tf_spmm_spmm_noalloc: null argument");
  if (m <= 0 || n_cols <= 0) return tf::fail(TF_ERR_ARG, "tf_spmm_spmm_noalloc: sizes must be positive");
  if ((long long)m * n_cols > kScratchFloats)
    return tf::fail(TF_ERR_ARG, "tf_spmm_spmm_noalloc: m * n_cols = " + std::to_string((long long)m * n_cols) +
                                    " exceeds the built-in intermediate of " + std::to_string(kScratchFloats) +
                                    " floats; use a plan (tf_plan_spmm_spmm) for larger problems");
  float *T = nullptr;
  int rc = scratch_for_current_device(&T);
  if (rc != TF_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  int vec, ch;
  const int grid = std::max(1, std::min((m + 63) / 64, 148 * 8));
  // T = A * C: every row of T is overwritten, so nothing of the previous call survives in the rows used
  tfk::choose_shape(n_cols, aligned16(C), &vec, &ch);
  cudaError_t e = tfk::launch_spmm(vec, ch, grid, Ap, Ai, Ax, m, C, n_cols, T, s);
  if (e != cudaSuccess) return tf::fail(TF_ERR_CUDA, std::string("first SpMM launch: ") + cudaGetErrorString(e));
  // D = A * T
  tfk::choose_shape(n_cols, aligned16(D), &vec, &ch);
  e = tfk::launch_spmm(vec, ch, grid, Ap, Ai, Ax, m, T, n_cols, D, s);
  if (e != cudaSuccess) return tf::fail(TF_ERR_CUDA, std::string("second SpMM launch: ") + cudaGetErrorString(e));
  return TF_OK;
}
