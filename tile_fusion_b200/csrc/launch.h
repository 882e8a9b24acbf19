// Host-callable launchers of the kernels in kernels.cu.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>

namespace tfk {
struct Params;

// vec = floats per lane (4, 2, 1), ch = vectors per lane (1, 2): column panel = 32*vec*ch.
void choose_shape(int n_cols, bool aligned16, int *vec, int *ch);
// mode: 0 SpMM-SpMM, 1 GeMM-SpMM, 2 SDDMM-SpMM
int stream_occupancy(int mode, int vec, int ch, bool ring, size_t dyn_smem);
cudaError_t launch_stream(int mode, int vec, int ch, bool ring, int grid, size_t dyn_smem, const Params &p,
                          cudaStream_t s);
cudaError_t launch_schedule_level(int mode, int vec, int ch, int grid, const Params &p, const int *ptr2,
                                  const int *id, const int *type, const int *ker, int part_begin, int part_end,
                                  cudaStream_t s);
cudaError_t launch_spmm(int vec, int ch, int grid, const int *ap, const int *ai, const float *ax, int m,
                        const float *x, int n_cols, float *out, cudaStream_t s);
// gather-tile pipeline (one CTA per SM): plans whose items are all gather tiles
size_t tile_pipeline_smem(int tile_slots, int tile_rows);
cudaError_t launch_tile_pipeline(int grid, const Params &p, cudaStream_t s);
cudaError_t launch_rows_fix(const int *rows, int n_rows, int n_cols, float *x, bool relu, cudaStream_t s);
cudaError_t launch_fill(bool normal, float *p, long long n, unsigned long long seed, long long off, float sigma,
                        cudaStream_t s);
}  // namespace tfk
