// Plane-marching executor for chains of two lattice (star-stencil) operators: parameters and launcher.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfk {

constexpr int kMarchW = 16, kMarchH = 8;    // grid points of a tile in x and y
constexpr int kMarchCols = 16;              // dense columns per chunk (64 bytes per row)
constexpr int kMarchStages = 3;             // planes of C in flight per CTA (measured: 3 beats 4 and 5; 2 starves)
constexpr int kMarchThreads = 128;          // 4 warps: 32 patches of 2 x 2 grid points x 4 lanes of 4 columns
constexpr int kMarchCtasPerSm = 2;          // two independent CTAs per SM: one loads while the other computes
constexpr int kMarchCBytes = (kMarchW + 4) * (kMarchH + 4) * kMarchCols * 4;                          // 15 360
constexpr int kMarchTBytes = ((kMarchW + 2) * (kMarchH + 2) * kMarchCols * 4 + 1023) / 1024 * 1024;  // 12 288
constexpr int kMarchMaxClassesDev = 63;
constexpr size_t kMarchSmemBytes = (size_t)kMarchStages * kMarchCBytes + 2 * kMarchTBytes + (kMarchStages + 1) * 8 + 1024;

struct MarchState {
  int ticket;    // next item
  int finished;  // CTAs that left the item loop
  int error;     // sticky: a bounded wait ran out
  int pad;
};

struct MarchParams {
  const unsigned *pcls_f, *pcls_a;  // class words of the first / second operator, [nz][pny][pnx]
  int ncls_f, ncls_a;               // the class with this index is the all-zero vector
  float *out;                       // D, nx * ny * nz rows of n_cols
  const float *t_lo, *t_hi;         // planes -1 and nz of T received from the neighbour ranks (null: none)
  const int4 *items;                // {x0, y0, zs, ze}, {first column, flags, 0, 0}
  int item_begin, item_end;         // tickets run over the items [item_begin, item_end)
  MarchState *st;
  int nx, ny, nz, pnx, pny, n_cols;
  int z_shift;                      // plane of C (in the tensor map) that holds the operand rows of plane 0
  int wait_limit;
  int first_idle_sm;                // CTAs that land on an SM with this id or a higher one leave at once (see api.cu)
  // Coefficient dictionaries, (classes + 1) x 2 float4 each: {z-, y-, x-, centre}, {x+, y+, z+, 0}.  They travel
  // as kernel parameters, i.e. in the constant bank: the four lanes that share a row -- usually the whole warp --
  // read the same entry, which the constant cache serves as one broadcast, while a 16-byte load from shared
  // memory costs four wavefronts of that pipe whatever the lanes share.
  float4 dict_f[2 * (kMarchMaxClassesDev + 1)], dict_a[2 * (kMarchMaxClassesDev + 1)];
};

// Tensor map of C as a 5-D fp32 tensor (n_cols, nx / 2, 2, ny, planes), box = 16 columns x (W+4)/2 x 2 x (H+4) x 1.
int march_make_map(CUtensorMap *out, const float *c, int n_cols, int nx, int ny, long long planes);
int march_ctas_per_sm();
cudaError_t launch_lattice_march(int grid, const CUtensorMap &tm_c, const MarchParams &p, cudaStream_t s);

}  // namespace tfk
