// Plane-marching executor for SpMM-SpMM chains whose two operators are star stencils on a grid
// (lattice.cpp): D = A * (F * C), one launch, the intermediate T = F * C never leaves the SM.
//
// A work item is an x-y tile of 16 x 16 grid points, a range of planes [zs, ze) and a chunk of 16 dense
// columns.  The CTA marches along z.  Per step k one plane of C -- the tile grown by two points on every
// side, 20 x 20 row chunks of 64 bytes -- arrives in shared memory through one 5-D TMA box load
// (cp.async.bulk.tensor, zero fill outside the grid) that was issued four steps earlier.  The tensor map
// splits x into (x / 2, x % 2) and lists x / 2 first, so a plane lands as [y][x % 2][x / 2][16 floats]: two
// patches that are neighbours in x then read addresses exactly 64 bytes apart in every load, i.e. opposite
// halves of the 32 banks, and the 128-bit loads of a quarter-warp never conflict.  A thread owns a 2 x 2 patch of grid points and four dense columns (one float4 per row):
//   * it reads the patch's own rows and its eight in-plane neighbours of C(k) once (12 loads for 4 rows,
//     instead of 7 per row),
//   * adds the z+ product to the rows T(k-1) it has been accumulating, which completes them; they go to a
//     double-buffered plane of T in shared memory (for the neighbours) and stay in registers (for itself),
//   * completes and stores the rows D(k-2), and starts T(k) and -- after the step's one CTA barrier --
//     D(k-1) from the neighbours' T(k-1).
// Products are added in sorted-column order (z-, y-, x-, centre, x+, y+, z+) with fused multiply-adds
// from a zero accumulator, which is the order of the reference's row loop (SpMM_SpMM.cpp:211-248,
// SpMM_SpMM_vectorized.cpp:876), so results are bit-identical to the CSR executors; an absent neighbour has
// coefficient 0.  T is needed one point beyond the tile: four extra warps compute that border ring (2 x 1
// and 1 x 2 strips).  Coefficients come from the class of each row (one byte per row, a 32-bit word per
// patch) through a small dictionary in shared memory; a warp whose rows are all of class 0 (interior rows)
// uses registers instead.
//
// Every wait is bounded: a thread whose wait runs out raises the abort vote of the step's barrier, the CTA
// leaves the item loop together, waits (bounded) for its copies in flight, sets the error flag and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lattice_march.h"

namespace tfk {

namespace {

constexpr int W = kMarchW, H = kMarchH;
constexpr int PC = W + 4;  // pitch (rows) of the staged C rectangle
constexpr int PT = W + 2;  // pitch of the T rectangle
constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity, int limit) {
  const unsigned a = smem_u32(bar);
  for (int i = 0; i < limit; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(a), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// One plane of C for a tile: coordinates (column, x / 2, x % 2, y, plane).
__device__ __forceinline__ void tma_load_plane(void *smem, const CUtensorMap *tm, int col, int xh, int y, int z,
                                               unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem)), "l"((unsigned long long)tm), "r"(smem_u32(bar)), "r"(col), "r"(xh), "r"(0), "r"(y), "r"(z)
      : "memory");
}

// Rectangles of P x (rows) row chunks of 64 bytes are kept as [y][x % 2][x / 2][64 B]: byte offset of
// column rx inside a y-row.
template <int P>
__device__ __forceinline__ int xoff(int rx) { return (rx & 1) * (P / 2 * 64) + (rx >> 1) * 64; }

__device__ __forceinline__ float4 lds4(const char *buf, int off) { return *reinterpret_cast<const float4 *>(buf + off); }
__device__ __forceinline__ void sts4(char *buf, int off, const float4 &v) { *reinterpret_cast<float4 *>(buf + off) = v; }
__device__ __forceinline__ float4 fma4(float a, const float4 &x, const float4 &c) {
  return make_float4(fmaf(a, x.x, c.x), fmaf(a, x.y, c.y), fmaf(a, x.z, c.z), fmaf(a, x.w, c.w));
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

struct Coef {
  float zm, ym, xm, c0, xp, yp, zp;
};
__device__ __forceinline__ Coef coef_from(const float4 &a, const float4 &b) {
  return Coef{a.x, a.y, a.z, a.w, b.x, b.y, b.z};
}

// Own rows and in-plane neighbours of a PX x PY patch in a rectangle of pitch P.  xo[a + 1] = byte offset of
// the patch's column a (-1 .. PX) inside a y-row, lane's 16 bytes included; yo = byte offset of the patch's
// first y-row.  nb: [0, PY) left column, [PY, 2PY) right column, [2PY, 2PY+PX) row below, then the row above.
template <int PX, int PY, int P>
__device__ __forceinline__ void load_nb(const char *buf, const int (&xo)[PX + 2], int yo, float4 (&nb)[2 * PX + 2 * PY]) {
#pragma unroll
  for (int b = 0; b < PY; ++b) {
    nb[b] = lds4(buf, yo + b * (P * 64) + xo[0]);
    nb[PY + b] = lds4(buf, yo + b * (P * 64) + xo[PX + 1]);
  }
#pragma unroll
  for (int a = 0; a < PX; ++a) {
    nb[2 * PY + a] = lds4(buf, yo - P * 64 + xo[a + 1]);
    nb[2 * PY + PX + a] = lds4(buf, yo + PY * (P * 64) + xo[a + 1]);
  }
}
template <int PX, int PY, int P>
__device__ __forceinline__ void load_own(const char *buf, const int (&xo)[PX + 2], int yo, float4 (&own)[PX * PY]) {
#pragma unroll
  for (int b = 0; b < PY; ++b)
#pragma unroll
    for (int a = 0; a < PX; ++a) own[b * PX + a] = lds4(buf, yo + b * (P * 64) + xo[a + 1]);
}

// acc[j] = the first six products of row j in sorted-column order: z- (from `prev`, the same grid point
// one plane down), y-, x-, centre, x+, y+ (this plane).  The z+ product is added one step later.
template <int PX, int PY>
__device__ __forceinline__ void stencil_partial(float4 (&acc)[PX * PY], const float4 (&prev)[PX * PY],
                                                const float4 (&own)[PX * PY], const float4 (&nb)[2 * PX + 2 * PY],
                                                const Coef (&cf)[PX * PY]) {
#pragma unroll
  for (int b = 0; b < PY; ++b)
#pragma unroll
    for (int a = 0; a < PX; ++a) {
      const int j = b * PX + a;
      float4 s = fma4(cf[j].zm, prev[j], zero4());
      s = fma4(cf[j].ym, b > 0 ? own[j - PX] : nb[2 * PY + a], s);
      s = fma4(cf[j].xm, a > 0 ? own[j - 1] : nb[b], s);
      s = fma4(cf[j].c0, own[j], s);
      s = fma4(cf[j].xp, a < PX - 1 ? own[j + 1] : nb[PY + b], s);
      s = fma4(cf[j].yp, b < PY - 1 ? own[j + PX] : nb[2 * PY + PX + a], s);
      acc[j] = s;
    }
}

// Class word of the patch that holds grid point (x, y) of plane z: classes of (2px+dx, 2py+dy), byte
// 2*dy+dx.  Outside the grid every row is of the zero class.
__device__ __forceinline__ unsigned class_word(const unsigned *pcls, int x, int y, int z, int nx, int ny, int nz,
                                               int pnx, int pny, unsigned zero_word) {
  if (x < 0 || x >= nx || y < 0 || y >= ny || z < 0 || z >= nz) return zero_word;
  return __ldg(pcls + ((size_t)z * pny + (y >> 1)) * pnx + (x >> 1));
}

// Coefficients of the PX x PY rows of a patch at (x, y) from its class word.
template <int PX, int PY>
__device__ __forceinline__ void patch_coefs(Coef (&cf)[PX * PY], unsigned word, int x, int y, const float4 *dict,
                                            const Coef &c0) {
  if (__all_sync(kFullMask, word == 0u)) {
#pragma unroll
    for (int j = 0; j < PX * PY; ++j) cf[j] = c0;
    return;
  }
#pragma unroll
  for (int b = 0; b < PY; ++b)
#pragma unroll
    for (int a = 0; a < PX; ++a) {
      const int byte = 2 * ((y + b) & 1) + ((x + a) & 1);
      const unsigned c = (word >> (8 * byte)) & 255u;
      cf[b * PX + a] = coef_from(dict[2 * c], dict[2 * c + 1]);
    }
}

struct Shared {
  char *cbuf, *tbuf;
  float4 *dict_f, *dict_a;
  unsigned long long *full;
};

// The border ring of T: a PX x PY strip at (x, y), first-operator work only.
template <int PX, int PY>
__device__ __forceinline__ bool march_border(const MarchParams &P, const Shared &S, int x, int y, int x0, int y0,
                                             int kfirst, int steps, int c0col, int c4, unsigned &n_use,
                                             const Coef &cF0) {
  int xoC[PX + 2], xoT[PX + 2];
#pragma unroll
  for (int a = -1; a <= PX; ++a) {
    xoC[a + 1] = xoff<PC>(x - x0 + 2 + a) + c4 * 16;
    xoT[a + 1] = xoff<PT>(x - x0 + 1 + a) + c4 * 16;
  }
  const int yoC = (y - y0 + 2) * (PC * 64), yoT = (y - y0 + 1) * (PT * 64);
  const unsigned zero_f = 0x01010101u * (unsigned)P.ncls_f;
  float4 cprev[PX * PY], accT[PX * PY];
  float czp[PX * PY];
#pragma unroll
  for (int j = 0; j < PX * PY; ++j) { cprev[j] = zero4(); accT[j] = zero4(); czp[j] = 0.f; }
  unsigned wf = class_word(P.pcls_f, x, y, kfirst, P.nx, P.ny, P.nz, P.pnx, P.pny, zero_f);
  const int zs = kfirst + 2, ze = kfirst + steps - 2;
  for (int step = 0; step < steps; ++step, ++n_use) {
    const int k = kfirst + step;
    const unsigned stage = n_use % kMarchStages;
    const bool ok = mbar_wait(&S.full[stage], (n_use / kMarchStages) & 1u, P.wait_limit);
    const char *cb = S.cbuf + stage * kMarchCBytes;
    float4 own[PX * PY], nb[2 * PX + 2 * PY];
    load_own<PX, PY, PC>(cb, xoC, yoC, own);
    load_nb<PX, PY, PC>(cb, xoC, yoC, nb);
    const unsigned wf_next = class_word(P.pcls_f, x, y, k + 1, P.nx, P.ny, P.nz, P.pnx, P.pny, zero_f);
    char *tb = S.tbuf + ((k - 1) & 1) * kMarchTBytes;
    const float *halo = (k - 1 == -1) ? P.t_lo : ((k - 1 == P.nz) ? P.t_hi : nullptr);
#pragma unroll
    for (int b = 0; b < PY; ++b)
#pragma unroll
      for (int a = 0; a < PX; ++a) {
        const int j = b * PX + a;
        float4 t = fma4(czp[j], own[j], accT[j]);
        if (halo) {
          const int gx = x + a, gy = y + b, col = c0col + 4 * c4;
          t = zero4();
          if (gx >= 0 && gx < P.nx && gy >= 0 && gy < P.ny && col < P.n_cols)
            t = __ldg(reinterpret_cast<const float4 *>(halo + ((size_t)gy * P.nx + gx) * P.n_cols + col));
        }
        sts4(tb, yoT + b * (PT * 64) + xoT[a + 1], t);
      }
    if (k >= zs - 1 && k <= ze) {
      Coef cf[PX * PY];
      patch_coefs<PX, PY>(cf, wf, x, y, S.dict_f, cF0);
      stencil_partial<PX, PY>(accT, cprev, own, nb, cf);
#pragma unroll
      for (int j = 0; j < PX * PY; ++j) czp[j] = cf[j].zp;
    }
#pragma unroll
    for (int j = 0; j < PX * PY; ++j) cprev[j] = own[j];
    wf = wf_next;
    if (__syncthreads_or(!ok)) return false;
  }
  return true;
}

}  // namespace

__global__ void __launch_bounds__(kMarchThreads, 1)
lattice_march_kernel(const __grid_constant__ CUtensorMap tm_c, const MarchParams P) {
  extern __shared__ char dyn[];
  __shared__ int ctl[2];
  char *sm = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~(uintptr_t)1023);
  Shared S;
  S.cbuf = sm;
  S.tbuf = sm + kMarchStages * kMarchCBytes;
  S.dict_f = reinterpret_cast<float4 *>(S.tbuf + 2 * kMarchTBytes);
  S.dict_a = S.dict_f + 2 * (kMarchMaxClassesDev + 1);
  S.full = reinterpret_cast<unsigned long long *>(S.dict_a + 2 * (kMarchMaxClassesDev + 1));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i < 2 * (P.ncls_f + 1); i += kMarchThreads) S.dict_f[i] = __ldg(P.dict_f + i);
  for (int i = tid; i < 2 * (P.ncls_a + 1); i += kMarchThreads) S.dict_a[i] = __ldg(P.dict_a + i);
  if (tid == 0) {
    for (int s = 0; s < kMarchStages; ++s) mbar_init(&S.full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const Coef cF0 = coef_from(S.dict_f[0], S.dict_f[1]);
  const Coef cA0 = coef_from(S.dict_a[0], S.dict_a[1]);
  const unsigned zero_f = 0x01010101u * (unsigned)P.ncls_f, zero_a = 0x01010101u * (unsigned)P.ncls_a;

  // lane -> patch: four lanes (16 columns) per patch; the two patches of a quarter-warp are neighbours in x
  const int c4 = lane & 3;
  const int pi = lane >> 2;  // 0 .. 7

  unsigned n_use = 0;  // plane loads consumed by this CTA so far: stage = n_use % stages, parity from n_use / stages
  unsigned n_iss = 0;  // plane loads issued so far (kept by the main warps; thread 0 issues them)
  bool failed = false;
  for (;;) {
    if (tid == 0) ctl[0] = atomicAdd(&P.st->ticket, 1);
    __syncthreads();
    const int it = P.item_begin + ctl[0];
    if (it >= P.item_end) break;
    const int4 ia = __ldg(P.items + 2 * it), ib = __ldg(P.items + 2 * it + 1);
    const int x0 = ia.x, y0 = ia.y, zs = ia.z, ze = ia.w, c0col = ib.x;
    const int kfirst = zs - 2, steps = ze - zs + 4;
    if (tid == 0) {
      for (int s = 0; s < min(kMarchStages, steps); ++s) {
        const unsigned stage = (n_use + s) % kMarchStages;
        mbar_expect_tx(&S.full[stage], kMarchCBytes);
        tma_load_plane(S.cbuf + stage * kMarchCBytes, &tm_c, c0col, x0 / 2 - 1, y0 - 2, kfirst + s + P.z_shift, &S.full[stage]);
      }
    }
    n_iss = n_use + min(kMarchStages, steps);
    if (warp >= 8) {
      // border ring of T: warps 8, 9 the rows below / above the tile, warps 10, 11 the columns left / right
      bool ok;
      // (the two groups of a quarter-warp take the left and the right strip of the same rows: their addresses
      // differ by an odd multiple of 64 bytes in both rectangles)
      if (warp == 8) ok = march_border<2, 1>(P, S, x0 + 2 * pi, y0 - 1, x0, y0, kfirst, steps, c0col, c4, n_use, cF0);
      else if (warp == 9) ok = march_border<2, 1>(P, S, x0 + 2 * pi, y0 + H, x0, y0, kfirst, steps, c0col, c4, n_use, cF0);
      else ok = march_border<1, 2>(P, S, (pi & 1) ? x0 + W : x0 - 1, y0 + 2 * (4 * (warp - 10) + (pi >> 1)), x0, y0, kfirst,
                                   steps, c0col, c4, n_use, cF0);
      if (!ok) { failed = true; break; }
      continue;
    }

    // ---- main warps: 2 x 2 patches of the tile, both products ----
    const int x = x0 + 2 * pi, y = y0 + 2 * warp;
    int xoC[4], xoT[4];
#pragma unroll
    for (int a = -1; a <= 2; ++a) {
      xoC[a + 1] = xoff<PC>(x - x0 + 2 + a) + c4 * 16;
      xoT[a + 1] = xoff<PT>(x - x0 + 1 + a) + c4 * 16;
    }
    const int yoC = (y - y0 + 2) * (PC * 64), yoT = (y - y0 + 1) * (PT * 64);
    const int col = c0col + 4 * c4;
    const bool col_ok = col < P.n_cols;
    float4 cprev[4], accT[4], tprev[4], accD[4];
    float czpT[4], czpD[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      cprev[j] = zero4(); accT[j] = zero4(); tprev[j] = zero4(); accD[j] = zero4();
      czpT[j] = 0.f; czpD[j] = 0.f;
    }
    unsigned wf = class_word(P.pcls_f, x, y, kfirst, P.nx, P.ny, P.nz, P.pnx, P.pny, zero_f);
    unsigned wa = zero_a;  // classes of the second operator's rows of plane k - 1
    bool ok_all = true;
    for (int step = 0; step < steps; ++step, ++n_use) {
      const int k = kfirst + step;
      const unsigned stage = n_use % kMarchStages;
      const bool ok = mbar_wait(&S.full[stage], (n_use / kMarchStages) & 1u, P.wait_limit);
      const char *cb = S.cbuf + stage * kMarchCBytes;
      float4 own[4], tcur[4];
      {
        float4 nb[8];
        load_own<2, 2, PC>(cb, xoC, yoC, own);
        load_nb<2, 2, PC>(cb, xoC, yoC, nb);
        const unsigned wf_next = class_word(P.pcls_f, x, y, k + 1, P.nx, P.ny, P.nz, P.pnx, P.pny, zero_f);
        const unsigned wa_next = class_word(P.pcls_a, x, y, k, P.nx, P.ny, P.nz, P.pnx, P.pny, zero_a);
        // T(k-1) is complete with its z+ product
        char *tb = S.tbuf + ((k - 1) & 1) * kMarchTBytes;
        const float *halo = (k - 1 == -1) ? P.t_lo : ((k - 1 == P.nz) ? P.t_hi : nullptr);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tcur[j] = fma4(czpT[j], own[j], accT[j]);
          if (halo) {
            const int gx = x + (j & 1), gy = y + (j >> 1);
            tcur[j] = zero4();
            if (gx < P.nx && gy < P.ny && col_ok)
              tcur[j] = __ldg(reinterpret_cast<const float4 *>(halo + ((size_t)gy * P.nx + gx) * P.n_cols + col));
          }
          sts4(tb, yoT + (j >> 1) * (PT * 64) + xoT[(j & 1) + 1], tcur[j]);
        }
        // D(k-2) is complete with its z+ product
        if (k - 2 >= zs && k - 2 < ze) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 d = fma4(czpD[j], tcur[j], accD[j]);
            const int gx = x + (j & 1), gy = y + (j >> 1);
            if (gx < P.nx && gy < P.ny && col_ok)
              *reinterpret_cast<float4 *>(P.out + (((size_t)(k - 2) * P.ny + gy) * P.nx + gx) * P.n_cols + col) = d;
          }
        }
        // T(k): everything but the z+ product
        if (k >= zs - 1 && k <= ze) {
          Coef cf[4];
          patch_coefs<2, 2>(cf, wf, x, y, S.dict_f, cF0);
          stencil_partial<2, 2>(accT, cprev, own, nb, cf);
#pragma unroll
          for (int j = 0; j < 4; ++j) czpT[j] = cf[j].zp;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) cprev[j] = own[j];
        wf = wf_next;
        // wa still holds the classes of plane k - 1 for the D(k-1) start below; wa_next those of plane k
        if (__syncthreads_or(!ok)) { ok_all = false; break; }
        if (step + kMarchStages < steps) {
          ++n_iss;
          if (tid == 0) {
            mbar_expect_tx(&S.full[stage], kMarchCBytes);
            tma_load_plane(S.cbuf + stage * kMarchCBytes, &tm_c, c0col, x0 / 2 - 1, y0 - 2, k + kMarchStages + P.z_shift, &S.full[stage]);
          }
        }
        // D(k-1): everything but the z+ product, from T(k-2) (registers), T(k-1) (registers and neighbours)
        if (k - 1 >= zs && k - 1 < ze) {
          float4 tn[8];
          load_nb<2, 2, PT>(tb, xoT, yoT, tn);
          Coef ca[4];
          patch_coefs<2, 2>(ca, wa, x, y, S.dict_a, cA0);
          stencil_partial<2, 2>(accD, tprev, tcur, tn, ca);
#pragma unroll
          for (int j = 0; j < 4; ++j) czpD[j] = ca[j].zp;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) tprev[j] = tcur[j];
        wa = wa_next;
      }
    }
    if (!ok_all) { failed = true; break; }
  }
  if (failed) {
    // Leave together: every thread of the CTA saw the same abort vote.  Copies still in flight must land
    // before the shared memory is given up; thread 0 waits for each stage it armed, again with a limit.
    if (tid == 0) {
      atomicExch(&P.st->error, 1);
      for (unsigned q = n_use; q != n_iss; ++q)
        mbar_wait(&S.full[q % kMarchStages], (q / kMarchStages) & 1u, P.wait_limit);
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int f = atomicAdd(&P.st->finished, 1);
    if (f == (int)gridDim.x - 1) {
      P.st->ticket = 0;
      P.st->finished = 0;
      __threadfence();
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int march_make_map(CUtensorMap *out, const float *c, int n_cols, int nx, int ny, long long planes) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  if (!fn) return -1;
  // (column, x / 2, x % 2, y, plane): nx is even, so row x = 2 * (x / 2) + x % 2 of a y-line
  const cuuint64_t row = (cuuint64_t)n_cols * 4;
  cuuint64_t gdim[5] = {(cuuint64_t)n_cols, (cuuint64_t)(nx / 2), 2, (cuuint64_t)ny, (cuuint64_t)planes};
  cuuint64_t gstride[4] = {2 * row, row, row * nx, row * nx * ny};
  cuuint32_t box[5] = {(cuuint32_t)kMarchCols, (cuuint32_t)((kMarchW + 4) / 2), 2, (cuuint32_t)(kMarchH + 4), 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(c), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

cudaError_t launch_lattice_march(int grid, const CUtensorMap &tm_c, const MarchParams &p, cudaStream_t s) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute((const void *)lattice_march_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kMarchSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  lattice_march_kernel<<<grid, kMarchThreads, kMarchSmemBytes, s>>>(tm_c, p);
  return cudaGetLastError();
}

}  // namespace tfk
