// Plane-marching executor for SpMM-SpMM chains whose two operators are star stencils on a grid
// (lattice.cpp): D = A * (F * C), one launch, the intermediate T = F * C never leaves the SM.
//
// A work item is an x-y tile of 16 x 8 grid points, a range of planes [zs, ze) and a chunk of 16 dense
// columns.  The CTA (four warps; two CTAs per SM, so one loads while the other computes) marches along z.
// Per step k one plane of C -- the tile grown by two points on every side, 20 x 12 row chunks of 64 bytes --
// arrives in shared memory through one 5-D TMA box load (cp.async.bulk.tensor, zero fill outside the grid)
// that was issued two steps earlier; the copies run on into the CTA's next item.  The tensor map splits x
// into (x / 2, x % 2) and lists x / 2 first, so a plane lands as [y][x % 2][x / 2][16 floats]: two patches
// that are neighbours in x then read addresses exactly 64 bytes apart in every load, i.e. opposite halves of
// the 32 banks, and the 128-bit loads of a quarter-warp never conflict.  A thread owns a 2 x 2 patch of grid
// points and four dense columns (one float4 per row):
//   * it reads the patch's own rows and its eight in-plane neighbours of C(k) once (12 loads for 4 rows,
//     instead of 7 per row),
//   * adds the z+ product to the rows T(k-1) it has been accumulating, which completes them; they go to a
//     double-buffered plane of T in shared memory (for the neighbours) and stay in registers (for itself),
//   * completes and stores the rows D(k-2), and starts T(k) and -- after the step's one CTA barrier --
//     D(k-1) from the neighbours' T(k-1).
// Products are added in sorted-column order (z-, y-, x-, centre, x+, y+, z+) with fused multiply-adds
// from a zero accumulator, which is the order of the reference's row loop (SpMM_SpMM.cpp:211-248,
// SpMM_SpMM_vectorized.cpp:876), so results are bit-identical to the CSR executors; an absent neighbour has
// coefficient 0.  T is needed one point beyond the tile: three of the four warps also compute two rows each of
// that border ring per 4-lane group.  Coefficients come from the class of each row (one byte per row, a 32-bit
// word per patch) through a small dictionary that travels in the kernel's parameters: the constant cache serves
// the lanes that share an entry in one broadcast, where a 16-byte load from shared memory costs four
// wavefronts of the pipe that is this kernel's busiest.
//
// Every wait is bounded: a thread whose wait runs out raises the CTA's abort flag, the CTA leaves the item
// loop together, waits (bounded) for its copies in flight, sets the error flag and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "lattice_march.h"

namespace tfk {

namespace {

constexpr int W = kMarchW, H = kMarchH;
constexpr int PC = W + 4;  // pitch (rows) of the staged C rectangle
constexpr int PT = W + 2;  // pitch of the T rectangle

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned a, unsigned parity, int limit) {
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
__device__ __forceinline__ void tma_load_plane(unsigned smem, const CUtensorMap *tm, int col, int xh, int y, int z,
                                               unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem), "l"((unsigned long long)tm), "r"(bar), "r"(col), "r"(xh), "r"(0), "r"(y), "r"(z)
      : "memory");
}

// Rectangles of P x (rows) row chunks of 64 bytes are kept as [y][x % 2][x / 2][64 B]: byte offset of
// column rx inside a y-row.
template <int P>
__device__ __forceinline__ int xoff(int rx) { return (rx & 1) * (P / 2 * 64) + (rx >> 1) * 64; }

// Shared memory is addressed by 32-bit shared-window addresses throughout (ld.shared / st.shared).
__device__ __forceinline__ float4 lds4(unsigned buf, int off) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(buf + off) : "memory");
  return v;
}
// The same with a compile-time byte offset in the instruction's address field.
template <int OFF>
__device__ __forceinline__ float4 lds4i(unsigned addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ void sts4i(unsigned addr, const float4 &v) {
  asm volatile("st.shared.v4.f32 [%0+%1], {%2, %3, %4, %5};" ::"r"(addr), "n"(OFF), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void sts4(unsigned buf, int off, const float4 &v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(buf + off), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 fma4(float a, const float4 &x, const float4 &c) {
  return make_float4(fmaf(a, x.x, c.x), fmaf(a, x.y, c.y), fmaf(a, x.z, c.z), fmaf(a, x.w, c.w));
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// In-plane neighbours of a 2 x 2 patch in a rectangle of pitch P.  xo[a + 1] = byte offset of the patch's
// column a (-1 .. 2) inside a y-row, lane's 16 bytes included; yo = byte offset of the patch's first y-row.
// nb: [0, 2) left column, [2, 4) right column, [4, 6) row below, [6, 8) row above.
// A patch starts at an even x of its tile (x - x0 = 2 * pi), so in a rectangle of pitch P whose column 0 holds
// x0 - R0 the patch's columns a = -1 .. 2 sit at fixed byte distances co<P, R0>(a) from `base` = the address of
// (column of x0 - R0 + 2 * pi ... i.e. pi * 64 bytes into the row, lane's 16 bytes included) of the patch's first
// y-row: one register addresses all twelve loads of a patch.
template <int P, int R0>
__host__ __device__ constexpr int co(int a) { return ((R0 + a) & 1) * (P / 2 * 64) + ((R0 + a) >> 1) * 64; }

// nb: [0, 2) left column, [2, 4) right column, [4, 6) row below, [6, 8) row above.
template <int P, int R0>
__device__ __forceinline__ void load_nb(unsigned base, float4 (&nb)[8]) {
  nb[0] = lds4i<co<P, R0>(-1)>(base);             nb[1] = lds4i<co<P, R0>(-1) + P * 64>(base);
  nb[2] = lds4i<co<P, R0>(2)>(base);              nb[3] = lds4i<co<P, R0>(2) + P * 64>(base);
  nb[4] = lds4i<co<P, R0>(0) - P * 64>(base);     nb[5] = lds4i<co<P, R0>(1) - P * 64>(base);
  nb[6] = lds4i<co<P, R0>(0) + 2 * P * 64>(base); nb[7] = lds4i<co<P, R0>(1) + 2 * P * 64>(base);
}
template <int P, int R0>
__device__ __forceinline__ void load_own(unsigned base, float4 (&own)[4]) {
  own[0] = lds4i<co<P, R0>(0)>(base);          own[1] = lds4i<co<P, R0>(1)>(base);
  own[2] = lds4i<co<P, R0>(0) + P * 64>(base); own[3] = lds4i<co<P, R0>(1) + P * 64>(base);
}

// Starts one row: acc = its first six products in sorted-column order -- z- (from `zm`, the same grid point one
// plane down), y-, x-, centre, x+, y+ (this plane); the z+ product is added one step later with the returned
// coefficient.  The coefficients are entry `cls` of a dictionary in the kernel's parameters (two 16-byte loads that
// the lanes of a warp mostly share).
__device__ __forceinline__ float row_start(float4 &acc, const float4 (&dict)[2 * (kMarchMaxClassesDev + 1)], unsigned cls,
                                           const float4 &zm, const float4 &ym, const float4 &xm, const float4 &c,
                                           const float4 &xp, const float4 &yp) {
  const float4 lo = dict[2 * cls], hi = dict[2 * cls + 1];
  float4 s = fma4(lo.x, zm, zero4());
  s = fma4(lo.y, ym, s);
  s = fma4(lo.z, xm, s);
  s = fma4(lo.w, c, s);
  s = fma4(hi.x, xp, s);
  acc = fma4(hi.y, yp, s);
  return hi.z;
}
// The four rows of a 2 x 2 patch; class of row j = byte j of `word`.
__device__ __forceinline__ void patch_start(float4 (&acc)[4], float (&czp)[4],
                                            const float4 (&dict)[2 * (kMarchMaxClassesDev + 1)], unsigned word,
                                            const float4 (&prev)[4], const float4 (&own)[4], const float4 (&nb)[8]) {
  czp[0] = row_start(acc[0], dict, word & 255u, prev[0], nb[4], nb[0], own[0], own[1], own[2]);
  czp[1] = row_start(acc[1], dict, (word >> 8) & 255u, prev[1], nb[5], own[0], own[1], nb[2], own[3]);
  czp[2] = row_start(acc[2], dict, (word >> 16) & 255u, prev[2], own[0], nb[1], own[2], own[3], nb[6]);
  czp[3] = row_start(acc[3], dict, word >> 24, prev[3], own[1], own[2], own[3], nb[3], nb[7]);
}

// Class words of one patch column: the word of plane z, or the all-zero class outside the grid.  Only the
// column's pointer is per thread; the plane pitch, the plane count and the all-zero word are the same for every
// column and come from the kernel's parameters.
struct ClassColumn {
  const unsigned *p;  // word of plane 0; null outside the grid
  __device__ __forceinline__ void init(const unsigned *pcls, int x, int y, int nx, int ny, int pnx) {
    p = (x >= 0 && x < nx && y >= 0 && y < ny) ? pcls + ((y >> 1) * pnx + (x >> 1)) : nullptr;
  }
  __device__ __forceinline__ unsigned at(int z, int nz, int plane_words, unsigned zero_word) const {
    return (p != nullptr && (unsigned)z < (unsigned)nz) ? __ldg(p + (size_t)z * plane_words) : zero_word;
  }
};

// 32-bit shared-window addresses of the CTA's buffers.
struct Shared {
  unsigned cbuf, tbuf;       // C stages, the two planes of T
  unsigned full;             // mbarriers, 8 bytes each: one per C stage (the plane has landed)
  unsigned tbar;             // one phase per step: every warp has stored its rows of T(k-1) (and read C(k))
  volatile int *abort;
};

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait that also gives up when another thread of the CTA already has.
__device__ __forceinline__ bool wait_or_abort(unsigned a, unsigned parity, int limit, volatile int *abort) {
  {
    unsigned done;   // the usual case: one try, no counters
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(a), "r"(parity) : "memory");
    if (done) return true;
  }
  for (int i = 0; i < limit; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(a), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255) == 255 && *abort) break;
  }
  *abort = 1;
  return false;
}

// One row of T(k-1) from the neighbour rank's plane (k-1 lies outside this rank's planes).
__device__ __forceinline__ float4 halo_row(const float *halo, int gx, int gy, int col, const MarchParams &P) {
  if (gx >= 0 && gx < P.nx && gy >= 0 && gy < P.ny && col < P.n_cols)
    return __ldg(reinterpret_cast<const float4 *>(halo + ((size_t)gy * P.nx + gx) * P.n_cols + col));
  return zero4();
}

// Planes of lead-in in front of the first output plane zs of an item: C(zs-2) and C(zs-1) enter T(zs-1) and
// T(zs).  Below plane 0 of a grid without a neighbour rank there is nothing -- C(-1), T(-1) are the zeros the
// registers start with -- so such an item starts at plane 0.
__device__ __forceinline__ int lead_in(int zs, const MarchParams &P) {
  return (zs == 0 && P.z_shift == 0 && P.t_lo == nullptr) ? 0 : 2;
}

// State a CTA carries from item to item.
struct CtaState {
  unsigned n_use;  // steps taken so far: step n uses C stage n % stages (parity of n / stages) and phase n of tbar
  unsigned n_iss;  // plane loads issued so far (kept by thread 0, which issues them)
};

// Rows of the ring of T around the tile that one 4-lane group computes besides its patch.
constexpr int kRing = 2;
static_assert(W == 16 && H == 8 && kMarchThreads == 128 && kMarchCols == 16,
              "the assignment of patches and ring rows to warps is written for 16 x 8 tiles of 16 columns and four warps");

// One work item, seen by one thread: its 2 x 2 patch of the tile at (x, y) (both products) and kRing single
// rows of the ring of T around the tile at (rx[r], ry[r]) (first product only; `ring` = this warp has any).
__device__ __forceinline__ bool run_item(const CUtensorMap *tm_c, const MarchParams &P, const Shared &S, CtaState &cs,
                                         int x0, int y0, int zs, int ze, int c0col, int x, int y, bool ring,
                                         const int (&rx)[kRing], const int (&ry)[kRing], bool pair_x,
                                         const volatile int *next, int &prefetched) {
  const int tid = threadIdx.x, lane = tid & 31, c4 = lane & 3;
  const int kfirst = zs - lead_in(zs, P), steps = ze - kfirst + 2;
  // byte offset of the patch's first y-row (at pi * 64 bytes into it, lane's 16 bytes included) in the C rectangle
  // (two points of rim: R0 = 2) and in the T rectangle (one point: R0 = 1)
  const int pi64 = (x - x0) * 32 + c4 * 16;
  const int boC = (y - y0 + 2) * (PC * 64) + pi64, boT = (y - y0 + 1) * (PT * 64) + pi64;
  // The group's two ring rows are neighbours (in x below / above the tile, in y beside it) and lie in one 2 x 2 class
  // patch.  Offsets of the first row, of its left neighbour and of the right neighbour (of the second row when
  // the pair lies along x) in the C rectangle, of the first row in the T rectangle; the second row's follow by
  // constants.
  const int ybr = (ry[0] - y0 + 2) * (PC * 64) + c4 * 16;
  const int rC = ybr + xoff<PC>(rx[0] - x0 + 2), rL = ybr + xoff<PC>(rx[0] - x0 + 1);
  const int rR = ybr + xoff<PC>(rx[0] - x0 + (pair_x ? 4 : 3));
  const int rT = (ry[0] - y0 + 1) * (PT * 64) + xoff<PT>(rx[0] - x0 + 1) + c4 * 16;
  const unsigned rsh0 = 8u * (2u * (ry[0] & 1) + (rx[0] & 1));  // bit position of the first row's class in the class word
  ClassColumn cr_col;
  cr_col.init(P.pcls_f, rx[0], ry[0], P.nx, P.ny, P.pnx);
  // second row: distances in the C rectangle, in the T rectangle and in the class word
  constexpr int kX1C = PC / 2 * 64, kY1C = PC * 64;       // x + 1 from an even column / y + 1
  constexpr int kX1T = 64 - PT / 2 * 64, kY1T = PT * 64;  // x + 1 from an odd column / y + 1
  const int col = c0col + 4 * c4;
  // rows of the patch that exist and whose columns exist: bit j
  unsigned live = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (x + (j & 1) < P.nx && y + (j >> 1) < P.ny && col < P.n_cols) live |= 1u << j;
  // D row (x, y) of plane k - 2 at step k; rows of the patch are n_cols and nx * n_cols floats further
  const size_t plane_floats = (size_t)P.nx * P.ny * P.n_cols;
  float *dptr = P.out + ((size_t)y * P.nx + x) * P.n_cols + col + (long long)(kfirst - 2) * (long long)plane_floats;
  const size_t drow = (size_t)P.nx * P.n_cols;
  ClassColumn cf_col, ca_col;
  cf_col.init(P.pcls_f, x, y, P.nx, P.ny, P.pnx);
  ca_col.init(P.pcls_a, x, y, P.nx, P.ny, P.pnx);
  const int plane_words = P.pnx * P.pny;
  const unsigned zero_f = 0x01010101u * (unsigned)P.ncls_f, zero_a = 0x01010101u * (unsigned)P.ncls_a;
  // The rows of T and D under way and the z+ coefficients they still need.  The own rows of C(k-1) / C(k), of
  // T(k-2) / T(k-1), the ring's own rows and the class words live in two sets of registers: set A is what the step
  // before left, set B what this step writes.
  float4 cA[4], cB[4], tA[4], tB[4], accT[4], accD[4], rA[kRing], rB[kRing], accR[kRing];
  float czpT[4], czpD[4], czpR[kRing];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    cA[j] = zero4(); tA[j] = zero4(); accT[j] = zero4(); accD[j] = zero4();
    czpT[j] = 0.f; czpD[j] = 0.f;
  }
#pragma unroll
  for (int r = 0; r < kRing; ++r) { rA[r] = zero4(); accR[r] = zero4(); czpR[r] = 0.f; }
  unsigned wrA = ring ? cr_col.at(kfirst, P.nz, plane_words, zero_f) : 0u, wrB;
  unsigned wfA = cf_col.at(kfirst, P.nz, plane_words, zero_f), wfB;
  unsigned waA = zero_a, waB;  // classes of the second operator's rows of plane k - 1

  // One step: plane C(k) arrives.  (cprev, tprev, rprev, wf, wa, wr) were written by the step before;
  // (own, tcur, rown, wf_next, wa_next, wr_next) are written here.
  auto one_step = [&](int step, float4 (&cprev)[4], float4 (&own)[4], float4 (&tprev)[4], float4 (&tcur)[4],
                      float4 (&rprev)[kRing], float4 (&rown)[kRing], unsigned wf, unsigned &wf_next, unsigned wa,
                      unsigned &wa_next, unsigned wr, unsigned &wr_next) -> bool {
    const int k = kfirst + step;
    const unsigned stage = cs.n_use % kMarchStages;
    if (!wait_or_abort(S.full + 8 * stage, (cs.n_use / kMarchStages) & 1u, P.wait_limit, S.abort)) return false;
    const unsigned cb = S.cbuf + stage * kMarchCBytes;
    float4 nb[8];
    const unsigned baseC = cb + boC;
    load_own<PC, 2>(baseC, own);
    load_nb<PC, 2>(baseC, nb);
    if (ring) {
      rown[0] = lds4(cb, rC);
      rown[1] = pair_x ? lds4i<kX1C>(cb + rC) : lds4i<kY1C>(cb + rC);
    }
    // T(k-1) is complete with its z+ product
    const unsigned tb = S.tbuf + ((k - 1) & 1) * kMarchTBytes;
    const float *halo = (k - 1 == -1) ? P.t_lo : ((k - 1 == P.nz) ? P.t_hi : nullptr);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tcur[j] = fma4(czpT[j], own[j], accT[j]);
      if (halo) tcur[j] = halo_row(halo, x + (j & 1), y + (j >> 1), col, P);
    }
    const unsigned baseT = tb + boT;
    // (the buffer of T(k-1) was last read in step k-2; this thread has waited for every warp's arrival of
    // step k-1, which each warp gives after its reads of step k-2)
    sts4i<co<PT, 1>(0)>(baseT, tcur[0]);           sts4i<co<PT, 1>(1)>(baseT, tcur[1]);
    sts4i<co<PT, 1>(0) + PT * 64>(baseT, tcur[2]); sts4i<co<PT, 1>(1) + PT * 64>(baseT, tcur[3]);
    if (ring) {
      float4 t0 = fma4(czpR[0], rown[0], accR[0]), t1 = fma4(czpR[1], rown[1], accR[1]);
      if (halo) { t0 = halo_row(halo, rx[0], ry[0], col, P); t1 = halo_row(halo, rx[1], ry[1], col, P); }
      sts4(tb, rT, t0);
      if (pair_x) sts4i<kX1T>(tb + rT, t1); else sts4i<kY1T>(tb + rT, t1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(S.tbar);
    // The class words of the next step are fetched only now: the arrive above is a release, which waits
    // for every load the thread has in flight, and a load from global memory can take a microsecond.
    wf_next = cf_col.at(k + 1, P.nz, plane_words, zero_f);
    wa_next = ca_col.at(k, P.nz, plane_words, zero_a);
    wr_next = ring ? cr_col.at(k + 1, P.nz, plane_words, zero_f) : 0u;
    // D(k-2) is complete with its z+ product
    if (k - 2 >= zs && k - 2 < ze) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 d = fma4(czpD[j], tcur[j], accD[j]);
        if (live >> j & 1u) *reinterpret_cast<float4 *>(dptr + (j & 1) * (size_t)P.n_cols + (j >> 1) * drow) = d;
      }
    }
    // T(k): everything but the z+ product
    if (k >= zs - 1 && k <= ze) {
      patch_start(accT, czpT, P.dict_f, wf, cprev, own, nb);
      if (ring) {
        // (the ring rows' neighbours are read only now, when the patch's are no longer needed; the stage is
        // refilled one step later, see below)
        const unsigned cls0 = (wr >> rsh0) & 255u;
        if (pair_x) {
          // the group's two ring rows are neighbours in x: each is the other's x- / x+ row
          const unsigned cls1 = (wr >> (rsh0 + 8u)) & 255u;
          const float4 ym0 = lds4i<-PC * 64>(cb + rC), xm0 = lds4(cb, rL), yp0 = lds4i<PC * 64>(cb + rC);
          czpR[0] = row_start(accR[0], P.dict_f, cls0, rprev[0], ym0, xm0, rown[0], rown[1], yp0);
          const float4 ym1 = lds4i<kX1C - PC * 64>(cb + rC), xp1 = lds4(cb, rR), yp1 = lds4i<kX1C + PC * 64>(cb + rC);
          czpR[1] = row_start(accR[1], P.dict_f, cls1, rprev[1], ym1, rown[0], rown[1], xp1, yp1);
        } else {
          // ... neighbours in y: each is the other's y- / y+ row
          const unsigned cls1 = (wr >> (rsh0 + 16u)) & 255u;
          const float4 ym0 = lds4i<-PC * 64>(cb + rC), xm0 = lds4(cb, rL), xp0 = lds4(cb, rR);
          czpR[0] = row_start(accR[0], P.dict_f, cls0, rprev[0], ym0, xm0, rown[0], xp0, rown[1]);
          const float4 xm1 = lds4i<kY1C>(cb + rL), xp1 = lds4i<kY1C>(cb + rR), yp1 = lds4i<2 * PC * 64>(cb + rC);
          czpR[1] = row_start(accR[1], P.dict_f, cls1, rprev[1], rown[0], xm1, rown[1], xp1, yp1);
        }
      }
    }
    // every warp has stored its rows of T(k-1) and is done with the plane C(k)
    if (!wait_or_abort(S.tbar, cs.n_use & 1u, P.wait_limit, S.abort)) return false;
    // Every warp has therefore finished step k-1, ring rows included (those read their plane after the
    // arrive): the stage of plane k-1 can take plane k-1 + stages.
    // When this item has no such plane left, the stage takes a plane of the CTA's next item (thread 0 knows
    // it: next[] = {valid, x0, y0, first plane, first column}), so the stream of copies does not stop between
    // items.
    if (step > 0 && tid == 0) {
      const unsigned prev_stage = (cs.n_use - 1) % kMarchStages;
      const int ahead = step - 1 + kMarchStages;
      if (ahead < steps) {
        ++cs.n_iss;
        mbar_expect_tx(S.full + 8 * prev_stage, kMarchCBytes);
        tma_load_plane(S.cbuf + prev_stage * kMarchCBytes, tm_c, c0col, x0 / 2 - 1, y0 - 2, kfirst + ahead + P.z_shift,
                       S.full + 8 * prev_stage);
      } else if (steps >= kMarchStages && next[0]) {   // (a shorter item left stages unarmed: no hand-over)
        ++cs.n_iss;
        ++prefetched;
        mbar_expect_tx(S.full + 8 * prev_stage, kMarchCBytes);
        tma_load_plane(S.cbuf + prev_stage * kMarchCBytes, tm_c, next[4], next[1] / 2 - 1, next[2] - 2,
                       next[3] + (ahead - steps) + P.z_shift, S.full + 8 * prev_stage);
      }
    }
    // D(k-1): everything but the z+ product, from T(k-2) (registers), T(k-1) (registers and neighbours)
    if (k - 1 >= zs && k - 1 < ze) {
      float4 tn[8];
      load_nb<PT, 1>(baseT, tn);
      patch_start(accD, czpD, P.dict_a, wa, tprev, tcur, tn);
    }
    ++cs.n_use;
    dptr += plane_floats;
    return true;
  };

  // (Taking two steps per turn with the register sets swapped would save these copies, but the loop body then no
  // longer fits the instruction cache as well: measured 5 % slower.)
  for (int step = 0; step < steps; ++step) {
    if (!one_step(step, cA, cB, tA, tB, rA, rB, wfA, wfB, waA, waB, wrA, wrB)) return false;
#pragma unroll
    for (int j = 0; j < 4; ++j) { cA[j] = cB[j]; tA[j] = tB[j]; }
#pragma unroll
    for (int r = 0; r < kRing; ++r) rA[r] = rB[r];
    wfA = wfB; waA = waB; wrA = wrB;
  }
  return true;
}

}  // namespace

__global__ void __launch_bounds__(kMarchThreads, kMarchCtasPerSm)
lattice_march_kernel(const __grid_constant__ CUtensorMap tm_c, const MarchParams P) {
  extern __shared__ char dyn[];
  __shared__ int ctl[2];
  __shared__ int nxt[5];
  Shared S;
  S.cbuf = (smem_u32(dyn) + 1023u) & ~1023u;
  S.tbuf = S.cbuf + kMarchStages * kMarchCBytes;
  S.full = S.tbuf + 2 * kMarchTBytes;
  S.tbar = S.full + 8 * kMarchStages;
  S.abort = &ctl[1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kMarchStages; ++s) mbar_init(S.full + 8 * s, 1);
    mbar_init(S.tbar, kMarchThreads / 32);
    ctl[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // lane -> patch: four lanes (16 columns) per patch; the two patches of a quarter-warp are neighbours in x.
  // Warp w owns the patches of the tile's rows 2w, 2w + 1.
  const int pi = lane >> 2;  // 0 .. 7
  // Ring rows of the group, relative to the tile origin.  In every load the two groups of a quarter-warp must
  // read addresses an odd multiple of 64 bytes apart: two columns apart below / above the tile, the left and
  // the right row of one y otherwise.
  int rdx[kRing], rdy[kRing];
  bool ring = true;
  // 48 rows, two per group of warps 0-2: below, above, left / right
#pragma unroll
  for (int r = 0; r < kRing; ++r) {
    if (warp < 2) { rdx[r] = 2 * pi + r; rdy[r] = warp == 0 ? -1 : H; }
    else { rdx[r] = (pi & 1) ? W : -1; rdy[r] = 2 * (pi >> 1) + r; }
  }
  ring = warp < 3;

  // SMs kept free for another kernel (the halo exchange of a multi-GPU step): the grid covers every SM, and the
  // CTAs that find themselves on one of the last SMs take no item.  A smaller grid would not do: the hardware
  // spreads a grid over all SMs before it doubles up, so no SM would stay empty.
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  const bool idle = (int)smid >= P.first_idle_sm;

  CtaState cs{0u, 0u};
  bool failed = false;
  // Thread 0 holds the ticket of the item after the current one and keeps that item's origin in shared memory:
  // the last steps of an item already fetch the first planes of the next (`pre` of them).
  int ticket_next = 0, pre = 0;
  if (tid == 0 && !idle) ticket_next = atomicAdd(&P.st->ticket, 1);
  for (; !idle;) {
    if (tid == 0) {
      ctl[0] = ticket_next;
      if (P.item_begin + ticket_next < P.item_end) {
        ticket_next = atomicAdd(&P.st->ticket, 1);
        const int nit = P.item_begin + ticket_next;
        nxt[0] = nit < P.item_end;
        if (nit < P.item_end) {
          const int4 na = __ldg(P.items + 2 * nit), nb = __ldg(P.items + 2 * nit + 1);
          nxt[1] = na.x; nxt[2] = na.y; nxt[3] = na.z - lead_in(na.z, P); nxt[4] = nb.x;
        }
      } else {
        nxt[0] = 0;
      }
    }
    __syncthreads();
    const int it = P.item_begin + ctl[0];
    if (it >= P.item_end || ctl[1]) break;
    const int4 ia = __ldg(P.items + 2 * it), ib = __ldg(P.items + 2 * it + 1);
    const int x0 = ia.x, y0 = ia.y, zs = ia.z, ze = ia.w, c0col = ib.x;
    const int kfirst = zs - lead_in(zs, P), steps = ze - kfirst + 2;
    if (tid == 0) {
      for (int s = pre; s < min(kMarchStages, steps); ++s) {
        const unsigned stage = (cs.n_use + s) % kMarchStages;
        mbar_expect_tx(S.full + 8 * stage, kMarchCBytes);
        tma_load_plane(S.cbuf + stage * kMarchCBytes, &tm_c, c0col, x0 / 2 - 1, y0 - 2, kfirst + s + P.z_shift, S.full + 8 * stage);
      }
      cs.n_iss = cs.n_use + min(kMarchStages, steps);
      pre = 0;
    }
    int rx[kRing], ry[kRing];
#pragma unroll
    for (int r = 0; r < kRing; ++r) { rx[r] = x0 + rdx[r]; ry[r] = y0 + rdy[r]; }
    if (!run_item(&tm_c, P, S, cs, x0, y0, zs, ze, c0col, x0 + 2 * pi, y0 + 2 * warp, ring, rx, ry, warp < 2, nxt, pre)) { failed = true; break; }
  }
  if (failed && tid == 0) atomicExch(&P.st->error, 1);
  // A thread that gave up has raised the CTA's abort flag; the others notice it in their own bounded waits
  // and arrive here too.  Copies still in flight must land before the shared memory is given up: thread 0
  // waits for each stage it armed, again with a limit.
  __syncthreads();
  if (ctl[1] && tid == 0) {
    atomicExch(&P.st->error, 1);
    for (unsigned q = cs.n_use; q != cs.n_iss; ++q) mbar_wait(S.full + 8 * (q % kMarchStages), (q / kMarchStages) & 1u, P.wait_limit);
  }
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

// CTAs of the kernel that fit one SM (0 on error).  The first call also raises the kernel's shared-memory limits.
int march_ctas_per_sm() {
  static int occ = -1;
  if (occ >= 0) return occ;
  const void *fn = (const void *)lattice_march_kernel;
  int n = 0;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMarchSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lattice_march_kernel, kMarchThreads, kMarchSmemBytes) != cudaSuccess)
    return 0;
  occ = n;
  return occ;
}

cudaError_t launch_lattice_march(int grid, const CUtensorMap &tm_c, const MarchParams &p, cudaStream_t s) {
  if (march_ctas_per_sm() <= 0) return cudaErrorLaunchOutOfResources;
  lattice_march_kernel<<<grid, kMarchThreads, kMarchSmemBytes, s>>>(tm_c, p);
  return cudaGetLastError();
}

}  // namespace tfk
