// Dense row-tile producer on the 5th-generation tensor cores (sm_100a):
//   T[r0 : r0+128, 0:N] = B[r0 : r0+128, 0:K] * W[0:K, 0:N]      fp32 in, fp32 out, 3xTF32 inside.
//
// Every fp32 operand is split as x = hi + lo with hi rounded to TF32 (10-bit mantissa); the product
// is accumulated in fp32 in tensor memory as hi*hi + hi*lo + lo*hi, which keeps the result within a
// few 1e-7 relative of the fp32 product (the dropped lo*lo term is below 2^-22).  W is split and
// transposed once per call by split_weight_kernel into Wt_hi / Wt_lo ([N][K], K contiguous), so both
// operands are K-major.  Per 32-wide K slice: TMA (cp.async.bulk.tensor, 128-byte swizzle) brings the
// raw B rows and the two W slices into shared memory, all threads split B in place (hi) and into a
// second buffer (lo), one thread issues 12 tcgen05.mma (4 K-steps of 8 x 3 products) and commits them
// to an mbarrier.  The accumulator (128 lanes x N columns) is read back with tcgen05.ld and stored
// as rows of T.  All waits are bounded: on expiry the error flag is set and the function returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.cuh"

namespace tfk {

constexpr int kTcRows = 128;      // rows per tile = MMA M
constexpr int kTcKSlice = 32;     // fp32 per 128-byte swizzle row
constexpr int kTcMaxN = 256;
constexpr int kTcTmemCols = 256;
// shared-memory layout of one slice (offsets from a 1024-byte aligned base)
constexpr int kTcOffAhi = 0;
constexpr int kTcOffAlo = kTcRows * 128;                    // 16 KB
constexpr int kTcOffWhi = 2 * kTcRows * 128;                // 32 KB
__host__ __device__ constexpr int tc_off_wlo(int n) { return kTcOffWhi + n * 128; }
__host__ __device__ constexpr int tc_smem_bytes(int n) { return kTcOffWhi + 2 * n * 128 + 1024; }  // + alignment slack

struct TcShared {
  unsigned long long bar_tma, bar_mma;
  unsigned tmem_base;
  int ok;
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded: returns false when the phase did not complete within `limit` polls
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
__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *tm, int c0, int c1, unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"((unsigned long long)tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc_sw128(unsigned smem_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (unsigned long long)1 << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= (unsigned long long)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= (unsigned long long)1 << 46;                         // descriptor version of sm_100
  d |= (unsigned long long)2 << 61;                         // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32, A and B tf32, both K-major, M = 128, N = n.
__device__ __forceinline__ unsigned umma_idesc_tf32(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(kTcRows >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Once per CTA, before any tile: warp 0 allocates tensor memory, thread 0 initialises the barriers.
__device__ __forceinline__ void tc_begin(TcShared &s) {
  if (threadIdx.x == 0) {
    mbar_init(&s.bar_tma, 1);
    mbar_init(&s.bar_mma, 1);
    s.ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    // the column count is an immediate: the resident-CTA calculation takes it from the instruction
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "n"(kTcTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Once per CTA, after the last tile (every thread has passed its last tensor-memory access).
__device__ __forceinline__ void tc_end(TcShared &s) {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(s.tmem_base), "n"(kTcTmemCols) : "memory");
  }
}

__device__ __forceinline__ float tf32_round(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

// One tile of up to 128 rows.  `phase` carries the barrier parities across calls (bit 0: TMA,
// bit 1: MMA).  Returns false if a bounded wait ran out (error flag set by the caller's protocol).
template <int NT, class DstRow>
__device__ __forceinline__ bool tc_gemm_rows(const CUtensorMap *tmA, const CUtensorMap *tmWhi, const CUtensorMap *tmWlo,
                                             int r0, int r_end, int K, int N, DstRow dst_row, char *smem1024,
                                             TcShared &s, unsigned &phase, int wait_limit) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float *a_hi = reinterpret_cast<float *>(smem1024 + kTcOffAhi);
  float *a_lo = reinterpret_cast<float *>(smem1024 + kTcOffAlo);
  char *w_hi = smem1024 + kTcOffWhi;
  char *w_lo = smem1024 + tc_off_wlo(N);
  const unsigned idesc = umma_idesc_tf32(N);
  const unsigned tmem_d = s.tmem_base;
  const int n_slices = (K + kTcKSlice - 1) / kTcKSlice;
  bool ok = true;
  for (int sl = 0; sl < n_slices; ++sl) {
    const int k0 = sl * kTcKSlice;
    if (tid == 0) {
      mbar_expect_tx(&s.bar_tma, (unsigned)(kTcRows * 128 + 2 * N * 128));
      tma_load_2d(a_hi, tmA, k0, r0, &s.bar_tma);
      tma_load_2d(w_hi, tmWhi, k0, 0, &s.bar_tma);
      tma_load_2d(w_lo, tmWlo, k0, 0, &s.bar_tma);
    }
    if (!mbar_wait(&s.bar_tma, phase & 1u, wait_limit)) { s.ok = 0; }
    phase ^= 1u;
    __syncthreads();
    if (!s.ok) { ok = false; break; }
    // split the raw rows: hi in place, lo beside it (same swizzled position)
    for (int i = tid; i < kTcRows * kTcKSlice; i += NT) {
      const float a = a_hi[i], h = tf32_round(a);
      a_hi[i] = h;
      a_lo[i] = a - h;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy (MMA) reads
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned ah = smem_u32(a_hi), al = smem_u32(a_lo), wh = smem_u32(w_hi), wl = smem_u32(w_lo);
#pragma unroll
      for (int j = 0; j < kTcKSlice / 8; ++j) {
        const unsigned o = j * 32;  // 8 tf32 = 32 bytes along K inside the swizzle row
        umma_tf32(tmem_d, umma_desc_sw128(ah + o), umma_desc_sw128(wh + o), idesc, (sl | j) ? 1u : 0u);
        umma_tf32(tmem_d, umma_desc_sw128(ah + o), umma_desc_sw128(wl + o), idesc, 1u);
        umma_tf32(tmem_d, umma_desc_sw128(al + o), umma_desc_sw128(wh + o), idesc, 1u);
      }
      umma_commit(&s.bar_mma);
    }
    // the slice buffers are reused by the next TMA: wait until the tensor core has read them
    if (!mbar_wait(&s.bar_mma, (phase >> 1) & 1u, wait_limit)) { s.ok = 0; }
    phase ^= 2u;
    __syncthreads();
    if (!s.ok) { ok = false; break; }
  }
  if (ok && warp < 4) {
    // epilogue: warp w reads tensor-memory lanes 32w .. 32w+31 (= tile rows), 32 columns at a time
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = r0 + warp * 32 + lane;
    for (int c = 0; c < N; c += 32) {
      unsigned v[32];
      const unsigned taddr = tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)c;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
            "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
            "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < r_end) {
        float *d = dst_row(row) + c;
        if (c + 32 <= N) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4 *>(d + 4 * q) = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                                 __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (c + q < N) d[q] = __uint_as_float(v[q]);
        }
      }
    }
  }
  // the next tile's first MMA overwrites the accumulator: every reader must be done
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  return ok;
}

}  // namespace tfk
