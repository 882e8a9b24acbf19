// Device side of the fused sparse-dense chains (sm_100a).
//
// One persistent kernel walks a ticket-ordered list of work items:
//   PRODUCE  rows of the intermediate T (CSR row gather of C, or a dense row tile B*W)
//   CONSUME  rows of D = A * T
//   SDDMM    rows of D = (A .* (Q K^T)) * V, the sampled values never stored
// Producers publish completed row blocks through a done-flag array and a
// contiguous watermark; consumers wait (bounded) on the watermark.  T is read
// with L2-only loads because other SMs write it during the same launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfk {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr unsigned kFull = 0xffffffffu;

struct ExecState {
  int ticket;    // next item
  int prod_wm;   // producer blocks [0, prod_wm) are complete
  int cons_wm;   // consumer blocks [0, cons_wm) are complete
  int finished;  // CTAs that left the item loop
  int error;     // sticky: a bounded wait ran out
  int pad[3];
};

struct Params {
  // first operator (SpMM producer) and second operator (consumer), device CSR
  const int *f_ap, *f_ai; const float *f_ax;
  const int *s_ap, *s_ai; const float *s_ax;
  const float *in0;  // C (SpMM-SpMM) | B dense (GeMM-SpMM) | Q (SDDMM)
  const float *in1;  // W (GeMM-SpMM) | K (SDDMM)
  const float *in2;  // V (SDDMM)
  float *inter;      // T: ring_rows (or all) rows of n_cols
  float *out;        // D
  const int4 *items; // two int4 per item
  int item_begin, item_end;
  int *prod_done, *cons_done;
  ExecState *st;
  int epoch;
  int n_cols;        // width of T and D
  int k_dim;         // GeMM: inner dimension; SDDMM: width of Q and K
  int m_local;       // rows of T produced here; columns >= m_local are halo rows
  int ring_rows;     // 0 = T holds every row
  int n_prod, n_cons;
  int relu, w_transposed;
  int reset_wm;      // last CTA clears the watermarks (last phase of a call)
  int spin_limit;    // polls before a wait gives up
};

// ---------------------------------------------------------------------------
// memory-model helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Publish block `b`: everything the CTA wrote (ordered before by the CTA barrier) is made
// visible, then the block's flag takes the value of this pass.
__device__ __forceinline__ void publish(int *done, int b, int epoch) {
  __threadfence();
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(done + b), "r"(epoch) : "memory");
}

// Bounded wait, executed by one whole warp, until blocks [0, need) of the other side are complete.
// `wm` is a lazy lower bound of the completed prefix: whoever verifies the flags [wm, need) raises
// it, so in steady state a waiter reads the watermark and one or two flags.  No thread ever walks
// the flag array serially.  Returns false if the wait gave up (or another CTA already had).
__device__ __forceinline__ bool wait_for(int *wm, const int *done, int need, int epoch, ExecState *st,
                                         int spin_limit, int lane) {
  int spins = 0;
  for (;;) {
    int w = 0;
    if (lane == 0) w = ld_acquire(wm);
    w = __shfl_sync(kFull, w, 0);
    if (w >= need) return true;
    bool all = true;
    for (int b = w + lane; b < need; b += 32) all = all && (ld_acquire(done + b) == epoch);
    if (__all_sync(kFull, all)) {
      if (lane == 0) { __threadfence(); atomicMax(wm, need); }
      return true;
    }
    int err = 0;
    if (lane == 0) err = (++spins > spin_limit) || (ld_acquire(&st->error) != 0);
    if (__shfl_sync(kFull, err, 0)) {
      if (lane == 0) atomicExch(&st->error, 1);
      return false;
    }
    __nanosleep(spins < 64 ? 64 : 512);
  }
}

// ---------------------------------------------------------------------------
// vector helpers: VEC floats per lane
// ---------------------------------------------------------------------------
template <int VEC> struct Vec;
template <> struct Vec<4> { typedef float4 T; };
template <> struct Vec<2> { typedef float2 T; };
template <> struct Vec<1> { typedef float T; };

template <int VEC, bool L2ONLY>
__device__ __forceinline__ void load_vec(float (&d)[VEC], const float *p) {
  typedef typename Vec<VEC>::T V;
  V v;
  if (L2ONLY) v = __ldcg(reinterpret_cast<const V *>(p));
  else v = __ldg(reinterpret_cast<const V *>(p));
  const float *f = reinterpret_cast<const float *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) d[i] = f[i];
}
template <int VEC>
__device__ __forceinline__ void store_vec(float *p, const float (&s)[VEC], bool relu) {
  typedef typename Vec<VEC>::T V;
  V v;
  float *f = reinterpret_cast<float *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) f[i] = relu ? fmaxf(s[i], 0.f) : s[i];
  *reinterpret_cast<V *>(p) = v;
}

// Row of the dense operand a column index refers to.
//   RING: T is a ring of ring_rows rows; `base` is a multiple of ring_rows at or below the
//         smallest column of the item, and every column of the item is below base + 2*ring_rows.
//   Columns >= m_local address halo rows stored after the local (or ring) rows.
template <bool RING>
__device__ __forceinline__ int map_row(int col, int base, int ring_rows, int m_local) {
  if (RING) {
    if (col >= m_local) return ring_rows + (col - m_local);
    int t = col - base;
    return t >= ring_rows ? t - ring_rows : t;
  }
  return col;
}

// acc[CH][VEC] += sum over nonzeros p in [p0, p1) of ax[p] * dense[row(ai[p]), lane's columns].
// Lanes fetch 32 (index, value) pairs at a time, coalesced, and broadcast them by shuffle;
// four gathers are in flight before their FMAs retire.
template <int VEC, int CH, bool L2ONLY, bool RING>
__device__ __forceinline__ void gather_row(float (&acc)[CH][VEC], const int *__restrict__ ai,
                                           const float *__restrict__ ax, int p0, int p1,
                                           const float *__restrict__ dense, int ld, int col0, int n_cols,
                                           int base, int ring_rows, int m_local, int lane) {
  for (int p = p0; p < p1; p += 32) {
    const int cnt = min(32, p1 - p);
    int row = 0;
    float val = 0.f;
    if (lane < cnt) {
      row = map_row<RING>(__ldg(ai + p + lane), base, ring_rows, m_local);
      val = __ldg(ax + p + lane);
    }
    int k = 0;
    for (; k + 4 <= cnt; k += 4) {
      float x[4][CH][VEC];
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = __shfl_sync(kFull, row, k + u);
        v[u] = __shfl_sync(kFull, val, k + u);
        const float *src = dense + (size_t)r * ld + col0;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int cc = (c * 32 + lane) * VEC;
          if (col0 + cc < n_cols) load_vec<VEC, L2ONLY>(x[u][c], src + cc);
          else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) x[u][c][i] = 0.f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[c][i] = fmaf(v[u], x[u][c][i], acc[c][i]);
    }
    for (; k < cnt; ++k) {
      const int r = __shfl_sync(kFull, row, k);
      const float v = __shfl_sync(kFull, val, k);
      const float *src = dense + (size_t)r * ld + col0;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int cc = (c * 32 + lane) * VEC;
        if (col0 + cc < n_cols) {
          float x[VEC];
          load_vec<VEC, L2ONLY>(x, src + cc);
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[c][i] = fmaf(v, x[i], acc[c][i]);
        }
      }
    }
  }
}

// out_row[lane's columns] = A[row,:] * dense, one warp per row, all column panels.
template <int VEC, int CH, bool L2ONLY, bool RING>
__device__ __forceinline__ void spmm_row_warp(const int *__restrict__ ap, const int *__restrict__ ai,
                                              const float *__restrict__ ax, int row,
                                              const float *__restrict__ dense, int n_cols, float *out_row,
                                              bool relu, int base, int ring_rows, int m_local, int lane) {
  const int p0 = __ldg(ap + row), p1 = __ldg(ap + row + 1);
  constexpr int PANEL = 32 * VEC * CH;
  for (int col0 = 0; col0 < n_cols; col0 += PANEL) {
    float acc[CH][VEC];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[c][i] = 0.f;
    gather_row<VEC, CH, L2ONLY, RING>(acc, ai, ax, p0, p1, dense, n_cols, col0, n_cols, base, ring_rows,
                                      m_local, lane);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int cc = col0 + (c * 32 + lane) * VEC;
      if (cc < n_cols) store_vec<VEC>(out_row + cc, acc[c], relu);
    }
  }
}

// A row too heavy for one warp: the CTA's warps split its nonzeros and add their partial
// sums through shared memory (panel by panel).
template <int VEC, int CH, bool L2ONLY, bool RING>
__device__ __forceinline__ void spmm_row_cta(const int *__restrict__ ap, const int *__restrict__ ai,
                                             const float *__restrict__ ax, int row,
                                             const float *__restrict__ dense, int n_cols, float *out_row,
                                             bool relu, int base, int ring_rows, int m_local,
                                             float *smem /* kWarps * 32*VEC*CH floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p0 = __ldg(ap + row), p1 = __ldg(ap + row + 1);
  const int per = ((p1 - p0 + kWarps - 1) / kWarps + 31) / 32 * 32;
  const int q0 = min(p1, p0 + warp * per), q1 = min(p1, q0 + per);
  constexpr int PANEL = 32 * VEC * CH;
  for (int col0 = 0; col0 < n_cols; col0 += PANEL) {
    float acc[CH][VEC];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[c][i] = 0.f;
    gather_row<VEC, CH, L2ONLY, RING>(acc, ai, ax, q0, q1, dense, n_cols, col0, n_cols, base, ring_rows,
                                      m_local, lane);
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) smem[warp * PANEL + (c * 32 + lane) * VEC + i] = acc[c][i];
    __syncthreads();
    for (int t = threadIdx.x; t < PANEL; t += kThreads) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += smem[w * PANEL + t];
      if (col0 + t < n_cols) out_row[col0 + t] = relu ? fmaxf(s, 0.f) : s;
    }
    __syncthreads();
  }
}

}  // namespace tfk
