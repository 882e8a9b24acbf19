// Kernels and launchers of the fused sparse-dense chains (sm_100a).  See kernels.cuh.
#include <cstdio>
#include <cstdlib>

#include "kernels.cuh"
#include "gemm_tc.cuh"
#include "launch.h"

namespace tfk {

// ---------------------------------------------------------------------------
// Dense row tile on the CUDA cores: T[rows, :] = B[rows, 0:K] * W  (fp32 FMA, k ascending).
// 64 x 64 output tile per pass, 16-deep k slices staged in shared memory, 4 x 4 per thread.
// W is K x N row-major, or N x K when w_transposed.
// ---------------------------------------------------------------------------
constexpr int GM = 64, GN = 64, GK = 16;

struct GemmSmem {
  float a[GK][GM + 4];
  float b[GK][GN + 4];
};

// dst_row(r) gives the output row pointer for source row r
template <class DstRow>
__device__ __forceinline__ void gemm_rows_cta(const float *__restrict__ B, const float *__restrict__ W,
                                              bool w_t, int rb, int re, int K, int N, DstRow dst_row,
                                              GemmSmem &sm) {
  // written for 256 threads; in a larger CTA the others only take part in the barriers
  const int tid = threadIdx.x, tx = tid & 15, ty = (tid >> 4) & 15;
  const bool on = tid < 256;
  for (int r0 = rb; r0 < re; r0 += GM) {
    for (int c0 = 0; c0 < N; c0 += GN) {
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
      for (int k0 = 0; k0 < K; k0 += GK) {
        // A slice: 64 rows x 16 k; thread loads 4 consecutive k of one row
        if (on) {
          const int r = tid >> 2, kk = (tid & 3) * 4;
          const int row = r0 + r;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int k = k0 + kk + u;
            sm.a[kk + u][r] = (row < re && k < K) ? __ldg(B + (size_t)row * K + k) : 0.f;
          }
        }
        // B slice: 16 k x 64 cols; thread loads 4 consecutive cols of one k
        if (on) {
          const int kk = tid >> 4, cc = (tid & 15) * 4;
          const int k = k0 + kk;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c0 + cc + u;
            float v = 0.f;
            if (k < K && c < N) v = w_t ? __ldg(W + (size_t)c * K + k) : __ldg(W + (size_t)k * N + c);
            sm.b[kk][cc + u] = v;
          }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
          float av[4], bv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) av[i] = sm.a[kk][ty * 4 + i];
#pragma unroll
          for (int j = 0; j < 4; ++j) bv[j] = sm.b[kk][tx * 4 + j];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = r0 + ty * 4 + i;
        if (on && row < re) {
          float *d = dst_row(row);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + tx * 4 + j;
            if (c < N) d[c] = acc[i][j];
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// SDDMM-SpMM row: D[row] = sum_p (ax[p] * <Q[row], K[col_p]>) * V[col_p]
// ---------------------------------------------------------------------------
// acc += sum over the nonzeros [q0, q1) of one row of ax[p] * <Q[row], K[col_p]> * V[col_p, panel columns].
// Eight nonzeros at a time: their K rows are read together (lane t holds the products of columns t,
// t + 32, ...), the eight partial dot products are reduced across the warp in one transposed pass (nine
// shuffles instead of forty), and the eight V rows are then gathered together.
template <int VEC, int CH>
__device__ __forceinline__ void sddmm_accumulate(const Params &P, const float *__restrict__ qrow, int q0, int q1,
                                                 int col0, float (&acc)[CH][VEC], int lane) {
  const int kq = P.k_dim, nv = P.n_cols;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  for (int p = q0; p < q1; p += 32) {
    const int cnt = min(32, q1 - p);
    int col = 0;
    float val = 0.f;
    if (lane < cnt) { col = __ldg(P.s_ai + p + lane); val = __ldg(P.s_ax + p + lane); }
    for (int k0 = 0; k0 < cnt; k0 += 8) {
      const float *krow[8];
      int cu[8];
      float part[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // lanes past the end name column 0 with value 0; their sums are dropped
        cu[u] = __shfl_sync(kFull, col, k0 + u);
        krow[u] = P.in1 + (size_t)cu[u] * kq;
        part[u] = 0.f;
      }
      for (int t = lane; t < kq; t += 32) {
        const float qv = __ldg(qrow + t);
#pragma unroll
        for (int u = 0; u < 8; ++u) part[u] = fmaf(qv, __ldg(krow[u] + t), part[u]);
      }
      // transposed reduction: afterwards the four lanes 4u .. 4u + 3 hold the dot product of nonzero k0 + u
      float h4[4], h2[2], dot;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float send = b4 ? part[i] : part[i + 4], keep = b4 ? part[i + 4] : part[i];
        h4[i] = keep + __shfl_xor_sync(kFull, send, 16);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float send = b3 ? h4[i] : h4[i + 2], keep = b3 ? h4[i + 2] : h4[i];
        h2[i] = keep + __shfl_xor_sync(kFull, send, 8);
      }
      {
        const float send = b2 ? h2[0] : h2[1], keep = b2 ? h2[1] : h2[0];
        dot = keep + __shfl_xor_sync(kFull, send, 4);
      }
      dot += __shfl_xor_sync(kFull, dot, 2);
      dot += __shfl_xor_sync(kFull, dot, 1);
      const float sc = dot * __shfl_sync(kFull, val, k0 + (lane >> 2));
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k0 + u < cnt) {  // uniform over the warp
          const float s = __shfl_sync(kFull, sc, 4 * u);
          const float *vrow = P.in2 + (size_t)cu[u] * nv + col0;
#pragma unroll
          for (int ch = 0; ch < CH; ++ch) {
            const int cc = (ch * 32 + lane) * VEC;
            if (col0 + cc < nv) {
              float x[VEC];
              load_vec<VEC, false>(x, vrow + cc);
#pragma unroll
              for (int i = 0; i < VEC; ++i) acc[ch][i] = fmaf(s, x[i], acc[ch][i]);
            }
          }
        }
      }
    }
  }
}

template <int VEC, int CH>
__device__ __forceinline__ void sddmm_row_warp(const Params &P, int row, int lane) {
  const int kq = P.k_dim, nv = P.n_cols;
  const int p0 = __ldg(P.s_ap + row), p1 = __ldg(P.s_ap + row + 1);
  const float *qrow = P.in0 + (size_t)row * kq;
  constexpr int PANEL = 32 * VEC * CH;
  for (int col0 = 0; col0 < nv; col0 += PANEL) {
    float acc[CH][VEC];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[c][i] = 0.f;
    sddmm_accumulate<VEC, CH>(P, qrow, p0, p1, col0, acc, lane);
    float *orow = P.out + (size_t)row * nv;
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const int cc = col0 + (ch * 32 + lane) * VEC;
      if (cc < nv) store_vec<VEC>(orow + cc, acc[ch], false);
    }
  }
}

// SDDMM-SpMM over the nonzeros [p0, p1) of one heavy row, split over the warps of the CTA; the partial
// rows are added through shared memory; ATOMIC: the range is one segment of the row, the sum is added to
// D[row] (zeroed before the pass) with atomicAdd.
template <int NT, int VEC, int CH, bool ATOMIC>
__device__ __forceinline__ void sddmm_range_cta(const Params &P, int row, int p0, int p1, float *smem) {
  constexpr int NW = NT / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kq = P.k_dim, nv = P.n_cols;
  const int per = ((p1 - p0 + NW - 1) / NW + 31) / 32 * 32;
  const int q0 = min(p1, p0 + warp * per), q1 = min(p1, q0 + per);
  const float *qrow = P.in0 + (size_t)row * kq;
  constexpr int PANEL = 32 * VEC * CH;
  for (int col0 = 0; col0 < nv; col0 += PANEL) {
    float acc[CH][VEC];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[c][i] = 0.f;
    sddmm_accumulate<VEC, CH>(P, qrow, q0, q1, col0, acc, lane);
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) smem[warp * PANEL + (c * 32 + lane) * VEC + i] = acc[c][i];
    __syncthreads();
    for (int t = threadIdx.x; t < PANEL; t += NT) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += smem[w * PANEL + t];
      if (col0 + t < nv) {
        if (ATOMIC) atomicAdd(P.out + (size_t)row * nv + col0 + t, s);
        else P.out[(size_t)row * nv + col0 + t] = s;
      }
    }
    __syncthreads();
  }
}

// The next row of an item for this warp: rows go to whichever warp is free, so that a block with a few
// long rows (power-law graphs) does not wait for the warp that drew them all.
__device__ __forceinline__ int next_row(int *counter, int row_begin, int lane) {
  int t = 0;
  if (lane == 0) t = atomicAdd(counter, 1);
  return row_begin + __shfl_sync(kFull, t, 0);
}

// ---------------------------------------------------------------------------
// The persistent executor
// ---------------------------------------------------------------------------
#ifndef TF_MIN_CTAS
#define TF_MIN_CTAS 4
#endif
constexpr int kHeavyNnz = 32 * kWarps;  // a single-row block at least this heavy is split over the CTA

union StreamSmem {
  GemmSmem g;
  float red[2048];  // warps * 32 * VEC * CH: 8 * 256 (direct) or 16 * 128 (gather-tile variant)
};

// TILED: the plan holds gather tiles (item kinds 4 and 5); their staging buffer allows two CTAs per
// SM, so that variant may use twice the registers.
template <int MODE, int VEC, int CH, bool RING, bool TILED>
__global__ void __launch_bounds__(TILED ? tiled_threads(MODE) : kThreads, TILED ? 2 : (MODE == 2 ? 3 : TF_MIN_CTAS))
    stream_kernel(const __grid_constant__ Params P) {
  constexpr int NT = TILED ? tiled_threads(MODE) : kThreads;
  constexpr int NW = NT / 32;
  constexpr bool HAS_TC = MODE == 1 && TILED;  // the dense producer may run on the tensor cores
  __shared__ StreamSmem sm;
  __shared__ int s_next;
  __shared__ int s_row;  // rows of the current item handed out so far (warps take the next row when they are free)
  __shared__ int s_ok;
  extern __shared__ float4 stage[];  // gather tiles: tile_slots * 8 float4, then tile_slots source row ids
  int *hrow = reinterpret_cast<int *>(stage + (size_t)P.tile_slots * 8);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  ExecState *st = P.st;
  const int n_items = P.item_end - P.item_begin;
  __shared__ TcShared tc;
  unsigned tc_phase = 0;
  char *smem1024 = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(stage) + 1023) & ~(uintptr_t)1023);
  const bool use_tc = HAS_TC && P.use_tc != 0;
  if (use_tc) tc_begin(tc);

  if (threadIdx.x == 0) { s_next = atomicAdd(&st->ticket, 1); s_row = 0; }
  __syncthreads();
  int cur = s_next;
  while (cur < n_items) {
    // take the next ticket now and keep it in a register: its latency hides behind this item
    int nxt = 0;
    if (threadIdx.x == 0) nxt = atomicAdd(&st->ticket, 1);
    const int4 ia = __ldg(P.items + 2 * (size_t)(P.item_begin + cur));
    const int4 ib = __ldg(P.items + 2 * (size_t)(P.item_begin + cur) + 1);
    const int kind = ia.x, block = ia.y, rb = ia.z, re = ia.w;
    const int need = ib.x, base = ib.y, send_row = ib.z;

    if (need > 0) {
      if (warp == 0) {
        const bool ok = (kind == 1 || kind == 5 || kind == 7)
                            ? wait_for(&st->prod_wm, P.prod_done, need, P.epoch, st, P.spin_limit, lane)
                            : wait_for(&st->cons_wm, P.cons_done, need, P.epoch, st, P.spin_limit, lane);
        if (lane == 0) s_ok = ok;
      }
      __syncthreads();
      if (!s_ok) break;
      // order this CTA's reads of T after the acquires made by warp 0
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
    }

    if (kind == 0 || kind == 3) {
      // ---- produce rows [rb, re) of T (kind 3: into the send buffer at row send_row) ----
      float *dst_base;
      int ring = 0, pbase = 0;
      if (kind == 3) dst_base = P.inter + (ptrdiff_t)(send_row - rb) * P.n_cols;  // phase 0: `inter` is the send buffer
      else { dst_base = P.inter; if (RING) { ring = P.ring_rows; pbase = base; } }
      auto dst_row = [&](int r) -> float * {
        int t = r;
        if (RING && kind == 0) { t = r - pbase; if (t >= ring) t -= ring; }
        return dst_base + (size_t)t * P.n_cols;
      };
      if (MODE == 1) {
        if (HAS_TC && use_tc) {
          if (!tc_gemm_rows<NT>(&P.tm_a, &P.tm_whi, &P.tm_wlo, rb, re, P.k_dim, P.n_cols, dst_row, smem1024, tc,
                                tc_phase, P.spin_limit)) {
            if (threadIdx.x == 0) atomicExch(&st->error, 1);
            break;
          }
        } else {
          gemm_rows_cta(P.in0, P.in1, P.w_transposed != 0, rb, re, P.k_dim, P.n_cols, dst_row, sm.g);
        }
      } else {
        if (re - rb == 1 && __ldg(P.f_ap + re) - __ldg(P.f_ap + rb) >= kHeavyNnz)
          spmm_row_cta<NT, VEC, CH, false, false>(P.f_ap, P.f_ai, P.f_ax, rb, P.in0, P.n_cols, dst_row(rb), false,
                                              0, 0, 0, sm.red);
        else {
          for (int r = next_row(&s_row, rb, lane); r < re; r = next_row(&s_row, rb, lane))
            spmm_row_warp<VEC, CH, false, false>(P.f_ap, P.f_ai, P.f_ax, r, P.in0, P.n_cols, dst_row(r),
                                                 false, 0, 0, 0, lane);
        }
      }
      if (kind == 0) {
        __syncthreads();
        if (threadIdx.x == 0) publish(P.prod_done, block, P.epoch);
      }
    } else if (kind == 1) {
      // ---- consume: D[rb, re) = A * T ----
      if (re - rb == 1 && __ldg(P.s_ap + re) - __ldg(P.s_ap + rb) >= kHeavyNnz)
        spmm_row_cta<NT, VEC, CH, true, RING>(P.s_ap, P.s_ai, P.s_ax, rb, P.inter, P.n_cols,
                                          P.out + (size_t)rb * P.n_cols, P.relu != 0, base, P.ring_rows,
                                          P.m_local, sm.red);
      else {
        for (int r = next_row(&s_row, rb, lane); r < re; r = next_row(&s_row, rb, lane))
          spmm_row_warp<VEC, CH, true, RING>(P.s_ap, P.s_ai, P.s_ax, r, P.inter, P.n_cols,
                                             P.out + (size_t)r * P.n_cols, P.relu != 0, base, P.ring_rows,
                                             P.m_local, lane);
      }
      if (RING) {
        __syncthreads();
        if (threadIdx.x == 0) publish(P.cons_done, block, P.epoch);
      }
    } else if (TILED && kind == 4) {
      // ---- produce the rows of one gather tile of the first operator ----
      const int ring = RING ? P.ring_rows : 0;
      auto dst_row = [&](int r) -> float * {
        int t = r;
        if (RING) { t = r - base; if (t >= ring) t -= ring; }
        return P.inter + (size_t)t * P.n_cols;
      };
      tile_gather<NT, false>(P.pt, rb, P.f_ap, P.f_ax, P.in0, P.n_cols, dst_row, false, 0, 0, 0, stage, hrow,
                             P.tile_slots);
      __syncthreads();
      if (threadIdx.x == 0) publish(P.prod_done, block, P.epoch);
    } else if (TILED && kind == 5) {
      // ---- consume: the rows of one gather tile of the second operator ----
      auto out_row = [&](int r) -> float * { return P.out + (size_t)r * P.n_cols; };
      tile_gather<NT, RING>(P.ct, rb, P.s_ap, P.s_ax, P.inter, P.n_cols, out_row, P.relu != 0, base, P.ring_rows,
                        P.m_local, stage, hrow, P.tile_slots);
      if (RING) {
        __syncthreads();
        if (threadIdx.x == 0) publish(P.cons_done, block, P.epoch);
      }
    } else if (kind == 6) {
      // ---- one segment of a heavy row of T: nonzeros [re, base), added atomically ----
      spmm_range_cta<NT, VEC, CH, false, false, true>(P.f_ai, P.f_ax, re, base, P.in0, P.n_cols,
                                                      P.inter + (size_t)rb * P.n_cols, false, 0, 0, 0, sm.red);
      __syncthreads();
      if (threadIdx.x == 0) publish(P.prod_done, block, P.epoch);
    } else if (kind == 7) {
      // ---- one segment of a heavy row of D ----
      spmm_range_cta<NT, VEC, CH, true, false, true>(P.s_ai, P.s_ax, re, base, P.inter, P.n_cols,
                                                     P.out + (size_t)rb * P.n_cols, false, 0, 0, P.m_local, sm.red);
    } else if (kind == 8) {
      // ---- one segment of a heavy SDDMM-SpMM row ----
      sddmm_range_cta<NT, VEC, CH, true>(P, rb, re, base, sm.red);
    } else if (kind == 2) {
      // ---- SDDMM-SpMM rows: a heavy row is shared by the CTA, the others go one per warp ----
      if (re - rb == 1 && __ldg(P.s_ap + re) - __ldg(P.s_ap + rb) >= kHeavyNnz) {
        sddmm_range_cta<NT, VEC, CH, false>(P, rb, __ldg(P.s_ap + rb), __ldg(P.s_ap + re), sm.red);
      } else
      for (int r = next_row(&s_row, rb, lane); r < re; r = next_row(&s_row, rb, lane)) sddmm_row_warp<VEC, CH>(P, r, lane);
    }
    __syncthreads();
    if (threadIdx.x == 0) { s_next = nxt; s_row = 0; }
    __syncthreads();
    cur = s_next;
  }
  if (use_tc) tc_end(tc);
  // the last CTA out rewinds the ticket counter (and, after the last phase, the watermarks)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int f = atomicAdd(&st->finished, 1);
    if (f == (int)gridDim.x - 1) {
      st->ticket = 0;
      st->finished = 0;
      if (P.reset_wm) { st->prod_wm = 0; st->cons_wm = 0; }
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------
// Schedule mode: one CTA per partition of a level of a reference-format schedule.
//   entries with type 0: produce that row of T; then, after a CTA barrier, entries with type 1:
//   consume.  Wave 2 partitions hold type-1 entries only.
// ---------------------------------------------------------------------------
struct SchedParams {
  const int *ptr2, *id, *type, *ker;  // device copies; ker may be null
  int part_begin, part_end;
};

template <int MODE, int VEC, int CH>
__global__ void __launch_bounds__(kThreads) schedule_level_kernel(const Params P, const SchedParams S) {
  __shared__ StreamSmem sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int w = S.part_begin + blockIdx.x; w < S.part_end; w += gridDim.x) {
    const int kb = __ldg(S.ptr2 + w), ke = __ldg(S.ptr2 + w + 1);
    if (MODE == 1) {
      // dense producer on the contiguous tile rows [id[kb], id[kb] + ts)
      const int ke1 = __ldg(S.ker + 2 * w);
      const int ts = ke1 - kb;
      if (ts > 0) {
        const int r0 = __ldg(S.id + kb);
        auto dst_row = [&](int r) -> float * { return P.inter + (size_t)r * P.n_cols; };
        gemm_rows_cta(P.in0, P.in1, P.w_transposed != 0, r0, r0 + ts, P.k_dim, P.n_cols, dst_row, sm.g);
      }
    } else {
      for (int k = kb + warp; k < ke; k += kWarps)
        if (__ldg(S.type + k) == 0) {
          const int r = __ldg(S.id + k);
          spmm_row_warp<VEC, CH, false, false>(P.f_ap, P.f_ai, P.f_ax, r, P.in0, P.n_cols,
                                               P.inter + (size_t)r * P.n_cols, false, 0, 0, 0, lane);
        }
    }
    __threadfence();
    __syncthreads();
    for (int k = kb + warp; k < ke; k += kWarps)
      if (__ldg(S.type + k) == 1) {
        const int r = __ldg(S.id + k);
        spmm_row_warp<VEC, CH, true, false>(P.s_ap, P.s_ai, P.s_ax, r, P.inter, P.n_cols,
                                            P.out + (size_t)r * P.n_cols, P.relu != 0, 0, 0, 0, lane);
      }
    __syncthreads();
  }
}

// rows[i] of a row-major matrix set to zero (before a pass that accumulates heavy rows atomically),
// or clamped at zero (after it, when the chain ends in a ReLU).
__global__ void rows_fix_kernel(const int *rows, int n_rows, int n_cols, float *x, int relu) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)n_rows * n_cols;
       i += (long long)gridDim.x * blockDim.x) {
    float *p = x + (size_t)__ldg(rows + i / n_cols) * n_cols + i % n_cols;
    *p = relu ? fmaxf(*p, 0.f) : 0.f;
  }
}

// Plain CSR SpMM, one warp per row (out = A * X).
template <int VEC, int CH>
__global__ void __launch_bounds__(kThreads) spmm_kernel(const int *ap, const int *ai, const float *ax, int m,
                                                        const float *x, int n_cols, float *out) {
  const int lane = threadIdx.x & 31;
  const int nw = gridDim.x * kWarps;
  // 8 consecutive rows per warp
  for (int r0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * 8; r0 < m; r0 += nw * 8)
    for (int r = r0; r < min(m, r0 + 8); ++r)
      spmm_row_warp<VEC, CH, false, false>(ap, ai, ax, r, x, n_cols, out + (size_t)r * n_cols, false, 0, 0, 0, lane);
}

// ---------------------------------------------------------------------------
// Seeded fills: u(seed, idx) = top 24 bits of splitmix64(seed * golden + idx) / 2^24
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  unsigned long long z = x + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float unit24(unsigned long long seed, unsigned long long idx) {
  return (float)(splitmix64(seed * 0x9E3779B97F4A7C15ull + idx) >> 40) * (1.0f / 16777216.0f);
}
__global__ void fill_uniform_kernel(float *p, long long n, unsigned long long seed, long long off) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = 2.0f * unit24(seed, (unsigned long long)(off + i)) - 1.0f;
}
__global__ void fill_normal_kernel(float *p, long long n, unsigned long long seed, long long off, float sigma) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float u1 = 1.0f - unit24(seed, 2ull * (unsigned long long)(off + i));
    const float u2 = unit24(seed, 2ull * (unsigned long long)(off + i) + 1ull);
    p[i] = sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
  }
}

// ---------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------
typedef void (*StreamFn)(const __grid_constant__ Params);
typedef void (*SchedFn)(const Params, const SchedParams);

template <int MODE, int VEC, int CH>
static StreamFn pick_ring(bool ring, bool tiled) {
  if (tiled) return ring ? stream_kernel<MODE, VEC, CH, true, true> : stream_kernel<MODE, VEC, CH, false, true>;
  return ring ? stream_kernel<MODE, VEC, CH, true, false> : stream_kernel<MODE, VEC, CH, false, false>;
}
template <int MODE>
static StreamFn pick_stream(int vec, int ch, bool ring, bool tiled) {
  if (vec == 4) return ch == 2 ? pick_ring<MODE, 4, 2>(ring, tiled) : pick_ring<MODE, 4, 1>(ring, tiled);
  if (vec == 2) return ch == 2 ? pick_ring<MODE, 2, 2>(ring, false) : pick_ring<MODE, 2, 1>(ring, false);
  return ch == 2 ? pick_ring<MODE, 1, 2>(ring, false) : pick_ring<MODE, 1, 1>(ring, false);
}
template <int MODE>
static SchedFn pick_sched(int vec, int ch) {
  if (vec == 4) return ch == 2 ? schedule_level_kernel<MODE, 4, 2> : schedule_level_kernel<MODE, 4, 1>;
  if (vec == 2) return ch == 2 ? schedule_level_kernel<MODE, 2, 2> : schedule_level_kernel<MODE, 2, 1>;
  return ch == 2 ? schedule_level_kernel<MODE, 1, 2> : schedule_level_kernel<MODE, 1, 1>;
}

void choose_shape(int n_cols, bool aligned16, int *vec, int *ch) {
  if (aligned16 && n_cols % 4 == 0 && n_cols > 64) { *vec = 4; *ch = n_cols > 128 ? 2 : 1; }
  else if (aligned16 && n_cols % 2 == 0) { *vec = 2; *ch = n_cols > 64 ? 2 : 1; }
  else { *vec = 1; *ch = n_cols > 32 ? 2 : 1; }
}

static StreamFn stream_fn(int mode, int vec, int ch, bool ring, bool tiled) {
  switch (mode) {
    case 0: return pick_stream<0>(vec, ch, ring, tiled);
    case 1: return pick_stream<1>(vec, ch, ring, tiled);
    default: return pick_stream<2>(vec, ch, false, false);
  }
}

int stream_occupancy(int mode, int vec, int ch, bool ring, size_t dyn_smem) {
  int nb = 0;
  const void *fn = (const void *)stream_fn(mode, vec, ch, ring, dyn_smem > 0);
  if (dyn_smem > 0 &&
      cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem) != cudaSuccess)
    return -1;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fn, dyn_smem > 0 ? tiled_threads(mode) : kThreads, dyn_smem);
  return e == cudaSuccess ? nb : -1;
}

cudaError_t launch_stream(int mode, int vec, int ch, bool ring, int grid, size_t dyn_smem, const Params &p,
                          cudaStream_t s) {
  StreamFn fn = stream_fn(mode, vec, ch, ring, dyn_smem > 0);
  if (dyn_smem > 0) {
    cudaError_t e = cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem);
    if (e != cudaSuccess) return e;
  }
  fn<<<grid, dyn_smem > 0 ? tiled_threads(mode) : kThreads, dyn_smem, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_schedule_level(int mode, int vec, int ch, int grid, const Params &p, const int *ptr2,
                                  const int *id, const int *type, const int *ker, int part_begin, int part_end,
                                  cudaStream_t s) {
  if (part_end <= part_begin) return cudaSuccess;
  SchedParams sp{ptr2, id, type, ker, part_begin, part_end};
  SchedFn f = mode == 1 ? pick_sched<1>(vec, ch) : pick_sched<0>(vec, ch);
  f<<<grid, kThreads, 0, s>>>(p, sp);
  return cudaGetLastError();
}

cudaError_t launch_spmm(int vec, int ch, int grid, const int *ap, const int *ai, const float *ax, int m,
                        const float *x, int n_cols, float *out, cudaStream_t s) {
  if (m <= 0) return cudaSuccess;
  if (vec == 4) { if (ch == 2) spmm_kernel<4, 2><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out);
                  else spmm_kernel<4, 1><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out); }
  else if (vec == 2) { if (ch == 2) spmm_kernel<2, 2><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out);
                       else spmm_kernel<2, 1><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out); }
  else { if (ch == 2) spmm_kernel<1, 2><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out);
         else spmm_kernel<1, 1><<<grid, kThreads, 0, s>>>(ap, ai, ax, m, x, n_cols, out); }
  return cudaGetLastError();
}

cudaError_t launch_rows_fix(const int *rows, int n_rows, int n_cols, float *x, bool relu, cudaStream_t s) {
  if (n_rows <= 0) return cudaSuccess;
  const long long total = (long long)n_rows * n_cols;
  rows_fix_kernel<<<(int)std::min<long long>((total + 255) / 256, 148LL * 8), 256, 0, s>>>(rows, n_rows, n_cols, x, relu ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t launch_fill(bool normal, float *p, long long n, unsigned long long seed, long long off, float sigma,
                        cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int grid = (int)std::min<long long>((n + 255) / 256, 148LL * 16);
  if (normal) fill_normal_kernel<<<grid, 256, 0, s>>>(p, n, seed, off, sigma);
  else fill_uniform_kernel<<<grid, 256, 0, s>>>(p, n, seed, off);
  return cudaGetLastError();
}

}  // namespace tfk
