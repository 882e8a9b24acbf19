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
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfk {

constexpr int kThreads = 256;       // CTA size of the direct kernels
constexpr int kWarps = kThreads / 32;
// CTA size of the gather-tile variant of the executor.  512 threads, two CTAs per SM: measured faster
// than 256 threads x four CTAs on the 128^3 case (1.30 vs 1.41 ms), whose smaller tiles reuse less.
__host__ __device__ constexpr int tiled_threads(int /*mode*/) { return 512; }
constexpr int kTiledThreadsMax = 512;
constexpr unsigned kFull = 0xffffffffu;

struct ExecState {
  int ticket;    // next item
  int prod_wm;   // producer blocks [0, prod_wm) are complete
  int cons_wm;   // consumer blocks [0, cons_wm) are complete
  int finished;  // CTAs that left the item loop
  int error;     // sticky: a bounded wait ran out
  int pad[3];
};

// Gather tiles of one operator: tile -> output rows, tile -> staged source rows (slot order),
// and per nonzero the slot its column occupies in the tile's staging buffer.
struct TileArrays {
  const int *row_ptr, *rows, *halo_ptr, *halo;
  const unsigned short *slot;
  // Row tables for the tile pipeline, one block per tile of kTileMetaPlanes planes of R pairs (R = the
  // tile's rows rounded up to 8): plane k < kTileMetaNnz holds {byte offset of the slot, value bits} of
  // nonzero k of every row ({0, 0} past the row's end), the last plane {row id or -1, row length}.
  const int2 *meta;
};
constexpr int kTileMetaNnz = 7;
constexpr int kTileMetaPlanes = kTileMetaNnz + 1;

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
  // tensor-core dense producer (GeMM-SpMM): TMA descriptors of B and of the split, transposed weight
  alignas(64) CUtensorMap tm_a, tm_whi, tm_wlo;
  int use_tc;
  TileArrays pt, ct; // gather tiles of the first / second operator (null when not tiled)
  int tile_slots;    // staging slots per CTA (dynamic shared memory holds tile_slots * 132 bytes)
  int tile_rows;     // tile pipeline: most rows of a tile, rounded up to 8
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

// A row too heavy for one warp: the CTA's warps split the nonzeros [p0, p1) of one row and add their
// partial sums through shared memory (panel by panel).  ATOMIC: the range is one segment of a row cut
// over several CTAs, the result is added to out_row (zeroed before the pass) with atomicAdd.
template <int NT, int VEC, int CH, bool L2ONLY, bool RING, bool ATOMIC>
__device__ __forceinline__ void spmm_range_cta(const int *__restrict__ ai, const float *__restrict__ ax, int p0,
                                               int p1, const float *__restrict__ dense, int n_cols,
                                               float *out_row, bool relu, int base, int ring_rows, int m_local,
                                               float *smem /* NT/32 * 32*VEC*CH floats */) {
  constexpr int NW = NT / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = ((p1 - p0 + NW - 1) / NW + 31) / 32 * 32;
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
    for (int t = threadIdx.x; t < PANEL; t += NT) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += smem[w * PANEL + t];
      if (col0 + t < n_cols) {
        if (ATOMIC) atomicAdd(out_row + col0 + t, s);
        else out_row[col0 + t] = relu ? fmaxf(s, 0.f) : s;
      }
    }
    __syncthreads();
  }
}

template <int NT, int VEC, int CH, bool L2ONLY, bool RING>
__device__ __forceinline__ void spmm_row_cta(const int *__restrict__ ap, const int *__restrict__ ai,
                                             const float *__restrict__ ax, int row,
                                             const float *__restrict__ dense, int n_cols, float *out_row,
                                             bool relu, int base, int ring_rows, int m_local, float *smem) {
  spmm_range_cta<NT, VEC, CH, L2ONLY, RING, false>(ai, ax, __ldg(ap + row), __ldg(ap + row + 1), dense, n_cols, out_row,
                                                   relu, base, ring_rows, m_local, smem);
}

// ---------------------------------------------------------------------------
// Gather tile: out[r, :] = sum_p ax[p] * src[col_p, :] for the rows r of one tile.
//
// The dense source rows the tile needs are staged once per 32-column chunk (128 B per row) in
// shared memory with 16-byte asynchronous copies that bypass L1, then every output row-chunk is
// computed by 8 lanes (one float4 each) reading its operands from shared memory: a staged row is
// fetched from L2 once and reused by every row of the tile that names it.  One warp works on four
// rows at a time; a 128-byte slot is read by one quarter-warp, which is conflict-free.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// SRC_RING: source rows live in the ring (or after it, for halo rows).  dst_row(r) gives the
// output row pointer.  A group of 4 lanes owns up to kTileRowsPerGroup rows of the tile and computes
// each row's 32-column chunk as two float4 per lane; their row ids, lengths and (slot, value) pairs
// -- lane l of the group holds nonzeros l and l + 4 -- are loaded once into registers and serve every
// column chunk, so the inner loop touches shared memory only.  The two groups that share a
// quarter-warp read opposite 64-byte halves of their slots in each load, which keeps the 128-bit
// shared loads conflict-free.
constexpr int kTileRowsPerGroup = 4;  // a tile holds at most NT rows (NT / 4 groups of 4 lanes)
constexpr int kTileMaxSlots = 1700;  // staging slots a tile may use (shared-memory capacity)

template <int NT, bool SRC_RING, class DstRow>
__device__ __forceinline__ void tile_gather(const TileArrays &ta, int tile, const int *__restrict__ ap,
                                            const float *__restrict__ ax, const float *__restrict__ src,
                                            int n_cols, DstRow dst_row, bool relu, int base, int ring_rows,
                                            int m_local, float4 *stage, int *hrow, int stage_slots) {
  const int rp = __ldg(ta.row_ptr + tile), nR = __ldg(ta.row_ptr + tile + 1) - rp;
  const int hp = __ldg(ta.halo_ptr + tile), nH = __ldg(ta.halo_ptr + tile + 1) - hp;
  const int g8 = threadIdx.x >> 3, l8 = threadIdx.x & 7;  // staging: 8 lanes per 128-byte slot
  constexpr int kTileGroups = NT / 4;
  const int g4 = threadIdx.x >> 2, l4 = threadIdx.x & 3;  // compute: 4 lanes per row
  const int colA = ((g4 & 1) * 16) + l4 * 4, colB = (((g4 & 1) ^ 1) * 16) + l4 * 4;  // floats within the chunk
  const char *sA = reinterpret_cast<const char *>(stage) + colA * 4;
  const char *sB = reinterpret_cast<const char *>(stage) + colB * 4;
  int rr[kTileRowsPerGroup], cnt[kTileRowsPerGroup], ms[kTileRowsPerGroup][2];
  float mv[kTileRowsPerGroup][2];
  int wmax = 0;
#pragma unroll
  for (int j = 0; j < kTileRowsPerGroup; ++j) {
    const int i = j * kTileGroups + g4;
    rr[j] = -1; cnt[j] = 0;
    ms[j][0] = ms[j][1] = 0; mv[j][0] = mv[j][1] = 0.f;
    if (i < nR) {
      rr[j] = __ldg(ta.rows + rp + i);
      const int p0 = __ldg(ap + rr[j]);
      cnt[j] = __ldg(ap + rr[j] + 1) - p0;
      // slots are kept as byte offsets into the staging buffer; padding names slot 0 with value 0
#pragma unroll
      for (int h = 0; h < 2; ++h)
        if (l4 + 4 * h < cnt[j]) {
          ms[j][h] = (int)__ldg(ta.slot + p0 + l4 + 4 * h) * 128;
          mv[j][h] = __ldg(ax + p0 + l4 + 4 * h);
        }
    }
    wmax = max(wmax, cnt[j]);
  }
  wmax = __reduce_max_sync(kFull, wmax);  // longest row this warp owns
  const int kshort = min(wmax, 8);
  // source row of every slot, resolved once per tile: all loads are in flight together
  __syncthreads();  // the previous tile's readers are done with hrow and the buffer
  {
    int v[kTileMaxSlots / NT + 1];
#pragma unroll
    for (int u = 0; u < kTileMaxSlots / NT + 1; ++u) {
      const int s = threadIdx.x + u * NT;
      v[u] = s < nH ? __ldg(ta.halo + hp + s) : 0;
    }
#pragma unroll
    for (int u = 0; u < kTileMaxSlots / NT + 1; ++u) {
      const int s = threadIdx.x + u * NT;
      if (s < nH) hrow[s] = map_row<SRC_RING>(v[u], base, ring_rows, m_local);
    }
  }
  // When the tile's staged rows fill at most half of the buffer, chunks are double-buffered: the
  // copies of chunk c + 1 are in flight while chunk c is computed.
  const bool dbl = 2 * nH <= stage_slots;
  const int half = dbl ? stage_slots / 2 * 128 : 0;  // byte offset of the second buffer
  auto issue = [&](int c0, int buf) {
    if (c0 + l8 * 4 < n_cols) {
      char *dst = reinterpret_cast<char *>(stage) + buf * half + l8 * 16;
      for (int s = g8; s < nH; s += NT / 8)
        cp_async16(dst + s * 128, src + (size_t)hrow[s] * n_cols + c0 + l8 * 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  __syncthreads();  // hrow is complete
  if (dbl) issue(0, 0);
  int cidx = 0;
  for (int c0 = 0; c0 < n_cols; c0 += 32, ++cidx) {
    const int buf = dbl ? (cidx & 1) : 0;
    if (dbl) {
      if (c0 + 32 < n_cols) { issue(c0 + 32, buf ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      issue(c0, 0);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const char *bA = sA + buf * half, *bB = sB + buf * half;
#pragma unroll
    for (int j = 0; j < kTileRowsPerGroup; ++j) {
      if (j * kTileGroups >= nR) continue;  // uniform over the CTA: no rows left for this round
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (k < kshort) {  // uniform over the warp
          const int off = __shfl_sync(kFull, ms[j][k >> 2], k & 3, 4);
          const float v = __shfl_sync(kFull, mv[j][k >> 2], k & 3, 4);
          const float4 x = *reinterpret_cast<const float4 *>(bA + off);
          const float4 y = *reinterpret_cast<const float4 *>(bB + off);
          if (k < cnt[j]) {
            a.x = fmaf(v, x.x, a.x); a.y = fmaf(v, x.y, a.y); a.z = fmaf(v, x.z, a.z); a.w = fmaf(v, x.w, a.w);
            b.x = fmaf(v, y.x, b.x); b.y = fmaf(v, y.y, b.y); b.z = fmaf(v, y.z, b.z); b.w = fmaf(v, y.w, b.w);
          }
        }
      }
      // rows with more than 8 nonzeros: the rest comes straight from the CSR arrays
      if (wmax > 8) {
        const int longest = __reduce_max_sync(kFull, cnt[j]);
        const int p0 = rr[j] >= 0 ? __ldg(ap + rr[j]) : 0;
        for (int q = 8; q < longest; q += 4) {
          int s2 = 0;
          float v2 = 0.f;
          if (q + l4 < cnt[j]) { s2 = (int)__ldg(ta.slot + p0 + q + l4) * 128; v2 = __ldg(ax + p0 + q + l4); }
          for (int k = 0; k < 4; ++k) {
            const int off = __shfl_sync(kFull, s2, k, 4);
            const float v = __shfl_sync(kFull, v2, k, 4);
            const float4 x = *reinterpret_cast<const float4 *>(bA + off);
            const float4 y = *reinterpret_cast<const float4 *>(bB + off);
            if (q + k < cnt[j]) {
              a.x = fmaf(v, x.x, a.x); a.y = fmaf(v, x.y, a.y); a.z = fmaf(v, x.z, a.z); a.w = fmaf(v, x.w, a.w);
              b.x = fmaf(v, y.x, b.x); b.y = fmaf(v, y.y, b.y); b.z = fmaf(v, y.z, b.z); b.w = fmaf(v, y.w, b.w);
            }
          }
        }
      }
      if (rr[j] >= 0) {
        if (relu) {
          a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f); a.z = fmaxf(a.z, 0.f); a.w = fmaxf(a.w, 0.f);
          b.x = fmaxf(b.x, 0.f); b.y = fmaxf(b.y, 0.f); b.z = fmaxf(b.z, 0.f); b.w = fmaxf(b.w, 0.f);
        }
        float *o = dst_row(rr[j]) + c0;
        if (c0 + colA < n_cols) *reinterpret_cast<float4 *>(o + colA) = a;
        if (c0 + colB < n_cols) *reinterpret_cast<float4 *>(o + colB) = b;
      }
    }
    __syncthreads();  // this chunk's readers are done before its buffer is filled again
  }
}

}  // namespace tfk
