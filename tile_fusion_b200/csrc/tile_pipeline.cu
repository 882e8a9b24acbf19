// Gather-tile pipeline: the persistent executor for plans whose items are all gather tiles.
//
// One CTA per SM, split into roles.  A control warp takes the tickets, waits (bounded) for the
// producer tiles an item depends on and posts a tile descriptor, up to four tiles ahead of the
// others, so the latency of the ticket, the item record and the flag checks stays off the data
// path.  Four staging warps copy the tile's source rows -- one 32-column chunk (128 bytes per row)
// at a time -- into one of three shared-memory buffers with 16-byte asynchronous copies whose
// completion is counted by an mbarrier.  Sixteen compute warps wait for a full
// buffer, form the tile's output rows for that chunk from shared memory, store them, and hand
// the buffer back.  Copies for chunk g + 1 (of this or of the next tile) are therefore in
// flight while chunk g is computed, and neither side ever meets the other at a CTA barrier.
//
// The tile's row table travels with its first chunk: eight planes of R (offset, value) pairs -- plane k < 7
// holds nonzero k of every row, the eighth the row id and length -- so that the eight rows a warp works
// on read one contiguous 64-byte line per nonzero and keep nothing about the tile in registers.
//
// Every wait is bounded: a wait that runs out sets the sticky error flag of the launch and the
// thread leaves its loop; the others then run out of their own waits and follow.
#include "kernels.cuh"
#include "gemm_tc.cuh"  // mbarrier helpers
#include "launch.h"

namespace tfk {

namespace {

constexpr int kPipeCompute = 512;  // 16 compute warps: 4 lanes per row, up to 4 rows per lane group
constexpr int kPipeStagers = 128;  // 4 staging warps: 8 lanes per 128-byte slot, 16 slots per step
constexpr int kPipeThreads = kPipeCompute + kPipeStagers + 32;  // + the control warp
constexpr int kPipeStages = 3;     // chunk buffers: two fills are in flight while one chunk is computed
constexpr int kPipeDepth = 4;      // tile descriptors in flight
constexpr int kPipeDoneDepth = 4;  // compute warps are at most kPipeStages chunks, hence tiles, apart
constexpr int kPipeReaders = (kPipeCompute + kPipeStagers) / 32;  // warps that read every descriptor
constexpr int kPipeGroups = kPipeCompute / 4;
constexpr int kPipeRounds = 3;     // rows per lane group: a tile holds at most 3 * 128 rows
constexpr int kPipeIdRegs = 4;     // source row ids per staging lane: 4 * 8 steps * 16 slot groups = 512 slots
constexpr int kPipeMaxSlots = kPipeIdRegs * 8 * 16;

struct PipeShared {
  unsigned long long full[kPipeStages];          // a chunk buffer holds its copies (one arrival per staging thread)
  unsigned long long empty[kPipeStages];          // its readers are done (one arrival per compute warp)
  unsigned long long desc_bar[kPipeDepth];   // descriptor posted (control warp)
  unsigned long long desc_free[kPipeDepth];  // every reader warp has copied it
  int desc[kPipeDepth][8];               // kind (-1: no more work), flag index, tile, rows (rounded up to 8),
                                         // staged rows, their offset in the halo list, offset of the row table
  int done_cnt[kPipeDoneDepth];          // compute warps that finished the tile
};

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait with a warp-uniform answer (the callers run warp collectives afterwards)
__device__ __forceinline__ bool warp_wait(unsigned long long *bar, unsigned parity, int limit) {
  return __all_sync(kFull, mbar_wait(bar, parity, limit));
}
// arrives once every asynchronous copy this thread issued so far has landed
__device__ __forceinline__ void cp_async_arrive(unsigned long long *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(kPipeThreads, 1) tile_pipeline_kernel(const __grid_constant__ Params P) {
  extern __shared__ float4 stage[];  // kPipeStages chunk buffers of tile_slots * 128 bytes, two row tables of 9 * tile_rows pairs
  __shared__ PipeShared sh;
  const int tid = threadIdx.x, lane = tid & 31;
  ExecState *st = P.st;
  const int n_items = P.item_end - P.item_begin;
  const int nchunks = (P.n_cols + 31) / 32;
  const int buf_bytes = P.tile_slots * 128;
  const int meta_bytes = kTileMetaPlanes * P.tile_rows * 8;
  char *meta_base = reinterpret_cast<char *>(stage) + kPipeStages * (size_t)buf_bytes;
  const int limit = P.spin_limit;
  if (tid == 0) {
    for (int b = 0; b < kPipeStages; ++b) { mbar_init(&sh.full[b], kPipeStagers); mbar_init(&sh.empty[b], kPipeCompute / 32); }
    for (int i = 0; i < kPipeDepth; ++i) {
      mbar_init(&sh.desc_bar[i], 1);
      mbar_init(&sh.desc_free[i], kPipeReaders);
    }
    for (int i = 0; i < kPipeDoneDepth; ++i) sh.done_cnt[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid >= kPipeCompute + kPipeStagers) {
    // ------------------------------------------------------------------ control warp
    int nxt = 0;
    if (lane == 0) nxt = atomicAdd(&st->ticket, 1);
    bool ok = true;
    for (int t = 0;; ++t) {
      const int slot = t & (kPipeDepth - 1);
      if (t >= kPipeDepth && !warp_wait(&sh.desc_free[slot], (t / kPipeDepth - 1) & 1, limit)) { ok = false; break; }
      const int cur = __shfl_sync(kFull, nxt, 0);
      int4 ia = make_int4(-1, 0, 0, 0), ib = make_int4(0, 0, 0, 0);
      if (cur < n_items) {
        if (lane == 0) nxt = atomicAdd(&st->ticket, 1);  // its latency hides behind this item's checks
        ia = __ldg(P.items + 2 * (size_t)(P.item_begin + cur));
        ib = __ldg(P.items + 2 * (size_t)(P.item_begin + cur) + 1);
        if (ib.x > 0) {
          const bool w = ia.x == 5 ? wait_for(&st->prod_wm, P.prod_done, ib.x, P.epoch, st, limit, lane)
                                   : wait_for(&st->cons_wm, P.cons_done, ib.x, P.epoch, st, limit, lane);
          if (!w) ia.x = -1;
        }
      }
      if (lane == 0) {
        volatile int *d = sh.desc[slot];
        d[0] = ia.x; d[1] = ia.y; d[2] = ia.z; d[3] = ia.w;
        d[4] = ib.y; d[5] = ib.z; d[6] = ib.w;
        mbar_arrive(&sh.desc_bar[slot]);
      }
      __syncwarp();
      if (ia.x < 0) break;
    }
    if (!ok) atomicExch(&st->error, 1);
  } else if (tid >= kPipeCompute) {
    // ------------------------------------------------------------------ staging warps
    const int ptid = tid - kPipeCompute;
    const int g8 = ptid >> 3, l8 = ptid & 7;
    unsigned g = 0;  // chunk sequence number of this CTA
    bool ok = true;
    for (int t = 0; ok; ++t) {
      const int slot = t & (kPipeDepth - 1);
      volatile int *d = sh.desc[slot];
      if (!warp_wait(&sh.desc_bar[slot], (t / kPipeDepth) & 1, limit)) { ok = false; break; }
      const int kind = d[0], nRt = d[3], nH = d[4], hp = d[5], moff = d[6];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.desc_free[slot]);
      if (kind < 0) break;
      // The control warp acquired (gpu scope) the flags of the tiles this one reads before it posted the
      // descriptor; the descriptor barrier (release / acquire within the CTA) carries that order over to
      // this thread's copies, which read T from L2.
      const TileArrays &ta = kind == 4 ? P.pt : P.ct;
      const float *src = kind == 4 ? P.in0 : P.inter;
      // the tile's source row ids, fetched in one batch: lane l of a slot group holds the ids of the
      // group's steps l, l + 8, ... (step i covers slot g8 + 16 i)
      int hid[kPipeIdRegs];
#pragma unroll
      for (int u = 0; u < kPipeIdRegs; ++u) {
        const int s = g8 + 16 * (u * 8 + l8);
        hid[u] = s < nH ? __ldg(ta.halo + hp + s) : 0;
      }
      for (int c = 0; c < nchunks; ++c, ++g) {
        const int buf = g % kPipeStages;
        if (!warp_wait(&sh.empty[buf], ((g / kPipeStages) & 1) ^ 1, limit)) { ok = false; break; }
        const int c0 = c * 32 + l8 * 4;
        char *dst = reinterpret_cast<char *>(stage) + (size_t)buf * buf_bytes + l8 * 16;
        const float *s0 = src + c0;
        const bool live = c0 < P.n_cols;
#pragma unroll
        for (int u = 0; u < kPipeIdRegs; ++u) {
          if (128 * u >= nH) break;  // uniform over the CTA
#pragma unroll
          for (int l = 0; l < 8; ++l) {
            const int s = g8 + 16 * (u * 8 + l);
            const int r = __shfl_sync(kFull, hid[u], l, 8);
            if (live && s < nH) cp_async16(dst + s * 128, s0 + (size_t)r * P.n_cols);
          }
        }
        if (c == 0) {  // the tile's row table (16-byte pieces, contiguous in global memory)
          // Its buffer served tile t - 2, whose last chunk is nchunks + 1 chunks back.  The wait above covers
          // the chunks up to g - kPipeStages; a closer one (single-chunk tiles) is waited for here.
          const unsigned gl = g - nchunks - 1;
          if (t >= 2 && nchunks + 1 < kPipeStages &&
              !warp_wait(&sh.empty[gl % kPipeStages], (gl / kPipeStages) & 1, limit)) { ok = false; break; }
          const int4 *msrc = reinterpret_cast<const int4 *>(ta.meta) + moff;
          char *mdst = meta_base + (size_t)(t & 1) * meta_bytes;
          const int n16 = kTileMetaPlanes * nRt / 2;
          for (int q = ptid; q < n16; q += kPipeStagers) cp_async16(mdst + q * 16, msrc + q);
        }
        cp_async_arrive(&sh.full[buf]);
      }
    }
    if (!ok) atomicExch(&st->error, 1);
  } else {
    // ------------------------------------------------------------------ compute warps
    const int g4 = tid >> 2, l4 = tid & 3;
    const int colA = ((g4 & 1) * 16) + l4 * 4, colB = (((g4 & 1) ^ 1) * 16) + l4 * 4;  // floats within the chunk
    unsigned g = 0;
    bool ok = true;
    for (int t = 0; ok; ++t) {
      const int slot = t & (kPipeDepth - 1);
      volatile int *d = sh.desc[slot];
      if (!warp_wait(&sh.desc_bar[slot], (t / kPipeDepth) & 1, limit)) { ok = false; break; }
      const int kind = d[0], block = d[1], nRt = d[3];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.desc_free[slot]);
      if (kind < 0) break;
      const bool first = kind == 4;
      const TileArrays &ta = first ? P.pt : P.ct;
      const int *ap = first ? P.f_ap : P.s_ap;
      const float *ax = first ? P.f_ax : P.s_ax;
      float *dst = first ? P.inter : P.out;
      const bool relu = !first && P.relu != 0;
      // row table of this tile: plane k at k * nRt pairs, the row ids and lengths in plane 8
      const int2 *meta = reinterpret_cast<const int2 *>(meta_base + (size_t)(t & 1) * meta_bytes);
      for (int c = 0; c < nchunks; ++c, ++g) {
        const int buf = g % kPipeStages;
        if (!warp_wait(&sh.full[buf], (g / kPipeStages) & 1, limit)) { ok = false; break; }
        const char *bA = reinterpret_cast<const char *>(stage) + (size_t)buf * buf_bytes + colA * 4;
        const char *bB = reinterpret_cast<const char *>(stage) + (size_t)buf * buf_bytes + colB * 4;
        const int c0 = c * 32;
#pragma unroll
        for (int j = 0; j < kPipeRounds; ++j) {
          if (j * kPipeGroups + (tid >> 5) * 8 >= nRt) continue;  // this warp has no rows in round j
          const int i = j * kPipeGroups + g4;
          const int2 rc = meta[kTileMetaNnz * nRt + i];  // row id (-1: padding), length
          const int longest = __reduce_max_sync(kFull, rc.y);
          const int kmax = min(longest, kTileMetaNnz);
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int k = 0; k < kTileMetaNnz; ++k) {
            if (k < kmax) {  // uniform over the warp
              const int2 m = meta[k * nRt + i];       // byte offset of the slot, value bits ({0, 0} past the row's end)
              const float v = __int_as_float(m.y);
              const float4 x = *reinterpret_cast<const float4 *>(bA + m.x);
              const float4 y = *reinterpret_cast<const float4 *>(bB + m.x);
              if (k < rc.y) {  // padding names slot 0, whose contents must not reach the sum
                a.x = fmaf(v, x.x, a.x); a.y = fmaf(v, x.y, a.y); a.z = fmaf(v, x.z, a.z); a.w = fmaf(v, x.w, a.w);
                b.x = fmaf(v, y.x, b.x); b.y = fmaf(v, y.y, b.y); b.z = fmaf(v, y.z, b.z); b.w = fmaf(v, y.w, b.w);
              }
            }
          }
          if (longest > kTileMetaNnz) {  // longer rows: the rest comes straight from the CSR arrays
            const int p0 = rc.x >= 0 ? __ldg(ap + rc.x) : 0;
            for (int q = kTileMetaNnz; q < longest; q += 4) {
              int s2 = 0;
              float v2 = 0.f;
              if (q + l4 < rc.y) { s2 = (int)__ldg(ta.slot + p0 + q + l4) * 128; v2 = __ldg(ax + p0 + q + l4); }
              for (int k = 0; k < 4; ++k) {
                const int off = __shfl_sync(kFull, s2, k, 4);
                const float v = __shfl_sync(kFull, v2, k, 4);
                const float4 x = *reinterpret_cast<const float4 *>(bA + off);
                const float4 y = *reinterpret_cast<const float4 *>(bB + off);
                if (q + k < rc.y) {
                  a.x = fmaf(v, x.x, a.x); a.y = fmaf(v, x.y, a.y); a.z = fmaf(v, x.z, a.z); a.w = fmaf(v, x.w, a.w);
                  b.x = fmaf(v, y.x, b.x); b.y = fmaf(v, y.y, b.y); b.z = fmaf(v, y.z, b.z); b.w = fmaf(v, y.w, b.w);
                }
              }
            }
          }
          if (rc.x >= 0) {
            if (relu) {
              a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f); a.z = fmaxf(a.z, 0.f); a.w = fmaxf(a.w, 0.f);
              b.x = fmaxf(b.x, 0.f); b.y = fmaxf(b.y, 0.f); b.z = fmaxf(b.z, 0.f); b.w = fmaxf(b.w, 0.f);
            }
            float *o = dst + (size_t)rc.x * P.n_cols + c0;
            if (c0 + colA < P.n_cols) *reinterpret_cast<float4 *>(o + colA) = a;
            if (c0 + colB < P.n_cols) *reinterpret_cast<float4 *>(o + colB) = b;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty[buf]);
      }
      if (!ok) break;
      if (first) {
        // the last compute warp to finish the tile publishes it
        __syncwarp();
        if (lane == 0) {
          // orders this warp's stores before the count within the CTA; the warp that publishes fences at
          // gpu scope, which covers everything that happened before its own increment
          __threadfence_block();
          int *cntp = &sh.done_cnt[t & (kPipeDoneDepth - 1)];
          if (atomicAdd(cntp, 1) == kPipeCompute / 32 - 1) {
            *cntp = 0;
            publish(P.prod_done, block, P.epoch);
          }
        }
      }
    }
    if (!ok) atomicExch(&st->error, 1);
  }
  // the last CTA out rewinds the ticket counter (and, after the last phase, the watermarks)
  __syncthreads();
  if (tid == 0) {
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

}  // namespace

// shared memory the pipeline needs for tiles of up to tile_slots staged rows and tile_rows rows; 0 when
// it cannot run them
size_t tile_pipeline_smem(int tile_slots, int tile_rows) {
  if (tile_slots <= 0 || tile_slots > kPipeMaxSlots || tile_rows <= 0 || tile_rows > kPipeRounds * kPipeGroups) return 0;
  return (size_t)kPipeStages * tile_slots * 128 + (size_t)2 * kTileMetaPlanes * tile_rows * 8;
}

cudaError_t launch_tile_pipeline(int grid, const Params &p, cudaStream_t s) {
  const size_t dyn = tile_pipeline_smem(p.tile_slots, p.tile_rows);
  if (dyn == 0) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute((const void *)tile_pipeline_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
  if (e != cudaSuccess) return e;
  tile_pipeline_kernel<<<grid, kPipeThreads, dyn, s>>>(p);
  return cudaGetLastError();
}

}  // namespace tfk
