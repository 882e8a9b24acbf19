// C ABI of libtilefusion_b200: plans (device-resident operators + item lists) and executors.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <climits>
#include <cstring>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <string>
#include <vector>

#include "gemm_tc_host.h"
#include "host_stage.h"
#include "kernels.cuh"
#include "lattice_march.h"
#include "launch.h"
#include "tf_internal.h"

namespace {

using tf::fail;

#define TF_CUDA(call)                                                                         \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return fail(TF_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));          \
  } while (0)

template <class T>
struct DevBuf {
  T *p = nullptr;
  size_t n = 0;
  ~DevBuf() { if (p) cudaFree(p); }
  int alloc(size_t count) {
    if (p) { cudaFree(p); p = nullptr; }
    n = count;
    if (count == 0) return TF_OK;
    cudaError_t e = cudaMalloc(&p, count * sizeof(T));
    if (e != cudaSuccess) { p = nullptr; return fail(TF_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e)); }
    return TF_OK;
  }
  int upload(const T *h, size_t count) {
    int rc = alloc(count);
    if (rc != TF_OK || count == 0) return rc;
    TF_CUDA(cudaMemcpy(p, h, count * sizeof(T), cudaMemcpyHostToDevice));
    return TF_OK;
  }
  int upload(const std::vector<T> &v) { return upload(v.data(), v.size()); }
};

struct DevCsr {
  int m = 0, n = 0;
  DevBuf<int> ap, ai;
  DevBuf<float> ax;
  int upload(const tf_csr &h) {
    m = h.m; n = h.n;
    int rc = ap.upload(h.ap, (size_t)h.m + 1);
    if (rc == TF_OK) rc = ai.upload(h.ai, (size_t)h.ap[h.m]);
    if (rc == TF_OK) rc = ax.upload(h.ax, (size_t)h.ap[h.m]);
    return rc;
  }
};

}  // namespace

struct tf_plan {
  int chain = 0;  // 0 SpMM-SpMM, 1 GeMM-SpMM, 2 SDDMM-SpMM
  int mode = TF_MODE_STREAM;
  int m = 0, n_cols = 0, k_dim = 0, halo_rows = 0;
  int first_cols = 0;  // columns of the first operator (rows of C)
  DevCsr first, second;
  bool first_is_second = false;
  tf::HostPlan hp;
  DevBuf<int4> items;
  DevBuf<int> seg_t, seg_out;  // rows of T / D that are accumulated atomically from segments of a heavy row
  DevBuf<int> prod_done, cons_done;
  DevBuf<tfk::ExecState> state;
  DevBuf<float> inter, sendbuf;
  // gather tiles (stream / unfused mode)
  struct DevTiling {
    DevBuf<int> row_ptr, rows, halo_ptr, halo;
    DevBuf<unsigned short> slot;
    DevBuf<int2> meta;
    std::vector<int> meta_off;  // per tile: offset of its row table, in 16-byte units
    bool on = false;
    // ap, ax: host CSR of the operator the tiling belongs to; with_meta: build the pipeline's row tables
    int upload(const tf::Tiling &t, const int *ap, const float *ax, bool with_meta) {
      on = t.tiled;
      if (!on) return TF_OK;
      int rc = TF_OK;
      if (with_meta) {
        const int nt = t.tiles();
        meta_off.assign(nt + 1, 0);
        size_t pairs = 0;
        for (int k = 0; k < nt; ++k) {
          meta_off[k] = (int)(pairs / 2);
          pairs += (size_t)tfk::kTileMetaPlanes * ((t.tile_row_ptr[k + 1] - t.tile_row_ptr[k] + 7) / 8 * 8);
        }
        std::vector<int2> m(pairs, make_int2(0, 0));
        for (int k = 0; k < nt; ++k) {
          const int rp = t.tile_row_ptr[k], nR = t.tile_row_ptr[k + 1] - rp, R = (nR + 7) / 8 * 8;
          int2 *blk = m.data() + 2 * (size_t)meta_off[k];
          for (int i = 0; i < R; ++i) blk[tfk::kTileMetaNnz * R + i] = make_int2(-1, 0);
          for (int i = 0; i < nR; ++i) {
            const int r = t.rows[rp + i], cnt = ap[r + 1] - ap[r];
            blk[tfk::kTileMetaNnz * R + i] = make_int2(r, cnt);
            for (int q = 0; q < std::min(cnt, tfk::kTileMetaNnz); ++q) {
              int2 e;
              e.x = (int)t.slot[ap[r] + q] * 128;
              std::memcpy(&e.y, &ax[ap[r] + q], 4);
              blk[q * R + i] = e;
            }
          }
        }
        rc = meta.upload(m);
      }
      if (rc == TF_OK) rc = row_ptr.upload(t.tile_row_ptr);
      if (rc == TF_OK) rc = rows.upload(t.rows);
      if (rc == TF_OK) rc = halo_ptr.upload(t.tile_halo_ptr);
      if (rc == TF_OK) rc = halo.upload(t.halo);
      if (rc == TF_OK) rc = slot.upload(t.slot);
      return rc;
    }
    tfk::TileArrays view() const {
      tfk::TileArrays a{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
      if (on) a = tfk::TileArrays{row_ptr.p, rows.p, halo_ptr.p, halo.p, slot.p, meta.p};
      return a;
    }
  } ptile, ctile;
  size_t dyn_smem = 0;
  int tile_slots = 0;
  bool pipe = false;  // every item of phases 1 and 2 is a gather tile: run them on the tile pipeline
  int pipe_grid = 0, pipe_rows = 0;
  // tensor-core dense producer
  bool use_tc = false;
  int sm_count = 0;
  DevBuf<float> w_hi, w_lo;  // split, transposed weight [n_cols][k]
  CUtensorMap tm_whi, tm_wlo;
  int tile_info[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // producer bx,by,bz,tiles ; consumer bx,by,bz,tiles
  // plane-marching executor (both operators are star stencils on one grid)
  struct March {
    bool on = false, same = false;  // same: one operator on both sides (B == A)
    bool identity_first = false;    // GeMM-SpMM: the first operator is the identity, the operand is the producer's T
    bool halo_lo = false, halo_hi = false;  // a neighbour rank below / above supplies plane -1 / nz of T
    int nx = 0, ny = 0, nz = 0, ncls_f = 0, ncls_a = 0, z_shift = 0, grid = 0, n_items = 0, n_phase1 = 0;
    long long planes_c = 0;
    DevBuf<unsigned> pcls_f, pcls_a;
    std::vector<float> dict_f, dict_a;   // host copies: the dictionaries travel as kernel parameters
    DevBuf<int4> items;
    int first_idle_sm = INT_MAX;
    int n_boundary = 0;              // rows of the neighbours' halo that this rank produces (phase 0)
    DevBuf<int> b_ap, b_ai;
    DevBuf<float> b_ax;
    DevBuf<tfk::MarchState> st;   // [0]: tickets of phase 1 (or of the whole grid), [1]: of phase 2 -- the two may run side by side
    std::vector<tf::MarchItem> host_items;
    // host-pointer path (single GPU): the grid again, cut into slabs of planes that run one launch each while the
    // planes of C for the next slab arrive and the planes of D of the one before leave
    struct Slab { int item_begin, item_end, z_begin, z_end; };
    std::vector<Slab> slabs;
  } march;
  // schedule mode
  DevBuf<int> s_ptr2, s_id, s_type, s_ker;
  int s_n1 = 0;
  std::vector<int> s_ptr1;
  bool s_has_ker = false;
  // host-pointer path: staging buffers, streams and the segments of the copy/compute pipeline
  struct Seg { int item_begin, item_end; long long in_rows, out_rows; };
  std::vector<Seg> segs;
  cudaStream_t s_h2d = nullptr, s_run = nullptr, s_d2h = nullptr;
  std::vector<cudaEvent_t> ev_in, ev_run;
  std::unique_ptr<tf::HostPipe> host_pipe;   // copies of the host-pointer calls; pinned slots for pageable arrays (host_stage.h)
  ~tf_plan() {
    for (cudaEvent_t e : ev_in) cudaEventDestroy(e);
    for (cudaEvent_t e : ev_run) cudaEventDestroy(e);
    if (s_h2d) cudaStreamDestroy(s_h2d);
    if (s_run) cudaStreamDestroy(s_run);
    if (s_d2h) cudaStreamDestroy(s_d2h);
  }
  DevBuf<float> h_in0, h_in1, h_in2, h_out;
  int grid = 0, vec = 1, ch = 1;
  int epoch = 1;  // flags start at 0, so no pass may use 0
  int spin_limit = 1 << 22;
  long long launches = 0;
  int device = 0;
};

namespace {

int device_ready(int *sm_count) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TF_ERR_CUDA, std::string("no usable CUDA device: ") + cudaGetErrorString(e));
  cudaDeviceProp prop;
  TF_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major < 10) return fail(TF_ERR_CUDA, "this library is built for sm_100a (B200) only");
  *sm_count = prop.multiProcessorCount;
  return TF_OK;
}

int default_rows_per_block(int n_cols, bool gemm) {
  if (gemm) return 64;
  return n_cols >= 128 ? 64 : 128;
}

// pt, ct: the gather tiles of a plan the tile pipeline runs; its tile items carry the extents of the
// tile ({kind, flag, tile, rows rounded up to 8} {need, staged rows, offset of the staged rows, offset
// of the row table}), so that the kernel needs no further lookup before it can start on a tile.
int upload_items(tf_plan &p, const tf::Tiling *pt = nullptr, const tf::Tiling *ct = nullptr) {
  std::vector<int4> raw(2 * p.hp.items.size());
  for (size_t i = 0; i < p.hp.items.size(); ++i) {
    const tf::Item &it = p.hp.items[i];
    raw[2 * i] = make_int4(it.kind, it.block, it.row_begin, it.row_end);
    raw[2 * i + 1] = make_int4(it.need, it.base, it.aux0, it.aux1);
    if (p.pipe && (it.kind == tf::ITEM_PRODUCE_TILED || it.kind == tf::ITEM_CONSUME_TILED)) {
      const tf::Tiling &t = it.kind == tf::ITEM_PRODUCE_TILED ? *pt : *ct;
      const int k = it.row_begin;
      const tf_plan::DevTiling &dt = it.kind == tf::ITEM_PRODUCE_TILED ? p.ptile : p.ctile;
      raw[2 * i].w = (t.tile_row_ptr[k + 1] - t.tile_row_ptr[k] + 7) / 8 * 8;
      raw[2 * i + 1] = make_int4(it.need, t.tile_halo_ptr[k + 1] - t.tile_halo_ptr[k], t.tile_halo_ptr[k], dt.meta_off[k]);
    }
  }
  int rc = p.items.upload(raw);
  if (rc == TF_OK && !p.hp.seg_t_rows.empty()) rc = p.seg_t.upload(p.hp.seg_t_rows);
  if (rc == TF_OK && !p.hp.seg_out_rows.empty()) rc = p.seg_out.upload(p.hp.seg_out_rows);
  return rc;
}

// Rows that segments of a heavy row add into start a pass at zero; a final ReLU is applied to them after it.
int segments_begin(tf_plan &p, const tfk::Params &P, cudaStream_t s) {
  TF_CUDA(tfk::launch_rows_fix(p.seg_t.p, (int)p.hp.seg_t_rows.size(), p.n_cols, p.inter.p, false, s));
  TF_CUDA(tfk::launch_rows_fix(p.seg_out.p, (int)p.hp.seg_out_rows.size(), p.n_cols, P.out, false, s));
  return TF_OK;
}
int segments_end(tf_plan &p, const tfk::Params &P, cudaStream_t s) {
  if (P.relu) TF_CUDA(tfk::launch_rows_fix(p.seg_out.p, (int)p.hp.seg_out_rows.size(), p.n_cols, P.out, true, s));
  return TF_OK;
}

int finish_plan(tf_plan &p, const tf_plan_opts &o, int sm_count, bool ring) {
  const bool a16 = true;  // buffers owned by the plan are 256-byte aligned; callers' pointers are checked per call
  tfk::choose_shape(p.n_cols, a16, &p.vec, &p.ch);
  if (p.dyn_smem > 0) { p.vec = 4; p.ch = 1; }
  int occ = tfk::stream_occupancy(p.chain, p.vec, p.ch, ring, p.dyn_smem);
  if (occ <= 0) return fail(TF_ERR_CUDA, "occupancy query failed for the executor kernel");
  // The resident-CTA query answers 1 for any kernel that allocates tensor memory.  Two CTAs of this
  // kernel fit an SM (256 of 512 tensor-memory columns each, half the shared memory, 64 registers), and
  // the executor does not depend on the answer for progress: only running CTAs hold tickets.
  if (p.use_tc && occ == 1 && p.dyn_smem <= 106 * 1024) occ = 2;
  if (o.ctas_per_sm > 0) occ = std::min(occ, o.ctas_per_sm);
  p.grid = sm_count * occ;
  return TF_OK;
}

int zero_state(tf_plan &p) {
  int rc = p.state.alloc(1);
  if (rc != TF_OK) return rc;
  TF_CUDA(cudaMemset(p.state.p, 0, sizeof(tfk::ExecState)));
  const size_t np = (size_t)p.hp.n_prod, nc = (size_t)p.hp.n_cons;
  rc = p.prod_done.alloc(std::max<size_t>(np, 1));
  if (rc == TF_OK) rc = p.cons_done.alloc(std::max<size_t>(nc, 1));
  if (rc != TF_OK) return rc;
  TF_CUDA(cudaMemset(p.prod_done.p, 0, p.prod_done.n * sizeof(int)));
  TF_CUDA(cudaMemset(p.cons_done.p, 0, p.cons_done.n * sizeof(int)));
  return TF_OK;
}

int check_opts(const tf_plan_opts *o, tf_plan_opts &out) {
  std::memset(&out, 0, sizeof(out));
  out.slack_blocks = -1;
  if (o) out = *o;
  if (out.mode < TF_MODE_STREAM || out.mode > TF_MODE_UNFUSED) return fail(TF_ERR_ARG, "plan: unknown mode");
  if (out.rows_per_block < 0 || out.halo_rows < 0 || out.n_boundary < 0) return fail(TF_ERR_ARG, "plan: negative option");
  if (out.tile_slots > tfk::kTileMaxSlots) return fail(TF_ERR_ARG, "plan: tile_slots above the shared-memory capacity");
  if (out.n_boundary > 0 && !out.boundary_rows) return fail(TF_ERR_ARG, "plan: boundary_rows is null");
  return TF_OK;
}

int load_schedule(tf_plan &p, const tf_schedule *s, bool need_ker) {
  if (!s) return fail(TF_ERR_ARG, "plan: TF_MODE_SCHEDULE needs a schedule");
  if (need_ker && !s->has_ker) return fail(TF_ERR_ARG, "plan: GeMM-SpMM needs a schedule with ker_begin (separated packing)");
  for (size_t k = 0; k < s->id.size(); ++k)
    if (s->id[k] < 0 || s->id[k] >= p.m || (s->type[k] != 0 && s->type[k] != 1))
      return fail(TF_ERR_ARG, "plan: schedule row id or type out of range");
  if (need_ker) {
    const int np = s->ptr1[s->n1];
    for (int w = 0; w < np; ++w) {
      const int kb = s->ptr2[w], ke1 = s->ker[2 * w];
      for (int k = kb; k < ke1; ++k)
        if (s->type[k] != 0 || s->id[k] != s->id[kb] + (k - kb))
          return fail(TF_ERR_ARG, "plan: GeMM-SpMM tiles must list consecutive first-loop rows");
      for (int k = ke1; k < s->ptr2[w + 1]; ++k)
        if (s->type[k] != 1) return fail(TF_ERR_ARG, "plan: ker_begin does not separate the two loops");
    }
  }
  p.s_n1 = s->n1;
  p.s_ptr1 = s->ptr1;
  p.s_has_ker = s->has_ker;
  int rc = p.s_ptr2.upload(s->ptr2);
  if (rc == TF_OK) rc = p.s_id.upload(s->id);
  if (rc == TF_OK) rc = p.s_type.upload(s->type);
  if (rc == TF_OK && s->has_ker) rc = p.s_ker.upload(s->ker);
  return rc;
}

void build_segments(tf_plan &p, int n_seg);

static_assert(tf::kMarchMaxClasses == tfk::kMarchMaxClassesDev, "host and device class limits differ");

// Plane-marching executor: taken when both operators of an SpMM-SpMM chain are star stencils on the same
// grid (lattice.cpp).  The general plan is built as well and serves calls whose operands are not 16-byte
// aligned.
// Fp == null: the first operator is the identity (GeMM-SpMM: the dense producer has written T, and the marching
// kernel computes D = A * (I * T); the products with the identity's zeros and its one are exact, so D is what the
// CSR consumer gives).
int build_march(tf_plan &p, const tf_csr *Fp, const tf_csr &A, int halo_rows, int sm_count, const std::vector<int> &boundary_rows) {
  tf::LatticeOp lf, la;
  int rc = TF_OK;
  if (Fp) {
    rc = tf::analyse_lattice_operator(Fp->m, Fp->n, Fp->ap, Fp->ai, Fp->ax, 0, lf);
    if (rc != TF_OK || !lf.ok) return rc;
  }
  if (Fp == &A && halo_rows == 0) la = lf;
  else {
    rc = tf::analyse_lattice_operator(A.m, A.n, A.ap, A.ai, A.ax, halo_rows, la);
    if (rc != TF_OK || !la.ok) return rc;
  }
  if (!Fp) {
    lf.ok = true; lf.nx = la.nx; lf.ny = la.ny; lf.nz = la.nz; lf.n_classes = 1;
    lf.dict.assign(16, 0.f);
    lf.dict[3] = 1.f;                    // class 0: centre coefficient 1; class 1: all zero
    lf.patch_cls = la.patch_cls;         // same rows exist: zero class where A has none
    for (uint32_t &w : lf.patch_cls) {
      uint32_t v = 0;
      for (int b = 0; b < 4; ++b) v |= (uint32_t)(((w >> (8 * b)) & 255u) == (uint32_t)la.n_classes ? 1u : 0u) << (8 * b);
      w = v;
    }
  }
  const tf_csr &F = Fp ? *Fp : A;
  if (la.nx != lf.nx || la.ny != lf.ny || la.nz != lf.nz) return TF_OK;
  if (halo_rows == 0 && (la.ghost_lo || la.ghost_hi)) return TF_OK;
  // with a neighbour rank below (above), the first operator must reach one plane of C below (above) the rank's
  // own: the boundary planes of T that the rank computes itself need them
  if (lf.ghost_lo > 1 || lf.ghost_hi > 1) return TF_OK;
  const int occ = tfk::march_ctas_per_sm();
  if (occ <= 0) return TF_OK;  // the kernel does not fit this device: general path
  tf_plan::March &M = p.march;
  M.nx = lf.nx; M.ny = lf.ny; M.nz = lf.nz;
  M.ncls_f = lf.n_classes; M.ncls_a = la.n_classes;
  M.z_shift = lf.ghost_lo;
  M.planes_c = (long long)lf.nz + lf.ghost_lo + lf.ghost_hi;
  M.halo_lo = halo_rows > 0 && la.ghost_lo; M.halo_hi = halo_rows > 0 && la.ghost_hi;
  // With a halo exchange in flight a few SMs are left to the NCCL send / receive kernels: the persistent CTAs of
  // phase 1 would otherwise hold every SM until they finish, and the exchange would only start then.
  // With neighbour ranks the last SMs stay free while phase 1 runs: the kernels of the halo exchange and phase 2
  // start there, beside the persistent CTAs.
  M.grid = sm_count * occ;
  M.first_idle_sm = halo_rows > 0 ? std::max(1, sm_count - 6) : INT_MAX;
  const int working = std::min(sm_count, M.first_idle_sm) * occ;
  // phase 1: the planes of D that need no plane of T from a neighbour rank; phase 2: the first and / or last plane
  const int z1 = M.halo_lo ? 1 : 0, z2 = M.nz - (M.halo_hi ? 1 : 0);
  tf::build_march_items(M.nx, M.ny, z1, z2, p.n_cols, tfk::kMarchW, tfk::kMarchH, tfk::kMarchCols, working, 1, M.host_items);
  M.n_phase1 = (int)M.host_items.size();
  if (M.halo_lo) tf::build_march_items(M.nx, M.ny, 0, 1, p.n_cols, tfk::kMarchW, tfk::kMarchH, tfk::kMarchCols, M.grid, 1, M.host_items);
  if (M.halo_hi && M.nz > 1)
    tf::build_march_items(M.nx, M.ny, M.nz - 1, M.nz, p.n_cols, tfk::kMarchW, tfk::kMarchH, tfk::kMarchCols, M.grid, 1, M.host_items);
  M.n_items = (int)M.host_items.size();
  if (halo_rows == 0 && M.nz >= 8) {
    const int n_slabs = std::min(32, M.nz / 4);
    for (int sl = 0; sl < n_slabs; ++sl) {
      const int za = (int)((long long)M.nz * sl / n_slabs), zb = (int)((long long)M.nz * (sl + 1) / n_slabs);
      const int b = (int)M.host_items.size();
      tf::build_march_items(M.nx, M.ny, za, zb, p.n_cols, tfk::kMarchW, tfk::kMarchH, tfk::kMarchCols, M.grid, 1, M.host_items);
      M.slabs.push_back(tf_plan::March::Slab{b, (int)M.host_items.size(), za, zb});
    }
  }
  std::vector<int4> raw(2 * M.host_items.size());
  for (size_t i = 0; i < M.host_items.size(); ++i) {
    const tf::MarchItem &it = M.host_items[i];
    raw[2 * i] = make_int4(it.x0, it.y0, it.zs, it.ze);
    raw[2 * i + 1] = make_int4(it.c0, it.flags, 0, 0);
  }
  rc = M.items.upload(raw);
  if (rc == TF_OK) rc = M.pcls_f.upload(lf.patch_cls);
  M.dict_f = lf.dict;
  M.same = Fp == &A && halo_rows == 0;
  M.identity_first = Fp == nullptr;
  if (rc == TF_OK && !M.same) rc = M.pcls_a.upload(la.patch_cls);
  M.dict_a = M.same ? lf.dict : la.dict;
  if (rc == TF_OK) rc = M.st.alloc(2);
  if (rc == TF_OK && Fp && !boundary_rows.empty()) {
    // phase 0 of such a plan: the boundary rows of the first operator as a CSR of their own, in send-buffer order
    std::vector<int> bp(1, 0), bi;
    std::vector<float> bx;
    for (int r : boundary_rows) {
      bi.insert(bi.end(), F.ai + F.ap[r], F.ai + F.ap[r + 1]);
      bx.insert(bx.end(), F.ax + F.ap[r], F.ax + F.ap[r + 1]);
      bp.push_back((int)bi.size());
    }
    M.n_boundary = (int)boundary_rows.size();
    rc = M.b_ap.upload(bp);
    if (rc == TF_OK) rc = M.b_ai.upload(bi);
    if (rc == TF_OK) rc = M.b_ax.upload(bx);
  }
  if (rc != TF_OK) return rc;
  TF_CUDA(cudaMemset(M.st.p, 0, 2 * sizeof(tfk::MarchState)));
  M.on = true;
  return TF_OK;
}

bool aligned(const void *q, size_t a);

// One launch over the march items [item_begin, item_end).
int run_march(tf_plan &p, const float *C, float *D, int item_begin, int item_end, bool with_halo, cudaStream_t s) {
  tf_plan::March &M = p.march;
  if (item_end <= item_begin) { p.launches = 0; return TF_OK; }
  CUtensorMap tm;
  const int mr = tfk::march_make_map(&tm, C, p.n_cols, M.nx, M.ny, M.planes_c);
  if (mr != 0) return fail(TF_ERR_CUDA, "cuTensorMapEncodeTiled failed for the dense operand (code " + std::to_string(mr) + ")");
  tfk::MarchParams Q;
  std::memset(&Q, 0, sizeof(Q));
  Q.pcls_f = M.pcls_f.p; Q.pcls_a = M.same ? M.pcls_f.p : M.pcls_a.p;
  std::memcpy(Q.dict_f, M.dict_f.data(), std::min(sizeof(Q.dict_f), M.dict_f.size() * sizeof(float)));
  std::memcpy(Q.dict_a, M.dict_a.data(), std::min(sizeof(Q.dict_a), M.dict_a.size() * sizeof(float)));
  Q.ncls_f = M.ncls_f; Q.ncls_a = M.ncls_a;
  Q.out = D;
  Q.items = M.items.p;
  Q.item_begin = item_begin; Q.item_end = item_end;
  Q.st = M.st.p + (with_halo ? 1 : 0);
  Q.nx = M.nx; Q.ny = M.ny; Q.nz = M.nz;
  Q.pnx = (M.nx + 1) / 2; Q.pny = (M.ny + 1) / 2;
  Q.n_cols = p.n_cols;
  Q.z_shift = M.z_shift;
  if (with_halo) {  // the received planes sit after the local rows of the intermediate: the lower neighbour's first
    const size_t plane = (size_t)M.nx * M.ny * p.n_cols;
    const float *halo = p.inter.p + (size_t)(p.hp.inter_rows - p.halo_rows) * p.n_cols;
    if (M.halo_lo) Q.t_lo = halo;
    if (M.halo_hi) Q.t_hi = halo + (M.halo_lo ? plane : 0);
  }
  Q.wait_limit = p.spin_limit;
  // phase 1 of a plan with neighbour ranks keeps the last SMs free; every other launch uses what it finds
  const bool keep_free = !with_halo && p.halo_rows > 0;
  Q.first_idle_sm = keep_free ? M.first_idle_sm : INT_MAX;
  TF_CUDA(tfk::launch_lattice_march(keep_free ? M.grid : std::min(M.grid, std::max(1, item_end - item_begin)), tm, Q, s));
  p.launches = 1;
  return TF_OK;
}

// Common plan construction for the two-operator chains.
int make_chain_plan(int chain, const tf_csr *A, const tf_csr *B, int k_dim, int n_cols, const tf_plan_opts *opts,
                    const tf_schedule *sched, tf_plan **out) {
  if (!A || !out) return fail(TF_ERR_ARG, "plan: null argument");
  if (n_cols <= 0) return fail(TF_ERR_ARG, "plan: dense width must be positive");
  tf_plan_opts o;
  int rc = check_opts(opts, o);
  if (rc != TF_OK) return rc;
  if (A->m <= 0) return fail(TF_ERR_ARG, "plan: matrix must have rows");
  if ((long long)A->m + o.halo_rows != A->n)
    return fail(TF_ERR_ARG, "plan: A must be m x (m + halo_rows): its columns index rows of the intermediate");
  rc = tf::check_csr(A->m, A->n, A->ap, A->ai, false);
  if (rc != TF_OK) return rc;
  if (!A->ax) return fail(TF_ERR_ARG, "plan: null value array");
  const tf_csr *F = chain == 0 ? (B ? B : A) : nullptr;
  if (F) {
    if (F->m != A->m) return fail(TF_ERR_ARG, "plan: B must have as many rows as A");
    if (F != A) {
      rc = tf::check_csr(F->m, F->n, F->ap, F->ai, false);
      if (rc != TF_OK) return rc;
      if (!F->ax) return fail(TF_ERR_ARG, "plan: null value array");
    }
    if (o.mode == TF_MODE_SCHEDULE && o.halo_rows) return fail(TF_ERR_UNSUPPORTED, "plan: schedule mode is single-GPU");
  }
  if (o.mode != TF_MODE_STREAM && (o.halo_rows || o.n_boundary))
    return fail(TF_ERR_UNSUPPORTED, "plan: halo exchange is available in stream mode only");
  int sm_count = 0;
  rc = device_ready(&sm_count);
  if (rc != TF_OK) return rc;

  std::unique_ptr<tf_plan> p(new tf_plan());
  cudaGetDevice(&p->device);
  p->chain = chain; p->mode = o.mode;
  p->m = A->m; p->n_cols = n_cols; p->k_dim = k_dim; p->halo_rows = o.halo_rows;
  rc = p->second.upload(*A);
  if (rc != TF_OK) return rc;
  if (F) {
    p->first_cols = F->n;
    if (F == A) p->first_is_second = true;
    else { rc = p->first.upload(*F); if (rc != TF_OK) return rc; }
  }

  tf::PlanParams pp;
  pp.m = A->m; pp.n_cols = n_cols;
  pp.producer_is_gemm = chain == 1;
  pp.rows_per_block = o.rows_per_block > 0 ? o.rows_per_block : default_rows_per_block(n_cols, chain == 1);
  pp.max_block_nnz = pp.rows_per_block * 32;
  pp.halo_rows = o.halo_rows;
  pp.boundary_rows.assign(o.boundary_rows, o.boundary_rows + o.n_boundary);
  for (int i = 0; i < o.n_boundary; ++i)
    if (pp.boundary_rows[i] < 0 || pp.boundary_rows[i] >= A->m || (i && pp.boundary_rows[i] <= pp.boundary_rows[i - 1]))
      return fail(TF_ERR_ARG, "plan: boundary_rows must be sorted local row ids");
  pp.ring_bytes = o.mode == TF_MODE_STREAM ? (o.ring_bytes == 0 ? (48LL << 20) : (long long)o.ring_bytes) : -1;

  // grid size first (the default slack depends on how many CTAs are resident); ring-ness does not
  // change the resource use enough to matter for this estimate
  rc = finish_plan(*p, o, sm_count, false);
  if (rc != TF_OK) return rc;
  pp.max_ctas = p->grid;
  pp.slack_blocks = o.mode == TF_MODE_UNFUSED ? (1 << 30) : o.slack_blocks;
  // gather tiles: 16-byte staging copies need rows that are multiples of 4 floats
  tf::Tiling pt, ct;
  // a tile holds one row per 4 lanes... of the CTA that runs it: 256 rows (sparse chains) or 512 (GeMM-SpMM)
  const int tile_rows = tfk::tiled_threads(chain);
  const int slots = o.tile_slots == 0 ? (chain == 1 ? tf::kDefaultTileSlots : tf::kDefaultTileSlotsSmall) : o.tile_slots;
  // SpMM-SpMM with both operators tiled runs on the tile pipeline (one CTA per SM, about four tiles in
  // flight each).  Its tiles are a little smaller: two chunk buffers and two row tables share the SM's
  // shared memory.  It has no ring addressing, so a ring is only kept when the caller asked for one.
  bool want_pipe = false;
  {
    const int ps = o.tile_slots == 0 ? tf::kPipeTileSlots : o.tile_slots;
    const size_t need = tfk::tile_pipeline_smem(ps, tf::kPipeTileRows);
    if (chain == 0 && F && o.mode != TF_MODE_SCHEDULE && o.tile_pipeline >= 0 && o.ring_bytes <= 0 &&
        o.tile_double_buffer <= 0 && n_cols % 4 == 0 && need > 0 && need <= 226 * 1024) {
      const int max_bz = o.tile_max_bz > 0 ? o.tile_max_bz : tf::kDefaultTileMaxBz;
      tf::build_tiling(F->m, F->ap, F->ai, ps, max_bz, tf::kPipeTileRows, pt);
      tf::build_tiling(A->m, A->ap, A->ai, ps, max_bz, tf::kPipeTileRows, ct);
      if (pt.tiled && ct.tiled) {
        want_pipe = true;
        p->tile_slots = ps;
        p->pipe_rows = tf::kPipeTileRows;
        p->dyn_smem = (size_t)ps * 132;  // for the launches of phase 0, which run on the two-CTA kernel
        rc = finish_plan(*p, o, sm_count, false);
        if (rc != TF_OK) return rc;
        pp.ring_bytes = -1;
        pp.max_ctas = 4 * sm_count;
      } else {
        pt = tf::Tiling();
        ct = tf::Tiling();
      }
    }
  }
  if (!want_pipe && o.mode != TF_MODE_SCHEDULE && slots > 0 && n_cols % 4 == 0) {
    const int max_bz = o.tile_max_bz > 0 ? o.tile_max_bz : tf::kDefaultTileMaxBz;
    const bool dbl = o.tile_double_buffer > 0 || (o.tile_double_buffer == 0 && tf::kDefaultTileDoubleBuffer);
    const int cap = dbl ? slots / 2 : slots;  // half-size tiles leave room for the next chunk's copies
    if (F) tf::build_tiling(F->m, F->ap, F->ai, cap, max_bz, tile_rows, pt);
    tf::build_tiling(A->m, A->ap, A->ai, cap, max_bz, tile_rows, ct);
    if (pt.tiled || ct.tiled) {
      p->dyn_smem = (size_t)slots * 132;  // 128 B of staging + one source row id per slot
      p->tile_slots = slots;
      rc = finish_plan(*p, o, sm_count, false);  // the staging buffer lowers the resident CTA count
      if (rc != TF_OK) return rc;
      pp.max_ctas = p->grid;
    }
  }
  // dense producer on the tensor cores: 128-row tiles, its K slices live in the same dynamic buffer
  const bool want_tc = chain == 1 && o.mode != TF_MODE_SCHEDULE && o.tensor_cores >= 0 && tfk::tc_supported(k_dim, n_cols);
  if (want_tc) {
    p->use_tc = true;
    p->dyn_smem = std::max(p->dyn_smem, (size_t)tfk::tc_smem_bytes_host(n_cols));
    if (o.rows_per_block == 0) pp.rows_per_block = tfk::kTcRowsHost;
    pp.max_block_nnz = pp.rows_per_block * 32;
    rc = p->w_hi.alloc((size_t)k_dim * n_cols);
    if (rc == TF_OK) rc = p->w_lo.alloc((size_t)k_dim * n_cols);
    if (rc == TF_OK) rc = tfk::tc_make_map(&p->tm_whi, p->w_hi.p, n_cols, k_dim, n_cols);
    if (rc == TF_OK) rc = tfk::tc_make_map(&p->tm_wlo, p->w_lo.p, n_cols, k_dim, n_cols);
    if (rc == TF_OK) rc = finish_plan(*p, o, sm_count, false);
    if (rc != TF_OK) return rc;
    pp.max_ctas = p->grid;
  }
  p->tile_info[0] = pt.bx; p->tile_info[1] = pt.by; p->tile_info[2] = pt.bz; p->tile_info[3] = pt.tiles();
  p->tile_info[4] = ct.bx; p->tile_info[5] = ct.by; p->tile_info[6] = ct.bz; p->tile_info[7] = ct.tiles();
  rc = tf::build_stream_plan(pp, F ? F->ap : nullptr, F ? F->ai : nullptr, A->ap, A->ai, &pt, &ct, p->hp);
  if (rc != TF_OK) return rc;
  rc = p->ptile.upload(pt, F ? F->ap : nullptr, F ? F->ax : nullptr, want_pipe);
  if (rc == TF_OK) rc = p->ctile.upload(ct, A->ap, A->ax, want_pipe);
  if (rc != TF_OK) return rc;
  p->pipe = want_pipe && p->hp.ring_rows == 0;
  for (int i = p->hp.phase_begin[1]; p->pipe && i < p->hp.phase_begin[3]; ++i)
    p->pipe = p->hp.items[i].kind == tf::ITEM_PRODUCE_TILED || p->hp.items[i].kind == tf::ITEM_CONSUME_TILED;
  p->pipe_grid = (o.halo_rows > 0 || o.n_boundary > 0) ? std::max(1, sm_count - 8) : sm_count;
  rc = finish_plan(*p, o, sm_count, p->hp.ring_rows > 0);
  if (rc != TF_OK) return rc;

  // with a halo exchange in flight, leave a few SMs half empty so that the NCCL send/recv kernels can
  // start while the persistent executor occupies the GPU (they would otherwise wait for it to drain)
  if ((o.halo_rows > 0 || o.n_boundary > 0) && p->grid > sm_count) p->grid = std::max(sm_count, p->grid - 16);
  // phase 0 items: boundary rows -> send buffer, in runs of consecutive rows
  if (!pp.boundary_rows.empty()) {
    std::vector<tf::Item> pre;
    size_t i = 0;
    while (i < pp.boundary_rows.size()) {
      size_t j = i + 1;
      while (j < pp.boundary_rows.size() && pp.boundary_rows[j] == pp.boundary_rows[j - 1] + 1 &&
             (int)(j - i) < pp.rows_per_block)
        ++j;
      tf::Item it{};
      it.kind = 3; it.row_begin = pp.boundary_rows[i]; it.row_end = pp.boundary_rows[i] + (int)(j - i);
      it.aux0 = (int)i;
      pre.push_back(it);
      i = j;
    }
    const int shift = (int)pre.size();
    p->hp.items.insert(p->hp.items.begin(), pre.begin(), pre.end());
    p->hp.phase_begin[1] += shift; p->hp.phase_begin[2] += shift; p->hp.phase_begin[3] += shift;
    rc = p->sendbuf.alloc(pp.boundary_rows.size() * (size_t)n_cols);
    if (rc != TF_OK) return rc;
  }
  if (o.mode == TF_MODE_STREAM && !o.halo_rows && !o.n_boundary) build_segments(*p, 16);
  rc = upload_items(*p, &pt, &ct);
  if (rc == TF_OK) rc = zero_state(*p);
  if (rc == TF_OK) rc = p->inter.alloc((size_t)p->hp.inter_rows * n_cols);
  if (rc != TF_OK) return rc;
  TF_CUDA(cudaMemset(p->inter.p, 0, p->inter.n * sizeof(float)));
  if (o.mode == TF_MODE_SCHEDULE) {
    rc = load_schedule(*p, sched, chain == 1);
    if (rc != TF_OK) return rc;
  }
  if (chain == 0 && F && o.mode == TF_MODE_STREAM && o.lattice_march >= 0 && o.ring_bytes <= 0 && n_cols % 4 == 0) {
    rc = build_march(*p, F, *A, o.halo_rows, sm_count, pp.boundary_rows);
    if (rc != TF_OK) return rc;
  }
  // GeMM-SpMM with a grid operator, the tensor-core producer and the whole intermediate in memory: the consumer is
  // the marching kernel
  if (chain == 1 && o.mode == TF_MODE_STREAM && o.lattice_march >= 0 && p->use_tc && p->hp.ring_rows == 0 && n_cols % 4 == 0) {
    rc = build_march(*p, nullptr, *A, o.halo_rows, sm_count, pp.boundary_rows);
    if (rc != TF_OK) return rc;
  }
  p->sm_count = sm_count;
  *out = p.release();
  return TF_OK;
}

tfk::Params base_params(tf_plan &p) {
  tfk::Params P;
  std::memset(&P, 0, sizeof(P));
  const DevCsr &f = p.first_is_second ? p.second : p.first;
  P.f_ap = f.ap.p; P.f_ai = f.ai.p; P.f_ax = f.ax.p;
  P.s_ap = p.second.ap.p; P.s_ai = p.second.ai.p; P.s_ax = p.second.ax.p;
  P.inter = p.inter.p;
  P.items = p.items.p;
  P.prod_done = p.prod_done.p; P.cons_done = p.cons_done.p;
  P.st = p.state.p;
  P.n_cols = p.n_cols; P.k_dim = p.k_dim; P.m_local = p.m;
  P.ring_rows = (int)p.hp.ring_rows;
  P.n_prod = p.hp.n_prod;
  P.n_cons = p.hp.n_cons;
  P.tile_rows = p.pipe_rows;
  P.pt = p.ptile.view();
  P.ct = p.ctile.view();
  P.tile_slots = p.tile_slots;
  P.spin_limit = p.spin_limit;
  return P;
}

bool aligned(const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; }
bool march_usable(const tf_plan &p, const float *C, const float *D) { return p.march.on && aligned(C, 16) && aligned(D, 16); }

// vector width usable with the caller's pointers (plan-owned buffers are always aligned)
void call_shape(const tf_plan &p, std::initializer_list<const void *> ptrs, int *vec, int *ch) {
  bool a16 = true;
  for (const void *q : ptrs) a16 = a16 && (!q || aligned(q, 16));
  tfk::choose_shape(p.n_cols, a16, vec, ch);
}

// Plans that run the staged kernel variant -- gather tiles or the tensor-core producer -- use 16-byte vector
// accesses on the dense operands whatever their width: refuse operands that are not aligned before any launch.
int check_tiled_alignment(const tf_plan &p, const tfk::Params &P) {
  if (p.dyn_smem > 0 && !(aligned(P.in0, 16) && (!P.out || aligned(P.out, 16))))
    return fail(TF_ERR_ARG, "this plan (gather tiles or tensor-core producer) needs 16-byte aligned dense operands "
                            "(build the plan with tile_slots < 0 and tensor_cores < 0 otherwise)");
  return TF_OK;
}

// Tensor-core producer: split the weight for this call and describe B to the TMA unit.
int prepare_tc(tf_plan &p, tfk::Params &P, cudaStream_t s) {
  P.use_tc = 0;
  if (!p.use_tc) return TF_OK;
  TF_CUDA(tfk::tc_split_weight(P.in1, P.w_transposed, p.k_dim, p.n_cols, p.w_hi.p, p.w_lo.p, s));
  int rc = tfk::tc_make_map(&P.tm_a, P.in0, p.m, p.k_dim, tfk::kTcRowsHost);
  if (rc != TF_OK) return rc;
  P.tm_whi = p.tm_whi;
  P.tm_wlo = p.tm_wlo;
  P.use_tc = 1;
  return TF_OK;
}

// One launch over the items [Q.item_begin, Q.item_end) of phases 1 and 2.
cudaError_t launch_items(tf_plan &p, int vec, int ch, bool ring, const tfk::Params &Q, cudaStream_t s) {
  if (p.pipe) return tfk::launch_tile_pipeline(p.pipe_grid, Q, s);
  return tfk::launch_stream(p.chain, vec, ch, ring, p.grid, p.dyn_smem, Q, s);
}

int run_phases(tf_plan &p, tfk::Params &P, int first_phase, int last_phase, cudaStream_t s) {
  int vec, ch;
  call_shape(p, {P.in0, P.in1, P.in2, P.out}, &vec, &ch);
  int rca = check_tiled_alignment(p, P);
  if (rca != TF_OK) return rca;
  if (p.dyn_smem > 0) { vec = 4; ch = 1; }  // the tiled kernel variant; its direct items loop over panels
  rca = prepare_tc(p, P, s);
  if (rca != TF_OK) return rca;
  const bool ring = p.hp.ring_rows > 0;
  if (first_phase <= 1 && last_phase >= 1) ++p.epoch;  // a new pass over the producer blocks
  P.epoch = p.epoch;
  p.launches = 0;
  if (first_phase <= 1 && last_phase >= 1) {
    rca = segments_begin(p, P, s);
    if (rca != TF_OK) return rca;
  }
  for (int ph = first_phase; ph <= last_phase; ++ph) {
    P.item_begin = p.hp.phase_begin[ph];
    P.item_end = p.hp.phase_begin[ph + 1];
    if (P.item_end <= P.item_begin) continue;
    tfk::Params Q = P;
    if (ph == 0) Q.inter = p.sendbuf.p;
    Q.reset_wm = (ph == 2) || (ph == 1 && p.hp.phase_begin[3] == p.hp.phase_begin[2] && last_phase >= 1);
    if (ph == 0) TF_CUDA(tfk::launch_stream(p.chain, vec, ch, ring, p.grid, p.dyn_smem, Q, s));
    else TF_CUDA(launch_items(p, vec, ch, ring, Q, s));
    ++p.launches;
  }
  if (last_phase == 2) return segments_end(p, P, s);
  return TF_OK;
}

// Segments of the item list for the host pipeline: after segment j, the producers listed so far have
// read input rows < in_rows, and every output row < out_rows is final.
void build_segments(tf_plan &p, int n_seg) {
  p.segs.clear();
  const int b = p.hp.phase_begin[1], e = p.hp.phase_begin[2];
  const int n = e - b;
  if (n <= 0 || p.hp.phase_begin[3] != e) return;
  n_seg = std::max(1, std::min(n_seg, n / std::max(1, p.grid)));
  if (!p.hp.seg_t_rows.empty() || !p.hp.seg_out_rows.empty()) n_seg = 1;  // rows finished by atomic adds: no early copies
  std::vector<int> suffix_min(n + 1, p.m);
  for (int i = n - 1; i >= 0; --i) {
    const tf::Item &it = p.hp.items[b + i];
    const bool cons = it.kind == tf::ITEM_CONSUME || it.kind == tf::ITEM_CONSUME_TILED;
    suffix_min[i] = std::min(suffix_min[i + 1], cons ? it.aux1 : p.m);
  }
  long long in_rows = 0;
  for (int s = 0; s < n_seg; ++s) {
    const int i0 = (int)((long long)n * s / n_seg), i1 = (int)((long long)n * (s + 1) / n_seg);
    for (int i = i0; i < i1; ++i) {
      const tf::Item &it = p.hp.items[b + i];
      if (it.kind == tf::ITEM_PRODUCE || it.kind == tf::ITEM_PRODUCE_TILED) in_rows = std::max<long long>(in_rows, it.aux0 + 1LL);
    }
    p.segs.push_back(tf_plan::Seg{b + i0, b + i1, in_rows, (long long)suffix_min[i1]});
  }
}

// Copies of one host-pointer call: plain for pinned arrays, through the pinned rings for pageable ones.
int begin_host_pipe(tf_plan &p, const void *h_in, const void *h_out) {
  if (!p.host_pipe) {
    const int t = (int)std::min(8u, std::max(2u, std::thread::hardware_concurrency() / 2));
    p.host_pipe.reset(new tf::HostPipe(t));
  }
  TF_CUDA(p.host_pipe->begin(p.device, tf::is_pageable(h_in), tf::is_pageable(h_out), (size_t)8 << 20, 16));
  return TF_OK;
}

// Host pipeline: the dense input is copied in row chunks on one stream, the item list runs in segments
// on a second as soon as the rows a segment reads have arrived, and finished output rows leave on a
// third.  in_rows x in_cols floats come from h_in; D is m x n_cols.
int run_host_pipeline(tf_plan &p, tfk::Params &P, const float *h_in, long long in_rows, int in_cols, float *d_in,
                      float *h_out, float *d_out) {
  if (!p.s_h2d) {
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_h2d, cudaStreamNonBlocking));
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_run, cudaStreamNonBlocking));
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_d2h, cudaStreamNonBlocking));
  }
  const int ns = (int)p.segs.size();
  while ((int)p.ev_in.size() < ns) {
    cudaEvent_t a, b;
    TF_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
    TF_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
    p.ev_in.push_back(a); p.ev_run.push_back(b);
  }
  int vec, ch;
  call_shape(p, {P.in0, P.in1, P.in2, P.out}, &vec, &ch);
  if (p.dyn_smem > 0) { vec = 4; ch = 1; }
  int rc = prepare_tc(p, P, p.s_run);
  if (rc != TF_OK) return rc;
  rc = begin_host_pipe(p, h_in, h_out);
  if (rc != TF_OK) return rc;
  const bool ring = p.hp.ring_rows > 0;
  ++p.epoch;
  P.epoch = p.epoch;
  p.launches = 0;
  long long in_done = 0, out_done = 0;
  rc = segments_begin(p, P, p.s_run);
  if (rc != TF_OK) return rc;
  for (int s = 0; s < ns; ++s) {
    const tf_plan::Seg &g = p.segs[s];
    const long long in_to = s == ns - 1 ? in_rows : std::min(in_rows, g.in_rows);
    if (in_to > in_done)
      TF_CUDA(p.host_pipe->upload(d_in + in_done * in_cols, h_in + in_done * in_cols, (size_t)(in_to - in_done) * in_cols * 4, p.s_h2d));
    in_done = std::max(in_done, in_to);
    TF_CUDA(cudaEventRecord(p.ev_in[s], p.s_h2d));
    TF_CUDA(cudaStreamWaitEvent(p.s_run, p.ev_in[s], 0));
    tfk::Params Q = P;
    Q.item_begin = g.item_begin; Q.item_end = g.item_end;
    Q.reset_wm = s == ns - 1;
    TF_CUDA(launch_items(p, vec, ch, ring, Q, p.s_run));
    ++p.launches;
    if (s == ns - 1) {
      rc = segments_end(p, P, p.s_run);
      if (rc != TF_OK) return rc;
    }
    TF_CUDA(cudaEventRecord(p.ev_run[s], p.s_run));
    const long long out_to = s == ns - 1 ? p.m : g.out_rows;
    if (out_to > out_done) {
      TF_CUDA(cudaStreamWaitEvent(p.s_d2h, p.ev_run[s], 0));
      TF_CUDA(p.host_pipe->download(h_out + out_done * p.n_cols, d_out + out_done * p.n_cols,
                               (size_t)(out_to - out_done) * p.n_cols * 4, p.s_d2h));
      out_done = out_to;
    }
  }
  TF_CUDA(p.host_pipe->finish());
  TF_CUDA(cudaStreamSynchronize(p.s_d2h));
  TF_CUDA(cudaStreamSynchronize(p.s_run));
  return TF_OK;
}

// The same pipeline for plane-marching plans: one launch per slab of planes.  A slab [za, zb) reads the planes
// za - 2 .. zb + 1 of C and completes the planes [za, zb) of D, so the copies run two planes ahead of the kernel
// and the output leaves slab by slab.  Pageable arrays go piece by piece through rings of pinned slots
// (host_stage.h).
int run_host_march(tf_plan &p, const float *h_in, float *d_in, float *h_out, float *d_out) {
  tf_plan::March &M = p.march;
  if (!p.s_h2d) {
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_h2d, cudaStreamNonBlocking));
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_run, cudaStreamNonBlocking));
    TF_CUDA(cudaStreamCreateWithFlags(&p.s_d2h, cudaStreamNonBlocking));
  }
  const int ns = (int)M.slabs.size();
  while ((int)p.ev_in.size() < ns) {
    cudaEvent_t a, b;
    TF_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
    TF_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
    p.ev_in.push_back(a); p.ev_run.push_back(b);
  }
  const size_t plane = (size_t)M.nx * M.ny * p.n_cols, plane_bytes = plane * sizeof(float);
  int rc = begin_host_pipe(p, h_in, h_out);
  if (rc != TF_OK) return rc;
  int planes_in = 0;
  long long launches = 0;
  for (int sl = 0; sl < ns; ++sl) {
    const tf_plan::March::Slab &g = M.slabs[sl];
    const int need = std::min(M.nz, g.z_end + 2);
    if (need > planes_in)
      TF_CUDA(p.host_pipe->upload(d_in + plane * planes_in, h_in + plane * planes_in, plane_bytes * (size_t)(need - planes_in), p.s_h2d));
    planes_in = std::max(planes_in, need);
    TF_CUDA(cudaEventRecord(p.ev_in[sl], p.s_h2d));
    TF_CUDA(cudaStreamWaitEvent(p.s_run, p.ev_in[sl], 0));
    rc = run_march(p, d_in, d_out, g.item_begin, g.item_end, false, p.s_run);
    if (rc != TF_OK) return rc;
    launches += p.launches;
    TF_CUDA(cudaEventRecord(p.ev_run[sl], p.s_run));
    TF_CUDA(cudaStreamWaitEvent(p.s_d2h, p.ev_run[sl], 0));
    TF_CUDA(p.host_pipe->download(h_out + plane * g.z_begin, d_out + plane * g.z_begin, plane_bytes * (size_t)(g.z_end - g.z_begin), p.s_d2h));
  }
  p.launches = launches;
  TF_CUDA(p.host_pipe->finish());
  TF_CUDA(cudaStreamSynchronize(p.s_d2h));
  TF_CUDA(cudaStreamSynchronize(p.s_run));
  return TF_OK;
}

int run_unfused(tf_plan &p, tfk::Params &P, cudaStream_t s) {
  // all producers are listed before all consumers: one launch per half, T through HBM
  int vec, ch;
  call_shape(p, {P.in0, P.in1, P.in2, P.out}, &vec, &ch);
  int rca = check_tiled_alignment(p, P);
  if (rca != TF_OK) return rca;
  if (p.dyn_smem > 0) { vec = 4; ch = 1; }
  rca = prepare_tc(p, P, s);
  if (rca != TF_OK) return rca;
  ++p.epoch;
  P.epoch = p.epoch;
  const int np = P.n_prod;
  p.launches = 0;
  rca = segments_begin(p, P, s);
  if (rca != TF_OK) return rca;
  tfk::Params Q = P;
  Q.item_begin = 0; Q.item_end = np; Q.reset_wm = 0;
  TF_CUDA(launch_items(p, vec, ch, false, Q, s));
  Q.item_begin = np; Q.item_end = (int)p.hp.items.size(); Q.reset_wm = 1;
  TF_CUDA(launch_items(p, vec, ch, false, Q, s));
  p.launches = 2;
  return segments_end(p, P, s);
}

int run_schedule(tf_plan &p, tfk::Params &P, cudaStream_t s) {
  int vec, ch;
  call_shape(p, {P.in0, P.in1, P.in2, P.out}, &vec, &ch);
  p.launches = 0;
  for (int l = 0; l < p.s_n1; ++l) {
    const int nparts = p.s_ptr1[l + 1] - p.s_ptr1[l];
    if (nparts <= 0) continue;
    const int grid = std::min(nparts, p.grid);
    TF_CUDA(tfk::launch_schedule_level(p.chain, vec, ch, grid, P, p.s_ptr2.p, p.s_id.p, p.s_type.p,
                                       p.s_has_ker ? p.s_ker.p : nullptr, p.s_ptr1[l], p.s_ptr1[l + 1], s));
    ++p.launches;
  }
  return TF_OK;
}

int run_chain(tf_plan &p, tfk::Params &P, cudaStream_t s) {
  if (p.mode == TF_MODE_SCHEDULE) return run_schedule(p, P, s);
  if (p.mode == TF_MODE_UNFUSED) return run_unfused(p, P, s);
  return run_phases(p, P, 1, 2, s);
}

int set_device(const tf_plan &p) {
  TF_CUDA(cudaSetDevice(p.device));
  return TF_OK;
}

}  // namespace

extern "C" {

int tf_plan_spmm_spmm(const tf_csr *A, const tf_csr *B, int n_cols, const tf_plan_opts *o,
                      const tf_schedule *sched, tf_plan **out) {
  return make_chain_plan(0, A, B, 0, n_cols, o, sched, out);
}

int tf_plan_gemm_spmm(const tf_csr *A, int k, int n_cols, const tf_plan_opts *o, const tf_schedule *sched,
                      tf_plan **out) {
  if (k <= 0) return fail(TF_ERR_ARG, "plan: inner dimension must be positive");
  return make_chain_plan(1, A, nullptr, k, n_cols, o, sched, out);
}

int tf_plan_sddmm_spmm(const tf_csr *A, int kq, int nv, const tf_plan_opts *opts, tf_plan **out) {
  if (!A || !out) return fail(TF_ERR_ARG, "plan: null argument");
  if (kq <= 0 || nv <= 0) return fail(TF_ERR_ARG, "plan: dense widths must be positive");
  tf_plan_opts o;
  int rc = check_opts(opts, o);
  if (rc != TF_OK) return rc;
  if (A->m <= 0 || A->n <= 0) return fail(TF_ERR_ARG, "plan: matrix must have rows and columns");
  rc = tf::check_csr(A->m, A->n, A->ap, A->ai, false);
  if (rc != TF_OK) return rc;
  if (!A->ax) return fail(TF_ERR_ARG, "plan: null value array");
  int sm_count = 0;
  rc = device_ready(&sm_count);
  if (rc != TF_OK) return rc;
  std::unique_ptr<tf_plan> p(new tf_plan());
  cudaGetDevice(&p->device);
  p->chain = 2; p->mode = TF_MODE_STREAM;
  p->m = A->m; p->n_cols = nv; p->k_dim = kq;
  rc = p->second.upload(*A);
  if (rc != TF_OK) return rc;
  p->first_is_second = true;
  tf::PlanParams pp;
  pp.m = A->m; pp.n_cols = nv;
  pp.rows_per_block = o.rows_per_block > 0 ? o.rows_per_block : 32;
  pp.max_block_nnz = pp.rows_per_block * 32;
  rc = tf::build_single_pass_plan(pp, A->ap, p->hp);
  if (rc == TF_OK) rc = finish_plan(*p, o, sm_count, false);
  if (rc == TF_OK) rc = upload_items(*p);
  if (rc == TF_OK) rc = zero_state(*p);
  if (rc != TF_OK) return rc;
  *out = p.release();
  return TF_OK;
}

void tf_plan_free(tf_plan *p) { delete p; }

int tf_plan_info(const tf_plan *p, long long info[8]) {
  if (!p || !info) return fail(TF_ERR_ARG, "tf_plan_info: null argument");
  info[0] = (long long)p->hp.items.size();
  info[1] = p->hp.n_prod;
  info[2] = p->hp.n_cons;
  info[3] = p->hp.ring_rows;
  info[4] = p->march.on ? p->march.grid : (p->pipe ? p->pipe_grid : p->grid);
  info[5] = p->march.on ? tfk::kMarchThreads : (p->pipe ? 672 : (p->dyn_smem > 0 ? tfk::tiled_threads(p->chain) : tfk::kThreads));
  info[6] = p->launches;
  info[7] = p->hp.inter_rows;
  return TF_OK;
}

int tf_plan_tile_info(const tf_plan *p, int info[8]) {
  if (!p || !info) return fail(TF_ERR_ARG, "tf_plan_tile_info: null argument");
  for (int i = 0; i < 8; ++i) info[i] = p->tile_info[i];
  return TF_OK;
}

int tf_plan_set_wait_limit(tf_plan *p, int polls) {
  if (!p || polls <= 0) return fail(TF_ERR_ARG, "tf_plan_set_wait_limit: bad argument");
  p->spin_limit = polls;
  return TF_OK;
}

int tf_plan_status(tf_plan *p, void *stream) {
  if (!p) return fail(TF_ERR_ARG, "tf_plan_status: null plan");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  TF_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (p->march.on) {
    tfk::MarchState ms[2];
    TF_CUDA(cudaMemcpy(ms, p->march.st.p, sizeof(ms), cudaMemcpyDeviceToHost));
    if (ms[0].error || ms[1].error) {
      cudaMemset(p->march.st.p, 0, sizeof(ms));
      return fail(TF_ERR_TIMEOUT, "a bounded in-kernel wait ran out; the output of the last call is not valid");
    }
  }
  tfk::ExecState st;
  TF_CUDA(cudaMemcpy(&st, p->state.p, sizeof(st), cudaMemcpyDeviceToHost));
  if (st.error) {
    // leave the plan usable: clear the executor state
    cudaMemset(p->state.p, 0, sizeof(st));
    return fail(TF_ERR_TIMEOUT, "a bounded in-kernel wait ran out; the output of the last call is not valid");
  }
  return TF_OK;
}

int tf_exec_spmm_spmm(tf_plan *p, const float *C, float *D, void *stream) {
  if (!p || !C || !D) return fail(TF_ERR_ARG, "tf_exec_spmm_spmm: null argument");
  if (p->chain != 0) return fail(TF_ERR_ARG, "tf_exec_spmm_spmm: plan was built for another chain");
  if (p->halo_rows || p->sendbuf.n) return fail(TF_ERR_ARG, "tf_exec_spmm_spmm: plan has halo rows, drive it with tf_exec_phase");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  if (march_usable(*p, C, D)) return run_march(*p, C, D, 0, p->march.n_items, false, (cudaStream_t)stream);
  tfk::Params P = base_params(*p);
  P.in0 = C; P.out = D;
  return run_chain(*p, P, (cudaStream_t)stream);
}

// GeMM-SpMM on a grid operator: the dense producer writes all rows of T (one launch of the tensor-core kernel), the
// marching kernel consumes them (items [item_begin, item_end)).
int run_gemm_march(tf_plan &p, const float *B, const float *W, int w_transposed, float *D, bool produce, int item_begin,
                   int item_end, bool with_halo, cudaStream_t s) {
  long long launches = 0;
  if (produce) {
    tfk::Params P = base_params(p);
    P.in0 = B; P.in1 = W; P.w_transposed = w_transposed;
    int rc = prepare_tc(p, P, s);
    if (rc != TF_OK) return rc;
    TF_CUDA(tfk::tc_launch_gemm(P.tm_a, P.tm_whi, P.tm_wlo, p.m, p.k_dim, p.n_cols, p.inter.p, &p.march.st.p[0].error, p.spin_limit,
                                p.sm_count, s));
    launches = 2;   // weight split + producer
  }
  int rc = run_march(p, p.inter.p, D, item_begin, item_end, with_halo, s);
  p.launches += launches;
  return rc;
}

bool gemm_march_usable(const tf_plan &p, const float *B, const float *D, int relu) {
  return p.chain == 1 && p.march.on && p.march.identity_first && !relu && aligned(B, 16) && aligned(D, 16);
}

int tf_exec_gemm_spmm(tf_plan *p, const float *B, const float *W, int w_transposed, int relu, float *D,
                      void *stream) {
  if (!p || !B || !W || !D) return fail(TF_ERR_ARG, "tf_exec_gemm_spmm: null argument");
  if (p->chain != 1) return fail(TF_ERR_ARG, "tf_exec_gemm_spmm: plan was built for another chain");
  if (p->halo_rows || p->sendbuf.n) return fail(TF_ERR_ARG, "tf_exec_gemm_spmm: plan has halo rows, drive it with tf_exec_phase");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  if (gemm_march_usable(*p, B, D, relu))
    return run_gemm_march(*p, B, W, w_transposed, D, true, 0, p->march.n_items, false, (cudaStream_t)stream);
  tfk::Params P = base_params(*p);
  P.in0 = B; P.in1 = W; P.out = D; P.w_transposed = w_transposed; P.relu = relu;
  return run_chain(*p, P, (cudaStream_t)stream);
}

int tf_exec_sddmm_spmm(tf_plan *p, const float *Q, const float *K, const float *V, float *D, void *stream) {
  if (!p || !Q || !K || !V || !D) return fail(TF_ERR_ARG, "tf_exec_sddmm_spmm: null argument");
  if (p->chain != 2) return fail(TF_ERR_ARG, "tf_exec_sddmm_spmm: plan was built for another chain");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  tfk::Params P = base_params(*p);
  P.in0 = Q; P.in1 = K; P.in2 = V; P.out = D;
  return run_phases(*p, P, 1, 1, (cudaStream_t)stream);
}

int tf_exec_phase(tf_plan *p, int phase, const float *in0, const float *in1, int w_transposed, int relu,
                  float *D, void *stream) {
  if (!p || !in0) return fail(TF_ERR_ARG, "tf_exec_phase: null argument");
  if (phase < 0 || phase > 2) return fail(TF_ERR_ARG, "tf_exec_phase: phase must be 0, 1 or 2");
  if (p->chain > 1 || p->mode != TF_MODE_STREAM) return fail(TF_ERR_ARG, "tf_exec_phase: stream-mode chain plans only");
  if (p->chain == 1 && !in1) return fail(TF_ERR_ARG, "tf_exec_phase: GeMM-SpMM needs the weight");
  if (phase > 0 && !D) return fail(TF_ERR_ARG, "tf_exec_phase: null output");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  // plane-marching plans: phase 0 (boundary rows of T for the neighbours: two planes at most) is a plain CSR product
  // of those rows into the send buffer -- a fraction of the time the general executor's launch takes for so little
  // work --, phases 1 and 2 run on the marching kernel, the second with the received planes of T
  if (phase == 0 && p->chain == 0 && p->march.on && p->march.n_boundary > 0 && aligned(in0, 16)) {
    const tf_plan::March &M = p->march;
    int vec, ch;
    tfk::choose_shape(p->n_cols, aligned(in0, 16) && aligned(p->sendbuf.p, 16), &vec, &ch);
    const int grid = std::max(1, std::min((M.n_boundary + tfk::kWarps - 1) / tfk::kWarps, 148 * 8));
    TF_CUDA(tfk::launch_spmm(vec, ch, grid, M.b_ap.p, M.b_ai.p, M.b_ax.p, M.n_boundary, in0, p->n_cols, p->sendbuf.p,
                             (cudaStream_t)stream));
    p->launches = 1;
    return TF_OK;
  }
  if (phase > 0 && gemm_march_usable(*p, in0, D, relu))
    return phase == 1 ? run_gemm_march(*p, in0, in1, w_transposed, D, true, 0, p->march.n_phase1, false, (cudaStream_t)stream)
                      : run_gemm_march(*p, in0, in1, w_transposed, D, false, p->march.n_phase1, p->march.n_items, true,
                                       (cudaStream_t)stream);
  if (phase > 0 && p->chain == 0 && march_usable(*p, in0, D))
    return phase == 1 ? run_march(*p, in0, D, 0, p->march.n_phase1, false, (cudaStream_t)stream)
                      : run_march(*p, in0, D, p->march.n_phase1, p->march.n_items, true, (cudaStream_t)stream);
  tfk::Params P = base_params(*p);
  P.in0 = in0; P.in1 = in1; P.out = D; P.w_transposed = w_transposed; P.relu = relu;
  return run_phases(*p, P, phase, phase, (cudaStream_t)stream);
}

int tf_plan_intermediate(tf_plan *p, float **dev_ptr, long long *rows, int *cols) {
  if (!p) return fail(TF_ERR_ARG, "tf_plan_intermediate: null plan");
  if (dev_ptr) *dev_ptr = p->inter.p;
  if (rows) *rows = p->hp.inter_rows;
  if (cols) *cols = p->n_cols;
  return TF_OK;
}

int tf_plan_exchange_buffers(tf_plan *p, float **send, long long *send_rows, float **halo, long long *halo_rows) {
  if (!p) return fail(TF_ERR_ARG, "tf_plan_exchange_buffers: null plan");
  if (send) *send = p->sendbuf.p;
  if (send_rows) *send_rows = p->n_cols ? (long long)(p->sendbuf.n / p->n_cols) : 0;
  if (halo) *halo = p->halo_rows ? p->inter.p + (size_t)(p->hp.inter_rows - p->halo_rows) * p->n_cols : nullptr;
  if (halo_rows) *halo_rows = p->halo_rows;
  return TF_OK;
}

// ---- host-pointer executors -------------------------------------------------
static int stage_in(DevBuf<float> &buf, const float *h, size_t count, cudaStream_t s) {
  if (buf.n < count) { int rc = buf.alloc(count); if (rc != TF_OK) return rc; }
  TF_CUDA(cudaMemcpyAsync(buf.p, h, count * sizeof(float), cudaMemcpyHostToDevice, s));
  return TF_OK;
}

static int finish_host(tf_plan *p, float *D, size_t count) {
  if (p->h_out.n < count) return fail(TF_ERR_ARG, "internal: output staging missing");
  TF_CUDA(cudaMemcpyAsync(D, p->h_out.p, count * sizeof(float), cudaMemcpyDeviceToHost, 0));
  return tf_plan_status(p, nullptr);
}

int tf_spmm_spmm_host(tf_plan *p, const float *C, float *D) {
  if (!p || !C || !D) return fail(TF_ERR_ARG, "tf_spmm_spmm_host: null argument");
  if (p->chain != 0) return fail(TF_ERR_ARG, "tf_spmm_spmm_host: plan was built for another chain");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  const size_t nd = (size_t)p->m * p->n_cols;
  if (!p->march.slabs.empty()) {
    const size_t nin = (size_t)p->first_cols * p->n_cols;
    if (p->h_in0.n < nin) rc = p->h_in0.alloc(nin);
    if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
    if (rc != TF_OK) return rc;
    if (march_usable(*p, p->h_in0.p, p->h_out.p)) {
      rc = run_host_march(*p, C, p->h_in0.p, D, p->h_out.p);
      if (rc != TF_OK) return rc;
      return tf_plan_status(p, nullptr);
    }
  }
  if (p->segs.size() > 1) {
    const size_t nin = (size_t)p->first_cols * p->n_cols;
    if (p->h_in0.n < nin) rc = p->h_in0.alloc(nin);
    if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
    if (rc != TF_OK) return rc;
    tfk::Params P = base_params(*p);
    P.in0 = p->h_in0.p; P.out = p->h_out.p;
    rc = run_host_pipeline(*p, P, C, p->first_cols, p->n_cols, p->h_in0.p, D, p->h_out.p);
    if (rc != TF_OK) return rc;
    return tf_plan_status(p, nullptr);
  }
  rc = stage_in(p->h_in0, C, (size_t)p->first_cols * p->n_cols, 0);
  if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
  if (rc == TF_OK) rc = tf_exec_spmm_spmm(p, p->h_in0.p, p->h_out.p, nullptr);
  if (rc != TF_OK) return rc;
  return finish_host(p, D, nd);
}

int tf_gemm_spmm_host(tf_plan *p, const float *B, const float *W, int w_transposed, int relu, float *D) {
  if (!p || !B || !W || !D) return fail(TF_ERR_ARG, "tf_gemm_spmm_host: null argument");
  if (p->chain != 1) return fail(TF_ERR_ARG, "tf_gemm_spmm_host: plan was built for another chain");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  const size_t nd = (size_t)p->m * p->n_cols;
  if (p->segs.size() > 1) {
    const size_t nin = (size_t)p->m * p->k_dim;
    if (p->h_in0.n < nin) rc = p->h_in0.alloc(nin);
    if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
    if (rc != TF_OK) return rc;
    if (!p->s_run) {
      TF_CUDA(cudaStreamCreateWithFlags(&p->s_h2d, cudaStreamNonBlocking));
      TF_CUDA(cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking));
      TF_CUDA(cudaStreamCreateWithFlags(&p->s_d2h, cudaStreamNonBlocking));
    }
    rc = stage_in(p->h_in1, W, (size_t)p->k_dim * p->n_cols, p->s_run);  // the weight first, on the stream that uses it
    if (rc != TF_OK) return rc;
    tfk::Params P = base_params(*p);
    P.in0 = p->h_in0.p; P.in1 = p->h_in1.p; P.out = p->h_out.p; P.w_transposed = w_transposed; P.relu = relu;
    rc = run_host_pipeline(*p, P, B, p->m, p->k_dim, p->h_in0.p, D, p->h_out.p);
    if (rc != TF_OK) return rc;
    return tf_plan_status(p, nullptr);
  }
  rc = stage_in(p->h_in0, B, (size_t)p->m * p->k_dim, 0);
  if (rc == TF_OK) rc = stage_in(p->h_in1, W, (size_t)p->k_dim * p->n_cols, 0);
  if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
  if (rc == TF_OK) rc = tf_exec_gemm_spmm(p, p->h_in0.p, p->h_in1.p, w_transposed, relu, p->h_out.p, nullptr);
  if (rc != TF_OK) return rc;
  return finish_host(p, D, nd);
}

int tf_sddmm_spmm_host(tf_plan *p, const float *Q, const float *K, const float *V, float *D) {
  if (!p || !Q || !K || !V || !D) return fail(TF_ERR_ARG, "tf_sddmm_spmm_host: null argument");
  if (p->chain != 2) return fail(TF_ERR_ARG, "tf_sddmm_spmm_host: plan was built for another chain");
  int rc = set_device(*p);
  if (rc != TF_OK) return rc;
  const size_t nd = (size_t)p->m * p->n_cols;
  rc = stage_in(p->h_in0, Q, (size_t)p->m * p->k_dim, 0);
  if (rc == TF_OK) rc = stage_in(p->h_in1, K, (size_t)p->second.n * p->k_dim, 0);
  if (rc == TF_OK) rc = stage_in(p->h_in2, V, (size_t)p->second.n * p->n_cols, 0);
  if (rc == TF_OK && p->h_out.n < nd) rc = p->h_out.alloc(nd);
  if (rc == TF_OK) rc = tf_exec_sddmm_spmm(p, p->h_in0.p, p->h_in1.p, p->h_in2.p, p->h_out.p, nullptr);
  if (rc != TF_OK) return rc;
  return finish_host(p, D, nd);
}

int tf_spmm_dev(const int *Ap, const int *Ai, const float *Ax, int m, const float *X, int n_cols, float *out,
                void *stream) {
  if (!Ap || !Ai || !Ax || !X || !out) return fail(TF_ERR_ARG, "tf_spmm_dev: null argument");
  if (m < 0 || n_cols <= 0) return fail(TF_ERR_ARG, "tf_spmm_dev: bad size");
  int vec, ch;
  tfk::choose_shape(n_cols, aligned(X, 16) && aligned(out, 16), &vec, &ch);
  const int grid = std::max(1, std::min((m + tfk::kWarps - 1) / tfk::kWarps, 148 * 8));
  TF_CUDA(tfk::launch_spmm(vec, ch, grid, Ap, Ai, Ax, m, X, n_cols, out, (cudaStream_t)stream));
  return TF_OK;
}

int tf_fill_uniform(float *dev, long long count, unsigned long long seed, long long offset, void *stream) {
  if (!dev || count < 0) return fail(TF_ERR_ARG, "tf_fill_uniform: bad argument");
  TF_CUDA(tfk::launch_fill(false, dev, count, seed, offset, 1.f, (cudaStream_t)stream));
  return TF_OK;
}

int tf_fill_normal(float *dev, long long count, unsigned long long seed, long long offset, float sigma,
                   void *stream) {
  if (!dev || count < 0) return fail(TF_ERR_ARG, "tf_fill_normal: bad argument");
  TF_CUDA(tfk::launch_fill(true, dev, count, seed, offset, sigma, (cudaStream_t)stream));
  return TF_OK;
}

}  // extern "C"
