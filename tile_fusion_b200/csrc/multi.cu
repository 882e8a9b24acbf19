// Row-block partitioned chains on several GPUs, one process (or thread) per GPU: the partition arrays, the
// halo exchange over NCCL and the three phases of a step behind one C entry point.
//
// The reference runs on one shared-memory host; the partition is this library's own.  Rule (deterministic,
// so every rank derives the same arrays):
//   * rank g owns the contiguous rows [bounds[g], bounds[g+1]) of A, of the intermediate T and of D;
//   * its halo is the sorted list of column ids of its rows of A that fall outside its own range; the rows
//     of T with those ids arrive from their owners and are stored after the local rows;
//   * its boundary is the sorted list of its own rows that appear in some other rank's halo; they are
//     produced first (phase 0) into a send buffer laid out in that order.
// Only halo rows of T travel, on a second stream, beside phase 1 (the rows that need no halo row).  Where every
// rank is a process of its own on one host, the copy engines write the send segments over NVLink straight into
// the neighbours' halo rows (mapped through CUDA IPC) and NCCL carries one-int tokens around the copies; else
// the rows go through ncclSend / ncclRecv in one group.  The communicator is created with at most four CTAs per
// NCCL kernel, so that those kernels fit on the SMs the persistent kernel of phase 1 leaves free.  NCCL is resolved
// at run time from the process (libnccl.so.2), so the library has no link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <climits>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "tf_internal.h"

namespace tf {

// ---------------------------------------------------------------------------
// partition arrays (host only)
// ---------------------------------------------------------------------------
std::vector<long long> halo_of(const long long *ai, long long nnz, long long r0, long long r1) {
  std::vector<long long> h;
  for (long long j = 0; j < nnz; ++j)
    if (ai[j] < r0 || ai[j] >= r1) h.push_back(ai[j]);
  std::sort(h.begin(), h.end());
  h.erase(std::unique(h.begin(), h.end()), h.end());
  return h;
}

int make_layout(int rank, int world, const long long *bounds, const std::vector<std::vector<long long>> &halos,
                RankLayout &out) {
  out = RankLayout();
  const long long r0 = bounds[rank], r1 = bounds[rank + 1];
  out.halo_ids = halos[rank];
  // received rows: the halo list is sorted, so the rows of one owner are consecutive
  size_t pos = 0;
  for (int p = 0; p < world; ++p) {
    size_t cnt = 0;
    while (pos + cnt < out.halo_ids.size() && out.halo_ids[pos + cnt] < bounds[p + 1]) ++cnt;
    if (cnt) out.recv.push_back(ExchangeSegment{p, (long long)pos, (long long)cnt, {}});
    pos += cnt;
  }
  // rows other ranks want from this one
  std::vector<std::vector<long long>> wanted(world);
  std::vector<long long> all;
  for (int g = 0; g < world; ++g) {
    if (g == rank) continue;
    for (long long id : halos[g])
      if (id >= r0 && id < r1) { wanted[g].push_back(id - r0); all.push_back(id - r0); }
  }
  std::sort(all.begin(), all.end());
  all.erase(std::unique(all.begin(), all.end()), all.end());
  out.boundary_rows = all;
  for (int g = 0; g < world; ++g) {
    if (wanted[g].empty()) continue;
    ExchangeSegment s{g, 0, (long long)wanted[g].size(), {}};
    std::vector<long long> idx(wanted[g].size());
    for (size_t i = 0; i < idx.size(); ++i)
      idx[i] = std::lower_bound(all.begin(), all.end(), wanted[g][i]) - all.begin();
    s.start = idx[0];
    if (idx.back() - idx[0] + 1 != (long long)idx.size()) s.index = idx;  // not contiguous: gathered before the send
    out.send.push_back(s);
  }
  return TF_OK;
}

}  // namespace tf

// Host-only view of the partition arrays of one rank (for callers that drive the phases themselves and for
// tests).  halo_ptr[world + 1] / halo_ids: every rank's halo list, concatenated.  Arrays are malloc'd (tf_free):
// boundary_rows (local ids), recv and send segments as {peer, start, count, contiguous} quadruples.
extern "C" int tf_partition_layout(int rank, int world, const long long *bounds, const long long *halo_ptr,
                                   const long long *halo_ids, long long **boundary_rows, long long *n_boundary,
                                   long long **recv, int *n_recv, long long **send, int *n_send) {
  if (!bounds || !halo_ptr || !boundary_rows || !n_boundary || !recv || !n_recv || !send || !n_send || rank < 0 || rank >= world)
    return tf::fail(TF_ERR_ARG, "tf_partition_layout: bad argument");
  std::vector<std::vector<long long>> halos(world);
  for (int g = 0; g < world; ++g) halos[g].assign(halo_ids + halo_ptr[g], halo_ids + halo_ptr[g + 1]);
  tf::RankLayout lay;
  tf::make_layout(rank, world, bounds, halos, lay);
  auto dup = [](const std::vector<long long> &v) {
    long long *b = (long long *)malloc(sizeof(long long) * std::max<size_t>(v.size(), 1));
    if (b && !v.empty()) std::copy(v.begin(), v.end(), b);
    return b;
  };
  auto flat = [](const std::vector<tf::ExchangeSegment> &s) {
    std::vector<long long> v;
    for (const auto &x : s) { v.push_back(x.peer); v.push_back(x.start); v.push_back(x.count); v.push_back(x.index.empty()); }
    return v;
  };
  *boundary_rows = dup(lay.boundary_rows); *n_boundary = (long long)lay.boundary_rows.size();
  *recv = dup(flat(lay.recv)); *n_recv = (int)lay.recv.size();
  *send = dup(flat(lay.send)); *n_send = (int)lay.send.size();
  return TF_OK;
}

// ---------------------------------------------------------------------------
// NCCL, resolved at run time
// ---------------------------------------------------------------------------
namespace {

using tf::fail;

typedef struct { char internal[128]; } NcclUniqueId;  // ncclUniqueId
typedef void *NcclComm;                               // ncclComm_t
// ncclConfig_t as NCCL 2.17 declared it (newer libraries accept it by its size and version fields and default what
// it lacks).  The one field set here is maxCTAs: the exchange kernel of a step must fit on the few SMs the
// marching kernel leaves free -- with NCCL's default of up to 32 CTAs most of them would wait for an SM until phase 1
// has ended, and the receive with them.
struct NcclConfig217 {
  size_t size;
  unsigned magic, version;
  int blocking, cga_cluster_size, min_ctas, max_ctas;
  const char *net_name;
};
constexpr int kExchangeCtas = 4;

struct Nccl {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommInitRankConfig)(NcclComm *, int, NcclUniqueId, int, NcclConfig217 *) = nullptr;  // optional (NCCL >= 2.17)
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*Send)(const void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*Recv)(void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
};
constexpr int kNcclInt8 = 0, kNcclInt32 = 2, kNcclFloat = 7;  // ncclInt8 / ncclChar, ncclInt32, ncclFloat32

Nccl &nccl() {
  static Nccl n;
  static bool tried = false;
  if (tried) return n;
  tried = true;
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return n;
  n.GetUniqueId = (int (*)(NcclUniqueId *))dlsym(h, "ncclGetUniqueId");
  n.CommInitRank = (int (*)(NcclComm *, int, NcclUniqueId, int))dlsym(h, "ncclCommInitRank");
  n.CommInitRankConfig = (int (*)(NcclComm *, int, NcclUniqueId, int, NcclConfig217 *))dlsym(h, "ncclCommInitRankConfig");
  n.CommDestroy = (int (*)(NcclComm))dlsym(h, "ncclCommDestroy");
  n.Send = (int (*)(const void *, size_t, int, int, NcclComm, cudaStream_t))dlsym(h, "ncclSend");
  n.Recv = (int (*)(void *, size_t, int, int, NcclComm, cudaStream_t))dlsym(h, "ncclRecv");
  n.AllGather = (int (*)(const void *, void *, size_t, int, NcclComm, cudaStream_t))dlsym(h, "ncclAllGather");
  n.GroupStart = (int (*)())dlsym(h, "ncclGroupStart");
  n.GroupEnd = (int (*)())dlsym(h, "ncclGroupEnd");
  n.GetErrorString = (const char *(*)(int))dlsym(h, "ncclGetErrorString");
  n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.Send && n.Recv && n.AllGather && n.GroupStart && n.GroupEnd;
  return n;
}

#define TF_NCCL(call)                                                                                         \
  do {                                                                                                        \
    int r__ = (call);                                                                                         \
    if (r__ != 0)                                                                                             \
      return fail(TF_ERR_CUDA, std::string(#call) + ": NCCL error " + std::to_string(r__) +                   \
                                   (nccl().GetErrorString ? std::string(" (") + nccl().GetErrorString(r__) + ")" : "")); \
  } while (0)
#define TF_CUDA(call)                                                                         \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return fail(TF_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));          \
  } while (0)

__global__ void gather_rows_kernel(const float *__restrict__ src, const long long *__restrict__ idx, long long n_rows,
                                   int n_cols, float *__restrict__ dst) {
  for (long long r = blockIdx.x; r < n_rows; r += gridDim.x)
    for (int c = threadIdx.x; c < n_cols; c += blockDim.x) dst[r * n_cols + c] = src[idx[r] * n_cols + c];
}

}  // namespace

struct tf_comm {
  NcclComm comm = nullptr;
  bool owned = false;
  int world = 0, rank = 0, device = 0;
};

struct tf_multi {
  tf_comm *c = nullptr;
  int chain = 0, n_cols = 0, k = 0;
  long long r0 = 0, r1 = 0, c_first = 0, c_rows = 0;
  tf::RankLayout lay;
  tf_plan *plan = nullptr;
  float *sendbuf = nullptr, *halobuf = nullptr;
  struct Gather { long long *idx = nullptr; float *stage = nullptr; };
  std::vector<Gather> gathers;  // per send segment (null when the segment is contiguous)
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr, arrived = nullptr;
  // Direct exchange (every rank a process of its own on one host, peer access between the GPUs): the send segments
  // are copied by the copy engines straight into the neighbours' halo rows, whose allocations are mapped here
  // through CUDA IPC; NCCL only carries one-int tokens.  Empty: the rows travel through ncclSend / ncclRecv.
  bool direct = false;
  std::vector<void *> peer_base;   // per send segment: the peer's mapped allocation (to be closed)
  std::vector<float *> peer_dst;   // per send segment: where its rows go in the peer's halo rows
  int *tokens = nullptr;           // device: [0] the token sent, [1 ..] tokens received
  // timing of the last step (tf_multi_trace): start, phase 0 done, exchange done, phase 2 done, phase 1 done, end
  bool trace = false;
  cudaEvent_t tev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  ~tf_multi() {
    for (auto &g : gathers) { if (g.idx) cudaFree(g.idx); if (g.stage) cudaFree(g.stage); }
    for (void *b : peer_base) if (b) cudaIpcCloseMemHandle(b);
    if (tokens) cudaFree(tokens);
    if (plan) tf_plan_free(plan);
    if (ready) cudaEventDestroy(ready);
    if (arrived) cudaEventDestroy(arrived);
    for (cudaEvent_t e : tev) if (e) cudaEventDestroy(e);
    if (comm_stream) cudaStreamDestroy(comm_stream);
  }
};

namespace {

struct ExchangeCard {   // what a rank tells the others about its halo rows
  cudaIpcMemHandle_t handle;   // of the allocation that holds them
  long long halo_offset;       // bytes from the allocation's start to the first halo row
  long long host, pid;
  int has_halo, pad;
};

// all-gather of one fixed-size record per rank through a device buffer
template <class T>
int gather_records(tf_multi &M, const T &mine, std::vector<T> &all) {
  const int world = M.c->world, rank = M.c->rank;
  all.resize(world);
  char *d = nullptr;
  TF_CUDA(cudaMalloc(&d, sizeof(T) * (size_t)world));
  TF_CUDA(cudaMemcpy(d + sizeof(T) * rank, &mine, sizeof(T), cudaMemcpyHostToDevice));
  TF_NCCL(nccl().AllGather(d + sizeof(T) * rank, d, sizeof(T), kNcclInt8, M.c->comm, M.comm_stream));
  TF_CUDA(cudaStreamSynchronize(M.comm_stream));
  TF_CUDA(cudaMemcpy(all.data(), d, sizeof(T) * (size_t)world, cudaMemcpyDeviceToHost));
  cudaFree(d);
  return TF_OK;
}

// Collective.  Maps the neighbours' halo rows into this process where that is possible; the direct exchange is
// used only if every rank could map all it needs (and none asked for ncclSend / ncclRecv: allow_direct).
int setup_direct_exchange(tf_multi &M, const std::vector<long long> &bounds, const std::vector<std::vector<long long>> &halos,
                          bool allow_direct) {
  const int world = M.c->world, rank = M.c->rank;
  if (world < 2) return TF_OK;
  ExchangeCard me;
  std::memset(&me, 0, sizeof(me));
  char host[256] = {0};
  gethostname(host, sizeof(host) - 1);
  for (const char *q = host; *q; ++q) me.host = me.host * 131 + (unsigned char)*q;
  me.pid = (long long)getpid();
  float *base = nullptr;
  long long rows = 0;
  int cols = 0;
  int rc = tf_plan_intermediate(M.plan, &base, &rows, &cols);
  if (rc != TF_OK) return rc;
  bool can = allow_direct;
  if (M.halobuf && base) {
    me.has_halo = 1;
    me.halo_offset = (long long)((const char *)M.halobuf - (const char *)base);
    if (cudaIpcGetMemHandle(&me.handle, base) != cudaSuccess) { (void)cudaGetLastError(); can = false; }
  }
  std::vector<ExchangeCard> cards;
  rc = gather_records(M, me, cards);
  if (rc != TF_OK) return rc;
  const tf::RankLayout &lay = M.lay;
  M.peer_base.assign(lay.send.size(), nullptr);
  M.peer_dst.assign(lay.send.size(), nullptr);
  for (size_t i = 0; i < lay.send.size() && can; ++i) {
    const int q = lay.send[i].peer;
    const ExchangeCard &cq = cards[q];
    if (!cq.has_halo || cq.host != me.host || cq.pid == me.pid) { can = false; break; }
    tf::RankLayout lq;   // where the peer expects this rank's rows
    tf::make_layout(q, world, bounds.data(), halos, lq);
    long long start = -1;
    for (const tf::ExchangeSegment &r : lq.recv)
      if (r.peer == rank && r.count == lay.send[i].count) start = r.start;
    if (start < 0) { can = false; break; }
    void *mapped = nullptr;
    if (cudaIpcOpenMemHandle(&mapped, cq.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      (void)cudaGetLastError();
      can = false;
      break;
    }
    M.peer_base[i] = mapped;
    M.peer_dst[i] = reinterpret_cast<float *>((char *)mapped + cq.halo_offset) + (size_t)start * M.n_cols;
  }
  std::vector<int> votes;
  rc = gather_records(M, (int)can, votes);
  if (rc != TF_OK) return rc;
  for (int v : votes) can = can && v != 0;
  if (!can) {
    for (void *&b : M.peer_base) if (b) { cudaIpcCloseMemHandle(b); b = nullptr; }
    M.peer_base.clear(); M.peer_dst.clear();
    return TF_OK;
  }
  TF_CUDA(cudaMalloc(&M.tokens, sizeof(int) * (2 + (size_t)world)));
  TF_CUDA(cudaMemset(M.tokens, 0, sizeof(int) * (2 + (size_t)world)));
  M.direct = true;
  return TF_OK;
}

// One-int messages between neighbours in one NCCL group: this rank sends to `to`, receives from `from`.
int token_round(tf_multi &M, const std::vector<int> &to, const std::vector<int> &from) {
  TF_NCCL(nccl().GroupStart());
  for (int q : to) TF_NCCL(nccl().Send(M.tokens, 1, kNcclInt32, q, M.c->comm, M.comm_stream));
  for (size_t i = 0; i < from.size(); ++i) TF_NCCL(nccl().Recv(M.tokens + 1 + i, 1, kNcclInt32, from[i], M.c->comm, M.comm_stream));
  TF_NCCL(nccl().GroupEnd());
  return TF_OK;
}

}  // namespace

extern "C" {

int tf_comm_unique_id(char id[128]) {
  if (!id) return fail(TF_ERR_ARG, "tf_comm_unique_id: null argument");
  if (!nccl().ok) return fail(TF_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded into this process");
  NcclUniqueId u;
  TF_NCCL(nccl().GetUniqueId(&u));
  std::memcpy(id, u.internal, 128);
  return TF_OK;
}

int tf_comm_create(const char id[128], int world, int rank, tf_comm **out) {
  if (!id || !out || world < 1 || rank < 0 || rank >= world) return fail(TF_ERR_ARG, "tf_comm_create: bad argument");
  if (!nccl().ok) return fail(TF_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded into this process");
  std::unique_ptr<tf_comm> c(new tf_comm());
  c->world = world; c->rank = rank; c->owned = true;
  TF_CUDA(cudaGetDevice(&c->device));
  NcclUniqueId u;
  std::memcpy(u.internal, id, 128);
  if (nccl().CommInitRankConfig) {
    NcclConfig217 cfg;
    cfg.size = sizeof(cfg); cfg.magic = 0xcafebeefu; cfg.version = 21700;
    cfg.blocking = INT_MIN; cfg.cga_cluster_size = INT_MIN;   // INT_MIN: left to the library
    cfg.min_ctas = 1; cfg.max_ctas = kExchangeCtas;
    cfg.net_name = nullptr;
    TF_NCCL(nccl().CommInitRankConfig(&c->comm, world, u, rank, &cfg));
  } else {
    TF_NCCL(nccl().CommInitRank(&c->comm, world, u, rank));
  }
  *out = c.release();
  return TF_OK;
}

int tf_comm_from_nccl(void *nccl_comm, int world, int rank, tf_comm **out) {
  if (!nccl_comm || !out || world < 1 || rank < 0 || rank >= world) return fail(TF_ERR_ARG, "tf_comm_from_nccl: bad argument");
  if (!nccl().ok) return fail(TF_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded into this process");
  std::unique_ptr<tf_comm> c(new tf_comm());
  c->comm = nccl_comm; c->world = world; c->rank = rank; c->owned = false;
  TF_CUDA(cudaGetDevice(&c->device));
  *out = c.release();
  return TF_OK;
}

void tf_comm_free(tf_comm *c) {
  if (!c) return;
  if (c->owned && c->comm && nccl().ok) nccl().CommDestroy(c->comm);
  delete c;
}

// Collective over the communicator: every rank calls it with its own rows.
int tf_multi_plan(tf_comm *c, int chain, long long r0, long long r1, const int *ap, const long long *ai, const float *ax,
                  int k, int n_cols, const tf_plan_opts *opts, tf_multi **out) {
  if (!c || !ap || !ai || !ax || !out || r1 <= r0) return fail(TF_ERR_ARG, "tf_multi_plan: bad argument");
  if (chain != 0 && chain != 1) return fail(TF_ERR_ARG, "tf_multi_plan: chain must be 0 (SpMM-SpMM) or 1 (GeMM-SpMM)");
  if (r1 - r0 > 0x7fffffffLL) return fail(TF_ERR_ARG, "tf_multi_plan: too many rows for one rank");
  TF_CUDA(cudaSetDevice(c->device));
  const int world = c->world, rank = c->rank;
  const int m = (int)(r1 - r0);
  const long long nnz = ap[m];
  std::unique_ptr<tf_multi> M(new tf_multi());
  M->c = c; M->chain = chain; M->n_cols = n_cols; M->k = k; M->r0 = r0; M->r1 = r1;
  TF_CUDA(cudaStreamCreateWithFlags(&M->comm_stream, cudaStreamNonBlocking));
  TF_CUDA(cudaEventCreateWithFlags(&M->ready, cudaEventDisableTiming));
  TF_CUDA(cudaEventCreateWithFlags(&M->arrived, cudaEventDisableTiming));

  // ---- every rank's bounds and halo list (two all-gathers of bytes) ----
  const std::vector<long long> mine = tf::halo_of(ai, nnz, r0, r1);
  std::vector<long long> head(3 * (size_t)world);  // {r0, r1, halo size} per rank
  {
    long long *d = nullptr;
    TF_CUDA(cudaMalloc(&d, sizeof(long long) * 3 * (size_t)world));
    const long long me[3] = {r0, r1, (long long)mine.size()};
    TF_CUDA(cudaMemcpy(d + 3 * rank, me, sizeof(me), cudaMemcpyHostToDevice));
    TF_NCCL(nccl().AllGather(d + 3 * rank, d, sizeof(me), kNcclInt8, c->comm, M->comm_stream));
    TF_CUDA(cudaStreamSynchronize(M->comm_stream));
    TF_CUDA(cudaMemcpy(head.data(), d, sizeof(long long) * head.size(), cudaMemcpyDeviceToHost));
    cudaFree(d);
  }
  std::vector<long long> bounds(world + 1);
  long long max_halo = 0;
  for (int g = 0; g < world; ++g) {
    bounds[g] = head[3 * g];
    if (g && head[3 * g] != head[3 * (g - 1) + 1]) return fail(TF_ERR_ARG, "tf_multi_plan: the ranks' row ranges must be consecutive");
    max_halo = std::max(max_halo, head[3 * g + 2]);
  }
  bounds[world] = head[3 * (world - 1) + 1];
  std::vector<std::vector<long long>> halos(world);
  if (max_halo > 0) {
    long long *d = nullptr;
    TF_CUDA(cudaMalloc(&d, sizeof(long long) * (size_t)max_halo * world));
    if (!mine.empty())
      TF_CUDA(cudaMemcpy(d + (size_t)max_halo * rank, mine.data(), sizeof(long long) * mine.size(), cudaMemcpyHostToDevice));
    TF_NCCL(nccl().AllGather(d + (size_t)max_halo * rank, d, sizeof(long long) * (size_t)max_halo, kNcclInt8, c->comm, M->comm_stream));
    TF_CUDA(cudaStreamSynchronize(M->comm_stream));
    std::vector<long long> all((size_t)max_halo * world);
    TF_CUDA(cudaMemcpy(all.data(), d, sizeof(long long) * all.size(), cudaMemcpyDeviceToHost));
    cudaFree(d);
    for (int g = 0; g < world; ++g) halos[g].assign(all.begin() + (size_t)max_halo * g, all.begin() + (size_t)max_halo * g + head[3 * g + 2]);
  }
  tf::make_layout(rank, world, bounds.data(), halos, M->lay);
  const tf::RankLayout &lay = M->lay;
  const long long n_halo = (long long)lay.halo_ids.size();

  // ---- the rank's operators in the executor's numbering ----
  std::vector<int> a_loc((size_t)nnz);
  for (long long j = 0; j < nnz; ++j) {
    const long long col = ai[j];
    if (col >= r0 && col < r1) a_loc[j] = (int)(col - r0);
    else a_loc[j] = m + (int)(std::lower_bound(lay.halo_ids.begin(), lay.halo_ids.end(), col) - lay.halo_ids.begin());
  }
  std::vector<int> bnd(lay.boundary_rows.begin(), lay.boundary_rows.end());
  tf_plan_opts o;
  std::memset(&o, 0, sizeof(o));
  o.slack_blocks = -1;
  if (opts) o = *opts;
  o.halo_rows = (int)n_halo;
  o.n_boundary = (int)bnd.size();
  o.boundary_rows = bnd.empty() ? nullptr : bnd.data();
  tf_csr A{m, m + (int)n_halo, ap, a_loc.data(), ax};
  int rc;
  if (chain == 0) {
    // first operator: the same rows, columns renumbered into the sorted list of rows of C they touch, which
    // must be one contiguous range [c_first, c_first + c_rows) of C (own rows plus ghost rows)
    std::vector<long long> ids(ai, ai + nnz);
    std::sort(ids.begin(), ids.end());
    ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
    if (ids.empty() || ids.back() - ids.front() + 1 != (long long)ids.size())
      return fail(TF_ERR_UNSUPPORTED, "tf_multi_plan: the rows of C a rank reads must form one contiguous range");
    M->c_first = ids.front(); M->c_rows = (long long)ids.size();
    std::vector<int> f_loc((size_t)nnz);
    for (long long j = 0; j < nnz; ++j) f_loc[j] = (int)(ai[j] - M->c_first);
    tf_csr F{m, (int)M->c_rows, ap, f_loc.data(), ax};
    rc = tf_plan_spmm_spmm(&A, &F, n_cols, &o, nullptr, &M->plan);
  } else {
    M->c_first = r0; M->c_rows = m;
    rc = tf_plan_gemm_spmm(&A, k, n_cols, &o, nullptr, &M->plan);
  }
  if (rc != TF_OK) return rc;
  long long sr = 0, hr = 0;
  rc = tf_plan_exchange_buffers(M->plan, &M->sendbuf, &sr, &M->halobuf, &hr);
  if (rc != TF_OK) return rc;
  M->gathers.resize(lay.send.size());
  for (size_t i = 0; i < lay.send.size(); ++i) {
    if (lay.send[i].index.empty()) continue;
    TF_CUDA(cudaMalloc(&M->gathers[i].idx, sizeof(long long) * lay.send[i].index.size()));
    TF_CUDA(cudaMemcpy(M->gathers[i].idx, lay.send[i].index.data(), sizeof(long long) * lay.send[i].index.size(), cudaMemcpyHostToDevice));
    TF_CUDA(cudaMalloc(&M->gathers[i].stage, sizeof(float) * lay.send[i].index.size() * n_cols));
  }
  rc = setup_direct_exchange(*M, bounds, halos, !(opts && opts->exchange < 0));
  if (rc != TF_OK) return rc;
  *out = M.release();
  return TF_OK;
}

void tf_multi_free(tf_multi *m) { delete m; }

// info = {local rows, halo rows, boundary rows, first row of C the rank reads, rows of C it reads, send peers,
// receive peers, kernels launched by the last step}
int tf_multi_info(const tf_multi *m, long long info[8]) {
  if (!m || !info) return fail(TF_ERR_ARG, "tf_multi_info: null argument");
  long long pi[8];
  tf_plan_info(m->plan, pi);
  info[0] = m->r1 - m->r0; info[1] = (long long)m->lay.halo_ids.size(); info[2] = (long long)m->lay.boundary_rows.size();
  info[3] = m->c_first; info[4] = m->c_rows; info[5] = (long long)m->lay.send.size(); info[6] = (long long)m->lay.recv.size();
  info[7] = pi[5];
  return TF_OK;
}

tf_plan *tf_multi_plan_handle(tf_multi *m) { return m ? m->plan : nullptr; }

// One step of the chain on this rank: phase 0, the exchange on the communicator's own stream, phase 1 beside it,
// phase 2 after the receive.  in0: the rank's rows of C ([c_first, c_first + c_rows), SpMM-SpMM) or of B
// (GeMM-SpMM); in1: the weight (GeMM-SpMM); D: the rank's rows of the result.  Work is enqueued; nothing waits.
int tf_multi_exec(tf_multi *m, const float *in0, const float *in1, int w_transposed, int relu, float *D, void *stream) {
  if (!m || !in0 || !D) return fail(TF_ERR_ARG, "tf_multi_exec: null argument");
  TF_CUDA(cudaSetDevice(m->c->device));
  cudaStream_t s = (cudaStream_t)stream;
  const tf::RankLayout &lay = m->lay;
  int rc;
  long long pinfo[8];
  tf_plan_info(m->plan, pinfo);
  const bool marching = pinfo[5] == 128 && m->chain == 0;
  const bool exchange = !lay.send.empty() || !lay.recv.empty();
  const bool tr = m->trace;
  if (tr) TF_CUDA(cudaEventRecord(m->tev[0], s));
  // Phase 0 (the boundary rows for the neighbours) is short and goes first, on every SM.
  if (!lay.boundary_rows.empty()) {
    rc = tf_exec_phase(m->plan, 0, in0, in1, w_transposed, relu, nullptr, s);
    if (rc != TF_OK) return rc;
  }
  if (tr) TF_CUDA(cudaEventRecord(m->tev[1], s));
  if (exchange) {
    TF_CUDA(cudaEventRecord(m->ready, s));
    TF_CUDA(cudaStreamWaitEvent(m->comm_stream, m->ready, 0));
    for (size_t i = 0; i < lay.send.size(); ++i)
      if (m->gathers[i].idx) {
        gather_rows_kernel<<<(unsigned)std::min<long long>(lay.send[i].count, 1184), 128, 0, m->comm_stream>>>(
            m->sendbuf, m->gathers[i].idx, lay.send[i].count, m->n_cols, m->gathers[i].stage);
        TF_CUDA(cudaGetLastError());
      }
    if (m->direct) {
      // (1) every rank tells the ranks that write into its halo rows that its previous step no longer reads them,
      // (2) the copy engines move the send segments into the neighbours' halo rows, (3) every rank tells the
      // owners of those rows that they are complete.  No SM moves data; the two token kernels are one CTA each.
      std::vector<int> senders, receivers;
      for (const tf::ExchangeSegment &r : lay.recv) senders.push_back(r.peer);
      for (const tf::ExchangeSegment &x : lay.send) receivers.push_back(x.peer);
      rc = token_round(*m, senders, receivers);
      if (rc != TF_OK) return rc;
      for (size_t i = 0; i < lay.send.size(); ++i) {
        const float *src = m->gathers[i].idx ? m->gathers[i].stage : m->sendbuf + (size_t)lay.send[i].start * m->n_cols;
        TF_CUDA(cudaMemcpyAsync(m->peer_dst[i], src, sizeof(float) * (size_t)lay.send[i].count * m->n_cols, cudaMemcpyDeviceToDevice,
                                m->comm_stream));
      }
      rc = token_round(*m, receivers, senders);
      if (rc != TF_OK) return rc;
    } else {
      TF_NCCL(nccl().GroupStart());
      for (size_t i = 0; i < lay.send.size(); ++i) {
        const float *src = m->gathers[i].idx ? m->gathers[i].stage : m->sendbuf + (size_t)lay.send[i].start * m->n_cols;
        TF_NCCL(nccl().Send(src, (size_t)lay.send[i].count * m->n_cols, kNcclFloat, lay.send[i].peer, m->c->comm, m->comm_stream));
      }
      for (const tf::ExchangeSegment &r : lay.recv)
        TF_NCCL(nccl().Recv(m->halobuf + (size_t)r.start * m->n_cols, (size_t)r.count * m->n_cols, kNcclFloat, r.peer, m->c->comm,
                            m->comm_stream));
      TF_NCCL(nccl().GroupEnd());
    }
    TF_CUDA(cudaEventRecord(m->arrived, m->comm_stream));
    if (tr) TF_CUDA(cudaEventRecord(m->tev[2], m->comm_stream));
  }
  if (marching && exchange) {
    // Plane-marching plans compute the intermediate inside phase 1, which therefore does not wait for anything.
    // Phase 2 (the first / last plane of D, with its own ticket state) follows the receive on the communication
    // stream and runs beside phase 1 -- on the SMs phase 1 leaves free for the exchange, then on those its CTAs
    // give up -- instead of after it.
    rc = tf_exec_phase(m->plan, 2, in0, in1, w_transposed, relu, D, m->comm_stream);
    if (rc != TF_OK) return rc;
    if (tr) TF_CUDA(cudaEventRecord(m->tev[3], m->comm_stream));
    TF_CUDA(cudaEventRecord(m->arrived, m->comm_stream));
    rc = tf_exec_phase(m->plan, 1, in0, in1, w_transposed, relu, D, s);
    if (rc != TF_OK) return rc;
    if (tr) TF_CUDA(cudaEventRecord(m->tev[4], s));
    TF_CUDA(cudaStreamWaitEvent(s, m->arrived, 0));
    if (tr) TF_CUDA(cudaEventRecord(m->tev[5], s));
    return TF_OK;
  }
  rc = tf_exec_phase(m->plan, 1, in0, in1, w_transposed, relu, D, s);
  if (rc != TF_OK) return rc;
  if (tr) TF_CUDA(cudaEventRecord(m->tev[4], s));
  if (exchange) TF_CUDA(cudaStreamWaitEvent(s, m->arrived, 0));
  rc = tf_exec_phase(m->plan, 2, in0, in1, w_transposed, relu, D, s);
  if (tr) {
    TF_CUDA(cudaEventRecord(m->tev[3], s));
    TF_CUDA(cudaEventRecord(m->tev[5], s));
  }
  return rc;
}

// on != 0: the following steps record their phases; ms (may be null) receives the times of the last traced step,
// measured from its start: {phase 0 done, exchange done, phase 2 done, phase 1 done, step done} (-1: not recorded).
int tf_multi_trace(tf_multi *m, int on, float ms[5]) {
  if (!m) return fail(TF_ERR_ARG, "tf_multi_trace: null argument");
  TF_CUDA(cudaSetDevice(m->c->device));
  if (ms) {
    for (int i = 0; i < 5; ++i) ms[i] = -1.f;
    if (m->trace && m->tev[0]) {
      TF_CUDA(cudaDeviceSynchronize());
      for (int i = 1; i < 6; ++i)
        if (cudaEventElapsedTime(&ms[i - 1], m->tev[0], m->tev[i]) != cudaSuccess) { ms[i - 1] = -1.f; (void)cudaGetLastError(); }
    }
  }
  if (on && !m->tev[0])
    for (cudaEvent_t &e : m->tev) TF_CUDA(cudaEventCreate(&e));
  m->trace = on != 0;
  return TF_OK;
}

int tf_multi_status(tf_multi *m, void *stream) {
  if (!m) return fail(TF_ERR_ARG, "tf_multi_status: null argument");
  TF_CUDA(cudaStreamSynchronize(m->comm_stream));
  return tf_plan_status(m->plan, stream);
}

}  // extern "C"
