// tile-fusion.h -- the C++ operator interface the reference documents (README.md:21-38):
//
//   swiftware::def::FusedSchedule swiftware::fusion::inspector(swiftware::def::CSRMatrix A, int NumThreads);
//   swiftware::fusion::spMMSpMMExecutor(CSRMatrix A, CSRMatrix B, Matrix C, Matrix D, FusedSchedule schedule, int NumThreads);
//   swiftware::fusion::geMMSpMMExecutor(CSRMatrix A, Matrix  B, Matrix C, Matrix D, FusedSchedule schedule, int NumThreads);
//   swiftware::CSRMatrix(int M, int N, int* Ap, int* Ai, float* Ax);   swiftware::Matrix(int M, int N, float* Data);
//
// with D = A * B * C.  The reference names this header but does not ship it; here it is a header-only
// layer over the C ABI of libtilefusion_b200 (tile_fusion_b200.h).  Matrices do not own their arrays.
// Dense data is host memory unless Matrix::onDevice is set.  Errors throw std::runtime_error.
#ifndef TILE_FUSION_H
#define TILE_FUSION_H

#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>

#include "tile_fusion_b200.h"

namespace swiftware {
namespace def {

struct CSRMatrix {
  int M, N;
  int *Ap, *Ai;
  float *Ax;
  CSRMatrix(int M_, int N_, int *Ap_, int *Ai_, float *Ax_) : M(M_), N(N_), Ap(Ap_), Ai(Ai_), Ax(Ax_) {}
  tf_csr view() const { return tf_csr{M, N, Ap, Ai, Ax}; }
  // Sampled checksum of the matrix (size, up to 2048 evenly spaced column ids and values): the plan cache keys on it
  // beside the array addresses, so that arrays refilled in place with another matrix get a new plan.  A change
  // that touches none of the sampled entries is not seen: build a new CSRMatrix over new arrays for new values.
  unsigned long long fingerprint() const {
    unsigned long long h = 1469598103934665603ull;
    auto mix = [&h](unsigned long long v) { h = (h ^ v) * 1099511628211ull; };
    const long long nnz = Ap[M];
    mix((unsigned long long)M); mix((unsigned long long)N); mix((unsigned long long)nnz);
    const long long step = nnz > 2048 ? nnz / 2048 : 1;
    for (long long j = 0; j < nnz; j += step) {
      unsigned bits;
      std::memcpy(&bits, &Ax[j], sizeof(bits));
      mix(((unsigned long long)(unsigned)Ai[j] << 32) | bits);
    }
    return h;
  }
};

struct Matrix {
  int M, N;
  float *Data;
  bool onDevice;
  Matrix(int M_, int N_, float *Data_, bool onDevice_ = false) : M(M_), N(N_), Data(Data_), onDevice(onDevice_) {}
};

// Mirrors sym_lib::ScheduleParameters (fusion/include/sparse-fusion/Fusion_Defs.h:21-55).
struct ScheduleParameters {
  int kind = TF_INSPECT_FIXED;
  int IterPerPartition = 2048;
  int TileM = 1250000;  // cache budget in bytes for the variable-tile inspectors
  int BCol = 32, CCol = 32;
  int DataSize = 4;
};

inline void check(int rc) {
  if (rc != TF_OK) throw std::runtime_error(std::string("tile-fusion: ") + tf_last_error());
}

// The schedule (sym_lib::MultiDimensionalSet) plus the device plans built from it on first use.
class FusedSchedule {
 public:
  FusedSchedule() = default;
  explicit FusedSchedule(tf_schedule *s) : impl_(std::make_shared<Impl>(s)) {}
  const tf_schedule *get() const { return impl_ ? impl_->s : nullptr; }
  int levels() const { int n1 = 0; check(tf_schedule_dims(get(), &n1, nullptr, nullptr, nullptr)); return n1; }
  int partitions() const { int np = 0; check(tf_schedule_dims(get(), nullptr, &np, nullptr, nullptr)); return np; }
  // LevelPtr, ParPtr, Partition, ParType, MixPtr of the reference's executors
  void arrays(const int **ptr1, const int **ptr2, const int **id, const int **type, const int **ker) const {
    check(tf_schedule_arrays(get(), ptr1, ptr2, id, type, ker));
  }
  // mode: TF_MODE_STREAM runs the library's own plan, TF_MODE_SCHEDULE follows this schedule tile by tile
  int mode = TF_MODE_STREAM;

  tf_plan *plan(int chain, const CSRMatrix &A, const CSRMatrix *B, int k, int n) const {
    if (!impl_) throw std::runtime_error("tile-fusion: empty schedule");
    auto key = std::make_tuple(chain, (const void *)A.Ap, B ? (const void *)B->Ap : nullptr, k, n, mode,
                               A.fingerprint() ^ (B ? 31 * B->fingerprint() : 0ull));
    auto it = impl_->plans.find(key);
    if (it != impl_->plans.end()) return it->second;
    tf_plan_opts o{};
    o.mode = mode;
    o.slack_blocks = -1;
    tf_plan *p = nullptr;
    tf_csr a = A.view();
    if (chain == 0) {
      tf_csr b = B ? B->view() : a;
      check(tf_plan_spmm_spmm(&a, B && B->Ap != A.Ap ? &b : nullptr, n, &o, impl_->s, &p));
    } else {
      check(tf_plan_gemm_spmm(&a, k, n, &o, impl_->s, &p));
    }
    impl_->plans[key] = p;
    return p;
  }

 private:
  struct Impl {
    tf_schedule *s;
    std::map<std::tuple<int, const void *, const void *, int, int, int, unsigned long long>, tf_plan *> plans;
    explicit Impl(tf_schedule *s_) : s(s_) {}
    ~Impl() {
      for (auto &kv : plans) tf_plan_free(kv.second);
      tf_schedule_free(s);
    }
  };
  std::shared_ptr<Impl> impl_;
};

}  // namespace def

using def::CSRMatrix;
using def::Matrix;

namespace fusion {

// README.md:25.  The two-argument form runs the fixed-tile inspector with its default
// IterPerPartition; the overload selects any of the reference inspectors.
inline def::FusedSchedule inspector(def::CSRMatrix A, int NumThreads, const def::ScheduleParameters &sp) {
  tf_sched_params p{sp.kind, NumThreads, sp.IterPerPartition, sp.TileM, sp.BCol, sp.CCol, sp.DataSize};
  tf_schedule *s = nullptr;
  def::check(tf_inspect(A.M, A.Ap, A.Ai, &p, &s));
  return def::FusedSchedule(s);
}
inline def::FusedSchedule inspector(def::CSRMatrix A, int NumThreads) {
  return inspector(A, NumThreads, def::ScheduleParameters());
}

// README.md:31.  D = A * (B * C), A and B sparse.  NumThreads is kept for source compatibility.
inline void spMMSpMMExecutor(def::CSRMatrix A, def::CSRMatrix B, def::Matrix C, def::Matrix D,
                             def::FusedSchedule schedule, int /*NumThreads*/) {
  if (C.N != D.N || D.M != A.M || C.M != B.N || B.M != A.N) throw std::runtime_error("tile-fusion: shapes do not chain");
  tf_plan *p = schedule.plan(0, A, &B, 0, C.N);
  if (C.onDevice && D.onDevice) def::check(tf_exec_spmm_spmm(p, C.Data, D.Data, nullptr));
  else if (!C.onDevice && !D.onDevice) def::check(tf_spmm_spmm_host(p, C.Data, D.Data));
  else throw std::runtime_error("tile-fusion: C and D must both be host or both be device data");
}

// README.md:32.  D = A * (B * C), B (M x K) and C (K x N) dense.
inline void geMMSpMMExecutor(def::CSRMatrix A, def::Matrix B, def::Matrix C, def::Matrix D,
                             def::FusedSchedule schedule, int /*NumThreads*/) {
  if (C.M != B.N || D.N != C.N || D.M != A.M || B.M != A.N) throw std::runtime_error("tile-fusion: shapes do not chain");
  tf_plan *p = schedule.plan(1, A, nullptr, B.N, C.N);
  const bool dev = B.onDevice && C.onDevice && D.onDevice, host = !B.onDevice && !C.onDevice && !D.onDevice;
  if (dev) def::check(tf_exec_gemm_spmm(p, B.Data, C.Data, 0, 0, D.Data, nullptr));
  else if (host) def::check(tf_gemm_spmm_host(p, B.Data, C.Data, 0, 0, D.Data));
  else throw std::runtime_error("tile-fusion: B, C and D must all be host or all be device data");
}

}  // namespace fusion
}  // namespace swiftware

#endif  // TILE_FUSION_H
