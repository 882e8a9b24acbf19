// Exercises include/tile-fusion.h the way the reference's README shows the API being used.
// Usage: api_test inspect | api_test run      (run needs a GPU)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "tile-fusion.h"

using namespace swiftware;

int main(int argc, char **argv) {
  const bool run = argc > 1 && std::strcmp(argv[1], "run") == 0;
  // 1-D 3-point Laplacian, n = 1000: the reference's fixed-tile inspector with 4 threads and
  // IterPerPartition 64 gives ptr1 = {0, 15, 30} and 972 fused rows
  const int n = 1000;
  std::vector<int> ap(n + 1, 0), ai;
  std::vector<float> ax;
  for (int i = 0; i < n; ++i) {
    if (i > 0) { ai.push_back(i - 1); ax.push_back(-1.f); }
    ai.push_back(i); ax.push_back(2.f);
    if (i < n - 1) { ai.push_back(i + 1); ax.push_back(-1.f); }
    ap[i + 1] = (int)ai.size();
  }
  def::CSRMatrix A(n, n, ap.data(), ai.data(), ax.data());
  def::ScheduleParameters sp;
  sp.IterPerPartition = 64;
  def::FusedSchedule s = fusion::inspector(A, 4, sp);
  const int *ptr1, *ptr2, *id, *type, *ker;
  s.arrays(&ptr1, &ptr2, &id, &type, &ker);
  if (s.levels() != 2 || ptr1[1] != 15 || ptr1[2] != 30 || ker[0] != 67 || ker[1] != 133) {
    std::printf("FAIL schedule %d %d %d %d %d\n", s.levels(), ptr1[1], ptr1[2], ker[0], ker[1]);
    return 1;
  }
  bool threw = false;
  try { fusion::inspector(def::CSRMatrix(n, n, ap.data(), ai.data(), ax.data()), 4, [] { def::ScheduleParameters q; q.kind = 9; return q; }()); }
  catch (const std::runtime_error &) { threw = true; }
  if (!threw) { std::printf("FAIL: bad inspector kind accepted\n"); return 1; }
  if (!run) { std::printf("OK inspect\n"); return 0; }

  // D = A * (A * 1): 2 on the first row, -1 on the second, 0 inside (the reference's demo input)
  const int N = 32;
  std::vector<float> c((size_t)n * N, 1.f), d((size_t)n * N, -7.f);
  for (int mode : {TF_MODE_STREAM, TF_MODE_SCHEDULE}) {
    s.mode = mode;
    std::fill(d.begin(), d.end(), -7.f);
    fusion::spMMSpMMExecutor(A, A, def::Matrix(n, N, c.data()), def::Matrix(n, N, d.data()), s, 4);
    double sum = 0;
    for (float v : d) sum += v;
    if (d[0] != 2.f || d[N] != -1.f || d[2 * N] != 0.f || sum != 2.0 * N) { std::printf("FAIL spmm-spmm mode %d sum %g\n", mode, sum); return 1; }
  }
  // D = A * (B * W) with B = ones (n x 8), W = ones (8 x N): B*W = 8, so D = 8 * (A * 1)
  std::vector<float> b((size_t)n * 8, 1.f), w((size_t)8 * N, 1.f);
  s.mode = TF_MODE_STREAM;
  fusion::geMMSpMMExecutor(A, def::Matrix(n, 8, b.data()), def::Matrix(8, N, w.data()), def::Matrix(n, N, d.data()), s, 4);
  if (d[0] != 8.f || d[N] != 0.f || d[(size_t)(n - 1) * N] != 8.f) { std::printf("FAIL gemm-spmm %g %g\n", d[0], d[N]); return 1; }
  std::printf("OK run\n");
  return 0;
}
