// Staging of pageable host arrays for the host-pointer executors.
//
// The reference's call sites hand over plain new[] / malloc arrays (SpMM_SpMM_Demo_Utils.h:43-60).  A
// cudaMemcpyAsync from or to such memory goes through the driver's own bounce buffer with one copying thread and
// does not overlap anything (measured on the 1 GB + 1 GB headline call: 150 ms against 24 ms with pinned arrays).
// Here the call copies plane-sized pieces with a few threads of its own between the caller's arrays and two rings
// of pinned slots, and the copy engines move the slots: upload, kernel and download overlap as they do for pinned
// arrays, and the host copies run at memory speed.
#pragma once
#include <cuda_runtime.h>

#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace tf {

// A few threads that copy one range together; copy() returns when the range is done.
class CopyCrew {
 public:
  explicit CopyCrew(int n) {
    for (int i = 0; i < n; ++i) threads_.emplace_back([this, i] { loop(i); });
  }
  ~CopyCrew() {
    {
      std::lock_guard<std::mutex> g(m_);
      stop_ = true;
      ++job_;
    }
    wake_.notify_all();
    for (std::thread &t : threads_) t.join();
  }
  void copy(void *dst, const void *src, size_t bytes) {
    const int n = (int)threads_.size();
    if (n == 0 || bytes < (1u << 20)) { std::memcpy(dst, src, bytes); return; }
    std::unique_lock<std::mutex> g(m_);
    dst_ = (char *)dst; src_ = (const char *)src; bytes_ = bytes; left_ = n;
    ++job_;
    wake_.notify_all();
    done_.wait(g, [this] { return left_ == 0; });
  }

 private:
  void loop(int me) {
    unsigned long long seen = 0;
    for (;;) {
      char *dst; const char *src; size_t bytes;
      {
        std::unique_lock<std::mutex> g(m_);
        wake_.wait(g, [&] { return job_ != seen; });
        seen = job_;
        if (stop_) return;
        dst = dst_; src = src_; bytes = bytes_;
      }
      const size_t n = threads_.size(), piece = ((bytes + n - 1) / n + 4095) / 4096 * 4096;
      const size_t a = std::min(bytes, piece * me), b = std::min(bytes, a + piece);
      if (b > a) std::memcpy(dst + a, src + a, b - a);
      {
        std::lock_guard<std::mutex> g(m_);
        if (--left_ == 0) done_.notify_all();
      }
    }
  }
  std::vector<std::thread> threads_;
  std::mutex m_;
  std::condition_variable wake_, done_;
  unsigned long long job_ = 0;
  bool stop_ = false;
  char *dst_ = nullptr;
  const char *src_ = nullptr;
  size_t bytes_ = 0;
  int left_ = 0;
};

// Two rings of pinned slots (one piece each) with the events that say when a slot may be reused.
struct StageRings {
  size_t piece_bytes = 0;
  int slots = 0;
  char *in = nullptr, *out = nullptr;             // slots * piece_bytes each, pinned
  std::vector<cudaEvent_t> in_sent, out_landed;   // per slot
  CopyCrew crew_in, crew_out;
  StageRings(int threads_in, int threads_out) : crew_in(threads_in), crew_out(threads_out) {}
  ~StageRings() {
    if (in) cudaFreeHost(in);
    if (out) cudaFreeHost(out);
    for (cudaEvent_t e : in_sent) cudaEventDestroy(e);
    for (cudaEvent_t e : out_landed) cudaEventDestroy(e);
  }
  cudaError_t reserve(size_t piece, int n_slots) {
    if (piece == piece_bytes && n_slots == slots) return cudaSuccess;
    if (in) { cudaFreeHost(in); in = nullptr; }
    if (out) { cudaFreeHost(out); out = nullptr; }
    cudaError_t e = cudaHostAlloc((void **)&in, piece * n_slots, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&out, piece * n_slots, cudaHostAllocDefault);
    while (e == cudaSuccess && (int)in_sent.size() < n_slots) {
      cudaEvent_t a = nullptr, b = nullptr;
      e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
      in_sent.push_back(a); out_landed.push_back(b);
    }
    if (e == cudaSuccess) { piece_bytes = piece; slots = n_slots; }
    return e;
  }
};

inline bool is_pageable(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { (void)cudaGetLastError(); return true; }
  return a.type == cudaMemoryTypeUnregistered;
}

}  // namespace tf
