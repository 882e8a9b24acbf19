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

// One call's copies.  upload() / download() are cudaMemcpyAsync on the given stream for pinned arrays; for pageable
// ones they go piece by piece through the rings: the calling thread fills upload slots (and waits for the copy engine
// before it reuses one), a second thread empties download slots into the caller's array as they land.
class HostPipe {
 public:
  explicit HostPipe(int threads) : rings_(threads, threads) {}
  ~HostPipe() { stop_drainer(); }

  cudaError_t begin(int device, bool stage_in, bool stage_out, size_t piece_bytes, int slots) {
    stop_drainer();
    stage_in_ = stage_in; stage_out_ = stage_out;
    n_up_ = 0; n_down_ = 0; drained_ = 0; failed_ = false; stop_ = false;
    jobs_.clear();
    if (!stage_in && !stage_out) return cudaSuccess;
    cudaError_t e = rings_.reserve(piece_bytes, slots);
    if (e != cudaSuccess) return e;
    if (stage_out) drainer_ = std::thread([this, device] { drain(device); });
    return cudaSuccess;
  }

  cudaError_t upload(void *d_dst, const void *h_src, size_t bytes, cudaStream_t s) {
    if (!stage_in_) return cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, s);
    const size_t piece = rings_.piece_bytes;
    for (size_t off = 0; off < bytes; off += piece, ++n_up_) {
      const size_t n = std::min(piece, bytes - off);
      const int slot = (int)(n_up_ % rings_.slots);
      cudaError_t e = n_up_ >= (unsigned long long)rings_.slots ? cudaEventSynchronize(rings_.in_sent[slot]) : cudaSuccess;
      if (e != cudaSuccess) return e;
      char *buf = rings_.in + (size_t)slot * piece;
      rings_.crew_in.copy(buf, (const char *)h_src + off, n);
      e = cudaMemcpyAsync((char *)d_dst + off, buf, n, cudaMemcpyHostToDevice, s);
      if (e == cudaSuccess) e = cudaEventRecord(rings_.in_sent[slot], s);
      if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
  }

  cudaError_t download(void *h_dst, const void *d_src, size_t bytes, cudaStream_t s) {
    if (!stage_out_) return cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, s);
    const size_t piece = rings_.piece_bytes;
    for (size_t off = 0; off < bytes; off += piece, ++n_down_) {
      const size_t n = std::min(piece, bytes - off);
      const int slot = (int)(n_down_ % rings_.slots);
      {
        std::unique_lock<std::mutex> g(m_);   // the slot's previous piece has reached the caller's array
        cv_.wait(g, [&] { return failed_ || drained_ + (unsigned long long)rings_.slots > n_down_; });
        if (failed_) return cudaErrorUnknown;
      }
      cudaError_t e = cudaMemcpyAsync(rings_.out + (size_t)slot * piece, (const char *)d_src + off, n, cudaMemcpyDeviceToHost, s);
      if (e == cudaSuccess) e = cudaEventRecord(rings_.out_landed[slot], s);
      if (e != cudaSuccess) return e;
      { std::lock_guard<std::mutex> g(m_); jobs_.push_back(Job{(char *)h_dst + off, n, slot}); }
      cv_.notify_all();
    }
    return cudaSuccess;
  }

  // every download has reached the caller's array
  cudaError_t finish() {
    if (!stage_out_) return cudaSuccess;
    {
      std::unique_lock<std::mutex> g(m_);
      cv_.wait(g, [&] { return failed_ || drained_ == n_down_; });
    }
    stop_drainer();
    return failed_ ? cudaErrorUnknown : cudaSuccess;
  }

 private:
  struct Job { char *dst; size_t bytes; int slot; };
  void drain(int device) {
    cudaSetDevice(device);
    for (size_t next = 0;; ++next) {
      Job j;
      {
        std::unique_lock<std::mutex> g(m_);
        cv_.wait(g, [&] { return stop_ || jobs_.size() > next; });
        if (jobs_.size() <= next) return;
        j = jobs_[next];
      }
      if (cudaEventSynchronize(rings_.out_landed[j.slot]) != cudaSuccess) {
        std::lock_guard<std::mutex> g(m_);
        failed_ = true;
        cv_.notify_all();
        return;
      }
      rings_.crew_out.copy(j.dst, rings_.out + (size_t)j.slot * rings_.piece_bytes, j.bytes);
      { std::lock_guard<std::mutex> g(m_); ++drained_; }
      cv_.notify_all();
    }
  }
  void stop_drainer() {
    { std::lock_guard<std::mutex> g(m_); stop_ = true; }
    cv_.notify_all();
    if (drainer_.joinable()) drainer_.join();
  }

  StageRings rings_;
  bool stage_in_ = false, stage_out_ = false;
  unsigned long long n_up_ = 0, n_down_ = 0, drained_ = 0;
  std::mutex m_;
  std::condition_variable cv_;
  std::vector<Job> jobs_;
  bool stop_ = false, failed_ = false;
  std::thread drainer_;
};

}  // namespace tf
