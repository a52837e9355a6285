// Stream-ordered scratch buffer: taken from the device's memory pool on the
// launching stream and returned to it (also stream-ordered) when the object
// goes out of scope, so kernels already queued on the stream keep a valid
// buffer and other streams never see it.
#pragma once
#include "common.cuh"

namespace mt {
struct TempBuf {
  void* ptr = nullptr;
  cudaStream_t st;
  bool ok_ = true;
  TempBuf(size_t bytes, cudaStream_t s) : st(s) {
    if (bytes == 0) return;
    cudaError_t e = cudaMallocAsync(&ptr, bytes, s);
    if (e != cudaSuccess) {
      set_error("scratch allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
      ok_ = false;
      ptr = nullptr;
    }
  }
  ~TempBuf() { if (ptr) cudaFreeAsync(ptr, st); }
  bool ok() const { return ok_; }
  TempBuf(const TempBuf&) = delete;
  TempBuf& operator=(const TempBuf&) = delete;
};
}  // namespace mt
