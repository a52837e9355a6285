// Event-pair timing of one class of kernel launches (see mt_prof_begin).
#pragma once
#include <cuda_runtime.h>

namespace mt {
enum { PROF_GEMM = 1, PROF_ATTN = 2 };
int prof_kind();
// Records an event before construction and one at destruction on `s` when the
// given class is being timed; otherwise does nothing.
struct ProfScope {
  ProfScope(int kind, cudaStream_t s, double flops);
  ~ProfScope();
  bool active_;
  cudaStream_t s_;
};
}  // namespace mt
