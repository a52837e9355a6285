// Internal GEMM interface shared by the tensor-core and CUDA-core kernels.
#pragma once
#include "common.cuh"

namespace mt {
struct GemmArgs {
  const void* A; const void* B; void* C; void* preact; const void* bias;
  int64_t M, N, K, lda, ldb, ldc;
  int trans_a, trans_b, in_dtype, out_dtype, act;
  float alpha;
  int accumulate;  // 0 store, 1 read-modify-write, 2 fp32 atomic add (split-K allowed)
};
int gemm_simt(const GemmArgs& g, cudaStream_t st);
bool gemm_tc_supported(const GemmArgs& g);
int gemm_tc(const GemmArgs& g, cudaStream_t st);
}  // namespace mt
