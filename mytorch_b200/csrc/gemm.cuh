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
  const void* aux = nullptr;  // [M,N] in the output dtype, row stride ldc
  int aux_mode = 0;           // see mt_gemm_ex
};

// Elementwise combination of the GEMM result with the aux operand (after bias/activation).
__device__ __forceinline__ float aux_apply(float x, float a, int mode) {
  switch (mode) {
    case 1: return x + a;                                   // residual add
    case 2: {                                               // x * gelu'(a)
      const float a2 = a * a;
      const float t = tanhf(0.7978845608f * (a + 0.044715f * a2 * a));
      return x * (0.5f * (1.f + t + a * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * a2)));
    }
    case 3: return x * 2.f * fmaxf(a, 0.f);                 // x * d/da relu(a)^2
    case 4: return a > 0.f ? x : 0.f;                       // x * d/da relu(a)
    default: return x;
  }
}
int gemm_simt(const GemmArgs& g, cudaStream_t st);
bool gemm_tc_supported(const GemmArgs& g);
int gemm_tc(const GemmArgs& g, cudaStream_t st);
}  // namespace mt
