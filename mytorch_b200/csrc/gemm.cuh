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
    case 5: return x * a;                                   // x * aux (aux = a stored derivative)
    case 6: return x * 2.f * sqrtf(fmaxf(a, 0.f));          // x * d/du relu(u)^2 with aux = relu(u)^2 itself
    default: return x;
  }
}
// `act` carries the activation in its low byte; with this bit the second output ("preact")
// receives the activation's derivative at the pre-activation instead of the pre-activation.
constexpr int kActStoreGrad = 0x100;
// d/dx act(x), exact tanh (CUDA-core path and reference for the tensor-core epilogue).
__device__ __forceinline__ float act_grad(float x, int act) {
  switch (act & 0xff) {
    case MT_ACT_GELU: {
      const float x2 = x * x;
      const float t = tanhf(0.7978845608f * (x + 0.044715f * x2 * x));
      return 0.5f * (1.f + t + x * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * x2));
    }
    case MT_ACT_RELU2: return 2.f * fmaxf(x, 0.f);
    case MT_ACT_RELU: return x > 0.f ? 1.f : 0.f;
    default: return 1.f;
  }
}
int gemm_simt(const GemmArgs& g, cudaStream_t st);
bool gemm_tc_supported(const GemmArgs& g);
int gemm_tc(const GemmArgs& g, cudaStream_t st);
}  // namespace mt
