// CUDA-core GEMM with fp32 accumulation: the full-precision path for fp32
// operands (tensor cores would round to tf32) and the fallback for half
// operands whose pointers or strides TMA cannot address. 64x64x16 tiles,
// 256 threads, 4x4 outputs per thread, any strides / transposes / tails.
#include "common.cuh"
#include "gemm.cuh"

namespace mt {

constexpr int SBM = 64, SBN = 64, SBK = 16;

__device__ __forceinline__ float act_apply(float x, int act) {
  switch (act) {
    case MT_ACT_GELU: {
      float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(inner));
    }
    case MT_ACT_RELU2: { float r = fmaxf(x, 0.f); return r * r; }
    case MT_ACT_RELU: return fmaxf(x, 0.f);
    default: return x;
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C, TO* __restrict__ preact,
                 const TI* __restrict__ bias, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                 int64_t ldc, int trans_a, int trans_b, int act, float alpha, int accumulate,
                 const TO* __restrict__ aux, int aux_mode) {
  __shared__ float As[SBK][SBM + 4];
  __shared__ float Bs[SBK][SBN + 4];
  const int tid = threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * SBM, n0 = (int64_t)blockIdx.x * SBN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += SBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = tid + i * 256;
      int m, k;
      if (trans_a) { m = idx % SBM; k = idx / SBM; } else { k = idx % SBK; m = idx / SBK; }
      int64_t gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < K) v = to_f(trans_a ? A[gk * lda + gm] : A[gm * lda + gk]);
      As[k][m] = v;
      int n, kb;
      if (trans_b) { kb = idx % SBK; n = idx / SBK; } else { n = idx % SBN; kb = idx / SBN; }
      int64_t gn = n0 + n, gkb = k0 + kb;
      float w = 0.f;
      if (gn < N && gkb < K) w = to_f(trans_b ? B[gn * ldb + gkb] : B[gkb * ldb + gn]);
      Bs[kb][n] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SBK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][tm + i]; b[i] = Bs[k][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = alpha * acc[i][j];
      if (bias) v += to_f(bias[gn]);
      if (preact) preact[gm * ldc + gn] = from_f<TO>((act & kActStoreGrad) ? act_grad(v, act) : v);
      v = act_apply(v, act & 0xff);
      if (aux_mode) v = aux_apply(v, to_f(aux[gm * ldc + gn]), aux_mode);
      if (accumulate) v += to_f(C[gm * ldc + gn]);
      C[gm * ldc + gn] = from_f<TO>(v);
    }
  }
}

int gemm_simt(const GemmArgs& g, cudaStream_t st) {
  if (g.M == 0 || g.N == 0) return MT_OK;
  dim3 grid((unsigned)((g.N + SBN - 1) / SBN), (unsigned)((g.M + SBM - 1) / SBM));
  MT_REQUIRE(grid.y <= 65535, "gemm: M too large for the CUDA-core kernel");
  MT_DISPATCH_FLOAT(g.in_dtype, TI, {
    MT_DISPATCH_FLOAT(g.out_dtype, TO, {
      gemm_simt_kernel<TI, TO><<<grid, 256, 0, st>>>((const TI*)g.A, (const TI*)g.B, (TO*)g.C, (TO*)g.preact,
                                                    (const TI*)g.bias, g.M, g.N, g.K, g.lda, g.ldb, g.ldc,
                                                    g.trans_a, g.trans_b, g.act, g.alpha, g.accumulate, (const TO*)g.aux, g.aux_mode);
    });
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // namespace mt
