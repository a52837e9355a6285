// Multi-tensor optimizer kernels: one launch covers every parameter tensor.
//
//  * gradient sum of squares + inf/nan flag (for clipping and the loss-scale
//    state machine), two fixed-order stages;
//  * fused AdamW: unscale, clip, moment update, parameter update with the
//    reference's decay-after-update order, low-precision copy, optional
//    gradient clear.
// HBM-bound. Algorithmic traffic per parameter for the fused AMP update:
// p,m,v read+write (24 B) + gradient read (4 B fp32 / 2 B half) + half write (2 B).
#include "common.cuh"
#include "tempbuf.cuh"

namespace mt {

constexpr int kChunk = 4096;
constexpr int kOptThreads = 256;

template <typename TG>
__global__ void __launch_bounds__(kOptThreads)
gradnorm_kernel(mt_tensor_list L, const float* __restrict__ inv_scale, float* __restrict__ partial_sq,
                float* __restrict__ partial_inf) {
  __shared__ float sh[32];
  const int64_t chunk = blockIdx.x;
  const int t = L.chunk_tensor[chunk];
  const int64_t off = L.chunk_offset[chunk];
  const int64_t size = L.size[t];
  const TG* g = (const TG*)L.g[t] + off;
  const int64_t n = size - off < kChunk ? size - off : kChunk;
  const float sc = inv_scale ? inv_scale[0] : 1.f;
  float sq = 0.f, bad = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += kOptThreads) {
    float x = to_f(g[i]) * sc;
    if (!isfinite(x)) bad = 1.f;
    sq += x * x;
  }
  sq = block_sum(sq, sh);
  bad = block_max(bad, sh);
  if (threadIdx.x == 0) { partial_sq[chunk] = sq; partial_inf[chunk] = bad; }
}

__global__ void __launch_bounds__(1024)
gradnorm_final_kernel(const float* __restrict__ partial_sq, const float* __restrict__ partial_inf, int64_t n,
                      float* __restrict__ sumsq, float* __restrict__ found_inf) {
  __shared__ float sh[32];
  float s = 0.f, b = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { s += partial_sq[i]; b = fmaxf(b, partial_inf[i]); }
  s = block_sum(s, sh);
  b = block_max(b, sh);
  if (threadIdx.x == 0) {
    if (sumsq) sumsq[0] = s;
    if (found_inf) found_inf[0] = (b > 0.f || !isfinite(s)) ? 1.f : 0.f;
  }
}

template <typename TG, typename TH>
__global__ void __launch_bounds__(kOptThreads)
adamw_kernel(mt_tensor_list L, float lr, double beta1d, double beta2d, float eps,
             const float* __restrict__ inv_scale, const float* __restrict__ sumsq, float max_norm,
             const float* __restrict__ found_inf, int zero_grad, double* __restrict__ step_state, int slot) {
  const int64_t chunk = blockIdx.x;
  const bool skip_step = found_inf && found_inf[0] != 0.f;
  // Step counter and running beta powers live on the device and advance only when the update is
  // applied. Every block reads slot `slot`; block 0 writes the other slot, which the next call reads.
  const double* cur = step_state + 4 * slot;
  const double b1p = cur[1] * beta1d, b2p = cur[2] * beta2d;
  if (chunk == 0 && threadIdx.x == 0) {
    double* nxt = step_state + 4 * (slot ^ 1);
    nxt[0] = skip_step ? cur[0] : cur[0] + 1.0;
    nxt[1] = skip_step ? cur[1] : b1p;
    nxt[2] = skip_step ? cur[2] : b2p;
  }
  const float lr_t = (float)((double)lr * sqrt(1.0 - b2p) / (1.0 - b1p));
  const float beta1 = (float)beta1d, beta2 = (float)beta2d;
  const int t = L.chunk_tensor[chunk];
  const int64_t off = L.chunk_offset[chunk];
  const int64_t size = L.size[t];
  const int64_t n = size - off < kChunk ? size - off : kChunk;
  TG* g = (TG*)L.g[t] + off;
  if (skip_step) {
    if (zero_grad) for (int64_t i = threadIdx.x; i < n; i += kOptThreads) g[i] = from_f<TG>(0.f);
    return;
  }
  float* p = (float*)L.p[t] + off;
  float* m = (float*)L.m[t] + off;
  float* v = (float*)L.v[t] + off;
  TH* ph = (L.p_half && L.p_half[t]) ? (TH*)L.p_half[t] + off : nullptr;
  const float wd = L.weight_decay[t];
  float gs = inv_scale ? inv_scale[0] : 1.f;
  if (max_norm > 0.f && sumsq) {
    float coef = max_norm / (sqrtf(sumsq[0]) + 1e-6f);
    if (coef < 1.f) gs *= coef;
  }
  const float omb1 = 1.f - beta1, omb2 = 1.f - beta2;
  for (int64_t i = threadIdx.x; i < n; i += kOptThreads) {
    float gi = to_f(g[i]) * gs;
    float mi = beta1 * m[i] + omb1 * gi;
    float vi = beta2 * v[i] + omb2 * gi * gi;
    float pi = p[i] - lr_t * mi / (sqrtf(vi) + eps);
    if (wd != 0.f) pi = pi - lr * wd * pi;
    m[i] = mi;
    v[i] = vi;
    p[i] = pi;
    if (ph) ph[i] = from_f<TH>(pi);
    if (zero_grad) g[i] = from_f<TG>(0.f);
  }
}

// Loss-scale state machine on the device. state = {scale, inv_total, unskipped, skipped_steps}
// with inv_total = 1 / (scale * accumulation_steps).
__global__ void scaler_update_kernel(float* state, const float* found_inf, float growth, float backoff,
                                     int interval, float inv_accum, int dynamic) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float scale = state[0], unskipped = state[2];
  const bool bad = found_inf && found_inf[0] != 0.f;
  if (bad) state[3] += 1.f;
  if (dynamic) {
    if (bad) {
      scale *= backoff;
      unskipped = 0.f;
    } else {
      unskipped += 1.f;
      if ((int)unskipped == interval) { scale *= growth; unskipped = 0.f; }
    }
  }
  state[0] = scale;
  state[1] = inv_accum / scale;
  state[2] = unskipped;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_scaler_update(float* state, const float* found_inf, float growth, float backoff, int interval,
                     float inv_accum, int dynamic, void* stream) {
  MT_REQUIRE(state, "scaler_update: bad arguments");
  scaler_update_kernel<<<1, 32, 0, as_stream(stream)>>>(state, found_inf, growth, backoff, interval, inv_accum, dynamic);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_gradnorm_multi(const mt_tensor_list* L, int g_dtype, const float* inv_scale_dev, float* sumsq,
                      float* found_inf, void* stream) {
  MT_REQUIRE(L && L->n_chunks >= 0 && L->n_tensors >= 0, "gradnorm_multi: bad list");
  cudaStream_t st = as_stream(stream);
  int64_t nc = L->n_chunks;
  TempBuf part((size_t)(nc > 0 ? nc : 1) * 2 * sizeof(float), st);
  if (!part.ok()) return MT_ERR_CUDA;
  float* psq = (float*)part.ptr;
  float* pinf = psq + (nc > 0 ? nc : 1);
  if (nc > 0) {
    MT_DISPATCH_FLOAT(g_dtype, TG, (gradnorm_kernel<TG><<<(unsigned)nc, kOptThreads, 0, st>>>(*L, inv_scale_dev, psq, pinf)));
    MT_LAUNCH_CHECK();
  }
  gradnorm_final_kernel<<<1, 1024, 0, st>>>(psq, pinf, nc, sumsq, found_inf);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_adamw_multi(const mt_tensor_list* L, int g_dtype, int half_dtype, float lr, double beta1,
                   double beta2, float eps, const float* inv_scale_dev, const float* sumsq_dev, float max_norm,
                   const float* found_inf_dev, int zero_grad, double* step_state, int slot, void* stream) {
  MT_REQUIRE(L && L->n_chunks >= 0 && L->n_tensors >= 0, "adamw_multi: bad list");
  MT_REQUIRE(step_state && (slot == 0 || slot == 1), "adamw_multi: step_state (8 doubles on the device) and slot 0/1 are required");
  if (L->n_chunks == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  if (half_dtype != MT_F16 && half_dtype != MT_BF16) half_dtype = MT_F16;  // only used when p_half is given
  MT_DISPATCH_FLOAT(g_dtype, TG, {
    if (half_dtype == MT_F16)
      adamw_kernel<TG, __half><<<(unsigned)L->n_chunks, kOptThreads, 0, st>>>(*L, lr, beta1, beta2, eps, inv_scale_dev, sumsq_dev, max_norm, found_inf_dev, zero_grad, step_state, slot);
    else
      adamw_kernel<TG, __nv_bfloat16><<<(unsigned)L->n_chunks, kOptThreads, 0, st>>>(*L, lr, beta1, beta2, eps, inv_scale_dev, sumsq_dev, max_norm, found_inf_dev, zero_grad, step_state, slot);
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // extern "C"
