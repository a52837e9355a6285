// Rotary embedding followed by parameter-free RMSNorm over head_dim, for the q and k
// projections of the nanochat attention, forward and backward, one pass over each tensor.
//
// Unfused this is three kernels per tensor and direction (copy, rotate in place, normalise),
// i.e. six reads and writes of q and of k; here each head vector is read once, rotated and
// normalised in registers and written once. HBM-bound: algorithmic traffic forward
// 2 * tokens * heads * head_dim * sizeof(T) per tensor (the cos/sin rows of a token are shared
// by all its heads and stay in cache), backward 3x (dy and y in, dx out).
//
// Layout: head h of token (b, t) starts at base + (b*seq + t) * ld + h * head_dim, so a
// [B,T,H,D] tensor (ld = H*D) and a column slice of a wider projection are both read in place.
// A warp owns one token; a head vector is spread over LPV = head_dim / (16 bytes / sizeof(T))
// lanes (one 16-byte vector per lane), 32 / LPV heads per iteration. The rotation pairs column
// c with c + head_dim/2, which sit LPV/2 lanes apart: one shuffle exchanges them.
#include <initializer_list>

#include "common.cuh"

namespace mt {

template <int N>
__device__ __forceinline__ void load_row_f32(const float* __restrict__ p, float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 4) {
    const float4 f = *reinterpret_cast<const float4*>(p + i);
    v[i] = f.x; v[i + 1] = f.y; v[i + 2] = f.z; v[i + 3] = f.w;
  }
}

template <int LPV>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPV / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, int LPV>
__global__ void __launch_bounds__(128)
rope_rmsnorm_fwd_kernel(const T* __restrict__ x0, const T* __restrict__ x1, T* __restrict__ y0, T* __restrict__ y1,
                        float* __restrict__ r0, float* __restrict__ r1, const float* __restrict__ cs,
                        const float* __restrict__ sn, int64_t tokens, int seq, int heads, int64_t ld_x, int64_t ld_y,
                        float eps) {
  constexpr int VN = Vec16<T>::N;
  constexpr int D = LPV * VN;
  constexpr int VPW = 32 / LPV;
  const T* __restrict__ x = blockIdx.y ? x1 : x0;
  T* __restrict__ y = blockIdx.y ? y1 : y0;
  float* __restrict__ rs = blockIdx.y ? r1 : r0;
  const int lane = threadIdx.x & 31;
  const int g = lane / LPV, l = lane % LPV;
  const int64_t token = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const int t = (int)(token % seq);
  float c[VN], s[VN];
  load_row_f32<VN>(cs + (int64_t)t * D + l * VN, c);
  load_row_f32<VN>(sn + (int64_t)t * D + l * VN, s);
  const float sign = l < LPV / 2 ? -1.f : 1.f;      // first half: x*cos - partner*sin; second: x*cos + partner*sin
  for (int h0 = 0; h0 < heads; h0 += VPW) {
    const int h = h0 + g;
    const bool active = h < heads;
    Vec16<T> v;
    if (active) v.load(x + token * ld_x + (int64_t)h * D + l * VN);
    else v.u = make_uint4(0, 0, 0, 0);
    Vec16<T> p;
    p.u.x = __shfl_xor_sync(0xffffffffu, v.u.x, LPV / 2);
    p.u.y = __shfl_xor_sync(0xffffffffu, v.u.y, LPV / 2);
    p.u.z = __shfl_xor_sync(0xffffffffu, v.u.z, LPV / 2);
    p.u.w = __shfl_xor_sync(0xffffffffu, v.u.w, LPV / 2);
    float r[VN], ss = 0.f;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      r[e] = v.get(e) * c[e] + sign * p.get(e) * s[e];
      ss += r[e] * r[e];
    }
    ss = group_sum<LPV>(ss);
    const float rstd = rsqrtf(ss * (1.f / D) + eps);
    if (active) {
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < VN; ++e) o.set(e, r[e] * rstd);
      o.store(y + token * ld_y + (int64_t)h * D + l * VN);
      if (l == 0) rs[token * heads + h] = rstd;
    }
  }
}

// dr = rstd * (dy - y * mean(dy * y)) is the RMSNorm backward written with the saved OUTPUT y
// (x_hat = y for a parameter-free norm), then dx = rotation of dr by the negative angle.
template <typename T, int LPV>
__global__ void __launch_bounds__(128)
rope_rmsnorm_bwd_kernel(const T* __restrict__ dy0, const T* __restrict__ dy1, const T* __restrict__ y0,
                        const T* __restrict__ y1, const float* __restrict__ r0, const float* __restrict__ r1,
                        T* __restrict__ dx0, T* __restrict__ dx1, const float* __restrict__ cs,
                        const float* __restrict__ sn, int64_t tokens, int seq, int heads, int64_t ld_dy, int64_t ld_y,
                        int64_t ld_dx) {
  constexpr int VN = Vec16<T>::N;
  constexpr int D = LPV * VN;
  constexpr int VPW = 32 / LPV;
  const T* __restrict__ dy = blockIdx.y ? dy1 : dy0;
  const T* __restrict__ y = blockIdx.y ? y1 : y0;
  const float* __restrict__ rs = blockIdx.y ? r1 : r0;
  T* __restrict__ dx = blockIdx.y ? dx1 : dx0;
  const int lane = threadIdx.x & 31;
  const int g = lane / LPV, l = lane % LPV;
  const int64_t token = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const int t = (int)(token % seq);
  float c[VN], s[VN];
  load_row_f32<VN>(cs + (int64_t)t * D + l * VN, c);
  load_row_f32<VN>(sn + (int64_t)t * D + l * VN, s);
  const float sign = l < LPV / 2 ? 1.f : -1.f;      // transpose of the forward rotation
  for (int h0 = 0; h0 < heads; h0 += VPW) {
    const int h = h0 + g;
    const bool active = h < heads;
    Vec16<T> gv, yv;
    float rstd = 0.f;
    if (active) {
      gv.load(dy + token * ld_dy + (int64_t)h * D + l * VN);
      yv.load(y + token * ld_y + (int64_t)h * D + l * VN);
      rstd = rs[token * heads + h];
    } else {
      gv.u = make_uint4(0, 0, 0, 0);
      yv.u = make_uint4(0, 0, 0, 0);
    }
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < VN; ++e) dot += gv.get(e) * yv.get(e);
    dot = group_sum<LPV>(dot) * (1.f / D);
    float dr[VN];
    Vec16<T> o;
#pragma unroll
    for (int e = 0; e < VN; ++e) dr[e] = rstd * (gv.get(e) - yv.get(e) * dot);
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      const float pe = __shfl_xor_sync(0xffffffffu, dr[e], LPV / 2);
      o.set(e, dr[e] * c[e] + sign * pe * s[e]);
    }
    if (active) o.store(dx + token * ld_dx + (int64_t)h * D + l * VN);
  }
}

template <typename T>
static bool rope_norm_shape_ok(int64_t head_dim, std::initializer_list<int64_t> lds, std::initializer_list<const void*> ptrs) {
  constexpr int VN = Vec16<T>::N;
  const int64_t lpv = head_dim / VN;
  if (head_dim % VN != 0 || (lpv != 2 && lpv != 4 && lpv != 8 && lpv != 16 && lpv != 32)) return false;
  for (int64_t ld : lds) if (ld % VN != 0) return false;
  for (const void* p : ptrs) if (p && !aligned16(p)) return false;
  return true;
}

template <typename T>
static int rope_rmsnorm_fwd_launch(const void* xq, const void* xk, void* yq, void* yk, float* rq, float* rk,
                                   const float* cs, const float* sn, int64_t tokens, int64_t seq, int64_t heads,
                                   int64_t head_dim, int64_t ld_x, int64_t ld_y, float eps, cudaStream_t st) {
  MT_REQUIRE((rope_norm_shape_ok<T>(head_dim, {ld_x, ld_y}, {xq, xk, yq, yk})),
             "rope_rmsnorm_fwd: head_dim must be 2, 4, 8, 16 or 32 16-byte vectors, tensors and strides 16-byte aligned");
  dim3 grid((unsigned)((tokens + 3) / 4), xk ? 2 : 1);
#define MT_RN(L) rope_rmsnorm_fwd_kernel<T, L><<<grid, 128, 0, st>>>((const T*)xq, (const T*)xk, (T*)yq, (T*)yk, rq, rk, cs, sn, tokens, (int)seq, (int)heads, ld_x, ld_y, eps)
  switch ((int)(head_dim / Vec16<T>::N)) {
    case 2: MT_RN(2); break;
    case 4: MT_RN(4); break;
    case 8: MT_RN(8); break;
    case 16: MT_RN(16); break;
    default: MT_RN(32);
  }
#undef MT_RN
  MT_LAUNCH_CHECK();
  return MT_OK;
}

template <typename T>
static int rope_rmsnorm_bwd_launch(const void* dyq, const void* dyk, const void* yq, const void* yk, const float* rq,
                                   const float* rk, void* dxq, void* dxk, const float* cs, const float* sn,
                                   int64_t tokens, int64_t seq, int64_t heads, int64_t head_dim, int64_t ld_dy,
                                   int64_t ld_y, int64_t ld_dx, cudaStream_t st) {
  MT_REQUIRE((rope_norm_shape_ok<T>(head_dim, {ld_dy, ld_y, ld_dx}, {dyq, dyk, yq, yk, dxq, dxk})),
             "rope_rmsnorm_bwd: head_dim must be 2, 4, 8, 16 or 32 16-byte vectors, tensors and strides 16-byte aligned");
  dim3 grid((unsigned)((tokens + 3) / 4), dyk ? 2 : 1);
#define MT_RN(L) rope_rmsnorm_bwd_kernel<T, L><<<grid, 128, 0, st>>>((const T*)dyq, (const T*)dyk, (const T*)yq, (const T*)yk, rq, rk, (T*)dxq, (T*)dxk, cs, sn, tokens, (int)seq, (int)heads, ld_dy, ld_y, ld_dx)
  switch ((int)(head_dim / Vec16<T>::N)) {
    case 2: MT_RN(2); break;
    case 4: MT_RN(4); break;
    case 8: MT_RN(8); break;
    case 16: MT_RN(16); break;
    default: MT_RN(32);
  }
#undef MT_RN
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_rope_rmsnorm_fwd(const void* xq, const void* xk, void* yq, void* yk, float* rstd_q, float* rstd_k,
                        const float* cos_t, const float* sin_t, int64_t batch, int64_t seq, int64_t heads,
                        int64_t head_dim, int64_t ld_x, int64_t ld_y, float eps, int dtype, void* stream) {
  MT_REQUIRE(xq && yq && rstd_q && cos_t && sin_t && batch >= 0 && seq > 0 && heads > 0 && head_dim > 0,
             "rope_rmsnorm_fwd: bad arguments");
  MT_REQUIRE(!xk || (yk && rstd_k), "rope_rmsnorm_fwd: a second input needs its outputs");
  MT_REQUIRE(ld_x >= heads * head_dim && ld_y >= heads * head_dim, "rope_rmsnorm_fwd: row stride below heads * head_dim");
  const int64_t tokens = batch * seq;
  if (tokens == 0) return MT_OK;
  MT_REQUIRE(aligned16(cos_t) && aligned16(sin_t), "rope_rmsnorm_fwd: cos/sin tables must be 16-byte aligned");
  MT_DISPATCH_FLOAT(dtype, T, return (rope_rmsnorm_fwd_launch<T>(xq, xk, yq, yk, rstd_q, rstd_k, cos_t, sin_t, tokens, seq, heads, head_dim, ld_x, ld_y, eps, as_stream(stream))));
  return MT_OK;
}

int mt_rope_rmsnorm_bwd(const void* dyq, const void* dyk, const void* yq, const void* yk, const float* rstd_q,
                        const float* rstd_k, void* dxq, void* dxk, const float* cos_t, const float* sin_t,
                        int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, int64_t ld_dy, int64_t ld_y,
                        int64_t ld_dx, int dtype, void* stream) {
  MT_REQUIRE(dyq && yq && rstd_q && dxq && cos_t && sin_t && batch >= 0 && seq > 0 && heads > 0 && head_dim > 0,
             "rope_rmsnorm_bwd: bad arguments");
  MT_REQUIRE(!dyk || (yk && rstd_k && dxk), "rope_rmsnorm_bwd: a second gradient needs its saved output, rstd and result");
  const int64_t hd = heads * head_dim;
  MT_REQUIRE(ld_dy >= hd && ld_y >= hd && ld_dx >= hd, "rope_rmsnorm_bwd: row stride below heads * head_dim");
  const int64_t tokens = batch * seq;
  if (tokens == 0) return MT_OK;
  MT_REQUIRE(aligned16(cos_t) && aligned16(sin_t), "rope_rmsnorm_bwd: cos/sin tables must be 16-byte aligned");
  MT_DISPATCH_FLOAT(dtype, T, return (rope_rmsnorm_bwd_launch<T>(dyq, dyk, yq, yk, rstd_q, rstd_k, dxq, dxk, cos_t, sin_t, tokens, seq, heads, head_dim, ld_dy, ld_y, ld_dx, as_stream(stream))));
  return MT_OK;
}

}  // extern "C"
