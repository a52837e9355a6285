// Elementwise and small reduction kernels: cast, fill, add, axpby, scale,
// row-vector add, column sum, activations (tanh-GELU, ReLU^2, ReLU) forward and
// backward, RoPE. All are HBM-bound: 16-byte vector accesses when pointers and
// counts allow, grid-stride loops sized from the SM count.
#include "common.cuh"
#include "tempbuf.cuh"

namespace mt {

static inline unsigned grid_for(int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// Generic unary/binary map over n elements; F is a functor on floats.
template <typename TI, typename TO, typename F>
__global__ void __launch_bounds__(256) map1_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t n, F f, int vec) {
  constexpr int VN = 8;  // elements per thread-iteration on the vector path
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    int64_t nv = n / VN;
    for (int64_t i = tid; i < nv; i += stride) {
      __align__(16) TI in[VN]; __align__(16) TO out[VN];
      if (sizeof(TI) == 2) *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(x + i * VN);
      else { reinterpret_cast<uint4*>(in)[0] = reinterpret_cast<const uint4*>(x + i * VN)[0];
             reinterpret_cast<uint4*>(in)[1] = reinterpret_cast<const uint4*>(x + i * VN)[1]; }
#pragma unroll
      for (int e = 0; e < VN; ++e) out[e] = from_f<TO>(f(to_f(in[e])));
      if (sizeof(TO) == 2) *reinterpret_cast<uint4*>(y + i * VN) = *reinterpret_cast<uint4*>(out);
      else { reinterpret_cast<uint4*>(y + i * VN)[0] = reinterpret_cast<uint4*>(out)[0];
             reinterpret_cast<uint4*>(y + i * VN)[1] = reinterpret_cast<uint4*>(out)[1]; }
    }
    for (int64_t i = nv * VN + tid; i < n; i += stride) y[i] = from_f<TO>(f(to_f(x[i])));
  } else {
    for (int64_t i = tid; i < n; i += stride) y[i] = from_f<TO>(f(to_f(x[i])));
  }
}

template <typename TA, typename TB, typename TO, typename F>
__global__ void __launch_bounds__(256) map2_kernel(const TA* __restrict__ a, const TB* __restrict__ b, TO* __restrict__ y, int64_t n, F f, int vec) {
  constexpr int VN = 8;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    int64_t nv = n / VN;
    for (int64_t i = tid; i < nv; i += stride) {
      __align__(16) TA ia[VN]; __align__(16) TB ib[VN]; __align__(16) TO out[VN];
      if (sizeof(TA) == 2) *reinterpret_cast<uint4*>(ia) = *reinterpret_cast<const uint4*>(a + i * VN);
      else { reinterpret_cast<uint4*>(ia)[0] = reinterpret_cast<const uint4*>(a + i * VN)[0];
             reinterpret_cast<uint4*>(ia)[1] = reinterpret_cast<const uint4*>(a + i * VN)[1]; }
      if (sizeof(TB) == 2) *reinterpret_cast<uint4*>(ib) = *reinterpret_cast<const uint4*>(b + i * VN);
      else { reinterpret_cast<uint4*>(ib)[0] = reinterpret_cast<const uint4*>(b + i * VN)[0];
             reinterpret_cast<uint4*>(ib)[1] = reinterpret_cast<const uint4*>(b + i * VN)[1]; }
#pragma unroll
      for (int e = 0; e < VN; ++e) out[e] = from_f<TO>(f(to_f(ia[e]), to_f(ib[e])));
      if (sizeof(TO) == 2) *reinterpret_cast<uint4*>(y + i * VN) = *reinterpret_cast<uint4*>(out);
      else { reinterpret_cast<uint4*>(y + i * VN)[0] = reinterpret_cast<uint4*>(out)[0];
             reinterpret_cast<uint4*>(y + i * VN)[1] = reinterpret_cast<uint4*>(out)[1]; }
    }
    for (int64_t i = nv * VN + tid; i < n; i += stride) y[i] = from_f<TO>(f(to_f(a[i]), to_f(b[i])));
  } else {
    for (int64_t i = tid; i < n; i += stride) y[i] = from_f<TO>(f(to_f(a[i]), to_f(b[i])));
  }
}

static inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }
template <typename T> static inline bool vec_ok(const void* p) { return sizeof(T) == 2 ? aligned16(p) : aligned32(p); }

template <typename TI, typename TO, typename F>
static int map1(const void* x, void* y, int64_t n, F f, cudaStream_t st) {
  if (n <= 0) return MT_OK;
  int vec = vec_ok<TI>(x) && vec_ok<TO>(y);
  map1_kernel<TI, TO, F><<<grid_for((n + 7) / 8, 256), 256, 0, st>>>((const TI*)x, (TO*)y, n, f, vec);
  MT_LAUNCH_CHECK();
  return MT_OK;
}
template <typename TA, typename TB, typename TO, typename F>
static int map2(const void* a, const void* b, void* y, int64_t n, F f, cudaStream_t st) {
  if (n <= 0) return MT_OK;
  int vec = vec_ok<TA>(a) && vec_ok<TB>(b) && vec_ok<TO>(y);
  map2_kernel<TA, TB, TO, F><<<grid_for((n + 7) / 8, 256), 256, 0, st>>>((const TA*)a, (const TB*)b, (TO*)y, n, f, vec);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

struct Identity { __device__ float operator()(float x) const { return x; } };
struct Const { float v; __device__ float operator()(float) const { return v; } };
struct Scale { float a; __device__ float operator()(float x) const { return a * x; } };
struct Add { __device__ float operator()(float a, float b) const { return a + b; } };
struct Axpby { float alpha, beta; __device__ float operator()(float x, float y) const { return alpha * x + beta * y; } };

// Activations. Constants follow the reference's tanh-GELU.
constexpr float kGeluA = 0.7978845608f, kGeluB = 0.044715f;
__device__ __forceinline__ float gelu_f(float x) {
  float inner = kGeluA * (x + kGeluB * x * x * x);
  return 0.5f * x * (1.f + tanhf(inner));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  float x2 = x * x;
  float t = tanhf(kGeluA * (x + kGeluB * x2 * x));
  float ig = kGeluA * (1.f + 3.f * kGeluB * x2);
  return 0.5f * (1.f + t + x * (1.f - t * t) * ig);
}
struct ActFwd {
  int act;
  __device__ float operator()(float x) const {
    switch (act) {
      case MT_ACT_GELU: return gelu_f(x);
      case MT_ACT_RELU2: { float r = fmaxf(x, 0.f); return r * r; }
      case MT_ACT_RELU: return fmaxf(x, 0.f);
      default: return x;
    }
  }
};
struct ActBwd {
  int act;
  __device__ float operator()(float x, float dy) const {
    switch (act) {
      case MT_ACT_GELU: return gelu_grad_f(x) * dy;
      case MT_ACT_RELU2: return 2.f * fmaxf(x, 0.f) * dy;
      case MT_ACT_RELU: return x > 0.f ? dy : 0.f;
      default: return dy;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(256) add_rowvec_kernel(const T* __restrict__ a, const T* __restrict__ v, T* __restrict__ out, int64_t rows, int64_t cols) {
  int64_t n = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f<T>(to_f(a[i]) + to_f(v[i % cols]));
}

// Column sum in two fixed-order stages: slabs of rows -> partial[slab][cols] -> out.
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T* __restrict__ a, float* __restrict__ partial, int64_t rows, int64_t cols, int64_t rows_per_slab) {
  __shared__ float sh[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
  float s = 0.f;
  if (c < cols) for (int64_t r = r0 + ty; r < r1; r += 8) s += to_f(a[r * cols + c]);
  sh[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][tx];
    partial[(int64_t)blockIdx.y * cols + c] = t;
  }
}
template <typename TO>
__global__ void colsum_final_kernel(const float* __restrict__ partial, TO* __restrict__ out, int nslab, int64_t cols, int accumulate) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int i = 0; i < nslab; ++i) s += partial[(int64_t)i * cols + c];
  out[c] = from_f<TO>(accumulate ? to_f(out[c]) + s : s);
}

template <typename T>
__global__ void __launch_bounds__(1024) sum_partial_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ partial) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s += to_f(x[i]);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(1024) sum_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) out[0] = s;
}

// RoPE, half-split pairing (d, d + D/2), in place on x [B,T,H,D].
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                                                   int64_t n_pairs, int64_t seq, int64_t heads, int half, float sign) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += (int64_t)gridDim.x * blockDim.x) {
    int d = (int)(i % half);
    int64_t bth = i / half;            // (b*T + t)*H + h
    int64_t t = (bth / heads) % seq;
    T* p = x + bth * (2 * half);
    float x1 = to_f(p[d]), x2 = to_f(p[d + half]);
    float c1 = cs[t * 2 * half + d], s1 = sn[t * 2 * half + d] * sign;
    float c2 = cs[t * 2 * half + d + half], s2 = sn[t * 2 * half + d + half] * sign;
    // y = x*cos + rotate_half(x)*sin, rotate_half(x) = [-x2, x1]
    p[d] = from_f<T>(x1 * c1 - x2 * s1);
    p[d + half] = from_f<T>(x2 * c2 + x1 * s2);
  }
}

}  // namespace mt

using namespace mt;

namespace mt {
// Token ids as stored on disk (uint16) widened to the int32 the embedding kernels index with.
__global__ void __launch_bounds__(256)
widen_u16_kernel(const uint16_t* __restrict__ src, int32_t* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = (int32_t)src[i];
}
}  // namespace mt

namespace mt {
// y = cap * tanh(x / cap): the soft cap nanochat puts on its logits.
template <typename T>
__global__ void __launch_bounds__(256)
softcap_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, float cap) {
  const float inv = 1.f / cap;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = from_f<T>(cap * tanhf(to_f(x[i]) * inv));
}
}  // namespace mt

extern "C" {

int mt_softcap(const void* x, void* y, int64_t n, float cap, int dtype, void* stream) {
  MT_REQUIRE(x && y && n >= 0 && cap > 0.f, "softcap: bad arguments");
  if (n == 0) return MT_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  MT_DISPATCH_FLOAT(dtype, T, (mt::softcap_kernel<T><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((const T*)x, (T*)y, n, cap)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_widen_u16_i32(const void* src, void* dst, int64_t n, void* stream) {
  MT_REQUIRE(src && dst && n >= 0, "widen_u16_i32: bad arguments");
  if (n == 0) return MT_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  mt::widen_u16_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((const uint16_t*)src, (int32_t*)dst, n);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_cast(const void* src, int sd, void* dst, int dd, int64_t n, void* stream) {
  MT_REQUIRE(src && dst && n >= 0, "cast: bad arguments");
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(sd, TI, { MT_DISPATCH_FLOAT(dd, TO, return (map1<TI, TO>(src, dst, n, Identity{}, st))); });
  return MT_OK;
}
int mt_fill(void* dst, int dtype, float value, int64_t n, void* stream) {
  MT_REQUIRE(dst && n >= 0, "fill: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (map1<T, T>(dst, dst, n, Const{value}, as_stream(stream))));
  return MT_OK;
}
int mt_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream) {
  MT_REQUIRE(a && b && out && n >= 0, "add: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (map2<T, T, T>(a, b, out, n, Add{}, as_stream(stream))));
  return MT_OK;
}
int mt_axpby(const void* x, float alpha, void* y, float beta, int64_t n, int xd, int yd, void* stream) {
  MT_REQUIRE(x && y && n >= 0, "axpby: bad arguments");
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(xd, TX, { MT_DISPATCH_FLOAT(yd, TY, return (map2<TX, TY, TY>(x, y, y, n, Axpby{alpha, beta}, st))); });
  return MT_OK;
}
int mt_scale(void* x, float alpha, int64_t n, int dtype, void* stream) {
  MT_REQUIRE(x && n >= 0, "scale: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (map1<T, T>(x, x, n, Scale{alpha}, as_stream(stream))));
  return MT_OK;
}
int mt_act_fwd(const void* x, void* y, int64_t n, int act, int dtype, void* stream) {
  MT_REQUIRE(x && y && n >= 0, "act_fwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (map1<T, T>(x, y, n, ActFwd{act}, as_stream(stream))));
  return MT_OK;
}
int mt_act_bwd(const void* x, const void* dy, void* dx, int64_t n, int act, int dtype, void* stream) {
  MT_REQUIRE(x && dy && dx && n >= 0, "act_bwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (map2<T, T, T>(x, dy, dx, n, ActBwd{act}, as_stream(stream))));
  return MT_OK;
}
int mt_add_rowvec(const void* a, const void* v, void* out, int64_t rows, int64_t cols, int dtype, void* stream) {
  MT_REQUIRE(a && v && out && rows >= 0 && cols > 0, "add_rowvec: bad arguments");
  if (rows == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(dtype, T, (add_rowvec_kernel<T><<<grid_for(rows * cols, 256), 256, 0, st>>>((const T*)a, (const T*)v, (T*)out, rows, cols)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}
int mt_colsum(const void* a, void* out, int64_t rows, int64_t cols, int dtype, int out_dtype, int accumulate, void* stream) {
  MT_REQUIRE(a && out && rows >= 0 && cols > 0, "colsum: bad arguments");
  cudaStream_t st = as_stream(stream);
  int nslab = (int)((rows + 255) / 256);
  if (nslab < 1) nslab = 1;
  if (nslab > 256) nslab = 256;
  int64_t rps = (rows + nslab - 1) / nslab;
  if (rps < 1) rps = 1;
  TempBuf part((size_t)nslab * cols * sizeof(float), st);
  if (!part.ok()) return MT_ERR_CUDA;
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)nslab);
  MT_DISPATCH_FLOAT(dtype, T, (colsum_partial_kernel<T><<<grid, 256, 0, st>>>((const T*)a, (float*)part.ptr, rows, cols, rps)));
  MT_LAUNCH_CHECK();
  MT_DISPATCH_FLOAT(out_dtype, TO, (colsum_final_kernel<TO><<<(unsigned)((cols + 127) / 128), 128, 0, st>>>((const float*)part.ptr, (TO*)out, nslab, cols, accumulate)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}
int mt_sum_f32(const void* x, int dtype, int64_t n, float* out, void* stream) {
  MT_REQUIRE(x && out && n >= 0, "sum: bad arguments");
  cudaStream_t st = as_stream(stream);
  int blocks = (int)((n + 4095) / 4096);
  if (blocks < 1) blocks = 1;
  if (blocks > 1024) blocks = 1024;
  TempBuf part((size_t)blocks * sizeof(float), st);
  if (!part.ok()) return MT_ERR_CUDA;
  MT_DISPATCH_FLOAT(dtype, T, (sum_partial_kernel<T><<<blocks, 1024, 0, st>>>((const T*)x, n, (float*)part.ptr)));
  MT_LAUNCH_CHECK();
  sum_final_kernel<<<1, 1024, 0, st>>>((const float*)part.ptr, blocks, out);
  MT_LAUNCH_CHECK();
  return MT_OK;
}
int mt_rope(void* x, const float* cs, const float* sn, int64_t batch, int64_t seq, int64_t heads, int64_t head_dim,
            int backward, int dtype, void* stream) {
  MT_REQUIRE(x && cs && sn && head_dim % 2 == 0 && head_dim > 0, "rope: bad arguments");
  int64_t n_pairs = batch * seq * heads * (head_dim / 2);
  if (n_pairs == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(dtype, T, (rope_kernel<T><<<grid_for(n_pairs, 256), 256, 0, st>>>((T*)x, cs, sn, n_pairs, seq, heads, (int)(head_dim / 2), backward ? -1.f : 1.f)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // extern "C"
