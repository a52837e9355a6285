// Row softmax (forward/backward) and cross entropy over the vocabulary
// (forward: one pass, online log-sum-exp in vocabulary chunks; backward:
// (softmax - onehot) * scale written over the logits).
//
// Algorithmic traffic: softmax fwd 2*R*C*s, bwd 3*R*C*s; cross entropy fwd
// R*C*s (one read), bwd 2*R*C*s (read + write).
#include "common.cuh"
#include "sm100.cuh"

namespace mt {

constexpr float kLog2e = 1.4426950408889634f;

// ------------------------------------------------------------- softmax ------
template <typename T, int MAXV>
__global__ void __launch_bounds__(128)
softmax_fwd_warp(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols) {
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / VN;
  Vec16<T> v[MAXV];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      v[i].load(x + row * cols + vi * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) mx = fmaxf(mx, v[i].get(e));
    }
  }
  mx = warp_max(mx);
  float f[MAXV][VN];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < VN; ++e) { f[i][e] = exp2f((v[i].get(e) - mx) * kLog2e); s += f[i][e]; }
    }
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < VN; ++e) o.set(e, f[i][e] * inv);
      o.store(y + row * cols + vi * VN);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
softmax_fwd_block(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols) {
  __shared__ float sh[32];
  const T* xr = x + (int64_t)blockIdx.x * cols;
  T* yr = y + (int64_t)blockIdx.x * cols;
  float mx = -INFINITY;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, to_f(xr[c]));
  mx = block_max(mx, sh);
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += exp2f((to_f(xr[c]) - mx) * kLog2e);
  s = block_sum(s, sh);
  const float inv = 1.f / s;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
    yr[c] = from_f<T>(exp2f((to_f(xr[c]) - mx) * kLog2e) * inv);
}

template <typename T, int MAXV>
__global__ void __launch_bounds__(128)
softmax_bwd_warp(const T* __restrict__ dy, const T* __restrict__ s, T* __restrict__ dx, int64_t rows, int cols) {
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / VN;
  Vec16<T> a[MAXV], b[MAXV];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      a[i].load(dy + row * cols + vi * VN);
      b[i].load(s + row * cols + vi * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) dot += a[i].get(e) * b[i].get(e);
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < VN; ++e) o.set(e, b[i].get(e) * (a[i].get(e) - dot));
      o.store(dx + row * cols + vi * VN);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
softmax_bwd_block(const T* __restrict__ dy, const T* __restrict__ s, T* __restrict__ dx, int64_t rows, int64_t cols) {
  __shared__ float sh[32];
  const int64_t off = (int64_t)blockIdx.x * cols;
  float dot = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) dot += to_f(dy[off + c]) * to_f(s[off + c]);
  dot = block_sum(dot, sh);
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
    dx[off + c] = from_f<T>(to_f(s[off + c]) * (to_f(dy[off + c]) - dot));
}

// ------------------------------------------------------- cross entropy ------
// tanh for the logit soft cap in a dozen instructions (tanhf costs several times that and the
// capped cross entropy evaluates it twice per logit): 1 - 2 / (e^{2x} + 1) with the hardware
// exp2 (relative error 2^-22), and the odd Taylor polynomial below |x| = 0.1 where that form
// cancels. Relative error at most 1e-6 over the whole range; saturates to +-1 exactly.
__device__ __forceinline__ float tanh_cap(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.8853900817779268f));   // e^{2x}
  const float big = 1.f - __fdividef(2.f, e + 1.f);
  const float x2 = x * x;
  const float small = x * fmaf(x2, fmaf(x2, fmaf(x2, -17.f / 315.f, 2.f / 15.f), -1.f / 3.f), 1.f);
  return fabsf(x) < 0.1f ? small : big;
}
// One MUFU instruction, relative error ~2^-11: at the level of the rounding that fp16 / bf16
// logits already carry, so the half-precision kernels use it (FAST) and halve the special-function
// work of the capped loss, which is bound by that unit (two passes x (tanh + exp) per logit).
__device__ __forceinline__ float tanh_mufu(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool FAST> __device__ __forceinline__ float tanh_sel(float x) { return FAST ? tanh_mufu(x) : tanh_cap(x); }
template <bool FAST = false>
__device__ __forceinline__ float softcap_f(float x, float cap) { return cap > 0.f ? cap * tanh_sel<FAST>(__fdividef(x, cap)) : x; }

constexpr int kCeThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_kernel(const T* __restrict__ logits, const int32_t* __restrict__ labels, float* __restrict__ loss,
              float* __restrict__ lse_out, int64_t classes, int64_t ld, float softcap, int vec_ok, int* __restrict__ flag,
              int64_t col_offset = 0, float* __restrict__ tgt = nullptr) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float shm[32], shs[32];
  const int64_t row = blockIdx.x;
  const T* xr = logits + row * ld;
  float m = -INFINITY, s = 0.f;  // running max (natural units) and sum of exp(x - m)
  int64_t vec_end = 0;
  if (vec_ok) {
    const int64_t nvec = classes / VN;
    vec_end = nvec * VN;
    for (int64_t vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
      Vec16<T> v;
      v.load(xr + vi * VN);
      float f[VN];
      float vm = -INFINITY;
#pragma unroll
      for (int e = 0; e < VN; ++e) { f[e] = softcap_f<sizeof(T) == 2>(v.get(e), softcap); vm = fmaxf(vm, f[e]); }
      if (vm > m) { s *= exp2f((m - vm) * kLog2e); m = vm; }
#pragma unroll
      for (int e = 0; e < VN; ++e) s += exp2f((f[e] - m) * kLog2e);
    }
  }
  for (int64_t c = vec_end + threadIdx.x; c < classes; c += kCeThreads) {
    float f = softcap_f<sizeof(T) == 2>(to_f(xr[c]), softcap);
    if (f > m) { s *= exp2f((m - f) * kLog2e); m = f; }
    s += exp2f((f - m) * kLog2e);
  }
  // combine (m, s) pairs across the block
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
    m = mm;
  }
  if (lane == 0) { shm[w] = m; shs[w] = s; }
  __syncthreads();
  if (w == 0) {
    m = lane < kCeThreads / 32 ? shm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? shs[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      float mm = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
      m = mm;
    }
    if (lane == 0 && tgt) {
      // vocabulary-chunk mode: merge this chunk's log-sum-exp into the running one and pick up
      // the target logit if the label falls inside the chunk [col_offset, col_offset + classes)
      const float lse_c = m + logf(s);
      const float old = lse_out[row];
      const float mx = fmaxf(old, lse_c);
      lse_out[row] = mx == -INFINITY ? -INFINITY : mx + logf(__expf(old - mx) + __expf(lse_c - mx));
      const int64_t lab = (int64_t)labels[row] - col_offset;
      if (lab >= 0 && lab < classes) tgt[row] = softcap_f<sizeof(T) == 2>(to_f(xr[lab]), softcap);
    } else if (lane == 0) {
      float lse = m + logf(s);
      lse_out[row] = lse;
      int32_t lab = labels[row];
      float l = 0.f;
      if (lab >= 0 && lab < classes) l = lse - softcap_f<sizeof(T) == 2>(to_f(xr[lab]), softcap);
      else if (lab != -100 && flag) atomicMax(flag, 2);  // label out of range: recorded, row ignored
      loss[row] = l;
    }
  }
}

// loss_sum[0] = sum(loss), valid_count[0] = #labels != -100; one block, fixed order.
__global__ void __launch_bounds__(1024)
ce_reduce_kernel(const float* __restrict__ loss, const int32_t* __restrict__ labels, int64_t rows,
                 float* __restrict__ loss_sum, float* __restrict__ valid_count, float* __restrict__ loss_mean) {
  __shared__ float sh[32];
  float s = 0.f, n = 0.f;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    s += loss[r];
    n += labels[r] != -100 ? 1.f : 0.f;
  }
  s = block_sum(s, sh);
  n = block_sum(n, sh);
  if (threadIdx.x == 0) {
    if (loss_sum) loss_sum[0] = s;
    if (valid_count) valid_count[0] = n;
    if (loss_mean) loss_mean[0] = s / n;
  }
}

// loss[row] = lse - target logit for rows whose label is not -100 (chunked forward, last step)
__global__ void __launch_bounds__(256)
ce_finish_kernel(const float* __restrict__ lse, const float* __restrict__ tgt, const int32_t* __restrict__ labels,
                 float* __restrict__ loss, int64_t rows) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) loss[r] = labels[r] != -100 ? lse[r] - tgt[r] : 0.f;
}

// valid_count[0] = #labels != -100 (one block); runs before the fused forward+gradient kernel,
// which needs the count for the 1/n of the mean.
__global__ void __launch_bounds__(1024)
ce_count_kernel(const int32_t* __restrict__ labels, int64_t rows, float* __restrict__ valid_count) {
  __shared__ float sh[32];
  float n = 0.f;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) n += labels[r] != -100 ? 1.f : 0.f;
  n = block_sum(n, sh);
  if (threadIdx.x == 0) valid_count[0] = n;
}

// Forward and gradient in one kernel: a block reads its row once for the log-sum-exp and at once
// a second time - while the row (100 KB at 50k classes) is still in L2 - to overwrite it with
// (softmax - onehot) * scale / n_valid. DRAM sees one read and one write of the logits instead
// of the two reads and one write of separate forward and backward kernels.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_grad_kernel(T* __restrict__ logits, const int32_t* __restrict__ labels, float* __restrict__ loss,
                   float* __restrict__ lse_out, float scale_host, const float* __restrict__ scale_dev,
                   const float* __restrict__ count_dev, int64_t classes, int64_t ld, float softcap, int vec_ok,
                   int* __restrict__ flag) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float shm[32], shs[32];
  __shared__ float row_lse;
  const int64_t row = blockIdx.x;
  T* xr = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  int64_t vec_end = 0;
  if (vec_ok) {
    const int64_t nvec = classes / VN;
    vec_end = nvec * VN;
    for (int64_t vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
      Vec16<T> v;
      v.load(xr + vi * VN);
      float f[VN];
      float vm = -INFINITY;
#pragma unroll
      for (int e = 0; e < VN; ++e) { f[e] = softcap_f<sizeof(T) == 2>(v.get(e), softcap); vm = fmaxf(vm, f[e]); }
      if (vm > m) { s *= exp2f((m - vm) * kLog2e); m = vm; }
#pragma unroll
      for (int e = 0; e < VN; ++e) s += exp2f((f[e] - m) * kLog2e);
    }
  }
  for (int64_t c = vec_end + threadIdx.x; c < classes; c += kCeThreads) {
    float f = softcap_f<sizeof(T) == 2>(to_f(xr[c]), softcap);
    if (f > m) { s *= exp2f((m - f) * kLog2e); m = f; }
    s += exp2f((f - m) * kLog2e);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
    m = mm;
  }
  if (lane == 0) { shm[w] = m; shs[w] = s; }
  __syncthreads();
  const int32_t label = labels[row];
  const bool valid = label >= 0 && label < classes;
  if (w == 0) {
    m = lane < kCeThreads / 32 ? shm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? shs[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      float mm = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
      m = mm;
    }
    if (lane == 0) {
      const float lse = m + logf(s);
      lse_out[row] = lse;
      row_lse = lse;
      float l = 0.f;
      if (valid) l = lse - softcap_f<sizeof(T) == 2>(to_f(xr[label]), softcap);
      else if (label != -100 && flag) atomicMax(flag, 2);  // label out of range: recorded, row ignored
      loss[row] = l;
    }
  }
  __syncthreads();   // the loss read its target logit before anything below overwrites the row
  const float l = row_lse;
  float scale = scale_host;
  if (scale_dev) scale *= scale_dev[0];
  scale = valid ? scale / count_dev[0] : 0.f;
  if (vec_ok) {
    const int64_t nvec = classes / VN;
    for (int64_t vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
      Vec16<T> v, o;
      v.load(xr + vi * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float x = v.get(e), f = x, dcap = 1.f;
        if (softcap > 0.f) { float t = tanh_sel<sizeof(T) == 2>(__fdividef(x, softcap)); f = softcap * t; dcap = 1.f - t * t; }
        float p = valid ? exp2f((f - l) * kLog2e) : 0.f;
        if (vi * VN + e == label) p -= 1.f;
        o.set(e, p * scale * dcap);
      }
      o.store(xr + vi * VN);
    }
  }
  for (int64_t c = vec_end + threadIdx.x; c < classes; c += kCeThreads) {
    float x = to_f(xr[c]), f = x, dcap = 1.f;
    if (softcap > 0.f) { float t = tanh_sel<sizeof(T) == 2>(__fdividef(x, softcap)); f = softcap * t; dcap = 1.f - t * t; }
    float p = valid ? exp2f((f - l) * kLog2e) : 0.f;
    if (c == label) p -= 1.f;
    xr[c] = from_f<T>(p * scale * dcap);
  }
}

// ce_fwd_grad_kernel with the row staged in shared memory. One thread starts bulk copies of the
// row (kCePieces pieces, one mbarrier each), so the whole row is in flight at once instead of one
// 16-byte load per thread; the block folds max / sum piece by piece as they land, then computes
// the gradient from shared memory and writes it straight over the row. Two blocks per SM: one
// row's arithmetic overlaps the other's copy. Needs classes a multiple of the 16-byte vector,
// 16-byte aligned rows and a row of at most kCeStagedMaxBytes.
constexpr int kCePieces = 4;
constexpr int kCeStagedMaxBytes = 110 * 1024;

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads, 2)
ce_fwd_grad_staged_kernel(T* __restrict__ logits, const int32_t* __restrict__ labels, float* __restrict__ loss,
                          float* __restrict__ lse_out, float scale_host, const float* __restrict__ scale_dev,
                          const float* __restrict__ count_dev, int classes, int64_t ld, float softcap,
                          int* __restrict__ flag) {
  constexpr int VN = Vec16<T>::N;
  extern __shared__ __align__(128) uint8_t ce_row[];   // [nvec * 16 bytes of logits][kCePieces mbarriers][abort word]
  __shared__ float shm[32], shs[32];
  __shared__ float row_lse;
  const int nvec = classes / VN;
  const int per = (nvec + kCePieces - 1) / kCePieces;
  const uint32_t sbase = sm100::smem_u32(ce_row);
  const uint32_t bar0 = sbase + (uint32_t)nvec * 16u;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ce_row + (size_t)nvec * 16 + 8 * kCePieces);
  const int64_t row = blockIdx.x;
  T* xr = logits + row * ld;
  const T* sr = reinterpret_cast<const T*>(ce_row);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int p = 0; p < kCePieces; ++p) sm100::mbar_init(bar0 + 8 * p, 1);
    sm100::fence_barrier_init();
    sm100::fence_proxy_async();
    for (int p = 0; p < kCePieces; ++p) {
      const int v0 = p * per, v1 = min(nvec, v0 + per);
      if (v1 <= v0) break;
      const uint32_t bytes = (uint32_t)(v1 - v0) * 16u;
      sm100::mbar_expect_tx(bar0 + 8 * p, bytes);
      sm100::bulk_load_1d(sbase + (uint32_t)v0 * 16u, xr + (int64_t)v0 * VN, bytes, bar0 + 8 * p);
    }
  }
  __syncthreads();
  float m = -INFINITY, s = 0.f;
  for (int p = 0; p < kCePieces; ++p) {
    const int v0 = p * per, v1 = min(nvec, v0 + per);
    if (v1 <= v0) break;
    if (!sm100::mbar_wait(bar0 + 8 * p, 0, abort_flag)) break;
    for (int vi = v0 + threadIdx.x; vi < v1; vi += kCeThreads) {
      Vec16<T> v;
      v.load(sr + (int64_t)vi * VN);
      float f[VN];
      float vm = -INFINITY;
#pragma unroll
      for (int e = 0; e < VN; ++e) { f[e] = softcap_f<sizeof(T) == 2>(v.get(e), softcap); vm = fmaxf(vm, f[e]); }
      if (vm > m) { s *= ex2_fast((m - vm) * kLog2e); m = vm; }
      const float mb = m * kLog2e;
#pragma unroll
      for (int e = 0; e < VN; ++e) s += ex2_fast(fmaf(f[e], kLog2e, -mb));
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
    m = mm;
  }
  if (lane == 0) { shm[w] = m; shs[w] = s; }
  __syncthreads();   // also: every wait above is over, so the abort word is final
  if (*abort_flag) {
    if (threadIdx.x == 0 && flag) atomicMax(flag, 103);   // a row copy did not arrive in time
    return;
  }
  const int32_t label = labels[row];
  const bool valid = label >= 0 && label < classes;
  if (w == 0) {
    m = lane < kCeThreads / 32 ? shm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? shs[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      float mm = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * exp2f((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mm) * kLog2e));
      m = mm;
    }
    if (lane == 0) {
      const float lse = m + logf(s);
      lse_out[row] = lse;
      row_lse = lse;
      float l = 0.f;
      if (valid) l = lse - softcap_f<sizeof(T) == 2>(to_f(sr[label]), softcap);
      else if (label != -100 && flag) atomicMax(flag, 2);  // label out of range: recorded, row ignored
      loss[row] = l;
    }
  }
  __syncthreads();
  const float lb = row_lse * kLog2e;
  float scale = scale_host;
  if (scale_dev) scale *= scale_dev[0];
  scale = valid ? scale / count_dev[0] : 0.f;
  const int label_vec = valid ? label / VN : -1, label_e = valid ? label % VN : 0;
  for (int vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
    Vec16<T> v, o;
    v.load(sr + (int64_t)vi * VN);
    float pe[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      float x = v.get(e), f = x, dcap = scale;
      if (softcap > 0.f) { float t = tanh_sel<sizeof(T) == 2>(__fdividef(x, softcap)); f = softcap * t; dcap = scale * (1.f - t * t); }
      float pr = valid ? ex2_fast(fmaf(f, kLog2e, -lb)) : 0.f;
      if (vi == label_vec && e == label_e) pr -= 1.f;
      pe[e] = pr * dcap;
    }
#pragma unroll
    for (int e = 0; e < VN; ++e) o.set(e, pe[e]);
    o.store(xr + (int64_t)vi * VN);
  }
}

// x[i] *= num[0] / den[0] (device scalars): corrects a gradient that was scaled for another
// upstream value than the one that finally arrived.
template <typename T>
__global__ void __launch_bounds__(256)
scale_ratio_kernel(T* __restrict__ x, int64_t n, const float* __restrict__ num, const float* __restrict__ den) {
  const float r = num[0] / den[0];
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = from_f<T>(to_f(x[i]) * r);
}

constexpr int kCeBwdChunk = 4096;  // elements of one row handled by one block

template <typename T>
__global__ void __launch_bounds__(256)
ce_bwd_kernel(const T* __restrict__ logits, const int32_t* __restrict__ labels, const float* __restrict__ lse,
              T* __restrict__ dlogits, float scale_host, const float* __restrict__ scale_dev,
              const float* __restrict__ count_dev, int64_t classes, int64_t ld, float softcap, int vec_ok,
              int64_t col_offset = 0, int chunk_mode = 0) {
  constexpr int VN = Vec16<T>::N;
  const int64_t row = blockIdx.y;
  const int64_t c0 = (int64_t)blockIdx.x * kCeBwdChunk;
  const int64_t c1 = c0 + kCeBwdChunk < classes ? c0 + kCeBwdChunk : classes;
  const int64_t lab = (int64_t)labels[row] - col_offset;   // label position relative to this chunk
  float scale = scale_host;
  if (scale_dev) scale *= scale_dev[0];
  if (count_dev) scale /= count_dev[0];
  // whole-vocabulary mode ignores any label outside [0, classes); in chunk mode only -100 is ignored
  const bool ignored = chunk_mode ? labels[row] == -100 : !(lab >= 0 && lab < classes);
  if (ignored) scale = 0.f;
  const float l = lse[row];
  const T* xr = logits + row * ld;
  T* dr = dlogits + row * ld;
  int64_t c = c0;
  if (vec_ok) {
    const int64_t v1 = c1 / VN * VN;
    for (int64_t cc = c0 + (int64_t)threadIdx.x * VN; cc < v1; cc += 256 * VN) {
      Vec16<T> v, o;
      v.load(xr + cc);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float x = v.get(e), f = x, dcap = 1.f;
        if (softcap > 0.f) { float t = tanh_sel<sizeof(T) == 2>(__fdividef(x, softcap)); f = softcap * t; dcap = 1.f - t * t; }
        float p = ignored ? 0.f : exp2f((f - l) * kLog2e);
        if (cc + e == lab) p -= 1.f;
        o.set(e, p * scale * dcap);
      }
      o.store(dr + cc);
    }
    c = v1 > c0 ? v1 : c0;
  }
  for (int64_t cc = c + threadIdx.x; cc < c1; cc += 256) {
    float x = to_f(xr[cc]), f = x, dcap = 1.f;
    if (softcap > 0.f) { float t = tanh_sel<sizeof(T) == 2>(__fdividef(x, softcap)); f = softcap * t; dcap = 1.f - t * t; }
    float p = ignored ? 0.f : exp2f((f - l) * kLog2e);
    if (cc == lab) p -= 1.f;
    dr[cc] = from_f<T>(p * scale * dcap);
  }
}

template <typename T>
static int softmax_launch(bool bwd, const void* a, const void* b, void* out, int64_t rows, int64_t cols, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  if (rows == 0) return MT_OK;
  bool vec = cols % VN == 0 && aligned16(a) && aligned16(out) && (!b || aligned16(b)) && cols / VN <= 32 * (bwd ? 4 : 8);
  const T* ap = (const T*)a; const T* bp = (const T*)b; T* op = (T*)out;
  if (vec) {
    int nvec = (int)(cols / VN);
    unsigned grid = (unsigned)((rows + 3) / 4);
    if (!bwd) {
#define MT_SF(MV) softmax_fwd_warp<T, MV><<<grid, 128, 0, st>>>(ap, op, rows, (int)cols)
      if (nvec <= 32) MT_SF(1); else if (nvec <= 64) MT_SF(2); else if (nvec <= 128) MT_SF(4); else MT_SF(8);
#undef MT_SF
    } else {
#define MT_SB(MV) softmax_bwd_warp<T, MV><<<grid, 128, 0, st>>>(ap, bp, op, rows, (int)cols)
      if (nvec <= 32) MT_SB(1); else if (nvec <= 64) MT_SB(2); else MT_SB(4);
#undef MT_SB
    }
  } else {
    if (!bwd) softmax_fwd_block<T><<<(unsigned)rows, 256, 0, st>>>(ap, op, rows, cols);
    else softmax_bwd_block<T><<<(unsigned)rows, 256, 0, st>>>(ap, bp, op, rows, cols);
  }
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int dtype, void* stream) {
  MT_REQUIRE(x && y && rows >= 0 && cols > 0, "softmax_fwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return softmax_launch<T>(false, x, nullptr, y, rows, cols, as_stream(stream)));
  return MT_OK;
}
int mt_softmax_bwd(const void* dy, const void* s, void* dx, int64_t rows, int64_t cols, int dtype, void* stream) {
  MT_REQUIRE(dy && s && dx && rows >= 0 && cols > 0, "softmax_bwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return softmax_launch<T>(true, dy, s, dx, rows, cols, as_stream(stream)));
  return MT_OK;
}

int mt_ce_fwd(const void* logits, const int32_t* labels, float* loss, float* lse, float* loss_sum,
              float* valid_count, float* loss_mean, int64_t rows, int64_t classes, int64_t ld, float softcap, int dtype,
              void* stream) {
  MT_REQUIRE(logits && labels && loss && lse && rows >= 0 && classes > 0 && ld >= classes, "ce_fwd: bad arguments");
  cudaStream_t st = as_stream(stream);
  if (rows > 0) {
    int* flag = device_flag_ptr();
    MT_DISPATCH_FLOAT(dtype, T, {
      int vec_ok = aligned16(logits) && (ld % Vec16<T>::N == 0);
      ce_fwd_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>((const T*)logits, labels, loss, lse, classes, ld, softcap, vec_ok, flag);
    });
    MT_LAUNCH_CHECK();
  }
  if (loss_sum || valid_count || loss_mean) {
    ce_reduce_kernel<<<1, 1024, 0, st>>>(loss, labels, rows, loss_sum, valid_count, loss_mean);
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

int mt_ce_fwd_grad(void* logits, const int32_t* labels, float* loss, float* lse, float* loss_sum, float* valid_count,
                   float* loss_mean, float scale_host, const float* scale_dev, int64_t rows, int64_t classes, int64_t ld,
                   float softcap, int dtype, void* stream) {
  MT_REQUIRE(logits && labels && loss && lse && valid_count && rows >= 0 && classes > 0 && ld >= classes,
             "ce_fwd_grad: bad arguments");
  cudaStream_t st = as_stream(stream);
  ce_count_kernel<<<1, 1024, 0, st>>>(labels, rows, valid_count);
  MT_LAUNCH_CHECK();
  if (rows > 0) {
    int* flag = device_flag_ptr();
    MT_DISPATCH_FLOAT(dtype, T, {
      constexpr int VN = Vec16<T>::N;
      int vec_ok = aligned16(logits) && (ld % VN == 0);
      const int64_t row_bytes = classes * (int64_t)sizeof(T);
      if (vec_ok && classes % VN == 0 && row_bytes <= kCeStagedMaxBytes) {
        const int smem = (int)row_bytes + 8 * kCePieces + 16;
        MT_CHECK_CUDA(cudaFuncSetAttribute(ce_fwd_grad_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ce_fwd_grad_staged_kernel<T><<<(unsigned)rows, kCeThreads, smem, st>>>((T*)logits, labels, loss, lse, scale_host, scale_dev,
                                                                             valid_count, (int)classes, ld, softcap, flag);
      } else {
        ce_fwd_grad_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>((T*)logits, labels, loss, lse, scale_host, scale_dev,
                                                                   valid_count, classes, ld, softcap, vec_ok, flag);
      }
    });
    MT_LAUNCH_CHECK();
  }
  if (loss_sum || loss_mean) {
    ce_reduce_kernel<<<1, 1024, 0, st>>>(loss, labels, rows, loss_sum, valid_count, loss_mean);
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

int mt_scale_ratio(void* x, int64_t n, const float* num, const float* den, int dtype, void* stream) {
  MT_REQUIRE(x && num && den && n >= 0, "scale_ratio: bad arguments");
  if (n == 0) return MT_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  MT_DISPATCH_FLOAT(dtype, T, (scale_ratio_kernel<T><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((T*)x, n, num, den)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_ce_bwd(const void* logits, const int32_t* labels, const float* lse, void* dlogits, float scale_host,
              const float* scale_dev, const float* count_dev, int64_t rows, int64_t classes, int64_t ld,
              float softcap, int dtype, void* stream) {
  MT_REQUIRE(logits && labels && lse && dlogits && rows >= 0 && classes > 0 && ld >= classes, "ce_bwd: bad arguments");
  MT_REQUIRE(rows <= 65535 * 1024, "ce_bwd: too many rows");
  if (rows == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  // rows on grid.y is limited to 65535: loop over slabs of rows
  const int64_t slab = 65535;
  for (int64_t r0 = 0; r0 < rows; r0 += slab) {
    int64_t nr = rows - r0 < slab ? rows - r0 : slab;
    dim3 grid((unsigned)((classes + kCeBwdChunk - 1) / kCeBwdChunk), (unsigned)nr);
    MT_DISPATCH_FLOAT(dtype, T, {
      int vec_ok = aligned16(logits) && aligned16(dlogits) && (ld % Vec16<T>::N == 0);
      ce_bwd_kernel<T><<<grid, 256, 0, st>>>((const T*)logits + r0 * ld, labels + r0, lse + r0, (T*)dlogits + r0 * ld,
                                             scale_host, scale_dev, count_dev, classes, ld, softcap, vec_ok);
    });
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

int mt_ce_chunk_fwd(const void* logits, const int32_t* labels, float* lse_running, float* tgt, int64_t rows,
                    int64_t chunk_classes, int64_t ld, int64_t col_offset, float softcap, int dtype, void* stream) {
  MT_REQUIRE(logits && labels && lse_running && tgt && rows >= 0 && chunk_classes > 0 && ld >= chunk_classes && col_offset >= 0,
             "ce_chunk_fwd: bad arguments");
  if (rows == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(dtype, T, {
    int vec_ok = aligned16(logits) && (ld % Vec16<T>::N == 0);
    ce_fwd_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>((const T*)logits, labels, nullptr, lse_running, chunk_classes, ld,
                                                            softcap, vec_ok, nullptr, col_offset, tgt);
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_ce_chunk_finish(const float* lse, const float* tgt, const int32_t* labels, float* loss, float* loss_sum,
                       float* valid_count, float* loss_mean, int64_t rows, void* stream) {
  MT_REQUIRE(lse && tgt && labels && loss && rows >= 0, "ce_chunk_finish: bad arguments");
  cudaStream_t st = as_stream(stream);
  if (rows > 0) {
    ce_finish_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(lse, tgt, labels, loss, rows);
    MT_LAUNCH_CHECK();
  }
  if (loss_sum || valid_count || loss_mean) {
    ce_reduce_kernel<<<1, 1024, 0, st>>>(loss, labels, rows, loss_sum, valid_count, loss_mean);
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

int mt_ce_chunk_bwd(const void* logits, const int32_t* labels, const float* lse, void* dlogits, float scale_host,
                    const float* scale_dev, const float* count_dev, int64_t rows, int64_t chunk_classes, int64_t ld,
                    int64_t col_offset, float softcap, int dtype, void* stream) {
  MT_REQUIRE(logits && labels && lse && dlogits && rows >= 0 && chunk_classes > 0 && ld >= chunk_classes && col_offset >= 0,
             "ce_chunk_bwd: bad arguments");
  if (rows == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  const int64_t slab = 65535;
  for (int64_t r0 = 0; r0 < rows; r0 += slab) {
    int64_t nr = rows - r0 < slab ? rows - r0 : slab;
    dim3 grid((unsigned)((chunk_classes + kCeBwdChunk - 1) / kCeBwdChunk), (unsigned)nr);
    MT_DISPATCH_FLOAT(dtype, T, {
      int vec_ok = aligned16(logits) && aligned16(dlogits) && (ld % Vec16<T>::N == 0);
      ce_bwd_kernel<T><<<grid, 256, 0, st>>>((const T*)logits + r0 * ld, labels + r0, lse + r0, (T*)dlogits + r0 * ld,
                                             scale_host, scale_dev, count_dev, chunk_classes, ld, softcap, vec_ok,
                                             col_offset, 1);
    });
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

}  // extern "C"
