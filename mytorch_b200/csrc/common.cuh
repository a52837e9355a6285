// Shared helpers for the mytorch_b200 kernels: status handling, dtype dispatch,
// vector load/store, warp/block reductions, launch accounting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include "../../include/mytorch_b200.h"

namespace mt {

void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int* device_flag_ptr();  // device pointer to the per-device status word (lazily created)

#define MT_CHECK_CUDA(expr)                                                        \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      mt::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return MT_ERR_CUDA;                                                          \
    }                                                                              \
  } while (0)

#define MT_REQUIRE(cond, ...)                 \
  do {                                        \
    if (!(cond)) {                            \
      mt::set_error(__VA_ARGS__);             \
      return MT_ERR_INVALID;                  \
    }                                         \
  } while (0)

#define MT_LAUNCH_CHECK()                                                          \
  do {                                                                             \
    cudaError_t _e = cudaGetLastError();                                           \
    if (_e != cudaSuccess) {                                                       \
      mt::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
      return MT_ERR_CUDA;                                                          \
    }                                                                              \
    mt::count_launch();                                                            \
  } while (0)

// Runs `body` with `T` bound to the C++ type of a floating dtype code.
#define MT_DISPATCH_FLOAT(dtype, T, ...)                                       \
  switch (dtype) {                                                             \
    case MT_F32:  { using T = float;          __VA_ARGS__; break; }            \
    case MT_F16:  { using T = __half;         __VA_ARGS__; break; }            \
    case MT_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; }            \
    default: mt::set_error("unsupported dtype code %d", (int)(dtype)); return MT_ERR_DTYPE; \
  }

inline size_t dtype_size(int dt) { return dt == MT_F32 ? 4 : 2; }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vector of T (4 floats or 8 halves).
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 u; T e[16 / sizeof(T)]; };
  __device__ __forceinline__ void load(const T* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = u; }
  __device__ __forceinline__ float get(int i) const { return to_f<T>(e[i]); }
  __device__ __forceinline__ void set(int i, float v) { e[i] = from_f<T>(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `sh` must hold 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -INFINITY;
  return warp_max(r);
}

int sm_count();

// Programmatic dependent launch. A kernel launched through launch_overlapped() may start while
// the kernel before it in the stream still runs; it must call grid_dependency_wait() before its
// first access to global memory (the call returns at once in a kernel launched the plain way).
// allow_dependents() lets the next kernel in the stream start as soon as every block of this one
// has passed the call. MT_PDL=0 in the environment turns the overlap off (overlap_launches()).
bool overlap_launches();
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                            Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace mt
