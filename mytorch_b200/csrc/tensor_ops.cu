// Layout and reduction helpers behind the Tensor glue ops (transpose, chunk, slicing,
// concatenate/stack, elementwise product, sums over an axis): a strided N-d copy, a product
// and a row sum. All HBM-bound; none of them is on the fused training path, which reads its
// operands in place through strides instead of copying them.
#include "common.cuh"

namespace mt {

constexpr int kMaxCopyDims = 6;
struct CopyDims {
  int ndim;
  int64_t shape[kMaxCopyDims];        // outermost first
  int64_t sstride[kMaxCopyDims];      // in elements; 0 broadcasts
  int64_t dstride[kMaxCopyDims];
};

// dst[idx . dstride] (+)= src[idx . sstride] over the index space `shape`. Threads walk the
// space in row-major order of `shape`, so whichever side is contiguous in its last dimension is
// accessed coalesced.
template <typename U, bool ACC, typename TF>
__global__ void __launch_bounds__(256) copy_strided_kernel(const U* __restrict__ src, U* __restrict__ dst, CopyDims d, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, so = 0, doff = 0;
#pragma unroll
    for (int k = kMaxCopyDims - 1; k >= 0; --k) {
      if (k < d.ndim) {
        const int64_t c = rem % d.shape[k];
        rem /= d.shape[k];
        so += c * d.sstride[k];
        doff += c * d.dstride[k];
      }
    }
    if (ACC) {
      TF* dp = reinterpret_cast<TF*>(dst) + doff;
      *dp = from_f<TF>(to_f(*dp) + to_f(reinterpret_cast<const TF*>(src)[so]));
    } else {
      dst[doff] = src[so];
    }
  }
}

struct Mul { __device__ float operator()(float a, float b) const { return a * b; } };

template <typename T>
__global__ void __launch_bounds__(256) mul_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = from_f<T>(to_f(a[i]) * to_f(b[i]));
}

// out[r] = sum_c a[r, c]: one warp per row, lanes stride the row, fixed shuffle tree.
template <typename T>
__global__ void __launch_bounds__(256) rowsum_kernel(const T* __restrict__ a, T* __restrict__ out, int64_t rows, int64_t cols, float alpha) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int64_t c = lane; c < cols; c += 32) s += to_f(a[row * cols + c]);
  s = warp_sum(s);
  if (lane == 0) out[row] = from_f<T>(s * alpha);
}

static inline unsigned blocks_for(int64_t n) {
  int64_t b = (n + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_copy_strided(const void* src, void* dst, int ndim, const int64_t* shape, const int64_t* src_strides,
                    const int64_t* dst_strides, int elem_bytes, int accumulate_dtype, void* stream) {
  MT_REQUIRE(src && dst && shape && src_strides && dst_strides && ndim >= 1 && ndim <= kMaxCopyDims,
             "copy_strided: 1 to %d dimensions", kMaxCopyDims);
  MT_REQUIRE(elem_bytes == 2 || elem_bytes == 4, "copy_strided: elements of 2 or 4 bytes");
  CopyDims d;
  d.ndim = ndim;
  int64_t n = 1;
  for (int k = 0; k < kMaxCopyDims; ++k) {
    d.shape[k] = k < ndim ? shape[k] : 1;
    d.sstride[k] = k < ndim ? src_strides[k] : 0;
    d.dstride[k] = k < ndim ? dst_strides[k] : 0;
    MT_REQUIRE(d.shape[k] >= 0, "copy_strided: negative extent");
    n *= d.shape[k];
  }
  if (n == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  if (accumulate_dtype < 0) {
    if (elem_bytes == 2) copy_strided_kernel<uint16_t, false, __half><<<blocks_for(n), 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, d, n);
    else copy_strided_kernel<uint32_t, false, float><<<blocks_for(n), 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, d, n);
  } else {
    MT_REQUIRE((int)dtype_size(accumulate_dtype) == elem_bytes, "copy_strided: accumulate dtype and element size disagree");
    switch (accumulate_dtype) {
      case MT_F32: copy_strided_kernel<uint32_t, true, float><<<blocks_for(n), 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, d, n); break;
      case MT_F16: copy_strided_kernel<uint16_t, true, __half><<<blocks_for(n), 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, d, n); break;
      case MT_BF16: copy_strided_kernel<uint16_t, true, __nv_bfloat16><<<blocks_for(n), 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, d, n); break;
      default: mt::set_error("copy_strided: unsupported dtype code %d", accumulate_dtype); return MT_ERR_DTYPE;
    }
  }
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_mul(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream) {
  MT_REQUIRE(a && b && out && n >= 0, "mul: bad arguments");
  if (n == 0) return MT_OK;
  MT_DISPATCH_FLOAT(dtype, T, (mul_kernel<T><<<blocks_for(n), 256, 0, as_stream(stream)>>>((const T*)a, (const T*)b, (T*)out, n)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_rowsum(const void* a, void* out, int64_t rows, int64_t cols, float alpha, int dtype, void* stream) {
  MT_REQUIRE(a && out && rows >= 0 && cols >= 0, "rowsum: bad arguments");
  if (rows == 0) return MT_OK;
  MT_DISPATCH_FLOAT(dtype, T, (rowsum_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, as_stream(stream)>>>((const T*)a, (T*)out, rows, cols, alpha)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // extern "C"
