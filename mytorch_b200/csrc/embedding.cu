// Embedding gather and its deterministic scatter-add.
//
// Forward: one warp per token, 16-byte vector copies of the row
// (traffic 2*tokens*dim*s). Backward: token indices are radix-sorted together
// with their positions (stable), then one warp per run of equal indices adds
// that run's gradient rows in position order into the fp32 weight gradient —
// no atomics, so the sum order and the result are reproducible.
#include "common.cuh"
#include <cub/device/device_radix_sort.cuh>

namespace mt {

template <typename T, bool POS>
__global__ void __launch_bounds__(128)
embedding_fwd_kernel(const T* __restrict__ w, const T* __restrict__ wpe, const int32_t* __restrict__ idx,
                     T* __restrict__ out, int64_t n, int64_t seq_len, int64_t dim, int64_t vocab, int vec, int* flag) {
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (tok >= n) return;
  int32_t id = idx[tok];
  bool bad = id < 0 || id >= vocab;
  if (bad) { if (lane == 0 && flag) atomicMax(flag, 1); }
  const T* src = w + (int64_t)(bad ? 0 : id) * dim;
  const T* pos = POS ? wpe + (tok % seq_len) * dim : nullptr;
  T* dst = out + tok * dim;
  if (vec) {
    for (int64_t c = (int64_t)lane * VN; c < dim; c += 32 * VN) {
      Vec16<T> v;
      if (bad) { for (int e = 0; e < VN; ++e) v.set(e, 0.f); } else v.load(src + c);
      if (POS) {
        Vec16<T> p;
        p.load(pos + c);
#pragma unroll
        for (int e = 0; e < VN; ++e) v.set(e, v.get(e) + p.get(e));
      }
      v.store(dst + c);
    }
  } else {
    for (int64_t c = lane; c < dim; c += 32) {
      float a = bad ? 0.f : to_f(src[c]);
      if (POS) a += to_f(pos[c]);
      dst[c] = from_f<T>(a);
    }
  }
}

__global__ void iota_kernel(int32_t* p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = (int32_t)i;
}

template <typename T>
__global__ void __launch_bounds__(128)
embedding_bwd_kernel(const T* __restrict__ dy, const int32_t* __restrict__ keys, const int32_t* __restrict__ pos,
                     float* __restrict__ dw, int64_t n, int64_t dim, int64_t vocab) {
  const int lane = threadIdx.x & 31;
  const int64_t j = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (j >= n) return;
  const int32_t key = keys[j];
  if (j > 0 && keys[j - 1] == key) return;   // not the head of a run
  if (key < 0 || key >= vocab) return;       // recorded by the forward pass; skipped here
  int64_t end = j + 1;
  while (end < n && keys[end] == key) ++end;
  float* dst = dw + (int64_t)key * dim;
  for (int64_t c = lane; c < dim; c += 32) {
    float acc = 0.f;
    for (int64_t r = j; r < end; ++r) acc += to_f(dy[(int64_t)pos[r] * dim + c]);
    dst[c] += acc;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
pos_embedding_bwd_kernel(const T* __restrict__ dy, float* __restrict__ dwpe, int64_t batch, int64_t seq_len, int64_t dim) {
  int64_t n = seq_len * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int64_t b = 0; b < batch; ++b) acc += to_f(dy[b * n + i]);
    dwpe[i] += acc;
  }
}

static size_t round256(size_t x) { return (x + 255) / 256 * 256; }
static size_t cub_sort_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int32_t*)nullptr, (int32_t*)nullptr,
                                  (const int32_t*)nullptr, (int32_t*)nullptr, (int)n);
  return bytes;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_embedding_fwd(const void* weight, const int32_t* idx, void* out, int64_t n, int64_t dim, int64_t vocab,
                     int dtype, void* stream) {
  MT_REQUIRE(weight && idx && out && n >= 0 && dim > 0 && vocab > 0, "embedding_fwd: bad arguments");
  if (n == 0) return MT_OK;
  int* flag = device_flag_ptr();
  MT_DISPATCH_FLOAT(dtype, T, {
    int vec = aligned16(weight) && aligned16(out) && dim % Vec16<T>::N == 0;
    embedding_fwd_kernel<T, false><<<(unsigned)((n + 3) / 4), 128, 0, as_stream(stream)>>>(
        (const T*)weight, nullptr, idx, (T*)out, n, 1, dim, vocab, vec, flag);
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_embedding_pos_fwd(const void* wte, const void* wpe, const int32_t* idx, void* out, int64_t n,
                         int64_t seq_len, int64_t dim, int64_t vocab, int dtype, void* stream) {
  MT_REQUIRE(wte && wpe && idx && out && n >= 0 && dim > 0 && vocab > 0 && seq_len > 0, "embedding_pos_fwd: bad arguments");
  if (n == 0) return MT_OK;
  int* flag = device_flag_ptr();
  MT_DISPATCH_FLOAT(dtype, T, {
    int vec = aligned16(wte) && aligned16(wpe) && aligned16(out) && dim % Vec16<T>::N == 0;
    embedding_fwd_kernel<T, true><<<(unsigned)((n + 3) / 4), 128, 0, as_stream(stream)>>>(
        (const T*)wte, (const T*)wpe, idx, (T*)out, n, seq_len, dim, vocab, vec, flag);
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

size_t mt_embedding_bwd_scratch_bytes(int64_t n) {
  if (n <= 0) return 256;
  return 3 * round256((size_t)n * 4) + round256(cub_sort_bytes(n));
}

int mt_embedding_bwd(const void* dy, const int32_t* idx, float* dweight, void* scratch, int64_t n, int64_t dim,
                     int64_t vocab, int dtype, void* stream) {
  MT_REQUIRE(dy && idx && dweight && scratch && n >= 0 && dim > 0 && vocab > 0, "embedding_bwd: bad arguments");
  MT_REQUIRE(n < (1ll << 31), "embedding_bwd: too many tokens");
  if (n == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
  char* base = (char*)scratch;
  size_t seg = round256((size_t)n * 4);
  int32_t* pos_in = (int32_t*)base;
  int32_t* keys_out = (int32_t*)(base + seg);
  int32_t* pos_out = (int32_t*)(base + 2 * seg);
  void* cub_tmp = base + 3 * seg;
  size_t cub_bytes = cub_sort_bytes(n);
  iota_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(pos_in, n);
  MT_LAUNCH_CHECK();
  // All 32 key bits take part: an out-of-range id (the forward pass flags those, the backward kernel
  // skips them) then sorts before or after every valid id instead of landing, by its low bits,
  // inside a run of equal valid ids and splitting it between two warps.
  MT_CHECK_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, idx, keys_out, pos_in, pos_out, (int)n, 0, 32, st));
  count_launch(3);
  MT_DISPATCH_FLOAT(dtype, T, (embedding_bwd_kernel<T><<<(unsigned)((n + 3) / 4), 128, 0, st>>>((const T*)dy, keys_out, pos_out, dweight, n, dim, vocab)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int mt_pos_embedding_bwd(const void* dy, float* dwpe, int64_t batch, int64_t seq_len, int64_t dim, int dtype, void* stream) {
  MT_REQUIRE(dy && dwpe && batch >= 0 && seq_len > 0 && dim > 0, "pos_embedding_bwd: bad arguments");
  int64_t n = seq_len * dim;
  int64_t blocks = (n + 255) / 256;
  MT_DISPATCH_FLOAT(dtype, T, (pos_embedding_bwd_kernel<T><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((const T*)dy, dwpe, batch, seq_len, dim)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // extern "C"
