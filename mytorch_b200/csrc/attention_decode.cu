// Attention of a few new query rows against a key/value cache (the inference step:
// gpt2_trainer/gpt2.py:29-86 Cache and :167-215 cached attention; Sq != Skv as in
// fused_ops/flash_cross_attention.py) and the append of new K/V rows to that cache.
//
// The cache is a preallocated ring [B, H, max_len, D]: appending never moves old rows, and once
// max_len rows are held the oldest is overwritten - the "drop the oldest token" policy of the
// reference's Cache.update without its concatenate-and-slice copies. Softmax attention does not
// depend on the order of the keys, so the ring order is immaterial for the result.
//
// Decode attention is HBM bound: it reads kv_len*D*2 elements of K and V per (batch, head) once.
// One CTA of four warps per (batch, head, query row); a lane owns whole keys (its dot product and
// its share of P.V need no cross-lane traffic), a warp walks the keys 32 at a time with an online
// softmax, the four warps' partial (max, sum, O) are merged through shared memory.
// Algorithmic bytes: 2*kv_len*D*s per (batch, head) (+ q and o rows).
#include "common.cuh"
#include "attention.cuh"

namespace mt {

constexpr int kDecWarps = 4;

template <typename T, int D>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, T* __restrict__ o,
                   mt_strides3 sq, mt_strides3 skv, mt_strides3 so, int heads, int group, int q_len, int kv_len,
                   float scale_log2, int causal_offset) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float q_s[D];
  __shared__ float red_m[kDecWarps], red_l[kDecWarps];
  __shared__ float red_o[kDecWarps][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = blockIdx.x % q_len;
  const int bh = blockIdx.x / q_len;
  const int b = bh / heads, h = bh % heads;
  const T* qrow = q + (int64_t)b * sq.b + (int64_t)h * sq.h + (int64_t)qi * sq.s;
  for (int d = threadIdx.x; d < D; d += blockDim.x) q_s[d] = to_f(qrow[d]) * scale_log2;
  __syncthreads();
  // keys this query may see: all of them, or those at positions <= causal_offset + qi
  const int n_keys = causal_offset < 0 ? kv_len : min(kv_len, causal_offset + qi + 1);
  const int hk = h / group;                      // key/value head of this query head (grouped-query attention)
  const T* kbase = kc + (int64_t)b * skv.b + (int64_t)hk * skv.h;
  const T* vbase = vc + (int64_t)b * skv.b + (int64_t)hk * skv.h;
  float m = -INFINITY, l = 0.f;
  float acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.f;
  for (int j0 = warp * 32; j0 < n_keys; j0 += kDecWarps * 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < n_keys) {
      const T* kr = kbase + (int64_t)j * skv.s;
      float dot = 0.f;
#pragma unroll
      for (int d = 0; d < D; d += VN) {
        Vec16<T> kv;
        kv.load(kr + d);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot = fmaf(kv.get(e), q_s[d + e], dot);
      }
      s = dot;   // already in the log2 domain
    }
    float mx = s;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m, mx);          // finite: the first key of a group always exists
    const float alpha = exp2f(m - m_new);      // 0 on the first group
    const float p = j < n_keys ? exp2f(s - m_new) : 0.f;
    l = l * alpha + p;
    m = m_new;
    if (j < n_keys) {
      const T* vr = vbase + (int64_t)j * skv.s;
#pragma unroll
      for (int d = 0; d < D; d += VN) {
        Vec16<T> vv;
        vv.load(vr + d);
#pragma unroll
        for (int e = 0; e < VN; ++e) acc[d + e] = fmaf(p, vv.get(e), acc[d + e] * alpha);
      }
    } else {
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] *= alpha;
    }
  }
  // lanes of a warp share m; sum l and O over lanes
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
#pragma unroll
  for (int d = 0; d < D; ++d) {
    float v = acc[d];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == (d & 31)) red_o[warp][d] = v;
  }
  if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, red_m[w]);
  float ll = 0.f;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) ll += red_m[w] == -INFINITY ? 0.f : red_l[w] * exp2f(red_m[w] - mm);
  T* orow = o + (int64_t)b * so.b + (int64_t)h * so.h + (int64_t)qi * so.s;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) v += red_m[w] == -INFINITY ? 0.f : red_o[w][d] * exp2f(red_m[w] - mm);
    orow[d] = from_f<T>(ll > 0.f ? v / ll : 0.f);
  }
}

// cache[b, h, (pos0 + i) % max_len, :] = new[b, h, i, :]
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_cache, T* __restrict__ v_cache,
                 mt_strides3 sk, mt_strides3 sv, mt_strides3 sc, int heads, int n_new, int pos0, int max_len, int D,
                 int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    int64_t r = i / D;
    const int t = (int)(r % n_new);
    r /= n_new;
    const int h = (int)(r % heads), b = (int)(r / heads);
    const int64_t dst = (int64_t)b * sc.b + (int64_t)h * sc.h + (int64_t)((pos0 + t) % max_len) * sc.s + d;
    k_cache[dst] = k_new[(int64_t)b * sk.b + (int64_t)h * sk.h + (int64_t)t * sk.s + d];
    v_cache[dst] = v_new[(int64_t)b * sv.b + (int64_t)h * sv.h + (int64_t)t * sv.s + d];
  }
}

template <typename T, int D>
static int launch_decode(const void* q, const void* kc, const void* vc, void* o, mt_strides3 sq, mt_strides3 skv,
                         mt_strides3 so, int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t kv_len,
                         float scale, int causal_offset, cudaStream_t st) {
  const int64_t blocks = batch * heads * q_len;
  attn_decode_kernel<T, D><<<(unsigned)blocks, kDecWarps * 32, 0, st>>>(
      (const T*)q, (const T*)kc, (const T*)vc, (T*)o, sq, skv, so, (int)heads, (int)(heads / kv_heads), (int)q_len,
      (int)kv_len, scale * 1.4426950408889634f, causal_offset);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_attn_decode_gqa(const void* q, const void* k_cache, const void* v_cache, void* o, mt_strides3 sq, mt_strides3 skv,
                       mt_strides3 so, int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t kv_len,
                       int64_t head_dim, float scale, int causal_offset, int dtype, void* stream) {
  MT_REQUIRE(q && k_cache && v_cache && o && batch >= 0 && heads > 0 && q_len >= 0 && kv_len >= 0 && head_dim > 0,
             "attn_decode: bad arguments");
  MT_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attn_decode: query heads must be a multiple of key/value heads");
  MT_REQUIRE(head_dim == 64 || head_dim == 128, "attn_decode: head_dim must be 64 or 128");
  MT_REQUIRE(batch * heads * q_len < (1ll << 31), "attn_decode: too many query rows");
  constexpr int64_t kAlign = 8;   // 16-byte vector loads of half rows (4 for fp32 rows is implied)
  MT_REQUIRE(skv.b % kAlign == 0 && skv.h % kAlign == 0 && skv.s % kAlign == 0 && aligned16(k_cache) && aligned16(v_cache),
             "attn_decode: cache rows must be 16-byte aligned");
  if (batch == 0 || q_len == 0) return MT_OK;
  cudaStream_t st = as_stream(stream);
#define MT_DEC(T)                                                                                                   \
  return head_dim == 64 ? launch_decode<T, 64>(q, k_cache, v_cache, o, sq, skv, so, batch, heads, kv_heads, q_len,  \
                                                kv_len, scale, causal_offset, st)                                    \
                        : launch_decode<T, 128>(q, k_cache, v_cache, o, sq, skv, so, batch, heads, kv_heads, q_len, \
                                                 kv_len, scale, causal_offset, st)
  MT_DISPATCH_FLOAT(dtype, T, MT_DEC(T));
#undef MT_DEC
  return MT_OK;
}

int mt_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* o, mt_strides3 sq, mt_strides3 skv,
                   mt_strides3 so, int64_t batch, int64_t heads, int64_t q_len, int64_t kv_len, int64_t head_dim,
                   float scale, int causal_offset, int dtype, void* stream) {
  return mt_attn_decode_gqa(q, k_cache, v_cache, o, sq, skv, so, batch, heads, heads, q_len, kv_len, head_dim, scale,
                            causal_offset, dtype, stream);
}

int mt_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, mt_strides3 sk, mt_strides3 sv,
                 mt_strides3 scache, int64_t batch, int64_t heads, int64_t n_new, int64_t pos0, int64_t max_len,
                 int64_t head_dim, int dtype, void* stream) {
  MT_REQUIRE(k_new && v_new && k_cache && v_cache && batch >= 0 && heads > 0 && n_new >= 0 && pos0 >= 0 && max_len > 0 &&
             head_dim > 0 && n_new <= max_len, "kv_append: bad arguments");
  const int64_t total = batch * heads * n_new * head_dim;
  if (total == 0) return MT_OK;
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  cudaStream_t st = as_stream(stream);
  MT_DISPATCH_FLOAT(dtype, T, (kv_append_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
      (const T*)k_new, (const T*)v_new, (T*)k_cache, (T*)v_cache, sk, sv, scache, (int)heads, (int)n_new, (int)pos0,
      (int)max_len, (int)head_dim, total)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

}  // extern "C"
