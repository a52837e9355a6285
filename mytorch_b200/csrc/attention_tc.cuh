// Helpers shared by the tensor-core attention kernels (forward and backward).
#pragma once
#include "common.cuh"
#include "attention.cuh"
#include "sm100.cuh"

namespace mt {

constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

// Position (1..3) of the seq / head / batch coordinate in each 4-D tensor map;
// the outer dimensions are ordered by ascending stride when the map is built.
struct MapPos { int s, h, b; };

// Tile order shared by the forward and backward kernels. Tiles are (block index along the
// sequence, (batch, head) pair). Heads are taken in groups of `gh`: within a group the order is
// block-major (all heads' heaviest block first), and a group is finished before the next begins.
// The CTAs that run at the same time therefore work on a few heads only, whose K/V (forward) or
// Q/dO/dQ (backward) stay in L2 while every block of the head is visited; with all heads in one
// group the concurrent CTAs would each stream a different head and the re-reads would come from
// DRAM. `slot` runs over the blocks in the order they should be taken (0 first).
__device__ __forceinline__ void decode_tile(int tile, int n_blocks, int bh_count, int gh, int& slot, int& bh) {
  const int per_group = gh * n_blocks;
  const int gi = tile / per_group, r = tile - gi * per_group;
  const int gh_cur = min(gh, bh_count - gi * gh);      // the last group may be smaller
  slot = r / gh_cur;
  bh = gi * gh + (r - slot * gh_cur);
}

__device__ __forceinline__ void load_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, MapPos pos, int d0, int row0,
                                          int h, int b) {
  int c[4];
  c[0] = d0; c[pos.s] = row0; c[pos.h] = h; c[pos.b] = b;
  sm100::tma_load_4d(dst, map, bar, c[0], c[1], c[2], c[3]);
}

__device__ __forceinline__ void prefetch_rows(const CUtensorMap* map, MapPos pos, int d0, int row0, int h, int b) {
  int c[4];
  c[0] = d0; c[pos.s] = row0; c[pos.h] = h; c[pos.b] = b;
  sm100::tma_prefetch_4d(map, c[0], c[1], c[2], c[3]);
}

// Store of a staged tile (64 of head_dim x `box rows` of seq) through the same kind of map.
__device__ __forceinline__ void store_rows(const CUtensorMap* map, uint32_t src, MapPos pos, int d0, int row0, int h, int b) {
  int c[4];
  c[0] = d0; c[pos.s] = row0; c[pos.h] = h; c[pos.b] = b;
  sm100::tma_store_4d(map, src, c[0], c[1], c[2], c[3]);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Three-input maximum in one instruction.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Two fp32 values in one 64-bit register pair, for the packed f32x2 arithmetic
// of sm_100 (one instruction per two elements).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

static inline bool strides_ok(const mt_strides3& s) { return s.b % 8 == 0 && s.h % 8 == 0 && s.s % 8 == 0; }

// 4-D map {head_dim, x, y, z} with (seq, head, batch) placed by ascending stride;
// the box covers 64 of head_dim and 128 rows of seq.
static inline int make_qkv_map(CUtensorMap* m, MapPos* pos, const void* p, int bf16, const mt_strides3& s, int64_t B, int64_t H,
                        int64_t S, int64_t D, uint32_t box_rows = 128) {
  struct Dim { uint64_t extent, stride; uint32_t box; int role; };
  Dim d[3] = {{(uint64_t)S, (uint64_t)s.s, box_rows, 0}, {(uint64_t)H, (uint64_t)s.h, 1, 1}, {(uint64_t)B, (uint64_t)s.b, 1, 2}};
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (d[j].stride < d[i].stride) { Dim t = d[i]; d[i] = d[j]; d[j] = t; }
  uint64_t dims[4] = {(uint64_t)D, d[0].extent, d[1].extent, d[2].extent};
  uint64_t str[3] = {d[0].stride, d[1].stride, d[2].stride};
  uint32_t box[4] = {64, d[0].box, d[1].box, d[2].box};
  for (int i = 0; i < 3; ++i) {
    if (d[i].role == 0) pos->s = i + 1;
    else if (d[i].role == 1) pos->h = i + 1;
    else pos->b = i + 1;
  }
  return make_tmap_nd(m, p, bf16, 4, dims, str, box);
}

bool attn_bwd_tc_supported(const AttnArgs& a);

}  // namespace mt
