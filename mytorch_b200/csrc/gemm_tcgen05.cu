// Tensor-core GEMM for sm_100a: C[M,N] = act(alpha * op(A) op(B) + bias) with
// fp16/bf16 operands and fp32 accumulation in tensor memory.
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 256 or 128).
// Warp roles:
//   warp 0    TMA producer: 128-byte-swizzled 64-deep K slices of A and B into
//             a ring of shared-memory stages (full/empty mbarriers);
//   warp 1    MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) per
//             16 of K, accumulating into one of two TMEM buffers, and commits
//             stage-release and accumulator-ready barriers;
//   warps 2-9 epilogue: tcgen05.ld the finished accumulator (thread = row, two
//             warps per 32-row slab, half of the columns each), apply alpha /
//             bias / activation, stage 32 x 128-byte slabs in shared memory and
//             hand them to TMA (store, or fp32 reduce-add for split-K) while
//             the MMA warp is already on the next tile in the other TMEM buffer.
// With CTA pairs (clusters of two, tcgen05 cta_group::2) the scheduled tile is
// 256 x BN: each CTA stages its own 128 rows of A and half of the B tile, rank 0
// issues the MMAs for both and each CTA drains its own 128 accumulator rows, so
// a byte of B fetched from L2 feeds twice the FLOPs.
// Operands may be K-major or MN-major in global memory (all four transpose
// combinations), selected by the TMA box and the UMMA descriptors; no
// transposed copies are made. Loads are plain (non-multicast) TMA.
//
// Roofline: tensor pipe; algorithmic work 2*M*N*K FLOP per launch.
#include "common.cuh"
#include "gemm.cuh"
#include "sm100.cuh"
#include "prof.cuh"
#include <atomic>
#include <mutex>
#include <string.h>
#include <type_traits>

namespace mt {

using namespace sm100;

constexpr int BM = 128, BK = 64;
constexpr int kEpiWarps = 8;                       // two warps per TMEM lane quarter, each half of the tile's columns
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kABytes = BM * BK * 2;  // 16 KB

// PAIR: two CTAs of a cluster share each MMA (cta_group::2): the pair's tile is
// 256 x BN, each CTA stages its own 128 rows of A and half of the B tile.
template <int BN, bool PAIR = false> struct GemmCfg {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;      // rows of the B tile this CTA stages
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = PAIR ? 6 : (BN == 256 ? 4 : 6);
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers
  static constexpr int kEpiBytes = kEpiWarps * 4096;  // per epilogue warp: one 32-row x 128-byte staging buffer
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 512 /*barriers*/;
  // Epilogues that move a second [M,N] tensor (an aux operand read, or a second output) can run
  // with one pipeline stage less and use its shared memory as a second staging buffer per warp.
  static constexpr bool kCanDoubleStage = kStageBytes >= kEpiBytes;
};

struct GemmParams {
  void* C; void* preact; const void* bias; const void* aux; int aux_mode;
  int64_t M, N, K, ldc;
  int out_dtype, in_bf16, act, accumulate, vec_store, tma_store;
  float alpha;
  int tiles_m, tiles_n, splits, kb_per_split, kb_total;
  int stages;   // pipeline stages in use: Cfg::kStages, or one less with the last stage's memory as second staging buffers
  int n_fast;   // order of the tile walk: 0 = neighbouring tiles share their columns (B panel), 1 = their rows (A panel)
  int* flag;
};

// tanh in one MUFU instruction (relative error ~2^-11, below the half-precision
// rounding of everything this kernel writes).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float aux_apply_tc(float x, float a, int mode) {
  switch (mode) {
    case 1: return x + a;
    case 2: {
      const float a2 = a * a;
      const float t = tanh_fast(0.7978845608f * (a + 0.044715f * a2 * a));
      return x * (0.5f * (1.f + t + a * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * a2)));
    }
    case 3: return x * 2.f * fmaxf(a, 0.f);
    case 4: return a > 0.f ? x : 0.f;
    case 5: return x * a;
    case 6: return x * 2.f * sqrtf(fmaxf(a, 0.f));
    default: return x;
  }
}

// tanh-GELU and its derivative on two values at once in half precision (fp16 outputs only: the
// result is rounded to half anyway). The polynomial, the tanh (one MUFU op for the pair) and the
// products run on packed half2 instructions, two to three times fewer issue slots than fp32.
// The argument of the tanh path is clamped to [-16, 16], where tanh has long saturated, so x*x
// cannot overflow and the derivative of a huge pre-activation is exactly 1 or 0, never NaN.
__device__ __forceinline__ __half2 tanh_h2(__half2 x) {
  uint32_t r, a = *reinterpret_cast<uint32_t*>(&x);
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(r) : "r"(a));
  return *reinterpret_cast<__half2*>(&r);
}
template <bool WITH_GRAD>
__device__ __forceinline__ void gelu_h2(float x0, float x1, uint32_t& y_bits, uint32_t& dy_bits) {
  const __half2 one = __float2half2_rn(1.f), half = __float2half2_rn(0.5f);
  const __half2 k = __float2half2_rn(0.7978845608f), kc = __float2half2_rn(0.7978845608f * 0.044715f);
  const __half2 x = __floats2half2_rn(x0, x1);
  const __half2 xc = __hmax2(__hmin2(x, __float2half2_rn(16.f)), __float2half2_rn(-16.f));
  const __half2 x2 = __hmul2(xc, xc);
  const __half2 t = tanh_h2(__hmul2(xc, __hfma2(kc, x2, k)));
  const __half2 opt = __hadd2(one, t);
  const __half2 y = __hmul2(__hmul2(half, x), opt);
  y_bits = *reinterpret_cast<const uint32_t*>(&y);
  if (WITH_GRAD) {
    const __half2 k3c = __float2half2_rn(3.f * 0.7978845608f * 0.044715f);
    const __half2 s = __hfma2(__hneg2(t), t, one);                    // 1 - t^2
    const __half2 r = __hmul2(__hmul2(xc, __hfma2(k3c, x2, k)), s);   // x (k + 3kc x^2)(1 - t^2)
    const __half2 dy = __hmul2(half, __hadd2(opt, r));
    dy_bits = *reinterpret_cast<const uint32_t*>(&dy);
  }
}

// Activation and its derivative of one pre-activation, sharing the tanh.
__device__ __forceinline__ void act_both_tc(float x, int act, float& y, float& dy) {
  switch (act) {
    case MT_ACT_GELU: {
      const float x2 = x * x;
      const float t = tanh_fast(0.7978845608f * (x + 0.044715f * x2 * x));
      y = 0.5f * x * (1.f + t);
      dy = 0.5f * (1.f + t + x * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * x2));
      return;
    }
    case MT_ACT_RELU2: { const float r = fmaxf(x, 0.f); y = r * r; dy = 2.f * r; return; }
    case MT_ACT_RELU: y = fmaxf(x, 0.f); dy = x > 0.f ? 1.f : 0.f; return;
    default: y = x; dy = 1.f; return;
  }
}

__device__ __forceinline__ float act_apply_tc(float x, int act) {
  switch (act) {
    case MT_ACT_GELU: {
      float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanh_fast(inner));
    }
    case MT_ACT_RELU2: { float r = fmaxf(x, 0.f); return r * r; }
    case MT_ACT_RELU: return fmaxf(x, 0.f);
    default: return x;
  }
}

// Writes 8 consecutive outputs of one row.
template <typename TO>
__device__ __forceinline__ void store8(TO* p, const float* v, int n_valid, bool vec, int accumulate) {
  if (vec && n_valid == 8) {
    if (sizeof(TO) == 2) {
      __align__(16) TO o[8];
      if (accumulate) {
        *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = from_f<TO>(to_f(o[e]) + v[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = from_f<TO>(v[e]);
      }
      *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(o);
    } else {
      float4* q = reinterpret_cast<float4*>(p);
      if (accumulate == 2) {
        atomicAdd(q, make_float4(v[0], v[1], v[2], v[3]));
        atomicAdd(q + 1, make_float4(v[4], v[5], v[6], v[7]));
      } else {
        float4 a = make_float4(v[0], v[1], v[2], v[3]), b = make_float4(v[4], v[5], v[6], v[7]);
        if (accumulate) {
          float4 c0 = q[0], c1 = q[1];
          a.x += c0.x; a.y += c0.y; a.z += c0.z; a.w += c0.w;
          b.x += c1.x; b.y += c1.y; b.z += c1.z; b.w += c1.w;
        }
        q[0] = a;
        q[1] = b;
      }
    }
  } else {
    for (int e = 0; e < n_valid; ++e) {
      if (accumulate == 2 && sizeof(TO) == 4) atomicAdd(reinterpret_cast<float*>(p) + e, v[e]);
      else p[e] = from_f<TO>(accumulate ? to_f(p[e]) + v[e] : v[e]);
    }
  }
}

template <typename TO> __device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<float>(float a, float) { return __float_as_uint(a); }

// One warp stages 32 rows x 128 bytes (its 32 TMEM lanes, CW columns) in shared
// memory with the 128-byte swizzle and hands it to TMA: coalesced global writes,
// rows/columns past M/N clipped by the tensor map, optional fp32 reduce-add.
template <typename TO, int CW>
__device__ __forceinline__ void stage_store(const CUtensorMap* map, const uint32_t* r, uint8_t* stage, int lane, int x,
                                            int y, bool reduce, int& sidx, bool keep_one = false) {
  uint8_t* buf = stage;
  // the last store out of this buffer has finished reading it: with two buffers used in turn that
  // is the store before the latest one, which may still be in flight
  if (lane == 0) { if (keep_one) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
  __syncwarp();
  uint8_t* rowp = buf + lane * 128;
#pragma unroll
  for (int c16 = 0; c16 < 8; ++c16) {
    uint4 v;
    if (sizeof(TO) == 4) {
      v = make_uint4(r[c16 * 4], r[c16 * 4 + 1], r[c16 * 4 + 2], r[c16 * 4 + 3]);
    } else {
      v.x = pack_pair<TO>(__uint_as_float(r[c16 * 8 + 0]), __uint_as_float(r[c16 * 8 + 1]));
      v.y = pack_pair<TO>(__uint_as_float(r[c16 * 8 + 2]), __uint_as_float(r[c16 * 8 + 3]));
      v.z = pack_pair<TO>(__uint_as_float(r[c16 * 8 + 4]), __uint_as_float(r[c16 * 8 + 5]));
      v.w = pack_pair<TO>(__uint_as_float(r[c16 * 8 + 6]), __uint_as_float(r[c16 * 8 + 7]));
    }
    *reinterpret_cast<uint4*>(rowp + ((c16 ^ (lane & 7)) << 4)) = v;
  }
  fence_proxy_async();
  __syncwarp();
  if (lane == 0) {
    if (reduce) tma_reduce_add_2d(map, smem_u32(buf), x, y);
    else tma_store_2d(map, smem_u32(buf), x, y);
    bulk_commit();
  }
  ++sidx;
}

// Starts the copy of one 32-row x 128-byte slab of the aux operand into the warp's staging buffer
// (one lane; the buffer's previous TMA store must have finished reading it).
__device__ __forceinline__ void aux_slab_load(const CUtensorMap* tmAux, uint8_t* stage, uint32_t aux_bar, int x, int y) {
  bulk_wait_read<0>();
  mbar_expect_tx(aux_bar, 4096);
  tma_load_2d(smem_u32(stage), tmAux, aux_bar, x, y);
}

template <int BN, typename TO>
__device__ __forceinline__ bool epilogue_staged(const GemmParams& P, const CUtensorMap* tmC, const CUtensorMap* tmPre,
                                                const CUtensorMap* tmAux, uint32_t taddr, uint8_t* stage, int lane, int y0,
                                                int64_t n0, bool add_bias, int& sidx, int col_begin, uint32_t aux_bar,
                                                uint32_t& aux_phase, bool aux_prefetched, volatile int* abort_flag,
                                                uint8_t* stage2 = nullptr, uint32_t aux_bar2 = 0, uint32_t* aux_phase2 = nullptr,
                                                bool aux_prefetched2 = false) {
  constexpr int CW = 128 / (int)sizeof(TO);   // accumulator columns per 128-byte staged row
  // Two staging buffers (half outputs: two slabs per warp and tile): slab 0 lives in `stage`,
  // slab 1 in `stage2` - the aux slabs of both are in flight before the accumulator is ready,
  // and one slab's TMA store reads its buffer while the next slab is computed into the other.
  // A second output goes through `stage2`, the first through `stage`.
  const bool dbl = stage2 != nullptr && BN / 2 / CW == 2;
  // This warp's half of the tile's columns is requested at once and waited for once.
  constexpr int GW = BN / 2;                  // columns per warp = per load group (128 or 64)
  const float alpha = P.alpha;
  const int act = P.act & 0xff;
  const bool store_grad = (P.act & kActStoreGrad) != 0;
#pragma unroll 1
  for (int g0 = col_begin; g0 < col_begin + GW; g0 += GW) {
    if (n0 + g0 >= P.N) break;                // warp-uniform
    uint32_t r[GW];
    tmem_ld32(taddr + g0, r);
    tmem_ld32(taddr + g0 + 32, r + 32);
    if (GW == 128) {
      tmem_ld32(taddr + g0 + 64, r + (GW == 128 ? 64 : 0));
      tmem_ld32(taddr + g0 + 96, r + (GW == 128 ? 96 : 0));
    }
    tmem_ld_wait();
#pragma unroll
    for (int cc = 0; cc < GW / CW; ++cc) {
      const int64_t col0 = n0 + g0 + cc * CW;
      if (col0 >= P.N) break;                 // warp-uniform
      uint32_t* rc = r + cc * CW;
      if (alpha != 1.f) {                     // uniform; the common alpha == 1 costs nothing
#pragma unroll
        for (int e = 0; e < CW; ++e) rc[e] = __float_as_uint(alpha * __uint_as_float(rc[e]));
      }
      if (add_bias) {                         // uniform; bias is read 8 columns at a time when aligned
        const bool vec_bias = (P.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(P.bias) & 15) == 0);
#pragma unroll
        for (int e8 = 0; e8 < CW; e8 += 8) {
          if (col0 + e8 >= P.N) break;
          float bv[8];
          if (vec_bias) {
            const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(P.bias) + col0 + e8);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (P.in_bf16) {
                bv[2 * u] = __uint_as_float(w[u] << 16);
                bv[2 * u + 1] = __uint_as_float(w[u] & 0xffff0000u);
              } else {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[u]);
                bv[2 * u] = __low2float(h);
                bv[2 * u + 1] = __high2float(h);
              }
            }
          } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int64_t col = col0 + e8 + u;
              bv[u] = col >= P.N ? 0.f
                      : P.in_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.bias)[col])
                                  : __half2float(reinterpret_cast<const __half*>(P.bias)[col]);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) rc[e8 + u] = __float_as_uint(__uint_as_float(rc[e8 + u]) + bv[u]);
        }
      }
      if (P.preact && store_grad) {
        // the second output receives act'(x): computed together with act(x) (one tanh), packed
        // into the staging rows eight columns at a time, while rc is overwritten with act(x)
        uint8_t* const gstage = dbl ? stage2 : stage;
        if (lane == 0) { if (dbl) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
        __syncwarp();
        constexpr int PER = 16 / (int)sizeof(TO);
        constexpr bool kHalfMath = std::is_same<TO, __half>::value;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          if (kHalfMath && act == MT_ACT_GELU) {
            // rc keeps gelu(x) as the exact float value of the half result: packing it again
            // for the output store below is lossless
            uint32_t yb[4], db[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              gelu_h2<true>(__uint_as_float(rc[v * 8 + 2 * u]), __uint_as_float(rc[v * 8 + 2 * u + 1]), yb[u], db[u]);
              const __half2 yh = *reinterpret_cast<const __half2*>(&yb[u]);
              rc[v * 8 + 2 * u] = __float_as_uint(__low2float(yh));
              rc[v * 8 + 2 * u + 1] = __float_as_uint(__high2float(yh));
            }
            *reinterpret_cast<uint4*>(gstage + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(db[0], db[1], db[2], db[3]);
            continue;
          }
          float d[PER];
#pragma unroll
          for (int u = 0; u < PER; ++u) {
            float yv;
            act_both_tc(__uint_as_float(rc[v * PER + u]), act, yv, d[u]);
            rc[v * PER + u] = __float_as_uint(yv);
          }
          uint4 q;
          if (sizeof(TO) == 4) {
            q = make_uint4(__float_as_uint(d[0]), __float_as_uint(d[1]), __float_as_uint(d[2]), __float_as_uint(d[3]));
          } else {
            q.x = pack_pair<TO>(d[0], d[1]); q.y = pack_pair<TO>(d[2 % PER], d[3 % PER]);
            q.z = pack_pair<TO>(d[4 % PER], d[5 % PER]); q.w = pack_pair<TO>(d[6 % PER], d[7 % PER]);
          }
          *reinterpret_cast<uint4*>(gstage + lane * 128 + ((v ^ (lane & 7)) << 4)) = q;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) { tma_store_2d(tmPre, smem_u32(gstage), (int)col0, y0); bulk_commit(); }
        ++sidx;
      } else {
        if (P.preact) stage_store<TO, CW>(tmPre, rc, dbl ? stage2 : stage, lane, (int)col0, y0, false, sidx, dbl);
        if (std::is_same<TO, __half>::value && act == MT_ACT_GELU) {
#pragma unroll
          for (int e = 0; e < CW; e += 2) {
            uint32_t yb, unused;
            gelu_h2<false>(__uint_as_float(rc[e]), __uint_as_float(rc[e + 1]), yb, unused);
            const __half2 yh = *reinterpret_cast<const __half2*>(&yb);
            rc[e] = __float_as_uint(__low2float(yh));
            rc[e + 1] = __float_as_uint(__high2float(yh));
          }
        } else if (act != MT_ACT_NONE) {
#pragma unroll
          for (int e = 0; e < CW; ++e) rc[e] = __float_as_uint(act_apply_tc(__uint_as_float(rc[e]), act));
        }
      }
      if (P.aux_mode) {
        // uniform: combine with the matching slab of the aux operand. It comes through the
        // staging buffer by TMA (coalesced, rows/columns past M/N read as zero); the first slab
        // of a tile was requested before the accumulator wait, the others are requested here.
        const bool second = dbl && !P.preact && cc == 1;          // slab 1 of a double-staged tile
        uint8_t* const astage = second ? stage2 : stage;
        if (!((second ? aux_prefetched2 : aux_prefetched) && g0 == col_begin && cc == (second ? 1 : 0))) {
          if (lane == 0) aux_slab_load(tmAux, astage, second ? aux_bar2 : aux_bar, (int)col0, y0);
        }
        if (second) {
          if (!__all_sync(0xffffffffu, mbar_wait(aux_bar2, *aux_phase2, abort_flag))) return false;
          *aux_phase2 ^= 1u;
        } else {
          if (!__all_sync(0xffffffffu, mbar_wait(aux_bar, aux_phase, abort_flag))) return false;
          aux_phase ^= 1u;
        }
        constexpr int PER = 16 / (int)sizeof(TO);       // elements per 16-byte chunk
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          Vec16<TO> a;
          a.load(reinterpret_cast<const TO*>(astage + lane * 128 + ((v ^ (lane & 7)) << 4)));
#pragma unroll
          for (int u = 0; u < PER; ++u)
            rc[v * PER + u] = __float_as_uint(aux_apply_tc(__uint_as_float(rc[v * PER + u]), a.get(u), P.aux_mode));
        }
        __syncwarp();
      }
      // first output: with two buffers and no second output, slab 1 goes through `stage2`
      stage_store<TO, CW>(tmC, rc, (dbl && !P.preact && cc == 1) ? stage2 : stage, lane, (int)col0, y0, P.accumulate != 0, sidx, dbl);
    }
  }
  return true;
}

template <bool A_MN, bool B_MN, int BN, bool PAIR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmPre,
               const __grid_constant__ CUtensorMap tmAux, const GemmParams P) {
  using Cfg = GemmCfg<BN, PAIR>;
  // In a pair, rank 0 issues the MMAs and owns the operand-ready and
  // accumulator-free barriers; both CTAs walk the same list of 256 x BN tiles.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TM = PAIR ? 2 * BM : BM;                  // rows of one scheduled tile
  constexpr int SMAX = Cfg::kStages;          // the shared-memory layout is that of the full pipeline
  const int S = P.stages;                     // stages in use (SMAX, or SMAX - 1 with a second staging buffer per warp)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 1024-byte alignment for the 128B swizzle
  uint8_t* base_ptr = smem_raw + (base - raw);
  uint8_t* epi_stage = base_ptr + SMAX * Cfg::kStageBytes;   // 1024-byte aligned (stage sizes are multiples of 1 KB)
  uint8_t* epi_stage2 = S < SMAX ? base_ptr + (SMAX - 1) * Cfg::kStageBytes : nullptr;   // the unused last stage
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + Cfg::kEpiBytes);
  // barrier slots: full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t bar0 = base + SMAX * Cfg::kStageBytes + Cfg::kEpiBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (SMAX + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * SMAX + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * SMAX + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SMAX + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto aux_bar = [&](int w) { return bar0 + 8u * (2 * SMAX + 5 + w); };   // two per epilogue warp: slab 0, slab 1

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SMAX; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), PAIR ? 2 * kEpiWarps : kEpiWarps); }
    for (int w = 0; w < 2 * kEpiWarps; ++w) mbar_init(aux_bar(w), 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this CTA's shared and tensor memory, so it may overlap the
  // tail of the previous kernel in the stream; global memory is read and written from here on.
  griddep_launch();
  griddep_wait();

  const int tiles_mn = P.tiles_m * P.tiles_n;
  const int total_tiles = tiles_mn * P.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = worker; t < total_tiles && ok; t += workers) {
        const int mn = t % tiles_mn, split = t / tiles_mn;
        const int tm_i = P.n_fast ? mn / P.tiles_n : mn % P.tiles_m, tn_i = P.n_fast ? mn % P.tiles_n : mn / P.tiles_m;
        const int m0 = tm_i * TM + (int)rank * BM;
        const int n0 = tn_i * BN + (int)rank * (PAIR ? BN / 2 : 0);   // this CTA's rows of the B tile
        const int kb0 = split * P.kb_per_split;
        const int kb1 = min(kb0 + P.kb_per_split, P.kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * Cfg::kStageBytes, sb = sa + kABytes;
          // Both CTAs' copies of a stage are counted on rank 0's barrier.
          const uint32_t fb = PAIR ? mapa_shared(full_bar(stage), 0) : full_bar(stage);
          if (!PAIR) mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
          else if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y) {
            if (PAIR) tma_load_2d_pair(dst, map, fb, x, y);
            else tma_load_2d(dst, map, fb, x, y);
          };
          const int k0 = kb * BK;
          if (!A_MN) {
            load(sa, &tmA, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) load(sa + j * (BK * 128), &tmA, m0 + j * 64, k0);
          }
          if (!B_MN) {
            load(sb, &tmB, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBRows / 64; ++j) load(sb + j * (BK * 128), &tmB, n0 + j * 64, k0);
          }
          ++issued;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && rank == 0) {
        // Bounded drain: let the copies already issued into each stage land
        // before the CTA's shared memory is released (in a pair, rank 0's
        // barriers count the peer's copies too, and the peer stays resident
        // until the cluster-wide join at the end).
        long long n = issued < S ? issued : S;
        int s = stage;
        uint32_t ph = phase;
        for (long long i = 0; i < n; ++i) {
          if (--s < 0) { s = S - 1; ph ^= 1u; }
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(s), ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = idesc_f16(P.in_bf16, A_MN, B_MN, TM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = worker; t < total_tiles && ok; t += workers, ++it) {
        const int split = t / tiles_mn;
        const int kb0 = split * P.kb_per_split;
        const int kb1 = min(kb0 + P.kb_per_split, P.kb_total);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(acce_bar(buf), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * Cfg::kStageBytes, sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? smem_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                     : smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                     : smem_desc_sw128(sb + k * 32, 16, 1024);
            if (PAIR) umma_f16_pair(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_f16(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // stage reusable once these MMAs have read it (in both CTAs of a pair)
          if (PAIR) umma_commit_pair(empty_bar(stage)); else umma_commit(empty_bar(stage));
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (ok) { if (PAIR) umma_commit_pair(accf_bar(buf)); else umma_commit(accf_bar(buf)); }  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    const int col_begin = ((warp - 2) >> 2) * (BN / 2);   // this warp's half of the tile's columns
    int it = 0;
    int sidx = 0;   // running count of staged stores of this warp (selects the staging buffer)
    uint32_t aux_phase = 0, aux_phase2 = 0;
    const uint32_t my_aux_bar = aux_bar(warp - 2), my_aux_bar2 = aux_bar(kEpiWarps + warp - 2);
    uint8_t* const stage2 = epi_stage2 ? epi_stage2 + (warp - 2) * 4096 : nullptr;
    const int slab_cols = P.out_dtype == MT_F32 ? 32 : 64;     // accumulator columns of one staged slab
    bool ok = true;
    for (int t = worker; t < total_tiles && ok; t += workers, ++it) {
      const int mn = t % tiles_mn;
      const bool add_bias = P.bias != nullptr && t / tiles_mn == 0;  // only the first K split adds it
      const int tm_i = P.n_fast ? mn / P.tiles_n : mn % P.tiles_m, tn_i = P.n_fast ? mn % P.tiles_n : mn / P.tiles_m;
      const int64_t m0 = (int64_t)tm_i * TM + (int64_t)rank * BM, n0 = (int64_t)tn_i * BN;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // the first aux slab of this tile travels while the accumulator is still being computed
      const bool aux_pre = P.tma_store && P.aux_mode && !P.preact && (int)m0 + quarter * 32 < P.M && n0 + col_begin < P.N;
      if (aux_pre && lane == 0)
        aux_slab_load(&tmAux, epi_stage + (warp - 2) * 4096, my_aux_bar, (int)n0 + col_begin, (int)m0 + quarter * 32);
      // with a second staging buffer (half outputs, two slabs per warp) the second slab travels too
      const bool aux_pre2 = aux_pre && stage2 != nullptr && slab_cols == 64 && BN / 2 == 128 && n0 + col_begin + 64 < P.N;
      if (aux_pre2 && lane == 0)
        aux_slab_load(&tmAux, stage2, my_aux_bar2, (int)n0 + col_begin + 64, (int)m0 + quarter * 32);
      // warp-uniform outcome: tcgen05.ld below needs all 32 lanes together
      if (!__all_sync(0xffffffffu, mbar_wait(accf_bar(buf), acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const int64_t row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      if (P.tma_store) {
        uint8_t* stage = epi_stage + (warp - 2) * 4096;
        const int y0 = (int)m0 + quarter * 32;
        if (y0 < P.M) {   // warp-uniform: a slab of 32 rows entirely past M has nothing to write
          bool fine;
          if (P.out_dtype == MT_F16) fine = epilogue_staged<BN, __half>(P, &tmC, &tmPre, &tmAux, taddr, stage, lane, y0, n0, add_bias, sidx, col_begin, my_aux_bar, aux_phase, aux_pre, abort_flag, stage2, my_aux_bar2, &aux_phase2, aux_pre2);
          else if (P.out_dtype == MT_BF16) fine = epilogue_staged<BN, __nv_bfloat16>(P, &tmC, &tmPre, &tmAux, taddr, stage, lane, y0, n0, add_bias, sidx, col_begin, my_aux_bar, aux_phase, aux_pre, abort_flag, stage2, my_aux_bar2, &aux_phase2, aux_pre2);
          else fine = epilogue_staged<BN, float>(P, &tmC, &tmPre, &tmAux, taddr, stage, lane, y0, n0, add_bias, sidx, col_begin, my_aux_bar, aux_phase, aux_pre, abort_flag, stage2, my_aux_bar2, &aux_phase2, aux_pre2);
          if (!fine) { ok = false; break; }
        }
      } else
#pragma unroll 1
      for (int c = col_begin / 32; c < (col_begin + BN / 2) / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        const int64_t col0 = n0 + c * 32;
        if (row < P.M && col0 < P.N) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int64_t col = col0 + g8 * 8;
            if (col >= P.N) break;
            const int n_valid = (int)(P.N - col < 8 ? P.N - col : 8);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float x = P.alpha * __uint_as_float(r[g8 * 8 + e]);
              if (add_bias && e < n_valid)
                x += P.in_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.bias)[col + e])
                               : __half2float(reinterpret_cast<const __half*>(P.bias)[col + e]);
              v[e] = x;
            }
            const int64_t off = row * P.ldc + col;
            if (P.preact) {
              float pv[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) pv[e] = (P.act & kActStoreGrad) ? act_grad(v[e], P.act) : v[e];
              if (P.out_dtype == MT_F16) store8(reinterpret_cast<__half*>(P.preact) + off, pv, n_valid, P.vec_store, 0);
              else if (P.out_dtype == MT_BF16) store8(reinterpret_cast<__nv_bfloat16*>(P.preact) + off, pv, n_valid, P.vec_store, 0);
              else store8(reinterpret_cast<float*>(P.preact) + off, pv, n_valid, P.vec_store, 0);
            }
            if ((P.act & 0xff) != MT_ACT_NONE) {
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = act_apply_tc(v[e], P.act & 0xff);
            }
            if (P.aux_mode) {
              for (int e = 0; e < n_valid; ++e) {
                const float a = P.out_dtype == MT_F16 ? __half2float(reinterpret_cast<const __half*>(P.aux)[off + e])
                              : P.out_dtype == MT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.aux)[off + e])
                                                       : reinterpret_cast<const float*>(P.aux)[off + e];
                v[e] = aux_apply(v[e], a, P.aux_mode);
              }
            }
            if (P.out_dtype == MT_F16) store8(reinterpret_cast<__half*>(P.C) + off, v, n_valid, P.vec_store, P.accumulate);
            else if (P.out_dtype == MT_BF16) store8(reinterpret_cast<__nv_bfloat16*>(P.C) + off, v, n_valid, P.vec_store, P.accumulate);
            else store8(reinterpret_cast<float*>(P.C) + off, v, n_valid, P.vec_store, P.accumulate);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {   // this warp is done with the buffer
        if (PAIR) mbar_arrive_cluster(mapa_shared(acce_bar(buf), 0));
        else mbar_arrive(acce_bar(buf));
      }
    }
    if (P.tma_store && lane == 0) bulk_wait_all<0>();   // staged stores must finish before shared memory goes away
  }

  // ---------------------------------------------------------------- teardown --
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA leaves, nor frees tensor memory, while its peer still works
  if (threadIdx.x == 0 && *abort_flag && P.flag) atomicMax(P.flag, 100);  // a bounded wait expired
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

static EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = (EncodeTiledFn)fn;
  });
  return g_encode;
}

int make_tmap_nd(CUtensorMap* map, const void* base_ptr, int is_bf16, int rank, const uint64_t* dims,
                 const uint64_t* strides_elems, const uint32_t* box) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MT_ERR_CUDA; }
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 1; i < rank; ++i) gstr[i - 1] = strides_elems[i - 1] * 2;  // bytes
  CUresult r = enc(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                   const_cast<void*>(base_ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return MT_ERR_CUDA; }
  return MT_OK;
}

int make_tmap_nd_typed(CUtensorMap* map, const void* base_ptr, int dt, int rank, const uint64_t* dims,
                       const uint64_t* strides_elems, const uint32_t* box) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MT_ERR_CUDA; }
  const uint64_t esize = dt == MT_F32 ? 4 : 2;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 1; i < rank; ++i) gstr[i - 1] = strides_elems[i - 1] * esize;
  CUtensorMapDataType t = dt == MT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                        : dt == MT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(map, t, (cuuint32_t)rank, const_cast<void*>(base_ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (typed map) failed with code %d", (int)r); return MT_ERR_CUDA; }
  return MT_OK;
}

int make_tmap_2d_typed(CUtensorMap* map, const void* base_ptr, int dt, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                       uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MT_ERR_CUDA; }
  const uint64_t esize = dt == MT_F32 ? 4 : 2;
  cuuint64_t gdim[2] = {inner, outer}, gstr[1] = {ld_elems * esize};
  cuuint32_t bx[2] = {box_inner, box_outer}, es[2] = {1, 1};
  CUtensorMapDataType t = dt == MT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                        : dt == MT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(map, t, 2, const_cast<void*>(base_ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (output map) failed with code %d", (int)r); return MT_ERR_CUDA; }
  return MT_OK;
}

int make_tmap_2d(CUtensorMap* map, const void* base_ptr, int is_bf16, uint64_t inner, uint64_t outer,
                 uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer}, str[1] = {ld_elems};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tmap_nd(map, base_ptr, is_bf16, 2, dims, str, box);
}

bool gemm_tc_supported(const GemmArgs& g) {
  if (g.in_dtype != MT_F16 && g.in_dtype != MT_BF16) return false;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
  if (!aligned16(g.A) || !aligned16(g.B)) return false;
  if (g.lda % 8 || g.ldb % 8) return false;
  if (g.M >= (1ll << 31) || g.N >= (1ll << 31) || g.K >= (1ll << 31)) return false;
  if (g.accumulate == 2 && g.out_dtype != MT_F32) return false;
  return true;
}

template <bool A_MN, bool B_MN, int BN>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tp,
                     const CUtensorMap& tx, const GemmParams& P, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BN, false>;
  static std::atomic<bool> attr_set[16];   // per device; racing first calls set the same attribute twice, harmlessly
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, false>;
  if (dev < 16 && !attr_set[dev].load(std::memory_order_acquire)) {
    MT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 1 : 0;
  MT_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tp, tx, P));
  count_launch();
  return MT_OK;
}

// CTA-pair variant: clusters of two CTAs; `pairs` = number of clusters to launch.
template <bool A_MN, bool B_MN, int BN>
static int launch_tc_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tp,
                          const CUtensorMap& tx, const GemmParams& P, int pairs, cudaStream_t st) {
  using Cfg = GemmCfg<BN, true>;
  static std::atomic<bool> attr_set[16];   // per device; racing first calls set the same attribute twice, harmlessly
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, true>;
  if (dev < 16 && !attr_set[dev].load(std::memory_order_acquire)) {
    MT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 2 : 1;
  MT_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tp, tx, P));
  count_launch();
  return MT_OK;
}

// Number of two-CTA clusters of the pair kernel that are resident at once on
// this device (an SM without a free partner in its GPC hosts none).
static int resident_pairs() {
  static std::atomic<int> cached[16];      // per device; racing first calls compute the same number
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return sm_count() / 2;
  if (int c = cached[dev].load(std::memory_order_acquire)) return c;
  using Cfg = GemmCfg<256, true>;
  auto kern = gemm_tc_kernel<false, false, 256, true>;
  int n = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) == cudaSuccess) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(sm_count() & ~1));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { n = 0; cudaGetLastError(); }
  } else {
    cudaGetLastError();
  }
  if (n <= 0 || n > sm_count() / 2) n = sm_count() / 2;
  cached[dev].store(n, std::memory_order_release);
  return n;
}

static int g_tile_policy = 0;   // 0 = choose by estimated efficiency, 1 = single-CTA tiles only, 2 = CTA pairs whenever M > 128

int gemm_tc(const GemmArgs& g, cudaStream_t st) {
  const int sms = sm_count();
  const int tiles_m = (int)((g.M + BM - 1) / BM);
  const int kb_total = (int)((g.K + BK - 1) / BK);
  // Choose the tile (single CTA 128 x BN, or CTA pair 256 x BN), BN and the
  // split count by estimated efficiency: wave quantisation on the workers
  // available, padded rows / columns, and the measured advantage of the wider
  // and the paired tiles (less operand traffic per FLOP).
  int best_bn = 256, best_splits = 1;
  bool best_pair = false;
  double best = -1.0;
  const int pairs_avail = resident_pairs();
  for (int pair = 0; pair < 2; ++pair) {
    if (pair && (g_tile_policy == 1 || g.M <= BM)) continue;
    if (!pair && g_tile_policy == 2 && g.M > BM) continue;
    const int tm = pair ? 2 * BM : BM;
    const int workers = pair ? pairs_avail : sms;
    const int tiles_rows = (int)((g.M + tm - 1) / tm);
    for (int bn : {256, 128}) {
      const int tiles = tiles_rows * (int)((g.N + bn - 1) / bn);
      const int max_splits = g.accumulate == 2 ? 16 : 1;
      for (int s = 1; s <= max_splits; ++s) {
        if (s > 1 && kb_total / s < 8) break;
        const int per = (kb_total + s - 1) / s;
        if ((s - 1) * per >= kb_total) continue;  // an empty split
        const long long work = (long long)tiles * s;
        const long long waves = (work + workers - 1) / workers;
        double eff = (double)work / (double)(waves * workers);
        // a pair's workers are two SMs each; unpaired SMs idle
        if (pair) eff *= (double)(2 * workers) / (double)sms;
        // padded work in the last row / column tile counts against the larger tile
        eff *= (double)g.N / (double)(((g.N + bn - 1) / bn) * bn);
        eff *= (double)g.M / (double)((long long)tiles_rows * tm);
        if (bn == 128) eff *= 0.92;
        if (pair) eff *= 1.12;
        eff *= 1.0 - 0.01 * (s - 1);
        if (eff > best) { best = eff; best_bn = bn; best_splits = s; best_pair = pair != 0; }
      }
    }
  }
  const int bn = best_bn;
  const bool pair = best_pair;
  GemmParams P;
  P.C = g.C; P.preact = g.preact; P.bias = g.bias; P.aux = g.aux; P.aux_mode = g.aux_mode;
  P.M = g.M; P.N = g.N; P.K = g.K; P.ldc = g.ldc;
  P.out_dtype = g.out_dtype; P.in_bf16 = g.in_dtype == MT_BF16; P.act = g.act; P.accumulate = g.accumulate;
  P.alpha = g.alpha;
  const int out_vec = g.out_dtype == MT_F32 ? 4 : 8;
  P.vec_store = aligned16(g.C) && (!g.preact || aligned16(g.preact)) && g.ldc % out_vec == 0;
  P.tiles_m = pair ? (int)((g.M + 2 * BM - 1) / (2 * BM)) : tiles_m;
  P.tiles_n = (int)((g.N + bn - 1) / bn);
  P.splits = best_splits;
  P.kb_total = kb_total;
  P.kb_per_split = (kb_total + best_splits - 1) / best_splits;
  P.flag = device_flag_ptr();
  const long long total = (long long)P.tiles_m * P.tiles_n * P.splits;
  {
    // Which tiles run side by side decides what DRAM sees. Walking the rows first (the default),
    // the tiles in flight share one B panel and each streams its own A panel, so A is read once
    // per column tile; walking the columns first, the tiles of one row panel run together and
    // share A, while B is read once per group of tiles in flight. An operand that fits the L2
    // is read from DRAM once either way. The lm_head's dX and dW GEMMs (A = the 1.65 GB of
    // dlogits, three column tiles) read 5 GB of DRAM the first way and 1.7 GB the second.
    const double bytes_a = (double)g.M * (double)g.K * 2.0, bytes_b = (double)g.N * (double)g.K * 2.0;
    const double l2 = 64e6;
    const long long workers_now = pair ? pairs_avail : sms;
    const double groups = (double)(((long long)P.tiles_m * P.tiles_n + workers_now - 1) / workers_now);
    const double traffic_rows_first = bytes_b + bytes_a * (bytes_a > l2 ? P.tiles_n : 1);
    const double traffic_cols_first = bytes_a + bytes_b * (bytes_b > l2 ? groups : 1);
    P.n_fast = traffic_cols_first < traffic_rows_first ? 1 : 0;
  }
  const int grid = pair ? (int)(total < pairs_avail ? total : pairs_avail)   // clusters
                        : (int)(total < sms ? total : sms);                  // CTAs

  CUtensorMap ta, tb;
  int rc;
  const int bf = P.in_bf16;
  if (!g.trans_a) rc = make_tmap_2d(&ta, g.A, bf, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, BM);
  else rc = make_tmap_2d(&ta, g.A, bf, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, 64, BK);
  if (rc) return rc;
  if (g.trans_b) rc = make_tmap_2d(&tb, g.B, bf, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BK, (uint32_t)(pair ? bn / 2 : bn));
  else rc = make_tmap_2d(&tb, g.B, bf, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, 64, BK);
  if (rc) return rc;

  // Output through staged TMA stores when the tensor map can describe C (16-byte aligned base and
  // row pitch); read-modify-write of a half output keeps the direct path.
  CUtensorMap tcm, tpm, txm;
  memset(&tcm, 0, sizeof(tcm));
  memset(&tpm, 0, sizeof(tpm));
  memset(&txm, 0, sizeof(txm));
  const size_t osz = g.out_dtype == MT_F32 ? 4 : 2;
  P.tma_store = aligned16(g.C) && (g.ldc * osz) % 16 == 0 && (!g.preact || aligned16(g.preact)) &&
                (!g.aux || aligned16(g.aux)) && !(g.accumulate && g.out_dtype != MT_F32);
  if (P.tma_store) {
    const uint32_t cw = (uint32_t)(128 / osz);
    rc = make_tmap_2d_typed(&tcm, g.C, g.out_dtype, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldc, cw, 32);
    if (rc) return rc;
    if (g.preact) {
      rc = make_tmap_2d_typed(&tpm, g.preact, g.out_dtype, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldc, cw, 32);
      if (rc) return rc;
    }
    if (g.aux) {   // read slab by slab into the epilogue's staging buffers
      rc = make_tmap_2d_typed(&txm, g.aux, g.out_dtype, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldc, cw, 32);
      if (rc) return rc;
    }
  }
  // An aux operand combined into a half-precision output: one pipeline stage less, its shared
  // memory becomes a second staging buffer per warp, so both aux slabs of a tile are in flight
  // before its accumulator is ready (fc2 forward + residual: 75 -> 70 us). A second OUTPUT gains
  // nothing from it and loses the stage (fc1 forward with the stored derivative: 84 -> 98 us), so
  // that variant keeps the full pipeline.
  {
    const bool second_tensor = g.aux != nullptr && g.preact == nullptr && P.tma_store && g.out_dtype != MT_F32;
    const int smax = pair ? GemmCfg<256, true>::kStages : (bn == 256 ? GemmCfg<256, false>::kStages : GemmCfg<128, false>::kStages);
    const bool can = pair ? (bn == 256 ? GemmCfg<256, true>::kCanDoubleStage : GemmCfg<128, true>::kCanDoubleStage)
                          : (bn == 256 ? GemmCfg<256, false>::kCanDoubleStage : GemmCfg<128, false>::kCanDoubleStage);
    P.stages = (second_tensor && can && bn == 256) ? smax - 1 : smax;
  }
  ProfScope prof(PROF_GEMM, st, 2.0 * (double)g.M * (double)g.N * (double)g.K);
  const bool a_mn = g.trans_a != 0, b_mn = g.trans_b == 0;
#define MT_TC(AM, BMN)                                                                                              \
  (pair ? (bn == 256 ? launch_tc_pair<AM, BMN, 256>(ta, tb, tcm, tpm, txm, P, grid, st)                                  \
                     : launch_tc_pair<AM, BMN, 128>(ta, tb, tcm, tpm, txm, P, grid, st))                                 \
        : (bn == 256 ? launch_tc<AM, BMN, 256>(ta, tb, tcm, tpm, txm, P, grid, st)                                       \
                     : launch_tc<AM, BMN, 128>(ta, tb, tcm, tpm, txm, P, grid, st)))
  if (!a_mn && !b_mn) return MT_TC(false, false);
  if (!a_mn && b_mn) return MT_TC(false, true);
  if (a_mn && !b_mn) return MT_TC(true, false);
  return MT_TC(true, true);
#undef MT_TC
}

}  // namespace mt

using namespace mt;

static int g_force_simt = 0;

extern "C" {

int mt_gemm_force_simt(int on) { g_force_simt = on; return MT_OK; }

int mt_gemm_tile_policy(int policy) {
  MT_REQUIRE(policy >= 0 && policy <= 2, "gemm_tile_policy: 0 (automatic), 1 (single-CTA tiles) or 2 (CTA pairs)");
  mt::g_tile_policy = policy;
  return MT_OK;
}

int mt_gemm_ex(const void* A, const void* B, void* C, void* preact, const void* bias, const void* aux, int aux_mode,
               int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
               int in_dtype, int out_dtype, int act, float alpha, int accumulate, void* stream);

int mt_gemm(const void* A, const void* B, void* C, void* preact, const void* bias, int64_t M, int64_t N, int64_t K,
            int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b, int in_dtype, int out_dtype, int act,
            float alpha, int accumulate, void* stream) {
  return mt_gemm_ex(A, B, C, preact, bias, nullptr, 0, M, N, K, lda, ldb, ldc, trans_a, trans_b, in_dtype, out_dtype, act,
                    alpha, accumulate, stream);
}

int mt_gemm_ex(const void* A, const void* B, void* C, void* preact, const void* bias, const void* aux, int aux_mode,
               int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
               int in_dtype, int out_dtype, int act, float alpha, int accumulate, void* stream) {
  MT_REQUIRE((aux != nullptr) == (aux_mode != 0) && aux_mode >= 0 && aux_mode <= 6, "gemm: aux operand and aux_mode must be given together");
  MT_REQUIRE((act & ~0x1ff) == 0 && (act & 0xff) <= MT_ACT_RELU, "gemm: unknown activation");
  MT_REQUIRE(!(act & 0x100) || preact, "gemm: storing the activation's derivative needs the second output");
  MT_REQUIRE(!(aux_mode && accumulate == 2), "gemm: an aux operand cannot be combined with split-K accumulation");
  MT_REQUIRE(A && B && C && M >= 0 && N >= 0 && K >= 0, "gemm: bad arguments");
  MT_REQUIRE(lda >= (trans_a ? M : K) && ldb >= (trans_b ? K : N) && ldc >= N, "gemm: leading dimension too small");
  MT_REQUIRE(accumulate >= 0 && accumulate <= 2, "gemm: bad accumulate mode");
  MT_REQUIRE(accumulate != 2 || out_dtype == MT_F32, "gemm: atomic accumulation needs an fp32 output");
  MT_REQUIRE(accumulate != 2 || ((act & 0xff) == MT_ACT_NONE && !preact), "gemm: split-K accumulation cannot apply an activation");
  if (M == 0 || N == 0) return MT_OK;
  GemmArgs g{A, B, C, preact, bias, M, N, K, lda, ldb, ldc, trans_a, trans_b, in_dtype, out_dtype, act, alpha, accumulate};
  g.aux = aux;
  g.aux_mode = aux_mode;
  cudaStream_t st = as_stream(stream);
  if (!g_force_simt && gemm_tc_supported(g)) return gemm_tc(g, st);
  return gemm_simt(g, st);
}

}  // extern "C"
