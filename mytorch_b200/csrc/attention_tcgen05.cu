// Tensor-core attention for sm_100a, fp16/bf16, causal or full.
//
// Forward: one CTA per (batch, head, block of 128 query rows).
//   warp 4    TMA producer: Q once, then K (two stages) and V (one stage) blocks
//             of 128 keys, 128-byte swizzled, read in place through 4-D tensor
//             maps {head_dim, seq, head, batch} (any batch/head/row strides);
//   warp 5    MMA issuer: S = Q K^T (128x128xD) into tensor memory, then
//             O += P V (128xDx128) with the accumulator kept in tensor memory;
//   warps 0-3 softmax: thread = query row = TMEM lane. Pass 1 reads S for the row
//             maximum, pass 2 re-reads it, computes exp2 in the scaled log2 domain,
//             accumulates the row sum and writes P (half) to shared memory in the
//             swizzled K-major layout the second MMA consumes. The running maximum
//             only moves (and O is only rescaled in tensor memory) when it grew by
//             more than 2^8, so most iterations skip the correction.
// head_dim 64 uses 97 KB of shared memory and 256 TMEM columns: two CTAs per SM
// overlap one CTA's softmax with the other's MMAs.
//
// Roofline: tensor pipe, 4*B*H*S^2*D FLOP (half of that when causal); at
// head_dim 64 the exp2 (MUFU) rate caps the kernel near half of the MMA peak.
#include "common.cuh"
#include "attention.cuh"
#include "sm100.cuh"
#include "attention_tc.cuh"

namespace mt {

using namespace sm100;

constexpr int kAttnThreads = 192;

template <int D> struct FwdCfg {
  static constexpr int kChunks = D / 64;               // 64-wide (128-byte) slices of head_dim
  static constexpr int kTile = 128 * D * 2;            // bytes of one 128-row Q/K/V block
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kTile;                  // two stages
  static constexpr int kOffV = kOffK + 2 * kTile;      // one stage
  static constexpr int kOffP = kOffV + kTile;          // 128 x 128 half
  static constexpr int kOffBar = kOffP + 128 * 128 * 2;
  static constexpr int kSmem = kOffBar + 256 + 1024;
  static constexpr int kTmemCols = 256;                // S: [0,128), O: [128,128+D)
};


struct AttnFwdParams {
  void* o; float* lse;
  MapPos pq, pk, pv;
  mt_strides3 so;
  int B, H, S, nqb, causal, is_bf16;
  float scale_log2;
  int* flag;
};


template <int D, typename T>
__global__ void __launch_bounds__(kAttnThreads, D == 64 ? 2 : 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnFwdParams P) {
  using Cfg = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar0 = base + Cfg::kOffBar;
  // barrier slots
  const uint32_t bar_q = bar0, bar_kfull0 = bar0 + 8, bar_kempty0 = bar0 + 24, bar_vfull = bar0 + 40,
                 bar_vempty = bar0 + 48, bar_s = bar0 + 56, bar_p = bar0 + 64, bar_o = bar0 + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + Cfg::kOffBar + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + Cfg::kOffBar + 100);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh_count = P.B * P.H;
  const int qb = P.nqb - 1 - (int)(blockIdx.x / bh_count);   // heaviest (last) query blocks first
  const int bh = blockIdx.x % bh_count;
  const int b = bh / P.H, h = bh % P.H;
  const int n_kv_total = (P.S + 127) / 128;
  const int n_kv = P.causal ? min(qb + 1, n_kv_total) : n_kv_total;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kfull0, 1); mbar_init(bar_kfull0 + 8, 1);
    mbar_init(bar_kempty0, 1); mbar_init(bar_kempty0 + 8, 1);
    mbar_init(bar_vfull, 1); mbar_init(bar_vempty, 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 128); mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 4) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
      mbar_expect_tx(bar_q, Cfg::kTile);
#pragma unroll
      for (int dc = 0; dc < Cfg::kChunks; ++dc)
        load_rows(base + Cfg::kOffQ + dc * 16384, &tmQ, bar_q, P.pq, dc * 64, qb * 128, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar_kempty0 + 8 * st, ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        mbar_expect_tx(bar_kfull0 + 8 * st, Cfg::kTile);
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
          load_rows(base + Cfg::kOffK + st * Cfg::kTile + dc * 16384, &tmK, bar_kfull0 + 8 * st, P.pk, dc * 64, j * 128, h, b);
        if (!mbar_wait(bar_vempty, (j & 1) ^ 1u, abort_flag)) break;
        mbar_expect_tx(bar_vfull, Cfg::kTile);
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
          load_rows(base + Cfg::kOffV + dc * 16384, &tmV, bar_vfull, P.pv, dc * 64, j * 128, h, b);
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = idesc_f16(P.is_bf16, 0, 0, 128, 128);
      const uint32_t idesc_o = idesc_f16(P.is_bf16, 0, 1, 128, D);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(bar_kfull0 + 8 * st, (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sq = base + Cfg::kOffQ, sk = base + Cfg::kOffK + st * Cfg::kTile;
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_s, smem_desc_sw128(sq + dc * 16384 + k * 32, 16, 1024),
                     smem_desc_sw128(sk + dc * 16384 + k * 32, 16, 1024), idesc_s, (dc | k) ? 1u : 0u);
        umma_commit(bar_kempty0 + 8 * st);
        umma_commit(bar_s);
        return true;
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(bar_p, j & 1, abort_flag)) break;      // P_j written, S_j consumed
        tc_fence_after();
        if (j + 1 < n_kv && !issue_s(j + 1)) break;
        if (!mbar_wait(bar_vfull, j & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t sp = base + Cfg::kOffP, sv = base + Cfg::kOffV;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16(tmem_o, smem_desc_sw128(sp + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
                   smem_desc_sw128(sv + ks * 2048, 16384, 1024), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(bar_vempty);
        umma_commit(bar_o);
      }
    }
  } else {
    // ------------------------------------------------------------- softmax --
    const int row = threadIdx.x;                      // 0..127 = TMEM lane
    const int q_glob = qb * 128 + row;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    uint8_t* p_smem = base_ptr + Cfg::kOffP;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, j & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (P.causal && j == qb) || ((j + 1) * 128 > P.S);
      // the whole row of S (128 fp32) in registers: four loads in flight, one wait
      uint32_t r[128];
      tmem_ld32(tmem_s + lane_addr, r);
      tmem_ld32(tmem_s + lane_addr + 32, r + 32);
      tmem_ld32(tmem_s + lane_addr + 64, r + 64);
      tmem_ld32(tmem_s + lane_addr + 96, r + 96);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 128; ++e) {
          const int col = j * 128 + e;
          if (col >= P.S || (P.causal && col > q_glob)) r[e] = 0xff800000u;   // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 128; e += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(r[e]));
        mx1 = fmaxf(mx1, __uint_as_float(r[e + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(r[e + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(r[e + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool resc = (m_new > m_used) && (m_used == -INFINITY || m_new - m_used > 8.f);
      float alpha = 1.f;
      if (resc) {
        alpha = m_used == -INFINITY ? 0.f : ex2_approx(m_used - m_new);
        l *= alpha;
        m_used = m_new;
      }
      if (j > 0) {   // P buffer free and O stable once the previous P V has completed
        if (!__all_sync(0xffffffffu, mbar_wait(bar_o, (j - 1) & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
      }
      const float msub = m_used == -INFINITY ? 0.f : m_used;   // a fully masked row has only -inf entries
      float l0 = 0.f, l1 = 0.f;
      uint8_t* prow = p_smem + row * 128;
#pragma unroll
      for (int c16 = 0; c16 < 16; ++c16) {          // 16-byte chunks of 8 columns
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(r[c16 * 8 + 2 * e]), P.scale_log2, -msub));
          const float p1 = ex2_approx(fmaf(__uint_as_float(r[c16 * 8 + 2 * e + 1]), P.scale_log2, -msub));
          l0 += p0;
          l1 += p1;
          pk[e] = pack2<T>(p0, p1);
        }
        // K-slice c16>>3 (64 columns each), chunk c16&7 within the 128-byte row, swizzled
        *reinterpret_cast<uint4*>(prow + (c16 >> 3) * 16384 + (((c16 & 7) ^ (row & 7)) << 4)) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l += l0 + l1;
      if (j > 0 && __any_sync(0xffffffffu, resc)) {   // rare: the running maximum moved by more than 2^8
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t t[32];
          tmem_ld32(tmem_o + lane_addr + c * 32, t);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
          tmem_st32(tmem_o + lane_addr + c * 32, t);
        }
        tmem_st_wait();
      }
      fence_proxy_async();      // generic-proxy writes of P -> visible to the tensor core
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok && __all_sync(0xffffffffu, mbar_wait(bar_o, (n_kv - 1) & 1, abort_flag))) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = reinterpret_cast<T*>(P.o) + (int64_t)b * P.so.b + (int64_t)h * P.so.h + (int64_t)q_glob * P.so.s;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_addr + c * 32, r);
        tmem_ld_wait();
        if (q_glob < P.S) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack2<T>(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
            v.y = pack2<T>(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
            v.z = pack2<T>(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
            v.w = pack2<T>(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
          }
        }
      }
      if (q_glob < P.S) P.lse[(int64_t)bh * P.S + q_glob] = (m_used + log2f(l)) * kLn2F;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && P.flag) atomicMax(P.flag, 101);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


bool attn_tc_supported(const AttnArgs& a, bool backward) {
  if (backward && !attn_bwd_tc_supported(a)) return false;
  if (a.dtype != MT_F16 && a.dtype != MT_BF16) return false;
  if (a.head_dim != 64 && a.head_dim != 128) return false;
  if (a.seq < 1 || a.batch < 1) return false;
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.o_out)) return false;
  if (!strides_ok(a.sq) || !strides_ok(a.sk) || !strides_ok(a.sv) || !strides_ok(a.so)) return false;
  if (a.batch * a.heads * ((a.seq + 127) / 128) >= (1ll << 31)) return false;
  return true;
}


template <int D, typename T>
static int launch_fwd(const AttnArgs& a, cudaStream_t st) {
  using Cfg = FwdCfg<D>;
  const int bf = a.dtype == MT_BF16;
  CUtensorMap tq, tk, tv;
  int rc;
  AttnFwdParams P;
  if ((rc = make_qkv_map(&tq, &P.pq, a.q, bf, a.sq, a.batch, a.heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tk, &P.pk, a.k, bf, a.sk, a.batch, a.heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tv, &P.pv, a.v, bf, a.sv, a.batch, a.heads, a.seq, D))) return rc;
  P.o = a.o_out; P.lse = a.lse; P.so = a.so;
  P.B = (int)a.batch; P.H = (int)a.heads; P.S = (int)a.seq; P.nqb = (int)((a.seq + 127) / 128);
  P.causal = a.causal; P.is_bf16 = bf; P.scale_log2 = a.scale * kLog2eF; P.flag = device_flag_ptr();
  auto kern = attn_fwd_tc_kernel<D, T>;
  MT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const unsigned grid = (unsigned)(P.nqb * P.B * P.H);
  kern<<<grid, kAttnThreads, Cfg::kSmem, st>>>(tq, tk, tv, P);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int attn_fwd_tc(const AttnArgs& a, cudaStream_t st) {
  if (a.head_dim == 64) {
    if (a.dtype == MT_F16) return launch_fwd<64, __half>(a, st);
    return launch_fwd<64, __nv_bfloat16>(a, st);
  }
  if (a.dtype == MT_F16) return launch_fwd<128, __half>(a, st);
  return launch_fwd<128, __nv_bfloat16>(a, st);
}


}  // namespace mt
