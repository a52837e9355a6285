// Tensor-core attention for sm_100a, fp16/bf16, causal or full.
//
// Forward: persistent, as many CTAs as are resident at once (two per SM at head_dim 64, one at
// 128), 320 threads each; a tile is one (batch, head, block of 128 query rows), and a CTA takes
// the next tile nobody has taken yet from a global counter (order: heads in groups that keep their
// K/V in L2, heaviest query blocks first).
//   warp 8    TMA producer, which also takes the tiles and hands them to the other warps through
//             a two-slot ring: a tile's Q (as soon as the previous tile's last score MMA has read
//             the Q buffer), then K and V blocks of 128 keys (two stages each, K one block ahead
//             of V, the rings running on across tiles), 128-byte swizzled, read in place
//             through 4-D tensor maps {head_dim, seq, head, batch} (any batch/head/row strides);
//   warp 9    MMA issuer: S = Q K^T (128x128xD) into tensor memory - issued for
//             block j+1 (or the next tile's first block) as soon as the softmax warps have
//             copied S_j to registers - then O += P V (128xDx128) with P read from tensor memory
//             and the accumulator kept in tensor memory;
//   warps 0-7 softmax: warps w and w+4 share the 32 query rows of TMEM lane quarter
//             w&3 and take 64 score columns each. A thread reads its half row once,
//             agrees with its partner on the row maximum through shared memory,
//             computes exp2 in the scaled log2 domain and writes P back to tensor
//             memory as packed half pairs. The running maximum only moves (and O is
//             only rescaled in tensor memory) when it grew by more than 2^8. On the
//             causal diagonal, 32-column groups that no row of the warp keeps are
//             skipped altogether. After a tile's last block the same warps scale O by 1/l and
//             send it out through staging buffers of their own (TMA store), while the producer
//             and the MMA warp are already on the next tile.
// head_dim 64 uses 99 KB of shared memory, 256 TMEM columns and 96 registers per thread, so two
// CTAs share an SM.
//
// Roofline: tensor pipe, 4*B*H*S^2*D FLOP (half of that when causal); at
// head_dim 64 the exp2 (MUFU, 16 per clock per SM) rate caps the kernel at half
// of the MMA peak.
#include "common.cuh"
#include "attention.cuh"
#include "sm100.cuh"
#include "attention_tc.cuh"
#include "tempbuf.cuh"

namespace mt {

using namespace sm100;

constexpr int kSoftmaxWarps = 8;                       // two per TMEM lane quarter: half a score row each
constexpr int kAttnThreads = 32 * kSoftmaxWarps + 64;  // + TMA producer warp + MMA issuer warp

template <int D> struct FwdCfg {
  static constexpr int kChunks = D / 64;               // 64-wide (128-byte) slices of head_dim
  static constexpr int kTile = 128 * D * 2;            // bytes of one 128-row Q/K/V block
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kTile;                  // two stages
  static constexpr int kOffV = kOffK + 2 * kTile;      // two stages
  static constexpr int kOffBar = kOffV + 2 * kTile;
  static constexpr int kOffX = kOffBar + 256;          // row statistics exchanged between the two half-row threads
  // No slack for aligning the base: the dynamic shared-memory window of a kernel
  // without static shared memory starts 1024-byte aligned (checked at entry).
  // O leaves through a staging area of its own (the K/V buffers already hold the next tile's
  // blocks by then): one 32-row x 128-byte buffer per storing warp
  static constexpr int kOffStage = (kOffX + 2 * 2 * 128 * 4 + 1023) / 1024 * 1024;   // swizzled: 1024-byte aligned
  static constexpr int kStageWarps = D == 64 ? 4 : 8;
  static constexpr int kSmem = kOffStage + kStageWarps * 4096;
  // Tensor memory: S fp32 [0,128), O fp32 [128,128+D), P as packed half pairs [128+D, 192+D)
  static constexpr int kTmemP = 128 + D;
  static constexpr int kTmemCols = D == 64 ? 256 : 512;
};


struct AttnFwdParams {
  float* lse;
  MapPos pq, pk, pv, po;
  int B, H, S, nqb, causal, is_bf16;
  int group;            // query heads per key/value head
  int gh;               // (batch, head) pairs per group of the CTA order
  float scale_log2;
  int* flag;
  int* tile_counter;    // zero at launch: the next tile nobody has taken yet
};


template <int D, typename T>
__global__ void __launch_bounds__(kAttnThreads, D == 64 ? 2 : 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                   const AttnFwdParams P) {
  using Cfg = FwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {   // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0 && P.flag) atomicMax(P.flag, 101);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + Cfg::kOffBar;
  // barrier slots
  const uint32_t bar_q = bar0, bar_kfull0 = bar0 + 8, bar_kempty0 = bar0 + 24, bar_vfull0 = bar0 + 40,
                 bar_vempty0 = bar0 + 56, bar_s = bar0 + 72, bar_p = bar0 + 80, bar_o = bar0 + 88,
                 bar_sfree = bar0 + 96, bar_pair0 = bar0 + 104,   // four pair barriers: +104 .. +135
                 bar_qfree = bar0 + 136, bar_tfull0 = bar0 + 160, bar_tempty0 = bar0 + 176;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + Cfg::kOffBar + 144);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + Cfg::kOffBar + 148);
  float* xchg = reinterpret_cast<float*>(base_ptr + Cfg::kOffX);   // [2 buffers][2 halves][128 rows]
  volatile int* tile_ring = reinterpret_cast<volatile int*>(base_ptr + Cfg::kOffBar + 152);   // two slots

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh_count = P.B * P.H;
  const int n_tiles = P.nqb * bh_count;
  const int n_kv_total = (P.S + 127) / 128;
  // The kernel is persistent: as many CTAs as are resident at once, each taking the next tile
  // nobody has taken yet from a global counter (so a CTA that starts late, or shares its SM with
  // another kernel, simply takes fewer). Tile order (decode_tile): heads in groups of P.gh, within
  // a group the heaviest (last) query blocks first, so that the CTAs working at one time read the K
  // and V of a few heads only and the light tiles fill the end. The producer thread takes the
  // tiles and hands each to the MMA and softmax warps through a two-slot ring in shared memory
  // (-1 = no more). Every role keeps a running block count, from which ring stages and barrier
  // parities follow; barriers and tensor memory are set up once, and the next tile's Q, K and
  // first scores are under way while this tile's O is still being written out.
  struct Tile { int qb, b, h, hk, n_kv; };
  auto decode = [&](int tile, Tile& t) {
    int slot, bh;
    decode_tile(tile, P.nqb, bh_count, P.gh, slot, bh);
    t.qb = P.nqb - 1 - slot;
    t.b = bh / P.H; t.h = bh % P.H;
    t.hk = t.h / P.group;                                // key/value head of this query head
    t.n_kv = P.causal ? min(t.qb + 1, n_kv_total) : n_kv_total;
  };

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kfull0, 1); mbar_init(bar_kfull0 + 8, 1);
    mbar_init(bar_kempty0, 1); mbar_init(bar_kempty0 + 8, 1);
    mbar_init(bar_vfull0, 1); mbar_init(bar_vfull0 + 8, 1);
    mbar_init(bar_vempty0, 1); mbar_init(bar_vempty0 + 8, 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 32 * kSoftmaxWarps); mbar_init(bar_o, 1); mbar_init(bar_sfree, kSoftmaxWarps);
    mbar_init(bar_qfree, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull0 + 8 * i, 1); mbar_init(bar_tempty0 + 8 * i, 1 + kSoftmaxWarps); }
    for (int i = 0; i < 4; ++i) mbar_init(bar_pair0 + 8 * i, 2);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kSoftmaxWarps + 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128, tmem_p = tmem_base + Cfg::kTmemP;

  if (warp == kSoftmaxWarps) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
      int gb = 0;                                        // blocks before this tile (running count)
      bool okp = true;
      Tile t;
      int tile_ahead = atomicAdd(P.tile_counter, 1);   // read one tile ahead: the round trip runs under the loads before
      for (int tn = 0; okp; ++tn) {
        // take the next tile and publish it (slot tn & 1 is free once the consumers have read tile tn - 2)
        if (!mbar_wait(bar_tempty0 + 8 * (tn & 1), ((tn >> 1) & 1) ^ 1u, abort_flag)) break;
        int tile = tile_ahead;
        if (tile < n_tiles) tile_ahead = atomicAdd(P.tile_counter, 1);
        if (tile >= n_tiles) tile = -1;
        tile_ring[tn & 1] = tile;
        mbar_arrive(bar_tfull0 + 8 * (tn & 1));
        if (tile < 0) break;
        decode(tile, t);
        // Q is read by every score MMA of a tile: the buffer is free once the previous tile's last one is done
        if (tn > 0 && !mbar_wait(bar_qfree, (tn - 1) & 1, abort_flag)) break;
        mbar_expect_tx(bar_q, Cfg::kTile);
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
          load_rows(base + Cfg::kOffQ + dc * 16384, &tmQ, bar_q, P.pq, dc * 64, t.qb * 128, t.h, t.b);
        // K runs one block ahead of V: the scores of block j+1 are issued while the
        // softmax of block j is still running, so K_{j+1} must already be on its way.
        auto load_k = [&](int j) -> bool {
          const int g = gb + j, st = g & 1;
          if (!mbar_wait(bar_kempty0 + 8 * st, ((g >> 1) & 1) ^ 1u, abort_flag)) return false;
          mbar_expect_tx(bar_kfull0 + 8 * st, Cfg::kTile);
#pragma unroll
          for (int dc = 0; dc < Cfg::kChunks; ++dc)
            load_rows(base + Cfg::kOffK + st * Cfg::kTile + dc * 16384, &tmK, bar_kfull0 + 8 * st, P.pk, dc * 64, j * 128, t.hk, t.b);
          return true;
        };
        okp = load_k(0);
        for (int j = 0; j < t.n_kv && okp; ++j) {
          if (j + 1 < t.n_kv && !load_k(j + 1)) { okp = false; break; }
          const int g = gb + j, st = g & 1;
          if (!mbar_wait(bar_vempty0 + 8 * st, ((g >> 1) & 1) ^ 1u, abort_flag)) { okp = false; break; }
          mbar_expect_tx(bar_vfull0 + 8 * st, Cfg::kTile);
#pragma unroll
          for (int dc = 0; dc < Cfg::kChunks; ++dc)
            load_rows(base + Cfg::kOffV + st * Cfg::kTile + dc * 16384, &tmV, bar_vfull0 + 8 * st, P.pv, dc * 64, j * 128, t.hk, t.b);
        }
        gb += t.n_kv;
      }
    }
  } else if (warp == kSoftmaxWarps + 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = idesc_f16(P.is_bf16, 0, 0, 128, 128);
      const uint32_t idesc_o = idesc_f16(P.is_bf16, 0, 1, 128, D);
      // every shared-memory descriptor is built once, ahead of the loop: after a barrier wait the
      // thread issues MMAs and nothing else
      uint64_t dq[4 * Cfg::kChunks], dk[2][4 * Cfg::kChunks], dv[2][8];
#pragma unroll
      for (int dc = 0; dc < Cfg::kChunks; ++dc)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          dq[dc * 4 + k] = smem_desc_sw128(base + Cfg::kOffQ + dc * 16384 + k * 32, 16, 1024);
#pragma unroll
          for (int st = 0; st < 2; ++st)
            dk[st][dc * 4 + k] = smem_desc_sw128(base + Cfg::kOffK + st * Cfg::kTile + dc * 16384 + k * 32, 16, 1024);
        }
#pragma unroll
      for (int st = 0; st < 2; ++st)
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          dv[st][ks] = smem_desc_sw128(base + Cfg::kOffV + st * Cfg::kTile + ks * 2048, 16384, 1024);
      // scores of running block g (its K is in ring stage g & 1)
      auto issue_s = [&](int g) -> bool {
        const int st = g & 1;
        if (!mbar_wait(bar_kfull0 + 8 * st, (g >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        if (st == 0) {
          umma_f16_x4(tmem_s, dq, dk[0], idesc_s, 0u);
          if (Cfg::kChunks == 2) umma_f16_x4(tmem_s, dq + 4 * (Cfg::kChunks - 1), dk[0] + 4 * (Cfg::kChunks - 1), idesc_s, 1u);
        } else {
          umma_f16_x4(tmem_s, dq, dk[1], idesc_s, 0u);
          if (Cfg::kChunks == 2) umma_f16_x4(tmem_s, dq + 4 * (Cfg::kChunks - 1), dk[1] + 4 * (Cfg::kChunks - 1), idesc_s, 1u);
        }
        umma_commit(bar_kempty0 + 8 * st);
        umma_commit(bar_s);
        return true;
      };
      int gb = 0;
      bool ok = true;
      Tile t;
      for (int tn = 0; ok; ++tn) {
        if (!mbar_wait(bar_tfull0 + 8 * (tn & 1), (tn >> 1) & 1, abort_flag)) break;
        const int tile = tile_ring[tn & 1];
        mbar_arrive(bar_tempty0 + 8 * (tn & 1));
        if (tile < 0) break;
        decode(tile, t);
        if (!mbar_wait(bar_q, tn & 1, abort_flag)) break;
        // the softmax warps have copied the previous tile's last scores to registers
        if (gb > 0 && !mbar_wait(bar_sfree, (gb - 1) & 1, abort_flag)) break;
        tc_fence_after();
        if (!issue_s(gb)) break;
        if (t.n_kv == 1) umma_commit(bar_qfree);        // the tile's last score MMA: Q may be replaced
        for (int j = 0; j < t.n_kv; ++j) {
          const int g = gb + j;
          if (j + 1 < t.n_kv) {
            // The softmax warps hold S_j in registers: the next block's scores are
            // computed while they work on this one.
            if (!mbar_wait(bar_sfree, g & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (!issue_s(g + 1)) { ok = false; break; }
            if (j + 2 == t.n_kv) umma_commit(bar_qfree);
          }
          if (!mbar_wait(bar_p, g & 1, abort_flag)) { ok = false; break; }      // P_j written
          tc_fence_after();
          if (!mbar_wait(bar_vfull0 + 8 * (g & 1), (g >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // A = P straight from tensor memory: 16 keys = 8 columns of packed half pairs per step
          if (g & 1) umma_f16_ts_x8(tmem_o, tmem_p, dv[1], idesc_o, j > 0 ? 1u : 0u);
          else umma_f16_ts_x8(tmem_o, tmem_p, dv[0], idesc_o, j > 0 ? 1u : 0u);
          umma_commit(bar_vempty0 + 8 * (g & 1));
          umma_commit(bar_o);
        }
        gb += t.n_kv;
      }
    }
  } else {
    // ------------------------------------------------------------- softmax --
    // Warps w and w+4 share the 32 query rows of TMEM lane quarter w&3; warp w
    // takes columns [0,64) of each score block, warp w+4 columns [64,128). The two
    // threads of a row agree on the running maximum through shared memory; their
    // partial row sums meet once, after the last block.
    const int qtr = warp & 3, hf = warp >> 2;
    const int row = qtr * 32 + lane;                  // query row within the block = TMEM lane
    const uint32_t lane_addr = (uint32_t)(qtr * 32) << 16;
    const uint32_t bar_pair = bar_pair0 + 8 * qtr;
    bool ok = true;
    int gb = 0, xu = 0;                               // running counts of blocks and of pair exchanges
    Tile t;
    // Both threads of a row see the same values, so `ok` and the rescale decision agree.
    auto pair_exchange = [&](int use, float mine, float& other) -> bool {
      float* slot = xchg + (use & 1) * 256;
      slot[hf * 128 + row] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pair);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_pair, use & 1, abort_flag))) return false;
      other = slot[(hf ^ 1) * 128 + row];
      return true;
    };
    for (int tn = 0; ok; ++tn) {
    if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull0 + 8 * (tn & 1), (tn >> 1) & 1, abort_flag))) { ok = false; break; }
    const int tile = tile_ring[tn & 1];
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_tempty0 + 8 * (tn & 1));
    if (tile < 0) break;
    decode(tile, t);
    const int qb = t.qb, b = t.b, h = t.h, n_kv = t.n_kv, bh = b * P.H + h;
    const int q_glob = qb * 128 + row;
    float m_used = -INFINITY, l = 0.f;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int g = gb + j;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, g & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      // Valid columns of this block for this row: c < lim. Whole 32-column groups
      // past every row of the warp are skipped (no max, no exp2, zeros written);
      // groups that every row keeps entirely need no per-element test.
      const int nvalid = min(128, P.S - j * 128);
      const bool diag = P.causal && j == qb;
      const int lim = (diag ? min(nvalid, row + 1) : nvalid) - hf * 64;             // in this thread's columns
      const int lim_max = (diag ? min(nvalid, qtr * 32 + 32) : nvalid) - hf * 64;   // warp-uniform
      const int lim_min = (diag ? min(nvalid, qtr * 32 + 1) : nvalid) - hf * 64;    // warp-uniform
      uint32_t r[64];
      tmem_ld32(tmem_s + lane_addr + hf * 64, r);
      tmem_ld32(tmem_s + lane_addr + hf * 64 + 32, r + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfree);          // S may be overwritten by the next block's scores
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (g * 32 < lim_max) {
          if ((g + 1) * 32 > lim_min) {
#pragma unroll
            for (int e = g * 32; e < g * 32 + 32; ++e)
              if (e >= lim) r[e] = 0xff800000u;   // -inf
          }
#pragma unroll
          for (int e = g * 32; e < g * 32 + 32; e += 8) {
            mx0 = max3(mx0, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
            mx1 = max3(mx1, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
            mx2 = max3(mx2, __uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
            mx3 = max3(mx3, __uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
          }
        }
      }
      const float mx_half = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2;
      float mx_other;
      if (!pair_exchange(xu++, mx_half, mx_other)) { ok = false; break; }
      const float m_new = fmaxf(m_used, fmaxf(mx_half, mx_other));
      const bool resc = (m_new > m_used) && (m_used == -INFINITY || m_new - m_used > 8.f);
      float alpha = 1.f;
      if (resc) {
        alpha = m_used == -INFINITY ? 0.f : ex2_approx(m_used - m_new);
        l *= alpha;
        m_used = m_new;
      }
      if (j > 0) {   // P buffer free and O stable once the previous P V has completed
        if (!__all_sync(0xffffffffu, mbar_wait(bar_o, (g - 1) & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
      }
      const float msub = m_used == -INFINITY ? 0.f : m_used;   // a fully masked row has only -inf entries
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t pk[16];                            // 32 probabilities as half pairs
        if (g * 32 < lim_max) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(r[g * 32 + 2 * e]), P.scale_log2, -msub));
            const float p1 = ex2_approx(fmaf(__uint_as_float(r[g * 32 + 2 * e + 1]), P.scale_log2, -msub));
            l0 += p0;
            l1 += p1;
            pk[e] = pack2<T>(p0, p1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
        }
        tmem_st16(tmem_p + lane_addr + hf * 32 + g * 16, pk);   // P never touches shared memory
      }
      l += l0 + l1;
      if (j > 0 && __any_sync(0xffffffffu, resc)) {   // rare: the running maximum moved by more than 2^8
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {            // this thread's half of the O columns
          uint32_t t[32];
          const uint32_t addr = tmem_o + lane_addr + hf * (D / 2) + c * 32;
          tmem_ld32(addr, t);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
          tmem_st32(addr, t);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (!ok) break;
    float l_other = 0.f;
    ok = pair_exchange(xu++, l, l_other);
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (gb + n_kv - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after();
      const float l_row = l + l_other;
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      // O leaves through shared memory: one warp per 32 rows x 64 columns stages 128-byte rows
      // (swizzled) in its own buffer and one lane issues a TMA store, which clips rows past the
      // sequence end. At head_dim 64 the warps of column half 1 have nothing to store.
      if (D == 128 || hf == 0) {
        const int dc = D == 128 ? hf : 0;
        uint8_t* stage = base_ptr + Cfg::kOffStage + warp * 4096;
        uint32_t r[64];
        tmem_ld32(tmem_o + lane_addr + dc * 64, r);
        tmem_ld32(tmem_o + lane_addr + dc * 64 + 32, r + 32);
        tmem_ld_wait();
        if (lane == 0) bulk_wait_read<0>();   // the previous tile's store has read the buffer
        __syncwarp();
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          uint4 v;
          v.x = pack2<T>(__uint_as_float(r[c16 * 8 + 0]) * inv, __uint_as_float(r[c16 * 8 + 1]) * inv);
          v.y = pack2<T>(__uint_as_float(r[c16 * 8 + 2]) * inv, __uint_as_float(r[c16 * 8 + 3]) * inv);
          v.z = pack2<T>(__uint_as_float(r[c16 * 8 + 4]) * inv, __uint_as_float(r[c16 * 8 + 5]) * inv);
          v.w = pack2<T>(__uint_as_float(r[c16 * 8 + 6]) * inv, __uint_as_float(r[c16 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((c16 ^ (lane & 7)) << 4)) = v;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          store_rows(&tmO, smem_u32(stage), P.po, dc * 64, qb * 128 + qtr * 32, h, b);
          bulk_commit();
        }
        __syncwarp();
      }
      if (hf == 0 && q_glob < P.S) P.lse[(int64_t)bh * P.S + q_glob] = (m_used + log2f(l_row)) * kLn2F;
    }
    gb += n_kv;
    }   // tiles
    if (lane == 0) bulk_wait_all<0>();   // the stores must be done with shared memory before the CTA exits
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && P.flag) atomicMax(P.flag, 101);
  if (warp == kSoftmaxWarps + 1) {
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
  CUtensorMap tq, tk, tv, to;
  int rc;
  AttnFwdParams P;
  if ((rc = make_qkv_map(&to, &P.po, a.o_out, bf, a.so, a.batch, a.heads, a.seq, D, 32))) return rc;
  if ((rc = make_qkv_map(&tq, &P.pq, a.q, bf, a.sq, a.batch, a.heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tk, &P.pk, a.k, bf, a.sk, a.batch, a.kv_heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tv, &P.pv, a.v, bf, a.sv, a.batch, a.kv_heads, a.seq, D))) return rc;
  P.lse = a.lse;
  P.group = (int)(a.heads / a.kv_heads);
  P.B = (int)a.batch; P.H = (int)a.heads; P.S = (int)a.seq; P.nqb = (int)((a.seq + 127) / 128);
  P.causal = a.causal; P.is_bf16 = bf; P.scale_log2 = a.scale * kLog2eF; P.flag = device_flag_ptr();
  // Heads per group of the CTA order: all of them while every head's K and V fit in L2 together,
  // else about as many as give each resident CTA (two per SM at head_dim 64, one at 128) two tiles.
  P.gh = (int)(a.batch * a.heads);
  if ((double)a.batch * a.kv_heads * a.seq * D * 4.0 > 64e6 && P.nqb > 1) {
    const int resident = sm_count() * (D == 64 ? 2 : 1);
    const int gh = 2 * resident / P.nqb > 1 ? 2 * resident / P.nqb : 1;
    if (gh < P.gh) P.gh = gh;
  }
  auto kern = attn_fwd_tc_kernel<D, T>;
  MT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const int64_t n_tiles = (int64_t)P.nqb * P.B * P.H;
  const int64_t resident = (int64_t)sm_count() * (D == 64 ? 2 : 1);
  const int64_t grid_i = n_tiles < resident ? n_tiles : resident;   // persistent
  TempBuf counter(sizeof(int), st);
  if (!counter.ok()) return MT_ERR_CUDA;
  MT_CHECK_CUDA(cudaMemsetAsync(counter.ptr, 0, sizeof(int), st));
  P.tile_counter = (int*)counter.ptr;
  const unsigned grid = (unsigned)grid_i;
  kern<<<grid, kAttnThreads, Cfg::kSmem, st>>>(tq, tk, tv, to, P);
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
