// Tensor-core attention backward for sm_100a, fp16/bf16, head_dim 64 or 128.
//
// A tile is one (batch, head, block of 128 key/value rows): the CTA that owns it walks the query
// blocks that attend to it (all of them, or those at/after the diagonal when causal). The kernel
// is persistent: one CTA per SM takes the next tile nobody has taken yet from a global counter
// (heaviest first; the producer thread fetches and hands the tile to the other roles through a
// two-slot ring in shared memory), tensor memory and barriers are set up once, and the roles
// run ahead across tile boundaries - the producer loads the next tile's K/V as soon as the last
// MMA reading the current ones has completed and keeps the Q/dO ring filled, the MMA warp issues
// the next tile's first S^T/dP^T while the elementwise warps still flush dQ and drain dK/dV of
// the current one.
// Per query block, five tcgen05 MMAs with accumulators in tensor memory:
//   S^T  = K Q^T            dP^T = V dO^T          (both 128x128xD, recomputed)
//   dV  += P^T dO           dK  += dS^T Q          (128xDx128, accumulated)
//   dQ   = dS K             (128xDx128, added to a fp32 buffer with TMA reduce-add,
//                            since every key block contributes to every dQ row)
// Warp roles: one warp TMA producer (K, V once per tile; Q, dO and the block's row statistics per
// query block, read in place through 4-D strided tensor maps), one warp MMA issuer, sixteen warps
// the elementwise stage: thread = key row = TMEM lane, four warps per lane quarter with 32 query
// columns each. It copies S^T and dP^T to registers, forms P^T = exp2(S^T*scale*log2e - lse*log2e)
// and dS^T = P^T (dP^T*scale - delta*scale), writes P^T to tensor memory as packed half pairs (the
// A operand of the dV MMA) and dS^T as half into shared memory in the swizzled layout that serves
// as K-major A operand for dK and, read the other way, as M-major A operand for dQ. No transposes
// are materialised anywhere. dK and dV leave through staged TMA stores.
//   head_dim 64: every accumulator has tensor-memory columns of its own and Q/dO come through a
// ring of three stages, so the next block's S^T/dP^T are issued as soon as the elementwise warps
// hold the current ones in registers, and a block's dQ is read out during the next block's MMAs.
//   head_dim 128: S^T, dP^T, dV and dK fill the 512 columns. Each warp writes its P^T over S^T
// columns that only it has read, and dQ is computed over dP^T; there is one buffer each for Q
// and dO. Per block the MMA order is dV, dK, dQ, S^T(next), dP^T(next): dV and dK
// free dO and Q, whose reloads (already in L2 by a prefetch) enter the TMA queue ahead of the dQ
// reduce-adds, S^T(next) only needs P^T consumed, dP^T(next) waits until dQ is in registers.
// The dQ reduce-add is the scarce resource at head_dim 128: reductions leave an SM at ~25 bytes
// per clock (measured; ~15 when all SMs send them), i.e. 2600-4300 cycles for the 64 KB of one
// block against 2520 cycles of MMA; it runs asynchronously out of staging buffers that nothing
// else uses.
// A small kernel run first writes the row statistics lse*log2e and delta*scale =
// scale*rowsum(O*dO), padded to whole blocks.
//
// Roofline: tensor pipe, 10*B*H*S^2*D FLOP (half when causal).
#include "common.cuh"
#include "attention.cuh"
#include "sm100.cuh"
#include "attention_tc.cuh"
#include "tempbuf.cuh"

namespace mt {

using namespace sm100;


template <int D> struct BwdCfg {
  // Elementwise warps: four per TMEM lane quarter, each taking 32 of the block's 128 query columns.
  static constexpr int kEwWarps = 16;
  static constexpr int kColsPerThread = 128 / (kEwWarps / 4);
  static constexpr int kThreads = 32 * (kEwWarps + 2);
  static constexpr int kChunks = D / 64;
  static constexpr int kTile = 128 * D * 2;                 // one 128-row block of K/V/Q/dO
  // head_dim 64: a ring of three Q+dO stages behind one barrier pair per stage. head_dim 128 has
  // room for one Q and one dO buffer, each with barriers of its own: Q is reloaded as soon as the
  // dK MMA (issued first) has read it, dO after the dV MMA; both were brought into L2 a block ahead.
  static constexpr bool kSplit = D == 128;
  static constexpr int kQStages = D == 64 ? 3 : 1;
  static constexpr int kDOStages = D == 64 ? 3 : 1;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTile;
  static constexpr int kOffQ = 2 * kTile;
  static constexpr int kOffDO = kOffQ + kQStages * kTile;
  static constexpr int kOffDST = kOffDO + kDOStages * kTile;
  // Staging for the TMA reduce-add of dQ and the TMA stores of dK/dV: a buffer of 32 rows x 128
  // bytes of its own for every warp that flushes (the eight warps of column groups 0 and 1 at
  // head_dim 64, all sixteen at head_dim 128). Reduce-adds leave an SM at about 25 bytes per clock
  // (15 when every SM sends them), so a block's dQ - 32 KB / 64 KB of fp32 - is on its way for
  // thousands of cycles: the buffers are not shared with anything, and a warp meets its buffer
  // again only a whole block later, when the reduce-add has long read it.
  static constexpr int kFlushWarps = D == 64 ? 8 : 16;
  static constexpr int kStageRows = 32;
  static constexpr int kStageBytes = kStageRows * 128;
  static constexpr int kOffStage = kOffDST + 32768;
  static constexpr int kOffStat = kOffStage + kFlushWarps * kStageBytes;   // per Q stage: lse*log2e [128], delta*scale [128] floats
  static constexpr int kOffBar = kOffStat + kQStages * 1024;
  // No slack for aligning the base: the dynamic shared-memory window of a kernel without static
  // shared memory starts 1024-byte aligned (checked at entry).
  static constexpr int kSmem = kOffBar + 256;
  static_assert(kSmem <= 232448, "shared memory of one CTA");
  // Tensor memory, 512 columns. head_dim 64: S^T, dP^T, dV, dK, dQ and P^T (packed half pairs)
  // each have their own. head_dim 128 fills all 512 with S^T, dP^T, dV and dK: every warp writes
  // its 16 packed columns of P^T over the first half of the 32 S^T columns that it alone has read
  // (no ordering among warps needed; the dV MMA takes its A operand in four pieces), and dQ is
  // computed over dP^T, which the elementwise warps have read by then.
  static constexpr int kTmemCols = 512;
  static constexpr int kColST = 0, kColDPT = 128, kColDV = 256, kColDK = 256 + D;
  static constexpr bool kAliasDQ = D == 128;
  static constexpr int kColDQ = kAliasDQ ? kColDPT : 256 + 2 * D;
  static constexpr int kColPT = kAliasDQ ? kColST : 256 + 3 * D;
};

struct AttnBwdParams {
  const float* stats;      // [2][B*H][nqb*128]: lse*log2e (+inf on padded rows), then delta*scale (0 on padded rows)
  float* dq_accum;
  void* dk; void* dv;
  MapPos pq, pk, pv, pdo, pdk, pdv;
  int B, H, S, nqb, causal, is_bf16;
  int Hkv, group;       // key/value heads; query heads per key/value head (H = Hkv * group)
  int gh;               // (batch, key/value head) pairs per group of the tile order
  int* tile_counter;    // zero at launch (the statistics kernel clears it): the next tile nobody has taken yet
  float scale, scale_log2;
  int* flag;
};

template <int D, typename T>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                   const __grid_constant__ CUtensorMap tmDV, const AttnBwdParams P) {
  using Cfg = BwdCfg<D>;
  constexpr int ST = Cfg::kQStages;             // Q ring (at head_dim 64 dO travels with it)
  constexpr int kBwdEwWarps = Cfg::kEwWarps;
  constexpr int CPT = Cfg::kColsPerThread;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {   // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0 && P.flag) atomicMax(P.flag, 102);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + Cfg::kOffBar;
  const uint32_t bar_kv = bar0, bar_qfull0 = bar0 + 8, bar_qempty0 = bar0 + 32, bar_sdp = bar0 + 56,
                 bar_pds = bar0 + 64, bar_dq = bar0 + 72, bar_dqfree = bar0 + 80, bar_sdpfree = bar0 + 88,
                 bar_kvfree = bar0 + 96, bar_dkvfree = bar0 + 104, bar_dofull = bar0 + 128, bar_doempty = bar0 + 136,
                 bar_kvissued = bar0 + 144, bar_tfull0 = bar0 + 152, bar_tempty0 = bar0 + 168;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + Cfg::kOffBar + 112);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + Cfg::kOffBar + 116);
  float* stat = reinterpret_cast<float*>(base_ptr + Cfg::kOffStat);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(base_ptr + Cfg::kOffBar + 120);   // two slots

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh_count = P.B * P.Hkv;           // (batch, key/value head) pairs
  const int n_tiles = P.nqb * bh_count;
  // Tile t -> (key block jb, (batch, key/value head)) by decode_tile: heads in groups of P.gh,
  // within a group small jb first (= most query blocks when causal, so heavy tiles come first and
  // the light ones fill the end). The tile's steps are the query blocks of
  // every query head that reads this key/value head: step i = (query head hk*group + i / n_qb,
  // query block q_start + i % n_qb); dK and dV accumulate over all of them. Every role walks the
  // same tile sequence and keeps a running count `g` of steps, from which ring stages and barrier
  // parities follow.

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 3; ++s) { mbar_init(bar_qfull0 + 8 * s, 1); mbar_init(bar_qempty0 + 8 * s, 1); }
    mbar_init(bar_sdp, 1); mbar_init(bar_pds, 32 * kBwdEwWarps); mbar_init(bar_dq, 1);
    mbar_init(bar_dqfree, 32 * kBwdEwWarps);
    mbar_init(bar_sdpfree, kBwdEwWarps);
    mbar_init(bar_kvfree, 1);
    mbar_init(bar_dkvfree, 8 * Cfg::kChunks);       // one arrival per warp that drains a 64-column piece of dK or dV
    mbar_init(bar_dofull, 1); mbar_init(bar_doempty, 1);
    mbar_init(bar_kvissued, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull0 + 8 * i, 1); mbar_init(bar_tempty0 + 8 * i, 1 + kBwdEwWarps); }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kBwdEwWarps + 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kBwdEwWarps) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
      // One step of this CTA's work: a query block of a tile. Steps are numbered g = 0, 1, ... across
      // tiles; `tn` counts the tiles.
      struct Step { int tn, i, n_q, n_qb, q_start, jb, b, h; bool valid; };
      // Takes the next tile nobody has taken yet as this CTA's tile number st.tn and publishes it
      // to the other roles (slot tn & 1 of the ring; -1 = no more); i = 0. The slot is free once the
      // consumers have read tile tn - 2.
      // (the counter is read one tile ahead: the atomic's round trip to L2 runs under the loads of
      // the tile before)
      int tile_ahead = atomicAdd(P.tile_counter, 1);
      auto fetch = [&](Step& st) {
        st.valid = false;
        if (!mbar_wait(bar_tempty0 + 8 * (st.tn & 1), ((st.tn >> 1) & 1) ^ 1u, abort_flag)) return;
        int tile = tile_ahead;
        if (tile < n_tiles) tile_ahead = atomicAdd(P.tile_counter, 1);
        if (tile >= n_tiles) tile = -1;
        tile_ring[st.tn & 1] = tile;
        mbar_arrive(bar_tfull0 + 8 * (st.tn & 1));
        if (tile < 0) return;
        int bkv;
        decode_tile(tile, P.nqb, bh_count, P.gh, st.jb, bkv);
        st.b = bkv / P.Hkv; st.h = bkv % P.Hkv;              // h: key/value head
        st.q_start = P.causal ? st.jb : 0;
        st.n_qb = P.nqb - st.q_start;
        st.n_q = st.n_qb * P.group;
        st.i = 0;
        st.valid = true;
      };
      auto advance = [&](Step& st) {
        if (++st.i < st.n_q) return;
        ++st.tn;
        fetch(st);
      };
      auto load_kv = [&](const Step& st) -> bool {
        // K and V of the previous tile are read until its last dQ MMA has completed
        if (st.tn > 0 && !mbar_wait(bar_kvfree, (st.tn - 1) & 1, abort_flag)) return false;
        mbar_expect_tx(bar_kv, 2 * Cfg::kTile);
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc) {
          load_rows(base + Cfg::kOffK + dc * 16384, &tmK, bar_kv, P.pk, dc * 64, st.jb * 128, st.h, st.b);
          load_rows(base + Cfg::kOffV + dc * 16384, &tmV, bar_kv, P.pv, dc * 64, st.jb * 128, st.h, st.b);
        }
        return true;
      };
      // Q of step g (and, at head_dim 64, its dO) with the block's row statistics
      auto load_q = [&](const Step& st, int g) -> bool {
        const int s = g % ST;
        if (!mbar_wait(bar_qempty0 + 8 * s, ((g / ST) & 1) ^ 1u, abort_flag)) return false;
        mbar_expect_tx(bar_qfull0 + 8 * s, (Cfg::kSplit ? 1 : 2) * Cfg::kTile + 1024);
        const int hq = st.h * P.group + st.i / st.n_qb, qi = st.q_start + st.i % st.n_qb;   // query head and block of this step
        const int64_t spad = (int64_t)P.nqb * 128;
        const float* src = P.stats + ((int64_t)st.b * P.H + hq) * spad + (int64_t)qi * 128;
        bulk_load_1d(base + Cfg::kOffStat + s * 1024, src, 512, bar_qfull0 + 8 * s);
        bulk_load_1d(base + Cfg::kOffStat + s * 1024 + 512, src + (int64_t)P.B * P.H * spad, 512, bar_qfull0 + 8 * s);
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc) {
          load_rows(base + Cfg::kOffQ + s * Cfg::kTile + dc * 16384, &tmQ, bar_qfull0 + 8 * s, P.pq, dc * 64, qi * 128, hq, st.b);
          if (!Cfg::kSplit)
            load_rows(base + Cfg::kOffDO + s * Cfg::kTile + dc * 16384, &tmDO, bar_qfull0 + 8 * s, P.pdo, dc * 64, qi * 128, hq, st.b);
        }
        return true;
      };
      Step cur;
      cur.tn = 0;
      fetch(cur);
      if (!Cfg::kSplit) {
        bool ok = true;
        for (int g = 0; cur.valid; ++g, advance(cur)) {
          // A tile's first Q/dO goes ahead of its K/V: the ring has room long before the previous
          // tile's last MMA lets go of K and V, and this thread would otherwise sit in that wait
          // with the Q/dO request still unissued.
          if (!load_q(cur, g)) { ok = false; break; }
          if (cur.i == 0 && !load_kv(cur)) { ok = false; break; }
          if (cur.i == 0) mbar_arrive(bar_kvissued);   // this tile's first loads are in the TMA queue
        }
        (void)ok;
      } else {
        // One buffer each for Q and dO: while step g is worked on, step g+1's Q and dO are brought
        // into L2; its dO is loaded as soon as the dV MMA of step g has completed, its Q after the
        // dK MMA (issued in that order) and, where step g+1 opens a tile, that tile's K and V follow.
        auto load_do = [&](const Step& st) {
          mbar_expect_tx(bar_dofull, Cfg::kTile);
          const int hq = st.h * P.group + st.i / st.n_qb, qi = st.q_start + st.i % st.n_qb;
#pragma unroll
          for (int dc = 0; dc < Cfg::kChunks; ++dc)
            load_rows(base + Cfg::kOffDO + dc * 16384, &tmDO, bar_dofull, P.pdo, dc * 64, qi * 128, hq, st.b);
        };
        bool ok = cur.valid;
        if (ok) ok = load_kv(cur);
        if (ok) ok = load_q(cur, 0);
        if (ok) load_do(cur);
        if (ok) mbar_arrive(bar_kvissued);
        Step nxt = cur;
        if (ok) advance(nxt);
        for (int g = 0; ok && nxt.valid; ++g) {
          {
            const int hq = nxt.h * P.group + nxt.i / nxt.n_qb, qi = nxt.q_start + nxt.i % nxt.n_qb;
#pragma unroll
            for (int dc = 0; dc < Cfg::kChunks; ++dc) {
              prefetch_rows(&tmDO, P.pdo, dc * 64, qi * 128, hq, nxt.b);
              prefetch_rows(&tmQ, P.pq, dc * 64, qi * 128, hq, nxt.b);
            }
          }
          if (!mbar_wait(bar_doempty, g & 1, abort_flag)) { ok = false; break; }   // dV of step g has read dO
          load_do(nxt);
          if (!load_q(nxt, g + 1)) { ok = false; break; }              // waits for dK of step g
          if (nxt.i == 0) {
            if (!load_kv(nxt)) { ok = false; break; }
            mbar_arrive(bar_kvissued);                 // the next tile's first loads are in the TMA queue
          }
          advance(nxt);
        }
      }
    }
  } else if (warp == kBwdEwWarps + 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_kk = idesc_f16(P.is_bf16, 0, 0, 128, 128);   // S^T, dP^T: both operands K-major
      const uint32_t idesc_kn = idesc_f16(P.is_bf16, 0, 1, 128, D);     // dV, dK: A K-major, B N-major
      const uint32_t idesc_mn = idesc_f16(P.is_bf16, 1, 1, 128, D);     // dQ: A M-major, B N-major
      const uint32_t sk = base + Cfg::kOffK, sv = base + Cfg::kOffV;
      const uint32_t sdst = base + Cfg::kOffDST;
      // Descriptors that do not depend on the Q/dO stage are built once; the stage's own are built
      // at the top of each step, BEFORE the barrier wait, so that after a wait this thread issues
      // MMAs and nothing else (it shares a scheduler with busy warps and every extra instruction
      // between wait and MMA costs 10-20 cycles of tensor-pipe idle time).
      constexpr int NS = 4 * Cfg::kChunks;              // MMAs of one S^T or dP^T
      uint64_t a_s[NS], a_dp[NS], a_dk[8], a_dq[8], b_dq[8];
#pragma unroll
      for (int dc = 0; dc < Cfg::kChunks; ++dc)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          a_s[dc * 4 + k] = smem_desc_sw128(sk + dc * 16384 + k * 32, 16, 1024);
          a_dp[dc * 4 + k] = smem_desc_sw128(sv + dc * 16384 + k * 32, 16, 1024);
        }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        a_dk[ks] = smem_desc_sw128(sdst + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);   // dS^T, K-major
        a_dq[ks] = smem_desc_sw128(sdst + ks * 2048, 16384, 1024);                          // dS^T, M-major
        b_dq[ks] = smem_desc_sw128(sk + ks * 2048, 16384, 1024);
      }
      auto issue_n = [&](uint32_t d, const uint64_t* a, const uint64_t* b, uint32_t idesc, uint32_t acc) {
        if (NS == 4) umma_f16_x4(d, a, b, idesc, acc);
        else umma_f16_x8(d, a, b, idesc, acc);
      };
      // S^T = K Q^T of query block g (running count) into tensor memory
      auto issue_s = [&](int g) -> bool {
        const int s = g % ST;
        const uint32_t sq = base + Cfg::kOffQ + s * Cfg::kTile;
        uint64_t b_s[NS];
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
#pragma unroll
          for (int k = 0; k < 4; ++k) b_s[dc * 4 + k] = smem_desc_sw128(sq + dc * 16384 + k * 32, 16, 1024);
        if (!mbar_wait(bar_qfull0 + 8 * s, (g / ST) & 1, abort_flag)) return false;
        tc_fence_after();
        issue_n(tmem_base + Cfg::kColST, a_s, b_s, idesc_kk, 0u);
        return true;
      };
      // dP^T = V dO^T of query block g; completes bar_sdp together with the S^T issued before it
      auto issue_dp = [&](int g) -> bool {
        const uint32_t sdo = base + Cfg::kOffDO + (g % Cfg::kDOStages) * Cfg::kTile;
        uint64_t b_dp[NS];
#pragma unroll
        for (int dc = 0; dc < Cfg::kChunks; ++dc)
#pragma unroll
          for (int k = 0; k < 4; ++k) b_dp[dc * 4 + k] = smem_desc_sw128(sdo + dc * 16384 + k * 32, 16, 1024);
        if (Cfg::kSplit) {
          if (!mbar_wait(bar_dofull, g & 1, abort_flag)) return false;
          // dQ of the previous block sits in these columns until the elementwise warps have read it
          if (g > 0 && !mbar_wait(bar_dqfree, (g - 1) & 1, abort_flag)) return false;
          tc_fence_after();
        }
        issue_n(tmem_base + Cfg::kColDPT, a_dp, b_dp, idesc_kk, 0u);
        umma_commit(bar_sdp);
        return true;
      };
      int g0 = 0;                                       // running count of query blocks at the start of the tile
      bool ok = true;
      for (int tn = 0; ok; ++tn) {
        if (!mbar_wait(bar_tfull0 + 8 * (tn & 1), (tn >> 1) & 1, abort_flag)) break;
        const int tile = tile_ring[tn & 1];
        mbar_arrive(bar_tempty0 + 8 * (tn & 1));
        if (tile < 0) break;
        int jb, bkv_unused;
        decode_tile(tile, P.nqb, bh_count, P.gh, jb, bkv_unused);
        const int n_q = (P.nqb - (P.causal ? jb : 0)) * P.group;
        if (!mbar_wait(bar_kv, tn & 1, abort_flag)) break;
        tc_fence_after();
        if (!Cfg::kAliasDQ) {
          // the elementwise warps have copied the previous block's S^T / dP^T (last block of the
          // previous tile) to registers
          if (g0 > 0 && !mbar_wait(bar_sdpfree, (g0 - 1) & 1, abort_flag)) break;
          tc_fence_after();
        }
        // (head_dim 128: every MMA of the previous tile has completed - K and V were only replaced
        // after that - so P^T in the S^T columns is dead; issue_dp waits for the last dQ's read-out)
        if (!issue_s(g0) || !issue_dp(g0)) break;
        for (int i = 0; i < n_q; ++i) {
          const int g = g0 + i;
          const int s = g % ST;
          const uint32_t sq = base + Cfg::kOffQ + s * Cfg::kTile;
          const uint32_t sdo = base + Cfg::kOffDO + (g % Cfg::kDOStages) * Cfg::kTile;
          if (!Cfg::kAliasDQ && i + 1 < n_q) {
            // The elementwise warps hold S^T / dP^T of block g in registers: the next block's are
            // computed while they work, ahead of everything else of this block.
            if (!mbar_wait(bar_sdpfree, g & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (!issue_s(g + 1) || !issue_dp(g + 1)) { ok = false; break; }
          }
          uint64_t b_dv[8], b_dk[8];
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            b_dv[ks] = smem_desc_sw128(sdo + ks * 2048, 16384, 1024);
            b_dk[ks] = smem_desc_sw128(sq + ks * 2048, 16384, 1024);
          }
          if (!mbar_wait(bar_pds, g & 1, abort_flag)) { ok = false; break; }     // P^T, dS^T written
          tc_fence_after();
          if (i == 0 && tn > 0) {
            // the first dV / dK MMA of a tile overwrites the accumulators: the previous tile's must
            // have been read out (the elementwise warps drain them before this tile's first block)
            if (!mbar_wait(bar_dkvfree, (tn - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
          }
          // dV += P^T dO (reduction over the 128 queries, A = P^T from tensor memory), dK += dS^T Q,
          // dQ = dS K (reduction over the 128 keys)
          if (!Cfg::kAliasDQ) {
            umma_f16_ts_x8(tmem_base + Cfg::kColDV, tmem_base + Cfg::kColPT, b_dv, idesc_kn, i > 0 ? 1u : 0u);
            umma_f16_x8(tmem_base + Cfg::kColDK, a_dk, b_dk, idesc_kn, i > 0 ? 1u : 0u);
            umma_commit(bar_qempty0 + 8 * s);   // Q and dO of this block are not read again (dQ needs neither)
            if (g > 0 && !mbar_wait(bar_dqfree, (g - 1) & 1, abort_flag)) { ok = false; break; }   // dQ columns read out
            tc_fence_after();
            umma_f16_x8(tmem_base + Cfg::kColDQ, a_dq, b_dq, idesc_mn, 0u);
            umma_commit(bar_dq);
          } else {
            // dV and dK first: they free the dO and Q buffers, and the loads of the next block must
            // enter the TMA queue before the 64 KB of dQ reduce-adds that follow the dQ MMA - a load
            // queued behind those waits a couple of thousand cycles.
            umma_f16_ts_x8_pairs(tmem_base + Cfg::kColDV, tmem_base + Cfg::kColPT, b_dv, idesc_kn, i > 0 ? 1u : 0u);
            umma_commit(bar_doempty);           // dO of this block is not read again
            umma_f16_x8(tmem_base + Cfg::kColDK, a_dk, b_dk, idesc_kn, i > 0 ? 1u : 0u);
            umma_commit(bar_qempty0 + 8 * s);   // Q of this block is not read again
            umma_f16_x8(tmem_base + Cfg::kColDQ, a_dq, b_dq, idesc_mn, 0u);
            umma_commit(bar_dq);
          }
          if (Cfg::kAliasDQ && i + 1 < n_q) {
            // The next block's S^T goes over P^T, which the dV MMA above (earlier in the pipe) was the
            // last to read; its dP^T goes over dQ and waits for the read-out inside issue_dp.
            if (!issue_s(g + 1) || !issue_dp(g + 1)) { ok = false; break; }
          }
        }
        umma_commit(bar_kvfree);            // completes with the tile's last dQ: K and V may be replaced
        g0 += n_q;
      }
    }
  } else {
    // ------------------------------------------------- elementwise stage --
    const int t = (warp & 3) * 32 + lane;             // key row within the block = TMEM lane
    const int hh = warp >> 2;                         // which CPT of the block's 128 query columns this warp handles
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* dst_row = base_ptr + Cfg::kOffDST + t * 128;
    bool ok = true;
    // adds the finished dQ block (TMEM) into the fp32 accumulator [B*H, S, D]: each warp stages its
    // 32 rows x 32 columns in swizzled shared memory and one lane issues a TMA reduce-add (rows past
    // the sequence end are clipped by the tensor map)
    // This warp's staging buffer (only warps that flush or drain have one)
    uint8_t* stage_buf = base_ptr + Cfg::kOffStage + (warp % Cfg::kFlushWarps) * Cfg::kStageBytes;
    constexpr int kPieces = 32 / Cfg::kStageRows;     // a warp's 32 rows leave in this many TMA operations
    constexpr int kDqChunks = D / 32;                 // 32-column pieces of dQ: column group hh flushes piece hh
    // Writes 128 bytes per row (`w`: this lane's row as 32 words) of rows
    // [piece * kStageRows, (piece + 1) * kStageRows) into the staging buffer, swizzled.
    auto stage_rows = [&](int piece, const uint32_t (&w)[32]) -> uint32_t {
      uint8_t* buf = stage_buf;
      if (lane == 0) bulk_wait_read<0>();             // the previous operation has finished reading the buffer
      __syncwarp();
      if (lane / Cfg::kStageRows == piece) {
        const int rr = lane % Cfg::kStageRows;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16)
          *reinterpret_cast<uint4*>(buf + rr * 128 + ((c16 ^ (rr & 7)) << 4)) =
              make_uint4(w[c16 * 4], w[c16 * 4 + 1], w[c16 * 4 + 2], w[c16 * 4 + 3]);
      }
      fence_proxy_async();
      __syncwarp();
      return smem_u32(buf);
    };
    // `gate` >= 0 (a tile's last block): the reduce-adds are held back until the producer has put
    // the next tile's first loads into the TMA queue - a load queued behind 32-64 KB of reduce-adds,
    // which leave the SM at ~25 bytes per clock, would wait thousands of cycles.
    auto flush_dq = [&](int qi, int bh, int gate) {   // bh: (batch, query head) index of the block
      if (hh < kDqChunks) {
        uint32_t r[32];
        tmem_ld32(tmem_base + Cfg::kColDQ + lane_addr + hh * 32, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar_dqfree);                      // the dQ columns may be overwritten: the rest works from registers
#pragma unroll
        for (int piece = 0; piece < kPieces; ++piece) {
          const uint32_t src = stage_rows(piece, r);
          if (lane == 0) {
            if (gate >= 0) mbar_wait(bar_kvissued, (uint32_t)gate, abort_flag);
            tma_reduce_add_3d(&tmDQ, src, hh * 32, qi * 128 + (warp & 3) * 32 + piece * Cfg::kStageRows, bh);
            bulk_commit();
          }
        }
      } else {
        mbar_arrive(bar_dqfree);
      }
    };
    int g0 = 0;                                       // running count of query blocks at the start of the tile
    int pend_qi = 0, pend_bh = 0;                     // head_dim 64: query block whose dQ is still in tensor memory
    for (int tn_ew = 0; ok; ++tn_ew) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull0 + 8 * (tn_ew & 1), (tn_ew >> 1) & 1, abort_flag))) { ok = false; break; }
      const int tile = tile_ring[tn_ew & 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty0 + 8 * (tn_ew & 1));
      if (tile < 0) break;
      int jb, bkv;
      decode_tile(tile, P.nqb, bh_count, P.gh, jb, bkv);
      const int b = bkv / P.Hkv, h = bkv % P.Hkv;     // h: key/value head
      const int q_start = P.causal ? jb : 0;
      const int n_qb = P.nqb - q_start;
      const int n_q = n_qb * P.group;
      const int kg = jb * 128 + t;                    // global key index
      // step i of the tile -> (batch, query head) index and query block
      auto bh_of = [&](int i) { return b * P.H + h * P.group + i / n_qb; };
      auto qi_of = [&](int i) { return q_start + i % n_qb; };
      for (int i = 0; i < n_q && ok; ++i) {
        const int g = g0 + i;
        const int qi = qi_of(i);
        // row statistics of this query block arrived with its Q/dO stage (bulk copy); the wait makes
        // that copy visible to this thread and returns at once, since S^T needed the stage too
        const float* lse2 = stat + (g % ST) * 256;
        const float* dlt = lse2 + 128;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_sdp, g & 1, abort_flag))) { ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(bar_qfull0 + 8 * (g % ST), (g / ST) & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        const bool diag = P.causal && qi == jb;
        const bool dead = kg >= P.S;                    // padded key row: contributes nothing
        {
          uint32_t s_[CPT], d_[CPT];
#pragma unroll
          for (int c = 0; c < CPT; c += 32) {
            tmem_ld32(tmem_base + Cfg::kColST + lane_addr + hh * CPT + c, s_ + c);
            tmem_ld32(tmem_base + Cfg::kColDPT + lane_addr + hh * CPT + c, d_ + c);
          }
          tmem_ld_wait();
          if (!Cfg::kAliasDQ) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sdpfree);   // S^T / dP^T columns may be overwritten
          }
          if (diag || __any_sync(0xffffffffu, dead)) {   // masked entries: score -inf -> p = 0, dS = 0
#pragma unroll
            for (int e = 0; e < CPT; ++e)
              if (dead || (diag && hh * CPT + e < t)) s_[e] = 0xff800000u;
          }
          if (!Cfg::kAliasDQ && i > 0) {
            // dS^T of the previous block is still an operand of its dQ MMA, which was issued after
            // the S^T/dP^T MMAs of this block: it must have completed before dS^T is overwritten
            // (at the first block of a tile the wait already happened before the previous tile's
            // last dQ flush)
            if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (g - 1) & 1, abort_flag))) { ok = false; break; }
          }
          uint32_t ptp[CPT / 2];                        // P^T of this thread as packed half pairs
          const float4* lse4 = reinterpret_cast<const float4*>(lse2 + hh * CPT);   // per query column, 16-byte loads
          const float4* dlt4 = reinterpret_cast<const float4*>(dlt + hh * CPT);
#pragma unroll
          for (int c16 = 0; c16 < CPT / 8; ++c16) {
            uint32_t pp[4], dd[4];
            const float4 la = lse4[c16 * 2], lb = lse4[c16 * 2 + 1], da = dlt4[c16 * 2], db = dlt4[c16 * 2 + 1];
            const float lv[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
            const float dl8[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float pv[2], dv[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int ce = c16 * 8 + 2 * e + u;              // this thread's column, of CPT
                const float p = ex2_approx(fmaf(__uint_as_float(s_[ce]), P.scale_log2, -lv[2 * e + u]));
                pv[u] = p;
                dv[u] = p * fmaf(__uint_as_float(d_[ce]), P.scale, -dl8[2 * e + u]);   // p (dP - delta) scale
              }
              pp[e] = pack2<T>(pv[0], pv[1]);
              dd[e] = pack2<T>(dv[0], dv[1]);
            }
            // byte offset of these 8 columns in the 128-row tile: 64-column chunk, then the swizzled 16-byte piece
            const int col8 = hh * (CPT / 8) + c16;
            const int off = (col8 >> 3) * 16384 + (((col8 & 7) ^ (t & 7)) << 4);
#pragma unroll
            for (int e = 0; e < 4; ++e) ptp[c16 * 4 + e] = pp[e];
            *reinterpret_cast<uint4*>(dst_row + off) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
            if ((c16 & 3) == 3)   // 32 finished columns = 16 packed words -> tensor memory
              tmem_st16(tmem_base + Cfg::kColPT + lane_addr + hh * (Cfg::kAliasDQ ? CPT : CPT / 2) + (c16 >> 2) * 16, ptp + (c16 >> 2) * 16);
          }
          tmem_st_wait();
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_pds);
        // dQ read-out. With its own TMEM columns the PREVIOUS block's dQ is flushed here, while the
        // tensor core works on this block - also across a tile boundary: a tile's last dQ stays in
        // tensor memory until the next tile's first block (the dQ MMA of that block waits for the
        // read-out as it does for any other), so the tile's end is not held up by a second batch of
        // reduce-adds right behind the previous one. When dQ aliases dP^T it has to be this block's.
        if (Cfg::kAliasDQ) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, g & 1, abort_flag))) { ok = false; break; }
          tc_fence_after();
          int gate = -1;
          if (i == n_q - 1) {
            // the producer published the tile after this one while it looked a step ahead; when
            // there is one, this tile's last reduce-adds wait until its first loads are queued
            if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull0 + 8 * ((tn_ew + 1) & 1), ((tn_ew + 1) >> 1) & 1, abort_flag))) { ok = false; break; }
            if (tile_ring[(tn_ew + 1) & 1] >= 0) gate = (tn_ew + 1) & 1;
          }
          flush_dq(qi, bh_of(i), gate);
        } else {
          if (g > 0) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (g - 1) & 1, abort_flag))) { ok = false; break; }
            tc_fence_after();
            flush_dq(pend_qi, pend_bh, -1);
          }
          pend_qi = qi; pend_bh = bh_of(i);
        }
      }
      if (!ok) break;
      if (!Cfg::kAliasDQ) {
        // the tile's last dQ; its completion also means every MMA of the tile is complete
        if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (g0 + n_q - 1) & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
      }
      // All MMAs of the tile are complete (its last bar_dq was waited above, in either variant).
      // Each 64-column piece of dK and of dV is drained by one column group: 32 key rows at a time
      // are staged (128-byte rows, swizzled) in the warp's buffer and stored by TMA, which clips
      // rows past the sequence end. Once the accumulators are in registers the MMA warp may start
      // the next tile's dV / dK.
      if (Cfg::kAliasDQ) {
        // here the dQ MMA is not the block's last: wait for the commit that follows the tile's last MMA
        if (!__all_sync(0xffffffffu, mbar_wait(bar_kvfree, tn_ew & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
      }
      if ((hh >> 1) < Cfg::kChunks) {
        // column group hh drains the 64-column piece hh >> 1 of dK (even hh) or dV (odd hh)
        const CUtensorMap* map = (hh & 1) ? &tmDV : &tmDK;
        const MapPos pos = (hh & 1) ? P.pdv : P.pdk;
        const int col0 = (hh & 1) ? Cfg::kColDV : Cfg::kColDK;
        const int dc = hh >> 1;
        uint32_t r[64];
        tmem_ld32(tmem_base + col0 + lane_addr + dc * 64, r);
        tmem_ld32(tmem_base + col0 + lane_addr + dc * 64 + 32, r + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dkvfree);
        uint32_t w[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) w[e] = pack2<T>(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
#pragma unroll
        for (int piece = 0; piece < kPieces; ++piece) {
          const uint32_t src = stage_rows(piece, w);
          if (lane == 0) {
            store_rows(map, src, pos, dc * 64, jb * 128 + (warp & 3) * 32 + piece * Cfg::kStageRows, h, b);
            bulk_commit();
          }
        }
      }
      g0 += n_q;
    }
    if (!Cfg::kAliasDQ && ok && g0 > 0) flush_dq(pend_qi, pend_bh, -1);   // the very last block's dQ
    if (lane == 0) bulk_wait_all<0>();   // reduces and stores must be done with shared memory before the CTA exits
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && P.flag) atomicMax(P.flag, 102);
  if (warp == kBwdEwWarps + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// Row statistics for the backward kernel, padded to whole 128-row blocks:
//   stats[0][bh][i] = lse[bh][i] * log2(e)            (+inf for i >= S: such a row gets p = 0)
//   stats[1][bh][i] = scale * sum_d o[i][d] * do[i][d]  (0 for i >= S)
// Eight threads per row read O and dO once; the same threads clear the row of the fp32 dQ
// accumulator [B*H, S, D] that the backward kernel adds into.
template <typename T>
__global__ void __launch_bounds__(256)
attn_bwd_stats_kernel(const T* __restrict__ o, const T* __restrict__ d_o, const float* __restrict__ lse,
                      float* __restrict__ stats, float* __restrict__ dq_accum, mt_strides3 so, mt_strides3 sdo, int heads,
                      int S, int spad, int D, int64_t total_rows, float scale, int* __restrict__ tile_counter) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *tile_counter = 0;   // the backward kernel's tile queue starts at 0
  constexpr int VN = Vec16<T>::N;
  const int sub = threadIdx.x & 7;
  const int64_t row = (int64_t)blockIdx.x * 32 + (threadIdx.x >> 3);   // over [B*H][spad]
  const int64_t bh = row / spad;
  const int i = (int)(row - bh * spad);
  const bool real = row < total_rows && i < S;
  float s = 0.f;
  if (real) {
    const int b = (int)(bh / heads), h = (int)(bh % heads);
    const T* op = o + (int64_t)b * so.b + (int64_t)h * so.h + (int64_t)i * so.s;
    const T* dp = d_o + (int64_t)b * sdo.b + (int64_t)h * sdo.h + (int64_t)i * sdo.s;
    for (int d = sub * VN; d < D; d += 8 * VN) {
      Vec16<T> a, g;
      a.load(op + d);
      g.load(dp + d);
#pragma unroll
      for (int e = 0; e < VN; ++e) s += a.get(e) * g.get(e);
    }
    float4* acc = reinterpret_cast<float4*>(dq_accum + (bh * S + i) * D);
    for (int d4 = sub; d4 < D / 4; d4 += 8) acc[d4] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (sub == 0 && row < total_rows) {
    stats[row] = real ? lse[bh * S + i] * kLog2eF : INFINITY;
    stats[total_rows + row] = real ? s * scale : 0.f;
  }
}

// dq[b,h,s,:] = (T) dq_accum[b,h,s,:]
template <typename T>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, mt_strides3 sdq, int H, int S, int D, int64_t n_vec) {
  const int vec_per_row = D / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int v = (int)(i - row * vec_per_row);
    const int64_t bh = row / S;
    const int s = (int)(row - bh * S);
    const int b = (int)(bh / H), h = (int)(bh % H);
    const float4 a0 = reinterpret_cast<const float4*>(acc + row * D + v * 8)[0];
    const float4 a1 = reinterpret_cast<const float4*>(acc + row * D + v * 8)[1];
    uint4 o;
    o.x = pack2<T>(a0.x, a0.y); o.y = pack2<T>(a0.z, a0.w); o.z = pack2<T>(a1.x, a1.y); o.w = pack2<T>(a1.z, a1.w);
    *reinterpret_cast<uint4*>(dq + (int64_t)b * sdq.b + (int64_t)h * sdq.h + (int64_t)s * sdq.s + v * 8) = o;
  }
}

bool attn_bwd_tc_supported(const AttnArgs& a) {
  if (!a.dq_accum) return false;
  if (!aligned16(a.o) || !aligned16(a.d_o) || !aligned16(a.dq) || !aligned16(a.dk) || !aligned16(a.dv) || !aligned16(a.dq_accum)) return false;
  if (!strides_ok(a.sdo) || !strides_ok(a.sdq) || !strides_ok(a.sdk) || !strides_ok(a.sdv)) return false;
  return true;
}

template <int D, typename T>
static int launch_bwd(const AttnArgs& a, cudaStream_t st) {
  using Cfg = BwdCfg<D>;
  const int bf = a.dtype == MT_BF16;
  int rc;
  const int nqb = (int)((a.seq + 127) / 128);
  const int64_t stat_rows = a.batch * a.heads * nqb * 128;
  TempBuf stats((size_t)stat_rows * 2 * sizeof(float) + 16, st);   // + the tile counter
  if (!stats.ok()) return MT_ERR_CUDA;
  int* tile_counter = reinterpret_cast<int*>(reinterpret_cast<float*>(stats.ptr) + stat_rows * 2);
  attn_bwd_stats_kernel<T><<<(unsigned)((stat_rows + 31) / 32), 256, 0, st>>>(
      (const T*)a.o, (const T*)a.d_o, a.lse, (float*)stats.ptr, a.dq_accum, a.so, a.sdo, (int)a.heads, (int)a.seq, nqb * 128, D,
      stat_rows, a.scale, tile_counter);
  MT_LAUNCH_CHECK();
  const int64_t n_acc = a.batch * a.heads * a.seq * D;
  CUtensorMap tq, tk, tv, tdo;
  AttnBwdParams P;
  if ((rc = make_qkv_map(&tq, &P.pq, a.q, bf, a.sq, a.batch, a.heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tk, &P.pk, a.k, bf, a.sk, a.batch, a.kv_heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tv, &P.pv, a.v, bf, a.sv, a.batch, a.kv_heads, a.seq, D))) return rc;
  if ((rc = make_qkv_map(&tdo, &P.pdo, a.d_o, bf, a.sdo, a.batch, a.heads, a.seq, D))) return rc;
  CUtensorMap tdk, tdv;
  if ((rc = make_qkv_map(&tdk, &P.pdk, a.dk, bf, a.sdk, a.batch, a.kv_heads, a.seq, D, Cfg::kStageRows))) return rc;
  if ((rc = make_qkv_map(&tdv, &P.pdv, a.dv, bf, a.sdv, a.batch, a.kv_heads, a.seq, D, Cfg::kStageRows))) return rc;
  CUtensorMap tdq;
  {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)a.seq, (uint64_t)(a.batch * a.heads)};
    uint64_t str[2] = {(uint64_t)D, (uint64_t)(a.seq * D)};
    uint32_t box[3] = {32, (uint32_t)Cfg::kStageRows, 1};
    if ((rc = make_tmap_nd_typed(&tdq, a.dq_accum, MT_F32, 3, dims, str, box))) return rc;
  }
  P.stats = (const float*)stats.ptr; P.dq_accum = a.dq_accum; P.dk = a.dk; P.dv = a.dv;
  P.B = (int)a.batch; P.H = (int)a.heads; P.S = (int)a.seq; P.nqb = (int)((a.seq + 127) / 128);
  P.Hkv = (int)a.kv_heads; P.group = (int)(a.heads / a.kv_heads);
  P.causal = a.causal; P.is_bf16 = bf; P.scale = a.scale; P.scale_log2 = a.scale * kLog2eF; P.flag = device_flag_ptr();
  auto kern = attn_bwd_tc_kernel<D, T>;
  MT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const int64_t n_tiles = (int64_t)P.nqb * P.B * P.Hkv;
  // Persistent, one CTA per SM; CTAs take tiles from a global counter, so the order below is also
  // the order in time. With every head in one group the CTAs that run at the same time each
  // stream a different head's Q, dO and dQ, which together no longer fit in L2 once there are many
  // long heads: then heads are taken in groups of about 2 * SMs / blocks-per-head, whose footprint
  // in L2 stays near 30 MB (head_dim 64) or 60 MB (128) whatever the sequence length.
  const int grid_i = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  P.gh = (int)(P.B * P.Hkv);
  P.tile_counter = tile_counter;
  const double footprint = (double)a.batch * a.heads * a.seq * D * 12.0;   // Q, dO, K, V (2 bytes each) + fp32 dQ
  // (only well beyond the 126 MB of L2: CTAs of one group work on the same heads at the same time
  // and their dQ reduce-adds then meet on the same rows - at 150 MB the groups cost 5-8 %, at 1 GB
  // they gain 15 %)
  if (P.nqb > 1 && n_tiles > 2 * (int64_t)sm_count() && footprint > 200e6) {
    const int gh = 2 * sm_count() / P.nqb > 1 ? 2 * sm_count() / P.nqb : 1;
    if (gh < P.gh) P.gh = gh;
  }
  const unsigned grid = (unsigned)grid_i;
  kern<<<grid, Cfg::kThreads, Cfg::kSmem, st>>>(tq, tk, tv, tdo, tdq, tdk, tdv, P);
  MT_LAUNCH_CHECK();
  const int64_t n_vec = n_acc / 8;
  int64_t blocks = (n_vec + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  dq_convert_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(a.dq_accum, (T*)a.dq, a.sdq, (int)a.heads, (int)a.seq, D, n_vec);
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int attn_bwd_tc(const AttnArgs& a, cudaStream_t st) {
  if (a.head_dim == 64) {
    if (a.dtype == MT_F16) return launch_bwd<64, __half>(a, st);
    return launch_bwd<64, __nv_bfloat16>(a, st);
  }
  if (a.dtype == MT_F16) return launch_bwd<128, __half>(a, st);
  return launch_bwd<128, __nv_bfloat16>(a, st);
}

}  // namespace mt
