// LayerNorm and RMSNorm, forward and backward.
//
// Fast path: one warp per row, the row held in registers as 16-byte vectors
// (lane owns vectors lane, lane+32, ...), fp32 math, two warp-shuffle
// reductions. Because a lane owns the same columns for every row it visits,
// the backward kernel keeps dgamma/dbeta partial sums in registers across
// rows; blocks write one partial row each and a second kernel adds them in a
// fixed order (no atomics: results are bit-reproducible). The backward for rows
// of 2-6 or 8 warps of vectors (the transformer widths) is a staged kernel: one
// block per SM, rows brought into a shared-memory ring by bulk copies.
// Fallback (unaligned or very wide rows): one block per row, scalar loads.
//
// Algorithmic traffic (HBM roofline): forward 2*rows*cols*sizeof(T); backward
// 3*rows*cols*sizeof(T) (+ negligible stats and partials).
#include <atomic>

#include "common.cuh"
#include "sm100.cuh"
#include "tempbuf.cuh"

namespace mt {

constexpr int kWarpsPerBlock = 4;

// ---------------------------------------------------------------- forward ---
template <typename T, int MAXV, bool RMS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_fwd_warp(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
              T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
              int64_t rows, int cols, float eps) {
  allow_dependents();
  grid_dependency_wait();
  constexpr int VN = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / VN;
  const T* xr = x + row * cols;
  Vec16<T> v[MAXV];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      v[i].load(xr + vi * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) s += RMS ? v[i].get(e) * v[i].get(e) : v[i].get(e);
    }
  }
  s = warp_sum(s);
  float mu = 0.f, rstd;
  if (RMS) {
    rstd = rsqrtf(s / cols + eps);
  } else {
    mu = s / cols;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
#pragma unroll
        for (int e = 0; e < VN; ++e) { float d = v[i].get(e) - mu; q += d * d; }
      }
    }
    q = warp_sum(q);
    rstd = rsqrtf(q / cols + eps);
  }
  if (lane == 0) {
    if (mean_out) mean_out[row] = mu;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * cols;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
      Vec16<T> g, b, o;
      if (gamma) g.load(gamma + vi * VN);
      if (beta) b.load(beta + vi * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float h = (v[i].get(e) - mu) * rstd;
        if (gamma) h *= g.get(e);
        if (beta) h += b.get(e);
        o.set(e, h);
      }
      o.store(yr + vi * VN);
    }
  }
}

template <typename T, bool RMS>
__global__ void __launch_bounds__(256)
norm_fwd_block(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
               T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
               int64_t rows, int64_t cols, float eps) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float a = to_f(xr[c]);
    s += RMS ? a * a : a;
  }
  s = block_sum(s, sh);
  float mu = 0.f, rstd;
  if (RMS) {
    rstd = rsqrtf(s / cols + eps);
  } else {
    mu = s / cols;
    float q = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { float d = to_f(xr[c]) - mu; q += d * d; }
    q = block_sum(q, sh);
    rstd = rsqrtf(q / cols + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mu;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * cols;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float h = (to_f(xr[c]) - mu) * rstd;
    if (gamma) h *= to_f(gamma[c]);
    if (beta) h += to_f(beta[c]);
    yr[c] = from_f<T>(h);
  }
}

// --------------------------------------------------------------- backward ---
// partial layout: [gridDim.x][2][cols] fp32 (dgamma partials, then dbeta).
template <typename T, int MAXV, bool RMS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_bwd_warp(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd_in,
              const T* __restrict__ dy, const T* __restrict__ gamma, T* __restrict__ dx,
              float* __restrict__ partial, int64_t rows, int cols, bool want_dg, bool want_db, bool dx_acc = false) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float red[kWarpsPerBlock][32 * VN + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols / VN;
  float dg[MAXV][VN], db[MAXV][VN];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int e = 0; e < VN; ++e) { dg[i][e] = 0.f; db[i][e] = 0.f; }
  Vec16<T> gv[MAXV];
  if (gamma) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) gv[i].load(gamma + vi * VN);
    }
  }
  const float inv_cols = 1.f / cols;
  for (int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + warp; row < rows;
       row += (int64_t)gridDim.x * kWarpsPerBlock) {
    const float mu = RMS ? 0.f : mean[row];
    const float rs = rstd_in[row];
    const T* xr = x + row * cols;
    const T* dyr = dy + row * cols;
    Vec16<T> xv[MAXV], dv[MAXV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
        xv[i].load(xr + vi * VN);
        dv[i].load(dyr + vi * VN);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          float xh = (xv[i].get(e) - mu) * rs;
          float d = dv[i].get(e);
          dg[i][e] += d * xh;
          db[i][e] += d;
          float dxh = gamma ? d * gv[i].get(e) : d;
          s1 += dxh;
          s2 += dxh * xh;
        }
      }
    }
    s1 = warp_sum(s1) * inv_cols;
    s2 = warp_sum(s2) * inv_cols;
    if (RMS) s1 = 0.f;
    T* dxr = dx + row * cols;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          float xh = (xv[i].get(e) - mu) * rs;
          float dxh = gamma ? dv[i].get(e) * gv[i].get(e) : dv[i].get(e);
          o.set(e, rs * (dxh - s1 - xh * s2));
        }
        if (dx_acc) {   // dx += result: the incoming buffer already holds the other branch's gradient
          Vec16<T> old;
          old.load(dxr + vi * VN);
#pragma unroll
          for (int e = 0; e < VN; ++e) o.set(e, o.get(e) + old.get(e));
        }
        o.store(dxr + vi * VN);
      }
    }
  }
  if (!want_dg && !want_db) return;
  // Reduce the per-warp partials of this block in a fixed order, one vector
  // slot at a time, and write the block's partial row.
  float* pg = partial + (size_t)blockIdx.x * 2 * cols;
  float* pb = pg + cols;
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 0 && !want_dg) continue;
    if (pass == 1 && !want_db) continue;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      __syncthreads();
#pragma unroll
      for (int e = 0; e < VN; ++e) red[warp][lane * VN + e] = pass == 0 ? dg[i][e] : db[i][e];
      __syncthreads();
      for (int t = threadIdx.x; t < 32 * VN; t += blockDim.x) {
        int col = (i * 32) * VN + t;
        if (col < cols) {
          float a = 0.f;
#pragma unroll
          for (int w = 0; w < kWarpsPerBlock; ++w) a += red[w][t];
          (pass == 0 ? pg : pb)[col] = a;
        }
      }
    }
  }
}

// Staged variant for rows of exactly NV*32 16-byte vectors (768 half columns: NV = 3, 1280: 5,
// 768 fp32 columns: 6). One block per SM:
// W row warps (15, 7 or 3) and one copy warp. Chunks of W consecutive rows are dealt to the blocks
// round robin, so at any moment the SMs read one moving window of the tensors (a contiguous range
// of rows per block balances better but was no faster at 16384 x 768 and slower at 65536 x 1280
// with three tensors). The copy warp's first
// lane walks the block's chunks and starts one bulk copy per tensor (x, dy and, when the result is added
// into dx, the old dx) into a ring of shared-memory stages, as far ahead as the ring allows,
// so the SM has 100-200 KB of reads in flight whatever the row warps are doing. Row warp w
// owns row w of every chunk: it waits for the stage, works from shared memory (two shuffle
// reductions, no block-wide barrier), stores dx straight from registers and hands the stage
// back. The row statistics are loaded one chunk ahead. A lane owns the same columns for every
// row, so dgamma/dbeta partials stay in registers; the block folds its W warps in a fixed order
// at the end and writes ONE partial row (one per SM instead of one per small block).
// Shared memory: [nstages][ntens][W][cols] of T, then eight "full" and eight "empty" mbarriers,
// the abort word, and gamma as fp32. Every wait is bounded; an expired one is recorded as 104.
template <typename T, int NV, bool PART>
struct StagedCfg {
  // registers a row warp's thread holds across rows (the column partials) and for one vector
  static constexpr int kLiveRegs = (PART ? NV * Vec16<T>::N * 2 : 0) + NV * 4;
  static constexpr int kWarps = (kLiveRegs > 60 || NV >= 8) ? 8 : 16;   // row warps + the copy warp: 255 or 128 registers per thread
};

template <typename T, int NV, bool RMS, bool PART>
__global__ void __launch_bounds__(StagedCfg<T, NV, PART>::kWarps * 32, 1)
norm_bwd_staged(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd_in,
                const T* __restrict__ dy, const T* __restrict__ gamma, T* dx, float* __restrict__ partial,
                int64_t rows, int W, int nstages, bool want_dg, bool want_db, bool dx_acc, int* __restrict__ flag) {
  allow_dependents();
  constexpr int VN = Vec16<T>::N;
  constexpr int cols = NV * 32 * VN;
  constexpr uint32_t row_bytes = cols * sizeof(T);
  extern __shared__ __align__(128) uint8_t stage_mem[];
  const uint32_t ntens = dx_acc ? 3u : 2u;
  const uint32_t tens_bytes = (uint32_t)W * row_bytes;
  const uint32_t stage_bytes = tens_bytes * ntens;
  uint8_t* bars = stage_mem + (size_t)nstages * stage_bytes;           // 144 bytes: full[8], empty[8], abort word
  const uint32_t bar_full = sm100::smem_u32(bars), bar_empty = bar_full + 64u;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 128);
  float4* sgamma = reinterpret_cast<float4*>(bars + 144);               // gamma as fp32, [VN / 4][NV * 32] float4
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < nstages; ++s) {
      sm100::mbar_init(bar_full + 8u * s, 1);
      sm100::mbar_init(bar_empty + 8u * s, (uint32_t)W);
    }
    sm100::fence_barrier_init();
    sm100::fence_proxy_async();
  }
  __syncthreads();
  grid_dependency_wait();      // everything above touches shared memory only and may run under the previous kernel's tail
  const int64_t nchunks = (rows + W - 1) / W;
  float dg[PART ? NV : 1][VN], db[PART ? NV : 1][VN];
#pragma unroll
  for (int i = 0; i < (PART ? NV : 1); ++i)
#pragma unroll
    for (int e = 0; e < VN; ++e) { dg[i][e] = 0.f; db[i][e] = 0.f; }

  if (warp == W) {
    if (lane == 0) {
      int k = 0;
      for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++k) {
        const int s = k % nstages;
        if (k >= nstages && !sm100::mbar_wait(bar_empty + 8u * s, (uint32_t)(k / nstages - 1) & 1u, abort_flag)) break;
        const int64_t r0 = c * W;
        const uint32_t nr = (uint32_t)(rows - r0 < W ? rows - r0 : W);
        const uint32_t bytes = nr * row_bytes;
        const uint32_t dst = sm100::smem_u32(stage_mem) + (uint32_t)s * stage_bytes;
        sm100::mbar_expect_tx(bar_full + 8u * s, bytes * ntens);
        sm100::bulk_load_1d(dst, x + r0 * cols, bytes, bar_full + 8u * s);
        sm100::bulk_load_1d(dst + tens_bytes, dy + r0 * cols, bytes, bar_full + 8u * s);
        if (dx_acc) sm100::bulk_load_1d(dst + 2u * tens_bytes, dx + r0 * cols, bytes, bar_full + 8u * s);
      }
    }
  } else {
    // gamma is converted to fp32 once and kept in shared memory (quarter q of vector v at
    // [q][v]: a lane's 16-byte reads are contiguous across the warp); the row warps meet at
    // their own named barrier, the copy warp is already loading.
    if (gamma) {
      for (int v = threadIdx.x; v < NV * 32; v += W * 32) {
        Vec16<T> g;
        g.load(gamma + v * VN);
#pragma unroll
        for (int q = 0; q < VN / 4; ++q)
          sgamma[q * (NV * 32) + v] = make_float4(g.get(4 * q), g.get(4 * q + 1), g.get(4 * q + 2), g.get(4 * q + 3));
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(W * 32) : "memory");
    const float inv_cols = 1.f / cols;
    float mu_next = 0.f, rs_next = 0.f;
    {
      const int64_t row = (int64_t)blockIdx.x * W + warp;
      if (row < rows) { mu_next = RMS ? 0.f : mean[row]; rs_next = rstd_in[row]; }
    }
    int k = 0;
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++k) {
      const int s = k % nstages;
      const int64_t row = c * W + warp;
      const float mu = mu_next, rs = rs_next;
      {
        const int64_t nrow = (c + gridDim.x) * W + warp;    // this warp's row of the block's next chunk
        if (nrow < rows) { mu_next = RMS ? 0.f : mean[nrow]; rs_next = rstd_in[nrow]; }
      }
      if (!sm100::mbar_wait(bar_full + 8u * s, (uint32_t)(k / nstages) & 1u, abort_flag)) break;
      if (row < rows) {
        const uint8_t* sbase = stage_mem + (size_t)s * stage_bytes + (size_t)warp * row_bytes;
        const T* sx = reinterpret_cast<const T*>(sbase);
        const T* sdy = reinterpret_cast<const T*>(sbase + tens_bytes);
        const T* sold = reinterpret_cast<const T*>(sbase + 2u * tens_bytes);
        const float nmr = -mu * rs;        // x-hat = x * rs + nmr
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int vi = lane + i * 32;
          Vec16<T> xv, dv;
          xv.load(sx + vi * VN);
          dv.load(sdy + vi * VN);
#pragma unroll
          for (int q = 0; q < VN / 4; ++q) {
            float gq[4] = {1.f, 1.f, 1.f, 1.f};
            if (gamma) { const float4 g4 = sgamma[q * (NV * 32) + vi]; gq[0] = g4.x; gq[1] = g4.y; gq[2] = g4.z; gq[3] = g4.w; }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = 4 * q + j;
              const float xh = fmaf(xv.get(e), rs, nmr);
              const float d = dv.get(e);
              if (PART) { dg[i][e] = fmaf(d, xh, dg[i][e]); db[i][e] += d; }
              const float dxh = gamma ? d * gq[j] : d;
              s1 += dxh;
              s2 = fmaf(dxh, xh, s2);
            }
          }
        }
        s1 = warp_sum(s1) * inv_cols;
        s2 = warp_sum(s2) * inv_cols;
        if (RMS) s1 = 0.f;
        // dx = rs * (dxh - s1 - xh * s2) = dxh * rs + (xh * (-s2 * rs) - s1 * rs)
        const float nc1 = -s1 * rs, nc2 = -s2 * rs;
        // Second pass: x and dy are read from the stage again instead of being held in registers
        // across the reductions (the column partials already take 16 registers per vector).
        T* dxr = dx + row * cols;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int vi = lane + i * 32;
          Vec16<T> xv, dv, o;
          xv.load(sx + vi * VN);
          dv.load(sdy + vi * VN);
#pragma unroll
          for (int q = 0; q < VN / 4; ++q) {
            float gq[4] = {1.f, 1.f, 1.f, 1.f};
            if (gamma) { const float4 g4 = sgamma[q * (NV * 32) + vi]; gq[0] = g4.x; gq[1] = g4.y; gq[2] = g4.z; gq[3] = g4.w; }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = 4 * q + j;
              const float xh = fmaf(xv.get(e), rs, nmr);
              const float dxh = gamma ? dv.get(e) * gq[j] : dv.get(e);
              o.set(e, fmaf(dxh, rs, fmaf(xh, nc2, nc1)));
            }
          }
          if (dx_acc) {
            Vec16<T> old;
            old.load(sold + vi * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) o.set(e, o.get(e) + old.get(e));
          }
          o.store(dxr + vi * VN);
        }
      }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(bar_empty + 8u * s);
    }
  }
  __syncthreads();   // every wait is over: the abort word is final and no copy is in flight
  if (*abort_flag) {
    if (threadIdx.x == 0 && flag) atomicMax(flag, 104);   // a stage did not arrive (or was not handed back) in time
    return;
  }
  if (!PART || (!want_dg && !want_db)) return;
  // Fold the W warps' column partials in warp order through the (now idle) stage memory.
  float* red = reinterpret_cast<float*>(stage_mem);      // [W][2][cols]
  if (warp < W) {
#pragma unroll
    for (int i = 0; i < (PART ? NV : 1); ++i)
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        red[(size_t)(warp * 2) * cols + (lane + i * 32) * VN + e] = dg[i][e];
        red[(size_t)(warp * 2 + 1) * cols + (lane + i * 32) * VN + e] = db[i][e];
      }
  }
  __syncthreads();
  float* pg = partial + (size_t)blockIdx.x * 2 * cols;
  for (int t = threadIdx.x; t < 2 * cols; t += blockDim.x) {
    if (t < cols ? !want_dg : !want_db) continue;
    float a = 0.f;
    for (int w = 0; w < W; ++w) a += red[(size_t)w * 2 * cols + t];
    pg[t] = a;
  }
}

template <typename T, bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_block(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd_in,
               const T* __restrict__ dy, const T* __restrict__ gamma, T* __restrict__ dx,
               int64_t rows, int64_t cols, bool dx_acc = false) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const float mu = RMS ? 0.f : mean[row];
  const float rs = rstd_in[row];
  const T* xr = x + row * cols;
  const T* dyr = dy + row * cols;
  float s1 = 0.f, s2 = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float xh = (to_f(xr[c]) - mu) * rs;
    float dxh = to_f(dyr[c]) * (gamma ? to_f(gamma[c]) : 1.f);
    s1 += dxh;
    s2 += dxh * xh;
  }
  s1 = block_sum(s1, sh) / cols;
  s2 = block_sum(s2, sh) / cols;
  if (RMS) s1 = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float xh = (to_f(xr[c]) - mu) * rs;
    float dxh = to_f(dyr[c]) * (gamma ? to_f(gamma[c]) : 1.f);
    const float r_ = rs * (dxh - s1 - xh * s2);
    dx[row * cols + c] = from_f<T>(dx_acc ? to_f(dx[row * cols + c]) + r_ : r_);
  }
}

// Column sums for the fallback path: block (32 x 8) owns 32 columns, walks all rows.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_colsum(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd_in,
                const T* __restrict__ dy, float* __restrict__ dgamma, float* __restrict__ dbeta,
                int64_t rows, int64_t cols, int accumulate) {
  __shared__ float sg[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  float g = 0.f, b = 0.f;
  if (c < cols) {
    for (int64_t r = ty; r < rows; r += 8) {
      float d = to_f(dy[r * cols + c]);
      float xh = (to_f(x[r * cols + c]) - (RMS ? 0.f : mean[r])) * rstd_in[r];
      g += d * xh;
      b += d;
    }
  }
  sg[ty][tx] = g;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float ag = 0.f, ab = 0.f;
    for (int i = 0; i < 8; ++i) { ag += sg[i][tx]; ab += sb[i][tx]; }
    if (dgamma) dgamma[c] = accumulate ? dgamma[c] + ag : ag;
    if (dbeta) dbeta[c] = accumulate ? dbeta[c] + ab : ab;
  }
}

// Sums the per-block partial rows in a fixed order, so the result does not depend on
// scheduling: block = 8 columns x 128 row groups; row group g adds rows g, g+128, ... in
// order (about ten independent loads per thread, all in flight together), then the groups
// are folded by a fixed tree (shuffles within a warp, shared memory across warps).
// Grid (ceil(cols / 8), 2): blockIdx.y = 0 reduces dgamma, 1 dbeta. Eight columns are one
// 32-byte sector of a partial row (the partials are read from L2), and a 768-column norm
// spreads its 1184 partial rows over 192 blocks.
constexpr int kFinalizeGroups = 128;
constexpr int kFinalizeCols = 8;
__global__ void __launch_bounds__(kFinalizeCols * kFinalizeGroups)
norm_bwd_finalize(const float* __restrict__ partial, int nblocks, int cols,
                  float* __restrict__ dgamma, float* __restrict__ dbeta, int accumulate) {
  allow_dependents();
  grid_dependency_wait();
  constexpr int kWarps = kFinalizeCols * kFinalizeGroups / 32;     // 32: each warp holds 4 row groups x 8 columns
  __shared__ float sm[kWarps][kFinalizeCols], sm2[kWarps / 4][kFinalizeCols];
  float* out = blockIdx.y ? dbeta : dgamma;
  if (!out) return;
  const int tx = threadIdx.x % kFinalizeCols, ty = threadIdx.x / kFinalizeCols;
  const int c = blockIdx.x * kFinalizeCols + tx;
  const int w = threadIdx.x >> 5;
  float v = 0.f;
  if (c < cols) {
    const float* p = partial + (size_t)blockIdx.y * cols + c;
#pragma unroll 10
    for (int i = ty; i < nblocks; i += kFinalizeGroups) v += p[(size_t)i * 2 * cols];
  }
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  if ((threadIdx.x & 31) < kFinalizeCols) sm[w][tx] = v;
  __syncthreads();
  if (threadIdx.x < kWarps * kFinalizeCols) {       // 256 threads: thread = (warp row ty, column tx)
    v = sm[ty][tx];
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    if ((threadIdx.x & 31) < kFinalizeCols) sm2[w][tx] = v;
  }
  __syncthreads();
  if (threadIdx.x < kFinalizeCols && c < cols) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps / 4; ++i) a += sm2[i][tx];
    out[c] = accumulate ? out[c] + a : a;
  }
}

template <typename T, bool RMS>
static int norm_fwd_launch(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                           float* rstd, int64_t rows, int64_t cols, float eps, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  const T* xp = (const T*)x; const T* gp = (const T*)gamma; const T* bp = (const T*)beta; T* yp = (T*)y;
  bool vec = cols % VN == 0 && aligned16(x) && aligned16(y) && (!gamma || aligned16(gamma)) &&
             (!beta || aligned16(beta)) && cols / VN <= 32 * 8;
  if (rows == 0) return MT_OK;
  if (vec) {
    int nvec = (int)(cols / VN);
    dim3 grid((unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock)), block(kWarpsPerBlock * 32);
#define MT_FWD(MV) MT_CHECK_CUDA(launch_overlapped(norm_fwd_warp<T, MV, RMS>, grid, block, 0, st, xp, gp, bp, yp, mean, rstd, rows, (int)cols, eps))
    if (nvec <= 32) MT_FWD(1); else if (nvec <= 64) MT_FWD(2); else if (nvec <= 128) MT_FWD(4); else MT_FWD(8);
#undef MT_FWD
  } else {
    norm_fwd_block<T, RMS><<<(unsigned)rows, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, cols, eps);
  }
  MT_LAUNCH_CHECK();
  return MT_OK;
}

// Column sums over no rows are zero: with nothing to launch the parameter gradients are
// still defined (left alone when they accumulate into existing values).
static int norm_bwd_no_rows(float* dgamma, float* dbeta, int64_t cols, int accumulate, cudaStream_t st) {
  if (accumulate & 1) return MT_OK;
  if (dgamma) MT_CHECK_CUDA(cudaMemsetAsync(dgamma, 0, (size_t)cols * sizeof(float), st));
  if (dbeta) MT_CHECK_CUDA(cudaMemsetAsync(dbeta, 0, (size_t)cols * sizeof(float), st));
  return MT_OK;
}

// Launches norm_bwd_staged (+ the finalize pass) for rows of NV*32 vectors. W row warps and the
// number of stages follow from the shared memory: the most warps that still leave three stages.
template <typename T, int NV, bool RMS, bool PART>
static int norm_bwd_staged_launch(const T* xp, const float* mean, const float* rstd, const T* dyp, const T* gp, T* dxp,
                                  float* dgamma, float* dbeta, int64_t rows, int accumulate, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  constexpr int cols = NV * 32 * VN;
  constexpr int row_bytes = cols * (int)sizeof(T);
  constexpr int kSmemMax = 232448;                 // dynamic shared memory one block may have
  constexpr int kBarBytes = 16 * 8 + 16;           // at most 8 stages of two mbarriers, and the abort word
  const int ntens = (accumulate & 2) ? 3 : 2;
  const int gamma_bytes = gp ? cols * (int)sizeof(float) : 0;
  int W = 0, nst = 0;
  for (int warps = StagedCfg<T, NV, PART>::kWarps;; warps /= 2) {
    W = warps - 1;
    nst = (kSmemMax - kBarBytes - gamma_bytes) / (W * row_bytes * ntens);
    if (nst >= 3 || warps == 4) break;
  }
  if (nst > 6) nst = 6;
  MT_REQUIRE(nst >= 2, "norm_bwd: a row of %d bytes does not fit the staged kernel", row_bytes);
  static std::atomic<bool> attr_set[16];
  int dev = 0;
  MT_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16 || !attr_set[dev].load(std::memory_order_acquire)) {
    MT_CHECK_CUDA(cudaFuncSetAttribute(norm_bwd_staged<T, NV, RMS, PART>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax));
    if (dev >= 0 && dev < 16) attr_set[dev].store(true, std::memory_order_release);
  }
  const int64_t nchunks = (rows + W - 1) / W;
  const int grid = (int)(nchunks < sm_count() ? nchunks : sm_count());
  const bool wg = PART && dgamma != nullptr, wb = PART && dbeta != nullptr;
  TempBuf part((wg || wb) ? (size_t)grid * 2 * cols * sizeof(float) : 0, st);
  if (!part.ok()) return MT_ERR_CUDA;
  const size_t smem = (size_t)nst * W * row_bytes * ntens + kBarBytes + gamma_bytes;
  MT_CHECK_CUDA(launch_overlapped(norm_bwd_staged<T, NV, RMS, PART>, dim3(grid), dim3((W + 1) * 32), smem, st, xp, mean, rstd,
                                  dyp, gp, dxp, (float*)part.ptr, rows, W, nst, wg, wb, (accumulate & 2) != 0, device_flag_ptr()));
  MT_LAUNCH_CHECK();
  if (wg || wb) {
    MT_CHECK_CUDA(launch_overlapped(norm_bwd_finalize, dim3((unsigned)((cols + kFinalizeCols - 1) / kFinalizeCols), 2),
                                    dim3(kFinalizeCols * kFinalizeGroups), 0, st, (const float*)part.ptr, grid, cols,
                                    dgamma, dbeta, accumulate & 1));
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}

template <typename T, bool RMS>
static int norm_bwd_launch(const void* x, const float* mean, const float* rstd, const void* dy,
                           const void* gamma, void* dx, float* dgamma, float* dbeta, int64_t rows,
                           int64_t cols, int accumulate, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  const T* xp = (const T*)x; const T* dyp = (const T*)dy; const T* gp = (const T*)gamma; T* dxp = (T*)dx;
  if (rows == 0) return norm_bwd_no_rows(dgamma, dbeta, cols, accumulate, st);
  const bool al = cols % VN == 0 && aligned16(x) && aligned16(dy) && aligned16(dx) && (!gamma || aligned16(gamma));
  const bool vec = al && cols / VN <= 32 * 4;
  const int nvec_all = (int)(cols / VN);
  if (al && cols % (32 * VN) == 0 && nvec_all / 32 >= 2 && (nvec_all / 32 <= 6 || nvec_all / 32 == 8)) {
    // rows of 2..6 or 8 warps of vectors (512..1536 and 2048 half columns, 256..768 and 1024 fp32
    // columns): staged through shared memory, one block per SM
    const int wpr = nvec_all / 32;
    const bool part = dgamma != nullptr || dbeta != nullptr || !RMS;
#define MT_STAGED(NV)                                                                                                      \
  return part ? norm_bwd_staged_launch<T, NV, RMS, true>(xp, mean, rstd, dyp, gp, dxp, dgamma, dbeta, rows, accumulate, st) \
              : norm_bwd_staged_launch<T, NV, RMS, RMS ? false : true>(xp, mean, rstd, dyp, gp, dxp, dgamma, dbeta, rows, accumulate, st)
    if (wpr == 2) MT_STAGED(2); else if (wpr == 3) MT_STAGED(3); else if (wpr == 4) MT_STAGED(4); else if (wpr == 5) MT_STAGED(5);
    else if (wpr == 6) MT_STAGED(6); else MT_STAGED(8);
#undef MT_STAGED
  }
  if (vec) {
    int nvec = (int)(cols / VN);
    int64_t want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    // One wave: as many blocks as are resident at once (the widest variant holds
    // three 128-thread blocks per SM), so no block waits for a second wave.
    const int per_sm = nvec <= 32 ? 8 : nvec <= 64 ? 5 : nvec <= 96 ? 4 : 3;
    int grid = (int)(want < (int64_t)sm_count() * per_sm ? want : (int64_t)sm_count() * per_sm);
    bool wg = dgamma != nullptr, wb = dbeta != nullptr;
    TempBuf part((wg || wb) ? (size_t)grid * 2 * cols * sizeof(float) : 0, st);
    if (!part.ok()) return MT_ERR_CUDA;
    dim3 block(kWarpsPerBlock * 32);
#define MT_BWD(MV) norm_bwd_warp<T, MV, RMS><<<grid, block, 0, st>>>(xp, mean, rstd, dyp, gp, dxp, (float*)part.ptr, rows, (int)cols, wg, wb, (accumulate & 2) != 0)
    if (nvec <= 32) MT_BWD(1); else if (nvec <= 64) MT_BWD(2); else if (nvec <= 96) MT_BWD(3); else MT_BWD(4);
#undef MT_BWD
    MT_LAUNCH_CHECK();
    if (wg || wb) {
      norm_bwd_finalize<<<dim3((unsigned)((cols + kFinalizeCols - 1) / kFinalizeCols), 2), kFinalizeCols * kFinalizeGroups, 0, st>>>((const float*)part.ptr, grid, (int)cols,
                                                                        dgamma, dbeta, accumulate & 1);
      MT_LAUNCH_CHECK();
    }
  } else {
    norm_bwd_block<T, RMS><<<(unsigned)rows, 256, 0, st>>>(xp, mean, rstd, dyp, gp, dxp, rows, cols, (accumulate & 2) != 0);
    MT_LAUNCH_CHECK();
    if (dgamma || dbeta) {
      norm_bwd_colsum<T, RMS><<<(unsigned)((cols + 31) / 32), 256, 0, st>>>(xp, mean, rstd, dyp, dgamma, dbeta,
                                                                           rows, cols, accumulate & 1);
      MT_LAUNCH_CHECK();
    }
  }
  return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                     int64_t rows, int64_t cols, float eps, int dtype, void* stream) {
  MT_REQUIRE(x && y && rows >= 0 && cols > 0, "layernorm_fwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (norm_fwd_launch<T, false>(x, gamma, beta, y, mean, rstd, rows, cols, eps, as_stream(stream))));
  return MT_OK;
}
int mt_layernorm_bwd(const void* x, const float* mean, const float* rstd, const void* dy, const void* gamma,
                     void* dx, float* dgamma, float* dbeta, int64_t rows, int64_t cols, int accumulate,
                     int dtype, void* stream) {
  MT_REQUIRE(x && dy && dx && mean && rstd && rows >= 0 && cols > 0, "layernorm_bwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (norm_bwd_launch<T, false>(x, mean, rstd, dy, gamma, dx, dgamma, dbeta, rows, cols, accumulate, as_stream(stream))));
  return MT_OK;
}
int mt_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int64_t rows, int64_t cols,
                   float eps, int dtype, void* stream) {
  MT_REQUIRE(x && y && rows >= 0 && cols > 0, "rmsnorm_fwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (norm_fwd_launch<T, true>(x, gamma, nullptr, y, nullptr, rstd, rows, cols, eps, as_stream(stream))));
  return MT_OK;
}
int mt_rmsnorm_bwd(const void* x, const float* rstd, const void* dy, const void* gamma, void* dx,
                   float* dgamma, int64_t rows, int64_t cols, int accumulate, int dtype, void* stream) {
  MT_REQUIRE(x && dy && dx && rstd && rows >= 0 && cols > 0, "rmsnorm_bwd: bad arguments");
  MT_DISPATCH_FLOAT(dtype, T, return (norm_bwd_launch<T, true>(x, nullptr, rstd, dy, gamma, dx, dgamma, nullptr, rows, cols, accumulate, as_stream(stream))));
  return MT_OK;
}

}  // extern "C"

// ---- LayerNorm backward without any allocation ------------------------------
// The two-stage column reduction of the backward pass needs a scratch area for
// per-block partial sums. mt_layernorm_bwd takes it from the stream-ordered
// pool; this variant keeps it in a fixed device array that lives in the
// library image, so the call itself never allocates or frees.
namespace mt {
constexpr int kNoAllocMaxBlocks = 256;   // partial rows (grid size cap)
constexpr int kNoAllocMaxCols = 1024;    // widest row accepted (128 16-byte vectors of fp16/bf16; fp32 rows: 512)
static __device__ __align__(256) float g_ln_scratch[kNoAllocMaxBlocks * 2 * kNoAllocMaxCols];  // 2 MiB per GPU

// Device address of g_ln_scratch per device; in host code the symbol's name is
// only a handle, so the address is looked up once per device and cached.
// Two host threads that race on the first call both look the address up and store the same
// value, so an atomic slot per device is enough.
static std::atomic<float*> g_ln_scratch_ptr[16];

static int ln_scratch_address(float** out) {
  int dev = 0;
  MT_CHECK_CUDA(cudaGetDevice(&dev));
  MT_REQUIRE(dev >= 0 && dev < 16, "layernorm_bwd_noalloc: device index %d out of range", dev);
  float* cached = g_ln_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!cached) {
    void* p = nullptr;
    MT_CHECK_CUDA(cudaGetSymbolAddress(&p, g_ln_scratch));
    cached = static_cast<float*>(p);
    g_ln_scratch_ptr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return MT_OK;
}

template <typename T>
static int layernorm_bwd_noalloc_launch(const void* x, const float* mean, const float* rstd, const void* dy,
                                        const void* gamma, void* dx, float* dgamma, float* dbeta, int64_t rows,
                                        int64_t cols, int accumulate, float* scratch, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  const T* xp = (const T*)x; const T* dyp = (const T*)dy; const T* gp = (const T*)gamma; T* dxp = (T*)dx;
  MT_REQUIRE(cols % VN == 0 && cols / VN <= 32 * 4 && aligned16(x) && aligned16(dy) && aligned16(dx) &&
             (!gamma || aligned16(gamma)),
             "layernorm_bwd_noalloc: needs 16-byte aligned tensors and cols a multiple of %d, at most %d", VN, 128 * VN);
  if (rows == 0) return norm_bwd_no_rows(dgamma, dbeta, cols, accumulate, st);
  const int nvec = (int)(cols / VN);
  int64_t want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int grid = (int)(want < kNoAllocMaxBlocks ? want : kNoAllocMaxBlocks);
  const bool wg = dgamma != nullptr, wb = dbeta != nullptr;
  dim3 block(kWarpsPerBlock * 32);
  // every block writes its whole partial row, so nothing in the shared scratch has to start at zero
#define MT_BWD(MV) norm_bwd_warp<T, MV, false><<<grid, block, 0, st>>>(xp, mean, rstd, dyp, gp, dxp, scratch, rows, (int)cols, wg, wb, (accumulate & 2) != 0)
  if (nvec <= 32) MT_BWD(1); else if (nvec <= 64) MT_BWD(2); else MT_BWD(4);
#undef MT_BWD
  MT_LAUNCH_CHECK();
  if (wg || wb) {
    norm_bwd_finalize<<<dim3((unsigned)((cols + kFinalizeCols - 1) / kFinalizeCols), 2), kFinalizeCols * kFinalizeGroups, 0, st>>>(scratch, grid, (int)cols, dgamma, dbeta, accumulate & 1);
    MT_LAUNCH_CHECK();
  }
  return MT_OK;
}
}  // namespace mt

extern "C" int mt_layernorm_bwd_noalloc(const void* x, const float* mean, const float* rstd, const void* dy,
                                        const void* gamma, void* dx, float* dgamma, float* dbeta, int64_t rows,
                                        int64_t cols, int accumulate, int dtype, void* stream) {
  using namespace mt;
  MT_REQUIRE(x && dy && dx && mean && rstd && rows >= 0 && cols > 0, "layernorm_bwd_noalloc: bad arguments");
  MT_REQUIRE(cols <= kNoAllocMaxCols,
             "layernorm_bwd_noalloc: %lld columns exceed the fixed scratch (at most %d columns); use mt_layernorm_bwd",
             (long long)cols, kNoAllocMaxCols);
  float* scratch = nullptr;
  int rc = ln_scratch_address(&scratch);
  if (rc) return rc;
  MT_DISPATCH_FLOAT(dtype, T, return (layernorm_bwd_noalloc_launch<T>(x, mean, rstd, dy, gamma, dx, dgamma, dbeta, rows, cols, accumulate, scratch, as_stream(stream))));
  return MT_OK;
}
