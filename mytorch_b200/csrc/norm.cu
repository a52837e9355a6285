// LayerNorm and RMSNorm, forward and backward.
//
// Fast path: one warp per row, the row held in registers as 16-byte vectors
// (lane owns vectors lane, lane+32, ...), fp32 math, two warp-shuffle
// reductions. Because a lane owns the same columns for every row it visits,
// the backward kernel keeps dgamma/dbeta partial sums in registers across
// rows; blocks write one partial row each and a second kernel adds them in a
// fixed order (no atomics: results are bit-reproducible).
// Fallback (unaligned or very wide rows): one block per row, scalar loads.
//
// Algorithmic traffic (HBM roofline): forward 2*rows*cols*sizeof(T); backward
// 3*rows*cols*sizeof(T) (+ negligible stats and partials).
#include <atomic>

#include "common.cuh"
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

// Row-team variant for rows of exactly WPR*32 16-byte vectors (768 half columns = 3 warps, 1280 =
// 5, 768 fp32 columns = 6): a block is one team, a thread owns ONE vector (8 half columns) of every row the block
// visits, so its dgamma/dbeta accumulators are 16 registers instead of the 48-64 of the
// warp-per-row kernel and more warps fit an SM. kTeamRows rows are in flight per thread; the row
// sums of the team's warps meet in shared memory (one __syncthreads per kTeamRows rows, double
// buffered). The block's column partials need no further reduction: thread t owns columns
// [t*VN, t*VN+VN). Same partial layout as norm_bwd_warp.
constexpr int kTeamRows = 2;     // rows in flight per thread (x and dy: 2 x 16 bytes each); three measured the same, four spill
template <typename T, int WPR, bool RMS>
__global__ void __launch_bounds__(WPR * 32, 768 / (WPR * 32))
norm_bwd_team(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd_in,
              const T* __restrict__ dy, const T* __restrict__ gamma, T* __restrict__ dx,
              float* __restrict__ partial, int64_t rows, bool want_dg, bool want_db, bool dx_acc) {
  allow_dependents();
  grid_dependency_wait();
  constexpr int VN = Vec16<T>::N;
  constexpr int RB = kTeamRows;
  constexpr int cols = WPR * 32 * VN;
  __shared__ float part[2][RB][WPR][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = threadIdx.x * VN;
  float dg[VN], db[VN];
#pragma unroll
  for (int e = 0; e < VN; ++e) { dg[e] = 0.f; db[e] = 0.f; }
  Vec16<T> gv;
  if (gamma) gv.load(gamma + c0);
  const float inv_cols = 1.f / cols;
  int it = 0;
  for (int64_t r0 = (int64_t)blockIdx.x * RB; r0 < rows; r0 += (int64_t)gridDim.x * RB, ++it) {
    Vec16<T> xv[RB], dv[RB];
    float mu[RB], rs[RB];
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      const int64_t row = r0 + j < rows ? r0 + j : rows - 1;   // clamped: rows past the end are recomputed, not stored
      xv[j].load(x + row * cols + c0);
      dv[j].load(dy + row * cols + c0);
      mu[j] = RMS ? 0.f : mean[row];
      rs[j] = rstd_in[row];
    }
    float (*pp)[WPR][2] = part[it & 1];
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        const float xh = (xv[j].get(e) - mu[j]) * rs[j];
        const float d = dv[j].get(e);
        const float dxh = gamma ? d * gv.get(e) : d;
        s1 += dxh;
        s2 += dxh * xh;
        if (r0 + j < rows) { dg[e] += d * xh; db[e] += d; }
      }
      s1 = warp_sum(s1);
      s2 = warp_sum(s2);
      if (lane == 0) { pp[j][warp][0] = s1; pp[j][warp][1] = s2; }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < RB; ++j) {
      if (r0 + j >= rows) break;
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) { s1 += pp[j][w][0]; s2 += pp[j][w][1]; }
      s1 *= inv_cols;
      s2 *= inv_cols;
      if (RMS) s1 = 0.f;
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        const float xh = (xv[j].get(e) - mu[j]) * rs[j];
        const float dxh = gamma ? dv[j].get(e) * gv.get(e) : dv[j].get(e);
        o.set(e, rs[j] * (dxh - s1 - xh * s2));
      }
      T* dxr = dx + (r0 + j) * cols + c0;
      if (dx_acc) {
        Vec16<T> old;
        old.load(dxr);
#pragma unroll
        for (int e = 0; e < VN; ++e) o.set(e, o.get(e) + old.get(e));
      }
      o.store(dxr);
    }
  }
  if (want_dg) {
    float* pg = partial + (size_t)blockIdx.x * 2 * cols + c0;
#pragma unroll
    for (int e = 0; e < VN; ++e) pg[e] = dg[e];
  }
  if (want_db) {
    float* pb = partial + (size_t)blockIdx.x * 2 * cols + cols + c0;
#pragma unroll
    for (int e = 0; e < VN; ++e) pb[e] = db[e];
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
    // columns): one thread per vector
    const int wpr = nvec_all / 32;
    const int per_sm = 768 / (wpr * 32);      // resident blocks (the kernel is compiled for this occupancy)
    int64_t want = (rows + kTeamRows - 1) / kTeamRows;
    int grid = (int)(want < (int64_t)sm_count() * per_sm ? want : (int64_t)sm_count() * per_sm);
    bool wg = dgamma != nullptr, wb = dbeta != nullptr;
    TempBuf part((wg || wb) ? (size_t)grid * 2 * cols * sizeof(float) : 0, st);
    if (!part.ok()) return MT_ERR_CUDA;
#define MT_TEAM(W) MT_CHECK_CUDA(launch_overlapped(norm_bwd_team<T, W, RMS>, dim3(grid), dim3(W * 32), 0, st, xp, mean, rstd, dyp, gp, dxp, (float*)part.ptr, rows, wg, wb, (accumulate & 2) != 0))
    if (wpr == 2) MT_TEAM(2); else if (wpr == 3) MT_TEAM(3); else if (wpr == 4) MT_TEAM(4); else if (wpr == 5) MT_TEAM(5);
    else if (wpr == 6) MT_TEAM(6); else MT_TEAM(8);
#undef MT_TEAM
    MT_LAUNCH_CHECK();
    if (wg || wb) {
      MT_CHECK_CUDA(launch_overlapped(norm_bwd_finalize, dim3((unsigned)((cols + kFinalizeCols - 1) / kFinalizeCols), 2),
                                      dim3(kFinalizeCols * kFinalizeGroups), 0, st, (const float*)part.ptr, grid, (int)cols,
                                      dgamma, dbeta, accumulate & 1));
      MT_LAUNCH_CHECK();
    }
    return MT_OK;
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
