// CUDA-core attention (forward and backward), fp32 math for any element type.
// It is the full-precision path for fp32 tensors (tensor cores would round the
// operands) and the fallback for shapes the tensor-core kernels do not take.
//
// One warp owns one query row (forward, dQ) or one key/value row (dK, dV) and
// walks the other sequence in tiles of 32 staged in shared memory; lanes split
// the 32 tile rows for the dot products and split head_dim for the
// accumulators. Online softmax in the forward; the backward recomputes
// probabilities from the saved log-sum-exp. No atomics: results are
// reproducible. Tensors are addressed as base + b*sb + h*sh + row*ss + d.
#include "common.cuh"
#include "attention.cuh"

namespace mt {

constexpr int kTile = 32;
constexpr int kMaxD = 128;
constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 2;
constexpr int kRowsPerBlock = kWarps * kRowsPerWarp;

template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* src, int64_t row_stride, int row0, int nrows_total,
                                          int D) {
  // dst[r][d] for r in [0,32): rows beyond the sequence are zero
  for (int i = threadIdx.x; i < kTile * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    int gr = row0 + r;
    dst[r * ld + d] = gr < nrows_total ? to_f(src[(int64_t)gr * row_stride + d]) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_fwd_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
              float* __restrict__ lse, mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 so,
              int heads, int group, int S, int D, float scale, int causal) {
  extern __shared__ float sm[];
  const int ld = D + 1;
  float* Ks = sm;                       // [32][ld]
  float* Vs = Ks + kTile * ld;          // [32][ld]
  float* Qs = Vs + kTile * ld;          // [rows_per_block][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int row_base = blockIdx.x * kRowsPerBlock;
  const T* qb = q + (int64_t)b * sq.b + (int64_t)h * sq.h;
  const T* kb = k + (int64_t)b * sk.b + (int64_t)(h / group) * sk.h;      // query head h reads key/value head h / group
  const T* vb = v + (int64_t)b * sv.b + (int64_t)(h / group) * sv.h;
  T* ob = o + (int64_t)b * so.b + (int64_t)h * so.h;
  for (int i = threadIdx.x; i < kRowsPerBlock * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    int gr = row_base + r;
    Qs[r * D + d] = gr < S ? to_f(qb[(int64_t)gr * sq.s + d]) * scale : 0.f;
  }
  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][kMaxD / 32];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) acc[r][c] = 0.f;
  }
  const int last_row = min(row_base + kRowsPerBlock, S) - 1;
  const int kv_end = causal ? last_row + 1 : S;
  for (int t0 = 0; t0 < kv_end; t0 += kTile) {
    __syncthreads();
    load_tile(Ks, ld, kb, sk.s, t0, S, D);
    load_tile(Vs, ld, vb, sv.s, t0, S, D);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lr = warp * kRowsPerWarp + r, gr = row_base + lr;
      if (gr >= S) continue;
      const int j = t0 + lane;
      float s = 0.f;
      const float* qr = Qs + lr * D;
      const float* kr = Ks + lane * ld;
      for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      const bool valid = j < S && (!causal || j <= gr);
      s = valid ? s : -INFINITY;
      const float mt_ = warp_max(s);
      if (mt_ == -INFINITY) continue;   // whole tile masked for this row
      const float mn = fmaxf(m[r], mt_);
      const float corr = m[r] == -INFINITY ? 0.f : __expf(m[r] - mn);
      const float p = valid ? __expf(s - mn) : 0.f;
      l[r] = l[r] * corr + warp_sum(p);
      m[r] = mn;
#pragma unroll
      for (int c = 0; c < kMaxD / 32; ++c) acc[r][c] *= corr;
      for (int jj = 0; jj < kTile; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
        for (int c = 0; c < kMaxD / 32; ++c) {
          int d = lane + c * 32;
          if (d < D) acc[r][c] = fmaf(pj, Vs[jj * ld + d], acc[r][c]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int gr = row_base + warp * kRowsPerWarp + r;
    if (gr >= S) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) {
      int d = lane + c * 32;
      if (d < D) ob[(int64_t)gr * so.s + d] = from_f<T>(acc[r][c] * inv);
    }
    if (lane == 0) lse[((int64_t)bh) * S + gr] = m[r] + __logf(l[r]);
  }
}

// delta[b,h,i] = sum_d dO[i,d] * O[i,d]. Eight lanes per row, 16-byte loads when
// head_dim and the strides allow (traffic: one read of O and dO).
template <typename T>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, mt_strides3 so,
                  mt_strides3 sdo, int heads, int S, int D, int64_t total_rows, int vec) {
  constexpr int VN = Vec16<T>::N;
  const int sub = threadIdx.x & 7;
  const int64_t row = (int64_t)blockIdx.x * 32 + (threadIdx.x >> 3);
  float s = 0.f;
  if (row < total_rows) {
    const int64_t bh = row / S;
    const int i = (int)(row - bh * S);
    const int b = (int)(bh / heads), h = (int)(bh % heads);
    const T* op = o + (int64_t)b * so.b + (int64_t)h * so.h + (int64_t)i * so.s;
    const T* dp = d_o + (int64_t)b * sdo.b + (int64_t)h * sdo.h + (int64_t)i * sdo.s;
    if (vec) {
      for (int d = sub * VN; d < D; d += 8 * VN) {
        Vec16<T> a, g;
        a.load(op + d);
        g.load(dp + d);
#pragma unroll
        for (int e = 0; e < VN; ++e) s += a.get(e) * g.get(e);
      }
    } else {
      for (int d = sub; d < D; d += 8) s += to_f(op[d]) * to_f(dp[d]);
    }
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (sub == 0 && row < total_rows) delta[row] = s;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_bwd_dq_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ d_o,
                 const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq, mt_strides3 sq,
                 mt_strides3 sk, mt_strides3 sv, mt_strides3 sdo, mt_strides3 sdq, int heads, int group, int S, int D,
                 float scale, int causal) {
  extern __shared__ float sm[];
  const int ld = D + 1;
  float* Ks = sm;
  float* Vs = Ks + kTile * ld;
  float* Qs = Vs + kTile * ld;                 // [rows][D], pre-scaled
  float* Gs = Qs + kRowsPerBlock * D;          // dO rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int row_base = blockIdx.x * kRowsPerBlock;
  const T* qb = q + (int64_t)b * sq.b + (int64_t)h * sq.h;
  const T* kb = k + (int64_t)b * sk.b + (int64_t)(h / group) * sk.h;      // query head h reads key/value head h / group
  const T* vb = v + (int64_t)b * sv.b + (int64_t)(h / group) * sv.h;
  const T* gb = d_o + (int64_t)b * sdo.b + (int64_t)h * sdo.h;
  T* dqb = dq + (int64_t)b * sdq.b + (int64_t)h * sdq.h;
  for (int i = threadIdx.x; i < kRowsPerBlock * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    int gr = row_base + r;
    Qs[r * D + d] = gr < S ? to_f(qb[(int64_t)gr * sq.s + d]) * scale : 0.f;
    Gs[r * D + d] = gr < S ? to_f(gb[(int64_t)gr * sdo.s + d]) : 0.f;
  }
  float acc[kRowsPerWarp][kMaxD / 32];
  float lrow[kRowsPerWarp], drow[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int gr = row_base + warp * kRowsPerWarp + r;
    lrow[r] = gr < S ? lse[(int64_t)bh * S + gr] : 0.f;
    drow[r] = gr < S ? delta[(int64_t)bh * S + gr] : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) acc[r][c] = 0.f;
  }
  const int last_row = min(row_base + kRowsPerBlock, S) - 1;
  const int kv_end = causal ? last_row + 1 : S;
  for (int t0 = 0; t0 < kv_end; t0 += kTile) {
    __syncthreads();
    load_tile(Ks, ld, kb, sk.s, t0, S, D);
    load_tile(Vs, ld, vb, sv.s, t0, S, D);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lr = warp * kRowsPerWarp + r, gr = row_base + lr;
      if (gr >= S) continue;
      const int j = t0 + lane;
      const float* qr = Qs + lr * D;
      const float* gr_ = Gs + lr * D;
      const float* kr = Ks + lane * ld;
      const float* vr = Vs + lane * ld;
      float s = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) { s = fmaf(qr[d], kr[d], s); dp = fmaf(gr_[d], vr[d], dp); }
      const bool valid = j < S && (!causal || j <= gr);
      const float p = valid ? __expf(s - lrow[r]) : 0.f;
      const float ds = p * (dp - drow[r]) * scale;
      for (int jj = 0; jj < kTile; ++jj) {
        const float dj = __shfl_sync(0xffffffffu, ds, jj);
#pragma unroll
        for (int c = 0; c < kMaxD / 32; ++c) {
          int d = lane + c * 32;
          if (d < D) acc[r][c] = fmaf(dj, Ks[jj * ld + d], acc[r][c]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int gr = row_base + warp * kRowsPerWarp + r;
    if (gr >= S) continue;
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) {
      int d = lane + c * 32;
      if (d < D) dqb[(int64_t)gr * sdq.s + d] = from_f<T>(acc[r][c]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_bwd_dkv_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ d_o,
                  const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dk,
                  T* __restrict__ dv, mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 sdo,
                  mt_strides3 sdk, mt_strides3 sdv, int heads, int group, int S, int D, float scale, int causal) {
  extern __shared__ float sm[];
  const int ld = D + 1;
  float* Qs = sm;                               // [32][ld] query tile (unscaled)
  float* Gs = Qs + kTile * ld;                  // [32][ld] dO tile
  float* Ks = Gs + kTile * ld;                  // [rows][D] this block's key rows
  float* Vs = Ks + kRowsPerBlock * D;           // [rows][D] value rows
  float* Ls = Vs + kRowsPerBlock * D;           // [32] lse of the query tile
  float* Ds = Ls + kTile;                       // [32] delta of the query tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // `heads` counts key/value heads here: the block owns rows of one key/value head and sums the
  // contributions of the `group` query heads that read it
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int row_base = blockIdx.x * kRowsPerBlock;
  const T* kb = k + (int64_t)b * sk.b + (int64_t)h * sk.h;
  const T* vb = v + (int64_t)b * sv.b + (int64_t)h * sv.h;
  for (int i = threadIdx.x; i < kRowsPerBlock * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    int gr = row_base + r;
    Ks[r * D + d] = gr < S ? to_f(kb[(int64_t)gr * sk.s + d]) : 0.f;
    Vs[r * D + d] = gr < S ? to_f(vb[(int64_t)gr * sv.s + d]) : 0.f;
  }
  float acck[kRowsPerWarp][kMaxD / 32], accv[kRowsPerWarp][kMaxD / 32];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) { acck[r][c] = 0.f; accv[r][c] = 0.f; }
  // causal: only queries i >= j contribute; start at the tile holding row_base
  const int q_begin = causal ? (row_base / kTile) * kTile : 0;
  for (int gq = 0; gq < group; ++gq) {
  const int hq = h * group + gq;
  const int64_t bhq = (int64_t)b * heads * group + hq;       // index of the query head in [B, H] (lse, delta)
  const T* qb = q + (int64_t)b * sq.b + (int64_t)hq * sq.h;
  const T* gb = d_o + (int64_t)b * sdo.b + (int64_t)hq * sdo.h;
  for (int t0 = q_begin; t0 < S; t0 += kTile) {
    __syncthreads();
    load_tile(Qs, ld, qb, sq.s, t0, S, D);
    load_tile(Gs, ld, gb, sdo.s, t0, S, D);
    if (threadIdx.x < kTile) {
      int gi = t0 + threadIdx.x;
      Ls[threadIdx.x] = gi < S ? lse[bhq * S + gi] : 0.f;
      Ds[threadIdx.x] = gi < S ? delta[bhq * S + gi] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lr = warp * kRowsPerWarp + r, gj = row_base + lr;
      if (gj >= S) continue;
      const int i = t0 + lane;                 // this lane's query
      const float* kr = Ks + lr * D;
      const float* vr = Vs + lr * D;
      const float* qr = Qs + lane * ld;
      const float* gr_ = Gs + lane * ld;
      float s = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) { s = fmaf(qr[d], kr[d], s); dp = fmaf(gr_[d], vr[d], dp); }
      const bool valid = i < S && (!causal || gj <= i);
      const float p = valid ? __expf(s * scale - Ls[lane]) : 0.f;
      const float ds = p * (dp - Ds[lane]) * scale;
      for (int ii = 0; ii < kTile; ++ii) {
        const float pi = __shfl_sync(0xffffffffu, p, ii);
        const float di = __shfl_sync(0xffffffffu, ds, ii);
#pragma unroll
        for (int c = 0; c < kMaxD / 32; ++c) {
          int d = lane + c * 32;
          if (d < D) {
            accv[r][c] = fmaf(pi, Gs[ii * ld + d], accv[r][c]);
            acck[r][c] = fmaf(di, Qs[ii * ld + d], acck[r][c]);
          }
        }
      }
    }
  }
  }
  T* dkb = dk + (int64_t)b * sdk.b + (int64_t)h * sdk.h;
  T* dvb = dv + (int64_t)b * sdv.b + (int64_t)h * sdv.h;
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int gj = row_base + warp * kRowsPerWarp + r;
    if (gj >= S) continue;
#pragma unroll
    for (int c = 0; c < kMaxD / 32; ++c) {
      int d = lane + c * 32;
      if (d < D) {
        dkb[(int64_t)gj * sdk.s + d] = from_f<T>(acck[r][c]);
        dvb[(int64_t)gj * sdv.s + d] = from_f<T>(accv[r][c]);
      }
    }
  }
}

int attn_delta(const AttnArgs& a, cudaStream_t st) {
  const int64_t rows = a.batch * a.heads * a.seq;
  if (rows == 0) return MT_OK;
  MT_DISPATCH_FLOAT(a.dtype, T, {
    constexpr int VN = Vec16<T>::N;
    auto ok = [&](const mt_strides3& s) { return s.b % VN == 0 && s.h % VN == 0 && s.s % VN == 0; };
    const int vec = a.head_dim % VN == 0 && aligned16(a.o) && aligned16(a.d_o) && ok(a.so) && ok(a.sdo);
    attn_delta_kernel<T><<<(unsigned)((rows + 31) / 32), 256, 0, st>>>(
        (const T*)a.o, (const T*)a.d_o, a.delta, a.so, a.sdo, (int)a.heads, (int)a.seq, (int)a.head_dim, rows, vec);
  });
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int attn_fwd_simt_launch(const AttnArgs& a, cudaStream_t st) {
  const int S = (int)a.seq, D = (int)a.head_dim;
  if (a.batch * a.heads * a.seq == 0) return MT_OK;
  MT_REQUIRE(D <= kMaxD && D > 0, "attention: head_dim must be in [1,128]");
  dim3 grid((S + kRowsPerBlock - 1) / kRowsPerBlock, (unsigned)(a.batch * a.heads));
  MT_REQUIRE(a.batch * a.heads <= 65535, "attention: batch*heads too large for the CUDA-core kernel");
  size_t smem = (size_t)(2 * kTile * (D + 1) + kRowsPerBlock * D) * sizeof(float);
  MT_DISPATCH_FLOAT(a.dtype, T, MT_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_simt<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536)));
  MT_DISPATCH_FLOAT(a.dtype, T, (attn_fwd_simt<T><<<grid, kWarps * 32, smem, st>>>(
      (const T*)a.q, (const T*)a.k, (const T*)a.v, (T*)a.o_out, a.lse, a.sq, a.sk, a.sv, a.so, (int)a.heads, (int)(a.heads / a.kv_heads), S, D, a.scale, a.causal)));
  MT_LAUNCH_CHECK();
  return MT_OK;
}

int attn_bwd_simt_launch(const AttnArgs& a, cudaStream_t st) {
  const int S = (int)a.seq, D = (int)a.head_dim;
  if (a.batch * a.heads * a.seq == 0) return MT_OK;
  MT_REQUIRE(D <= kMaxD && D > 0, "attention: head_dim must be in [1,128]");
  MT_REQUIRE(a.batch * a.heads <= 65535, "attention: batch*heads too large for the CUDA-core kernel");
  int rc = attn_delta(a, st);
  if (rc) return rc;
  dim3 grid((S + kRowsPerBlock - 1) / kRowsPerBlock, (unsigned)(a.batch * a.heads));
  size_t smem_dq = (size_t)(2 * kTile * (D + 1) + 2 * kRowsPerBlock * D) * sizeof(float);
  size_t smem_dkv = (size_t)(2 * kTile * (D + 1) + 2 * kRowsPerBlock * D + 2 * kTile) * sizeof(float);
  MT_DISPATCH_FLOAT(a.dtype, T, {
    MT_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dq_simt<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
    MT_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_simt<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
    attn_bwd_dq_simt<T><<<grid, kWarps * 32, smem_dq, st>>>((const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.d_o,
        a.lse, a.delta, (T*)a.dq, a.sq, a.sk, a.sv, a.sdo, a.sdq, (int)a.heads, (int)(a.heads / a.kv_heads), S, D, a.scale, a.causal);
    dim3 grid_kv((S + kRowsPerBlock - 1) / kRowsPerBlock, (unsigned)(a.batch * a.kv_heads));
    attn_bwd_dkv_simt<T><<<grid_kv, kWarps * 32, smem_dkv, st>>>((const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.d_o,
        a.lse, a.delta, (T*)a.dk, (T*)a.dv, a.sq, a.sk, a.sv, a.sdo, a.sdk, a.sdv, (int)a.kv_heads, (int)(a.heads / a.kv_heads),
        S, D, a.scale, a.causal);
  });
  MT_LAUNCH_CHECK();
  count_launch(1);
  return MT_OK;
}

}  // namespace mt
