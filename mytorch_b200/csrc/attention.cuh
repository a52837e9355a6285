// Internal attention interface shared by the tensor-core and CUDA-core kernels.
#pragma once
#include "common.cuh"

namespace mt {
struct AttnArgs {
  const void *q, *k, *v, *o, *d_o;
  void* o_out;
  float* lse;
  void *dq, *dk, *dv;
  float* delta;
  float* dq_accum;
  mt_strides3 sq, sk, sv, so, sdo, sdq, sdk, sdv;
  int64_t batch, heads, seq, head_dim;
  int64_t kv_heads;   // heads of k, v, dk, dv; query head h reads key/value head h / (heads / kv_heads)
  float scale;
  int causal, dtype;
};
int attn_delta(const AttnArgs& a, cudaStream_t st);
int attn_fwd_simt_launch(const AttnArgs& a, cudaStream_t st);
int attn_bwd_simt_launch(const AttnArgs& a, cudaStream_t st);
bool attn_tc_supported(const AttnArgs& a, bool backward);
int attn_fwd_tc(const AttnArgs& a, cudaStream_t st);
int attn_bwd_tc(const AttnArgs& a, cudaStream_t st);
}  // namespace mt
