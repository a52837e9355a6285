// C entry points for attention: argument checks and the choice between the
// tensor-core kernels (fp16/bf16, head_dim 64 or 128, aligned strides) and the
// CUDA-core kernels (everything else, and all fp32).
#include "common.cuh"
#include "attention.cuh"
#include "prof.cuh"

using namespace mt;

static int g_attn_force_simt = 0;

extern "C" {

int mt_attn_force_simt(int on) { g_attn_force_simt = on; return MT_OK; }

int mt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, mt_strides3 sq, mt_strides3 sk,
                mt_strides3 sv, mt_strides3 so, int64_t batch, int64_t heads, int64_t seq, int64_t head_dim,
                float scale, int causal, int dtype, void* stream) {
  return mt_attn_fwd_gqa(q, k, v, o, lse, sq, sk, sv, so, batch, heads, heads, seq, head_dim, scale, causal, dtype, stream);
}

int mt_attn_fwd_gqa(const void* q, const void* k, const void* v, void* o, float* lse, mt_strides3 sq, mt_strides3 sk,
                    mt_strides3 sv, mt_strides3 so, int64_t batch, int64_t heads, int64_t kv_heads, int64_t seq,
                    int64_t head_dim, float scale, int causal, int dtype, void* stream) {
  MT_REQUIRE(q && k && v && o && lse && batch >= 0 && heads > 0 && seq >= 0 && head_dim > 0, "attn_fwd: bad arguments");
  MT_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attn_fwd: %lld query heads are not a multiple of %lld key/value heads",
             (long long)heads, (long long)kv_heads);
  AttnArgs a{};
  a.kv_heads = kv_heads;
  a.q = q; a.k = k; a.v = v; a.o_out = o; a.lse = lse;
  a.sq = sq; a.sk = sk; a.sv = sv; a.so = so;
  a.batch = batch; a.heads = heads; a.seq = seq; a.head_dim = head_dim;
  a.scale = scale; a.causal = causal; a.dtype = dtype;
  cudaStream_t st = as_stream(stream);
  const double flops = 4.0 * batch * heads * (double)seq * seq * head_dim * (causal ? 0.5 : 1.0);
  ProfScope prof(PROF_ATTN, st, flops);
  if (!g_attn_force_simt && attn_tc_supported(a, false)) return attn_fwd_tc(a, st);
  return attn_fwd_simt_launch(a, st);
}

int mt_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                void* dq, void* dk, void* dv, float* delta, float* dq_accum, mt_strides3 sq, mt_strides3 sk,
                mt_strides3 sv, mt_strides3 so, mt_strides3 sdo, mt_strides3 sdq, mt_strides3 sdk, mt_strides3 sdv,
                int64_t batch, int64_t heads, int64_t seq, int64_t head_dim, float scale, int causal, int dtype,
                void* stream) {
  return mt_attn_bwd_gqa(q, k, v, o, d_o, lse, dq, dk, dv, delta, dq_accum, sq, sk, sv, so, sdo, sdq, sdk, sdv, batch, heads,
                         heads, seq, head_dim, scale, causal, dtype, stream);
}

int mt_attn_bwd_gqa(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                    void* dq, void* dk, void* dv, float* delta, float* dq_accum, mt_strides3 sq, mt_strides3 sk,
                    mt_strides3 sv, mt_strides3 so, mt_strides3 sdo, mt_strides3 sdq, mt_strides3 sdk, mt_strides3 sdv,
                    int64_t batch, int64_t heads, int64_t kv_heads, int64_t seq, int64_t head_dim, float scale,
                    int causal, int dtype, void* stream) {
  MT_REQUIRE(q && k && v && o && d_o && lse && dq && dk && dv && delta && batch >= 0 && heads > 0 && seq >= 0 &&
             head_dim > 0, "attn_bwd: bad arguments");
  MT_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attn_bwd: %lld query heads are not a multiple of %lld key/value heads",
             (long long)heads, (long long)kv_heads);
  AttnArgs a{};
  a.kv_heads = kv_heads;
  a.q = q; a.k = k; a.v = v; a.o = o; a.d_o = d_o; a.lse = const_cast<float*>(lse);
  a.dq = dq; a.dk = dk; a.dv = dv; a.delta = delta; a.dq_accum = dq_accum;
  a.sq = sq; a.sk = sk; a.sv = sv; a.so = so; a.sdo = sdo; a.sdq = sdq; a.sdk = sdk; a.sdv = sdv;
  a.batch = batch; a.heads = heads; a.seq = seq; a.head_dim = head_dim;
  a.scale = scale; a.causal = causal; a.dtype = dtype;
  cudaStream_t st = as_stream(stream);
  const double flops = 10.0 * batch * heads * (double)seq * seq * head_dim * (causal ? 0.5 : 1.0);
  ProfScope prof(PROF_ATTN, st, flops);
  if (!g_attn_force_simt && dq_accum && attn_tc_supported(a, true)) return attn_bwd_tc(a, st);
  return attn_bwd_simt_launch(a, st);
}

}  // extern "C"
