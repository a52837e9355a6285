// Tensor-core attention for sm_100a (placeholder translation unit: the
// tcgen05 kernels are not enabled yet, so every shape takes the CUDA-core path).
#include "common.cuh"
#include "attention.cuh"

namespace mt {
bool attn_tc_supported(const AttnArgs&, bool) { return false; }
int attn_fwd_tc(const AttnArgs&, cudaStream_t) { set_error("tensor-core attention not built"); return MT_ERR_UNSUPPORTED; }
int attn_bwd_tc(const AttnArgs&, cudaStream_t) { set_error("tensor-core attention not built"); return MT_ERR_UNSUPPORTED; }
}  // namespace mt
