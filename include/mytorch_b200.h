/*
 * mytorch_b200 — C ABI of the sm_100a library behind MyTorch's GPT training step.
 *
 * Every entry point is what a Python `ctypes` binding of the reference would
 * bind in place of one of its Triton/CuPy calls; the comment above each group
 * names the reference function it replaces (path:line inside the reference
 * project). Conventions:
 *   - plain device pointers, sizes and scalars; the CALLER owns every buffer
 *     (the library keeps no reference after a call returns, except for objects
 *     with an explicit destroy call);
 *   - `dtype` is an mt_dtype code for the floating-point tensors of the call;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     no compute entry point synchronises with the host;
 *   - the return value is an mt_status (0 = ok); mt_last_error() returns the
 *     text of the last failure on the calling thread.
 * Rows are the flattened leading dimensions ([B,T,E] is passed as rows=B*T).
 */
#ifndef MYTORCH_B200_H
#define MYTORCH_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { MT_F32 = 0, MT_F16 = 1, MT_BF16 = 2 } mt_dtype;
typedef enum {
  MT_OK = 0, MT_ERR_INVALID = 1, MT_ERR_DTYPE = 2, MT_ERR_CUDA = 3,
  MT_ERR_NCCL = 4, MT_ERR_TIMEOUT = 5, MT_ERR_UNSUPPORTED = 6, MT_ERR_DEVICE_FLAG = 7
} mt_status;
typedef enum { MT_ACT_NONE = 0, MT_ACT_GELU = 1, MT_ACT_RELU2 = 2, MT_ACT_RELU = 3 } mt_act;
#define MT_ACT_STORE_GRAD 0x100   /* mt_gemm / mt_gemm_ex only, see there */

/* ---- runtime: device arrays, copies, streams, events ----------------------
 * Replaces the CuPy allocator / cp.asarray / cp.asnumpy / cp.cuda.Event used
 * through mytorch/_array.py:199-249 and mytorch/tensor.py:221-261. */
const char* mt_last_error(void);
int mt_version(void);
int mt_device_count(int* count);
int mt_set_device(int device);
int mt_get_device(int* device);
int mt_device_sm_count(int* count);
int mt_malloc(void** ptr, size_t bytes, void* stream);      /* stream-ordered, pooled */
int mt_free(void* ptr, void* stream);
int mt_host_alloc(void** ptr, size_t bytes);                /* pinned host memory */
int mt_host_free(void* ptr);
int mt_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
int mt_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int mt_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int mt_memset(void* dst, int byte, size_t bytes, void* stream);
int mt_stream_create(void** stream);
int mt_stream_destroy(void* stream);
int mt_stream_sync(void* stream);
int mt_device_sync(void);
int mt_event_create(void** event);
int mt_event_destroy(void* event);
int mt_event_record(void* event, void* stream);
int mt_event_sync(void* event);
int mt_event_elapsed_ms(void* start, void* stop, float* ms);
int mt_stream_wait_event(void* stream, void* event);
int mt_mem_info(size_t* free_bytes, size_t* total_bytes);
/* Device status word: kernels that give up on a bounded wait or see an
 * out-of-range index record a code here instead of trapping (the largest code
 * seen is kept). Reads it back (synchronising `stream`) and clears it.
 * 0 = nothing recorded; 1 = embedding index out of range (row skipped);
 * 2 = cross-entropy label out of range (row ignored); an expired bounded wait:
 * 100 = tensor-core GEMM, 101 = attention forward, 102 = attention backward,
 * 103 = staged cross entropy, 104 = staged LayerNorm / RMSNorm backward. */
int mt_device_flag_read(int* flag, void* stream);

/* Per-kernel-class timing with CUDA events on the launching stream.
 * kind: 0 = off, 1 = tensor-core GEMM launches, 2 = attention launches. */
int mt_prof_begin(int kind);
int mt_prof_end(double* total_ms, int64_t* launches, double* total_flops);
int64_t mt_launch_count(void);            /* kernels launched by this library so far */
/* NVTX range on the calling thread (visible in a timeline profiler, free without one). The
 * ctypes layer opens one per library call when MT_TRACE=nvtx is set in the environment, and
 * times every call with CUDA events when MT_TRACE=time is (the reference's per-closure timer
 * of mytorch/tensor.py:221-261 is Tensor.backward(time_backward=True)). */
int mt_range_push(const char* name);
int mt_range_pop(void);

/* ---- elementwise (CuPy ufuncs reached through mytorch/_array.py:422-470 and
 * the autograd closures of mytorch/tensor.py:272-330, 596-640) -------------- */
int mt_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream);
/* uint16 token ids (the on-disk format of gpt2_trainer/train_gpt2.py:150) -> int32 indices,
 * so that batches cross PCIe at two bytes per token. */
int mt_widen_u16_i32(const void* src_u16, void* dst_i32, int64_t n, void* stream);
/* y = cap * tanh(x / cap), the logit soft cap of the nanochat model's inference branch
 * (nanochat_trainer/core/nanochat_gpt.py:336). */
int mt_softcap(const void* x, void* y, int64_t n, float cap, int dtype, void* stream);
int mt_fill(void* dst, int dtype, float value, int64_t n, void* stream);
int mt_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);          /* out = a + b */
int mt_axpby(const void* x, float alpha, void* y, float beta, int64_t n, int x_dtype, int y_dtype, void* stream); /* y = alpha*x + beta*y */
int mt_scale(void* x, float alpha, int64_t n, int dtype, void* stream);
int mt_add_rowvec(const void* a, const void* v, void* out, int64_t rows, int64_t cols, int dtype, void* stream); /* out[r,:] = a[r,:] + v */
int mt_colsum(const void* a, void* out, int64_t rows, int64_t cols, int dtype, int out_dtype, int accumulate, void* stream); /* out[c] (+)= sum_r a[r,c] */
int mt_sum_f32(const void* x, int dtype, int64_t n, float* out, void* stream);                    /* out[0] = sum x (fp32) */

/* Layout ops of the autograd Tensor that copy: transpose (mytorch/tensor.py:1381), chunk (:1598),
 * slicing in __getitem__ (:1314), concatenate / stack (mytorch/ops.py:62-160), the broadcast in the
 * backward of sum / mean (mytorch/tensor.py:1734-1955); the elementwise product of
 * Tensor.__mul__ (:596) and the reduction of sum / mean over the last axis.
 * mt_copy_strided walks an index space of up to 6 dimensions (outermost first) and copies, or with
 * accumulate_dtype >= 0 adds (dst += src in that mt_dtype), one element of elem_bytes (2 or 4) per
 * index: dst[sum idx*dst_strides] = src[sum idx*src_strides], strides in elements, a source
 * stride of 0 broadcasts. mt_rowsum: out[r] = alpha * sum_c a[r,c] (fp32 sum, fixed order). */
int mt_copy_strided(const void* src, void* dst, int ndim, const int64_t* shape, const int64_t* src_strides,
                    const int64_t* dst_strides, int elem_bytes, int accumulate_dtype, void* stream);
int mt_mul(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);          /* out = a * b */
int mt_rowsum(const void* a, void* out, int64_t rows, int64_t cols, float alpha, int dtype, void* stream);

/* fused_activation_forward / fused_activation_backward
 * (mytorch/nn/functional/fused_ops/activations.py:212, :273) */
int mt_act_fwd(const void* x, void* y, int64_t n, int act, int dtype, void* stream);
int mt_act_bwd(const void* x, const void* dy, void* dx, int64_t n, int act, int dtype, void* stream);

/* fused_layernorm_forward / fused_layernorm_backward
 * (mytorch/nn/functional/fused_ops/layernorm.py:244, :342). mean/rstd are fp32
 * [rows]. dgamma/dbeta are fp32 [cols] and may be NULL. `accumulate` is a bit
 * mask: 1 = add to dgamma/dbeta instead of overwriting them, 2 = add to dx
 * (dx then enters holding the gradient of the residual branch, so the block's
 * `x + f(norm(x))` backward needs no separate add). Column sums are two-stage
 * and deterministic. The same mask applies to mt_rmsnorm_bwd. */
int mt_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                     float* mean, float* rstd, int64_t rows, int64_t cols, float eps,
                     int dtype, void* stream);
int mt_layernorm_bwd(const void* x, const float* mean, const float* rstd, const void* dy,
                     const void* gamma, void* dx, float* dgamma, float* dbeta,
                     int64_t rows, int64_t cols, int accumulate, int dtype, void* stream);

/* LayerNorm backward that never allocates. It has no counterpart in the
 * reference (every reference op allocates its outputs and temporaries).
 * It is for callers that must not touch the device allocator while they run:
 * a host that has handed all device memory to its own arena, code running
 * where cudaMalloc/cudaFree would serialise or fail (for example inside a
 * region that forbids allocation), or a deployment with a fixed memory budget
 * that is audited up front. Same arguments (the `accumulate` bit mask included)
 * and results as mt_layernorm_bwd; the per-block partial sums of dgamma/dbeta go
 * to a fixed 2 MiB device array inside the library image (every GPU that loads
 * the library holds it until exit).
 * Limits: cols at most 1024 (fp16/bf16) or 512 (fp32) and a multiple of 8
 * (fp16/bf16) or 4 (fp32), tensors 16-byte aligned; anything else is rejected
 * with MT_ERR_INVALID and a message naming the limit. The first call on
 * a device looks up the array's device address (cudaGetSymbolAddress) and caches
 * it, so make that first call before starting any stream capture. All calls
 * share the one array and it keeps the previous call's contents (each call
 * overwrites every slot it reads, so nothing needs clearing): two calls that
 * overlap on the GPU, e.g. on different streams, race on it. */
int mt_layernorm_bwd_noalloc(const void* x, const float* mean, const float* rstd, const void* dy,
                             const void* gamma, void* dx, float* dgamma, float* dbeta,
                             int64_t rows, int64_t cols, int accumulate, int dtype, void* stream);

/* fused_rmsnorm_forward / fused_rmsnorm_backward
 * (mytorch/nn/functional/fused_ops/rmsnorm.py:159, :251) */
int mt_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd,
                   int64_t rows, int64_t cols, float eps, int dtype, void* stream);
int mt_rmsnorm_bwd(const void* x, const float* rstd, const void* dy, const void* gamma,
                   void* dx, float* dgamma, int64_t rows, int64_t cols, int accumulate,
                   int dtype, void* stream);

/* fused_softmax_forward / fused_softmax_backward
 * (mytorch/nn/functional/fused_ops/softmax.py:358, :408) */
int mt_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int dtype, void* stream);
int mt_softmax_bwd(const void* dy, const void* s, void* dx, int64_t rows, int64_t cols, int dtype, void* stream);

/* fused_cross_entropy_forward / fused_cross_entropy_backward
 * (mytorch/nn/functional/fused_ops/cross_entropy.py:263, :324). `ld` is the row
 * stride of logits in elements (>= classes). Labels are int32, -100 = ignored.
 * fwd writes loss[rows], lse[rows] (fp32) and, where the pointers are not NULL,
 * the device scalars loss_sum = sum(loss), valid_count = number of rows whose
 * label is not -100, loss_mean = loss_sum / valid_count (summed in a fixed order).
 * bwd writes (softmax - onehot) * scale into dlogits (may alias logits);
 * scale = scale_host * (*scale_dev if given) / (*count_dev if given), so the
 * upstream gradient and the valid-row count never have to be read back to the host. */
int mt_ce_fwd(const void* logits, const int32_t* labels, float* loss, float* lse,
              float* loss_sum, float* valid_count, float* loss_mean, int64_t rows, int64_t classes,
              int64_t ld, float softcap, int dtype, void* stream);
int mt_ce_bwd(const void* logits, const int32_t* labels, const float* lse, void* dlogits,
              float scale_host, const float* scale_dev, const float* count_dev,
              int64_t rows, int64_t classes, int64_t ld, float softcap, int dtype, void* stream);
/* Forward and gradient of the mean cross entropy in one pass over the logits (no reference
 * counterpart as one call; the math is fused_cross_entropy_forward followed by
 * fused_cross_entropy_backward, fused_ops/cross_entropy.py:263,324): on return `logits` holds
 * (softmax - onehot) * scale_host * scale_dev[0] / n_valid (0 on ignored rows), loss/lse/loss_sum/
 * valid_count/loss_mean as mt_ce_fwd. The upstream gradient of the mean loss has to be known at
 * this point (scale_dev, a device scalar; NULL = 1); mt_scale_ratio corrects the result if another
 * value arrives later. Each block reads its row twice back to back, so DRAM sees one read and one
 * write of the logits. */
int mt_ce_fwd_grad(void* logits, const int32_t* labels, float* loss, float* lse, float* loss_sum,
                   float* valid_count, float* loss_mean, float scale_host, const float* scale_dev,
                   int64_t rows, int64_t classes, int64_t ld, float softcap, int dtype, void* stream);
/* x[i] *= num[0] / den[0], both device scalars. */
int mt_scale_ratio(void* x, int64_t n, const float* num, const float* den, int dtype, void* stream);

/* Cross entropy over the vocabulary IN CHUNKS, for a fused lm_head + loss that
 * never holds the [rows, vocab] logits: the caller computes the logits of one
 * vocabulary chunk [col_offset, col_offset + chunk_classes) with mt_gemm and
 * hands them over. No counterpart in the reference, which materialises the
 * logits (gpt2_trainer/gpt2.py:368) and then calls fused_cross_entropy_*.
 *   fwd:    merges the chunk's log-sum-exp into lse_running[rows] (initialise it
 *           to -inf) and stores the target logit in tgt[rows] when the label
 *           lies inside the chunk;
 *   finish: loss[row] = lse - tgt for labels != -100, plus the same device
 *           scalars as mt_ce_fwd;
 *   bwd:    dlogits_chunk = (exp(logit - lse) - [col == label]) * scale from
 *           recomputed chunk logits and the FINAL lse (may alias the logits). */
int mt_ce_chunk_fwd(const void* logits_chunk, const int32_t* labels, float* lse_running, float* tgt,
                    int64_t rows, int64_t chunk_classes, int64_t ld, int64_t col_offset,
                    float softcap, int dtype, void* stream);
int mt_ce_chunk_finish(const float* lse, const float* tgt, const int32_t* labels, float* loss,
                       float* loss_sum, float* valid_count, float* loss_mean, int64_t rows, void* stream);
int mt_ce_chunk_bwd(const void* logits_chunk, const int32_t* labels, const float* lse, void* dlogits,
                    float scale_host, const float* scale_dev, const float* count_dev,
                    int64_t rows, int64_t chunk_classes, int64_t ld, int64_t col_offset,
                    float softcap, int dtype, void* stream);

/* fused_embedding_forward / fused_embedding_backward
 * (mytorch/nn/functional/fused_ops/embedding.py:108, :219). Indices int32.
 * An out-of-range index sets the device status word and is skipped.
 * bwd adds into dweight (fp32 [vocab, dim]); rows are summed in token order
 * (sorted segments, no atomics), so the result is deterministic. `scratch`
 * must hold mt_embedding_bwd_scratch_bytes(n_tokens) bytes. */
int mt_embedding_fwd(const void* weight, const int32_t* idx, void* out, int64_t n_tokens,
                     int64_t dim, int64_t vocab, int dtype, void* stream);
size_t mt_embedding_bwd_scratch_bytes(int64_t n_tokens);
int mt_embedding_bwd(const void* dy, const int32_t* idx, float* dweight, void* scratch,
                     int64_t n_tokens, int64_t dim, int64_t vocab, int dtype, void* stream);
/* GPT-2 embedding pair fused: out = wte[idx] + wpe[pos], pos = token % seq_len
 * (gpt2_trainer/gpt2.py:105-119). */
int mt_embedding_pos_fwd(const void* wte, const void* wpe, const int32_t* idx, void* out,
                         int64_t n_tokens, int64_t seq_len, int64_t dim, int64_t vocab,
                         int dtype, void* stream);
/* dwpe[t,:] += sum_b dy[b,t,:]  (fp32 accumulate) */
int mt_pos_embedding_bwd(const void* dy, float* dwpe, int64_t batch, int64_t seq_len,
                         int64_t dim, int dtype, void* stream);

/* fused_rope_forward / fused_rope_backward
 * (mytorch/nn/functional/fused_ops/rope.py:178, :265): x [B,T,H,D] in place,
 * cos/sin fp32 [T,D] (halves duplicated), backward = rotation by -angle. */
int mt_rope(void* x, const float* cos, const float* sin, int64_t batch, int64_t seq,
            int64_t heads, int64_t head_dim, int backward, int dtype, void* stream);

/* Rotary embedding THEN parameter-free RMSNorm over head_dim, on q and on k, in one pass over
 * each tensor: the three statements of nanochat_trainer/core/nanochat_gpt.py:119-124
 * (apply_rotary_pos_embed, norm(q), norm(k)), i.e. fused_rope_forward (fused_ops/rope.py:178)
 * followed by fused_rmsnorm_forward with gamma = None (fused_ops/rmsnorm.py:159), and their
 * backward passes in reverse order. Head h of token (b, t) starts at
 * base + (b*seq + t) * ld + h * head_dim elements, so [B,T,H,D] tensors (ld = H*D) and column
 * slices of a wider projection are read in place. xk/yk/rstd_k (dyk/...) may be NULL to process
 * one tensor. rstd is fp32 [B*T*H]. The rotation happens in fp32 registers (the reference
 * rounds the rotated values to the activation dtype before the norm).
 * bwd takes the SAVED OUTPUT y (for a norm without gamma, x_hat = y) and rstd:
 *   dr = rstd * (dy - y * mean(dy * y)),  dx = rotation of dr by the negative angle.
 * head_dim must be 2, 4, 8, 16 or 32 16-byte vectors (64 or 128 for fp16/bf16). */
int mt_rope_rmsnorm_fwd(const void* xq, const void* xk, void* yq, void* yk, float* rstd_q, float* rstd_k,
                        const float* cos, const float* sin, int64_t batch, int64_t seq, int64_t heads,
                        int64_t head_dim, int64_t ld_x, int64_t ld_y, float eps, int dtype, void* stream);
int mt_rope_rmsnorm_bwd(const void* dyq, const void* dyk, const void* yq, const void* yk,
                        const float* rstd_q, const float* rstd_k, void* dxq, void* dxk,
                        const float* cos, const float* sin, int64_t batch, int64_t seq, int64_t heads,
                        int64_t head_dim, int64_t ld_dy, int64_t ld_y, int64_t ld_dx, int dtype, void* stream);

/* fused_linear_forward (mytorch/nn/functional/fused_ops/linear.py:118),
 * fused_grouped_matmul (mytorch/nn/functional/fused_ops/matmul.py:842) and
 * cupy.matmul reached from mytorch/nn/functional/layers/linear.py:86,104,123.
 *   C[M,N] = act(alpha * op(A)·op(B) + bias)    (+ C if accumulate)
 * op(A) is [M,K]: trans_a=0 -> A stored [M,K] (lda>=K); trans_a=1 -> A stored [K,M].
 * op(B) is [K,N]: trans_b=0 -> B stored [K,N] (ldb>=N); trans_b=1 -> B stored [N,K].
 * Linear forward is (trans_a=0, trans_b=1); dgrad (0,0); wgrad (1,0).
 * in_dtype f16/bf16 runs on tcgen05 tensor cores (fp32 accumulate in TMEM)
 * when pointers/strides are 16-byte aligned, else on a CUDA-core kernel;
 * in_dtype f32 runs on the CUDA-core kernel in full fp32.
 * bias: [N] in in_dtype or NULL. preact: optional second output receiving the
 * value before the activation (same dtype/ld as C), or NULL.
 * accumulate: 0 = overwrite, 1 = C += result (read-modify-write),
 * 2 = split-K with fp32 atomic adds (C must be fp32; order not deterministic). */
int mt_gemm(const void* A, const void* B, void* C, void* preact, const void* bias,
            int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
            int trans_a, int trans_b, int in_dtype, int out_dtype, int act,
            float alpha, int accumulate, void* stream);
/* mt_gemm with one more elementwise operand, for the fusions of a transformer
 * block: aux is [M,N] in the output dtype with row stride ldc and is combined
 * with the result AFTER bias and activation:
 *   aux_mode 1: C = result + aux            (residual add: x + Linear(...),
 *               gpt2_trainer/gpt2.py:308-311)
 *   aux_mode 2: C = result * gelu'(aux)     (backward of Linear(act="gelu"),
 *               mytorch/nn/functional/layers/linear.py:193-221 + activations.py:182)
 *   aux_mode 3: C = result * 2*relu(aux)    (backward of relu_squared)
 *   aux_mode 4: C = result * (aux > 0)      (backward of relu)
 *   aux_mode 5: C = result * aux            (aux already holds a derivative, see below)
 *   aux_mode 6: C = result * 2*sqrt(aux)    (backward of relu_squared from its OUTPUT: with
 *               aux = relu(u)^2 the derivative 2*relu(u) is 2*sqrt(aux), so the forward pass
 *               keeps nothing but the activation it needs anyway)
 * `act` may be OR'ed with MT_ACT_STORE_GRAD: the second output (`preact`) then receives the
 * activation's derivative at the pre-activation, act'(A*B + bias), instead of the
 * pre-activation itself - what the backward pass multiplies by (aux_mode 5), computed where the
 * tanh of the forward activation is already at hand.
 * aux_mode 0 / aux NULL is mt_gemm. Not combinable with accumulate = 2. */
int mt_gemm_ex(const void* A, const void* B, void* C, void* preact, const void* bias,
               const void* aux, int aux_mode, int64_t M, int64_t N, int64_t K,
               int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
               int in_dtype, int out_dtype, int act, float alpha, int accumulate, void* stream);
/* Forces the CUDA-core kernel (1) or restores automatic choice (0); used by
 * the tests to cross-check the tensor-core path on the device. */
int mt_gemm_force_simt(int on);
/* Tile shape of the tensor-core kernel: 0 = chosen per call by estimated
 * efficiency (default), 1 = one CTA per 128-row tile only, 2 = pairs of CTAs
 * sharing 256-row tiles whenever M > 128. No reference counterpart; the tests
 * use it to run both tile shapes on the same inputs. */
int mt_gemm_tile_policy(int policy);

/* fused_sdpa_forward / fused_sdpa_backward
 * (mytorch/nn/functional/fused_ops/flash_attention.py:1269, :1441), causal or
 * full softmax(QK^T*scale)V. Tensors are addressed with explicit element
 * strides (batch, head, row; the head_dim stride is 1), so the per-head
 * interleaved [q|k|v] projection of gpt2_trainer/gpt2.py:168-177 and
 * [B,H,S,D] tensors are both read in place. lse is fp32 [B,H,S], natural log.
 * bwd needs delta scratch fp32 [B,H,S] and, for the tensor-core path, a fp32
 * dq accumulator of B*H*S*D floats (dq_accum; may be NULL on the CUDA-core path). */
typedef struct { int64_t b, h, s; } mt_strides3;
int mt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 so,
                int64_t batch, int64_t heads, int64_t seq, int64_t head_dim,
                float scale, int causal, int dtype, void* stream);
int mt_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_accum,
                mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 so, mt_strides3 sdo,
                mt_strides3 sdq, mt_strides3 sdk, mt_strides3 sdv,
                int64_t batch, int64_t heads, int64_t seq, int64_t head_dim,
                float scale, int causal, int dtype, void* stream);
/* The same with grouped-query heads (fused_ops/flash_attention.py:445-455, 1014-1018,
 * 1171-1176; the nanochat model's num_kv_heads, nanochat_trainer/core/nanochat_gpt.py:31-32,
 * 78-90): k, v, dk and dv have kv_heads heads, query head h reads key/value head
 * h / (heads / kv_heads), and dk / dv sum the contributions of the query heads of their group.
 * heads must be a multiple of kv_heads; kv_heads = heads is mt_attn_fwd / mt_attn_bwd. */
int mt_attn_fwd_gqa(const void* q, const void* k, const void* v, void* o, float* lse,
                    mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 so,
                    int64_t batch, int64_t heads, int64_t kv_heads, int64_t seq, int64_t head_dim,
                    float scale, int causal, int dtype, void* stream);
int mt_attn_bwd_gqa(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                    const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_accum,
                    mt_strides3 sq, mt_strides3 sk, mt_strides3 sv, mt_strides3 so, mt_strides3 sdo,
                    mt_strides3 sdq, mt_strides3 sdk, mt_strides3 sdv,
                    int64_t batch, int64_t heads, int64_t kv_heads, int64_t seq, int64_t head_dim,
                    float scale, int causal, int dtype, void* stream);
int mt_attn_force_simt(int on);

/* The inference step: attention of q_len new query rows against a key/value cache, and the
 * append of new rows to that cache (Cache.update and the cached branch of the attention module,
 * gpt2_trainer/gpt2.py:29-86, :167-215; Sq != Skv as in fused_ops/flash_cross_attention.py).
 * The cache is a ring [B, H, max_len, D] addressed with strides: row (pos0 + i) % max_len receives
 * new row i, so once max_len rows are held the oldest is overwritten (the reference drops the
 * oldest token by concatenating and slicing). mt_attn_decode attends to rows [0, kv_len) of the
 * cache; causal_offset < 0 means every query sees every key (the reference's choice once the
 * cache is non-empty), otherwise query i sees rows <= causal_offset + i (valid before the ring
 * wraps). head_dim 64 or 128; cache rows 16-byte aligned. */
int mt_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* o,
                   mt_strides3 sq, mt_strides3 skv, mt_strides3 so,
                   int64_t batch, int64_t heads, int64_t q_len, int64_t kv_len, int64_t head_dim,
                   float scale, int causal_offset, int dtype, void* stream);
/* The same with the cache holding kv_heads heads per batch and query head h reading head
 * h / (heads / kv_heads) of it (grouped-query attention, nanochat_gpt.py:78-90, 126-160). */
int mt_attn_decode_gqa(const void* q, const void* k_cache, const void* v_cache, void* o,
                       mt_strides3 sq, mt_strides3 skv, mt_strides3 so,
                       int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t kv_len,
                       int64_t head_dim, float scale, int causal_offset, int dtype, void* stream);
int mt_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                 mt_strides3 sk, mt_strides3 sv, mt_strides3 scache,
                 int64_t batch, int64_t heads, int64_t n_new, int64_t pos0, int64_t max_len,
                 int64_t head_dim, int dtype, void* stream);

/* AdamW.step (mytorch/optim/optimizers.py:342-371), GradScaler.unscale_grads +
 * the inf/nan scan (mytorch/accelerate.py:71-89, 716-729), clip_grad_norm_
 * (mytorch/accelerate.py:799-856) and the master->half copy of
 * OptimizerWrapper.step (mytorch/accelerate.py:342-361), over MANY tensors per
 * launch. A tensor list is described by device arrays built once by the caller:
 *   ptr tables (void*[n]), sizes (int64[n]), and a chunk table mapping each
 *   4096-element chunk to (tensor, offset) so one grid covers all tensors. */
typedef struct {
  void** p;          /* fp32 master parameters                      [n] */
  void** g;          /* gradients (g_dtype)                          [n] */
  void** m;          /* fp32 first moment                            [n] */
  void** v;          /* fp32 second moment                           [n] */
  void** p_half;     /* optional low-precision copies, or NULL table [n] */
  const int64_t* size;       /* elements per tensor                  [n] */
  const float* weight_decay; /* per tensor                           [n] */
  const int32_t* chunk_tensor;  /* [n_chunks] */
  const int64_t* chunk_offset;  /* [n_chunks] */
  int64_t n_tensors, n_chunks;
} mt_tensor_list;
/* sumsq[0] += sum g^2 (fp32, of g * *inv_scale if inv_scale != NULL);
 * found_inf[0] = 1.0 if any g is inf/nan. Both device scalars. */
int mt_gradnorm_multi(const mt_tensor_list* L, int g_dtype, const float* inv_scale_dev,
                      float* sumsq, float* found_inf, void* stream);
/* One launch: g' = g * (*inv_scale) * clip_coef where
 * clip_coef = min(1, max_norm / (sqrt(*sumsq) + 1e-6)) (max_norm <= 0: no clip);
 * skipped entirely when *found_inf != 0. Then the reference AdamW update
 * (decay applied after the Adam step, eps not bias-corrected) and, if p_half
 * is given, the low-precision copy. zero_grad != 0 clears g afterwards.
 * The step count and the running powers of the betas stay on the device, so a
 * step skipped because of *found_inf leaves them where they were, as the
 * reference does by not calling optimizer.step() on an overflow
 * (mytorch/accelerate.py:342-352): step_state is 8 doubles, two slots of
 * {t, beta1^t, beta2^t, unused}. A call reads slot `slot` (state after the last
 * applied step; initialise to {0, 1, 1, 0}) and writes the other one; the caller
 * alternates `slot` on every call, applied or not. The kernel uses
 * lr_t = lr * sqrt(1 - beta2^(t+1)) / (1 - beta1^(t+1)). */
int mt_adamw_multi(const mt_tensor_list* L, int g_dtype, int half_dtype,
                   float lr, double beta1, double beta2, float eps,
                   const float* inv_scale_dev, const float* sumsq_dev, float max_norm,
                   const float* found_inf_dev, int zero_grad, double* step_state, int slot,
                   void* stream);

/* GradScaler.update (mytorch/accelerate.py:91-121) on the device, so the step never
 * waits for the host: state = {scale, 1/(scale*accum_steps), clean-step counter,
 * skipped-step counter} (4 floats). On *found_inf != 0 the scale is multiplied by
 * `backoff` and the counter reset; otherwise the counter grows and at `interval`
 * the scale is multiplied by `growth`. dynamic = 0 keeps the scale fixed (fp32 /
 * bf16 training) and only refreshes state[1] and the skipped-step counter. */
int mt_scaler_update(float* state, const float* found_inf, float growth, float backoff,
                     int interval, float inv_accum, int dynamic, void* stream);

/* cupyx.distributed.NCCLBackend as used by mytorch/accelerate.py:154-159
 * (init), :249-250 (broadcast), :732-736/:757-772/:833-837 (all_reduce),
 * :873-880 (barrier), :1050-1052 (stop). NCCL is loaded with dlopen at first
 * use. The 128-byte unique id is produced on rank 0 and carried to the other
 * ranks by the caller (TCP store on CUPYX_DISTRIBUTED_HOST/PORT). */
int mt_comm_unique_id(void* id128);
int mt_comm_init(void** comm, const void* id128, int rank, int world_size);
int mt_comm_broadcast(void* comm, void* buf, int64_t count, int dtype, int root, void* stream);
/* op: 0 = sum, 1 = max, 2 = avg */
int mt_comm_allreduce(void* comm, const void* send, void* recv, int64_t count, int dtype, int op, void* stream);
int mt_comm_barrier(void* comm, void* stream);
int mt_comm_abort(void* comm);
int mt_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* MYTORCH_B200_H */
