"""The reference's fused-op interface, backed by the sm_100a library.

Same function names, argument meaning and return values as
`mytorch/nn/functional/fused_ops/__init__.py:1-13` of the reference (the 18
functions on the GPT training path), taking and returning device arrays
(anything exposing `__cuda_array_interface__`; results are `DeviceArray`).
The callee allocates outputs, as the reference does. Differences that are
deliberate and visible to callers:
  * statistics (mean, rstd, lse) and parameter gradients are fp32 whatever the
    activation dtype (the reference keeps LayerNorm stats in the input dtype,
    fused_ops/layernorm.py:270-271);
  * `fused_sdpa_forward` returns a natural-log LSE; it is only ever consumed
    by `fused_sdpa_backward` of the same library;
  * nothing here synchronises with the host.
"""
import ctypes as C
import math

from . import _lib
from .array import DeviceArray, as_device_array, stream

_A = as_device_array


def _ptr(x):
    return None if x is None else _A(x).ptr


def _check_float(*arrs):
    dt = None
    for a in arrs:
        if a is None:
            continue
        if a.dtype not in ("float32", "float16", "bfloat16"):
            raise TypeError(f"floating dtype expected, got {a.dtype}")
        if dt is not None and a.dtype != dt:
            raise TypeError(f"mismatched dtypes: {a.dtype} vs {dt}")
        dt = a.dtype
    return dt


# ------------------------------------------------------------------ matmul ----
def gemm(a, b, trans_a=False, trans_b=False, out=None, bias=None, act=None, preact=False,
         out_dtype=None, alpha=1.0, accumulate=0, aux=None, aux_mode=0):
    """out = combine(act(alpha * op(a) @ op(b) + bias), aux); see mt_gemm / mt_gemm_ex in
    the C header (aux_mode 1 adds aux, 2/3/4 multiply by gelu'/relu2'/relu' of aux, 5 by aux).
    preact=True also returns the pre-activation; preact="grad" returns the activation's
    derivative at the pre-activation instead."""
    a, b = _A(a), _A(b)
    dt = _check_float(a, b, bias)
    assert a.ndim == 2 and b.ndim == 2
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    Kb, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions must match: {a.shape} x {b.shape} (trans {trans_a},{trans_b})")
    out_dtype = out_dtype or (out.dtype if out is not None else dt)
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an existing output")
        out = DeviceArray.empty((M, N), out_dtype)
    pre = DeviceArray.empty((M, N), out_dtype) if preact else None
    if aux is not None:
        aux = _A(aux)
        assert aux.size == M * N and aux.dtype == out.dtype, "aux must be [M,N] in the output dtype"
    _lib.gemm_ex(a.ptr, b.ptr, out.ptr, _ptr(pre), _ptr(bias), _ptr(aux), int(aux_mode if aux is not None else 0),
                 M, N, K, a.shape[1], b.shape[1], N, int(trans_a), int(trans_b), a.code, out.code,
                 _lib.ACT[act] | (0x100 if preact == "grad" else 0), float(alpha), int(accumulate), stream())
    return (out, pre) if preact else out


def fused_grouped_matmul(a, b):
    """c[M,N] = a[M,K] @ b[K,N]  (fused_ops/matmul.py:842)."""
    return gemm(a, b)


def fused_linear_forward(a, w, b=None, act_func=None):
    """y = act(a[B,I] @ w[I,O] + b); returns (preact, postact) — postact is None
    without an activation (fused_ops/linear.py:118)."""
    if act_func is None:
        return gemm(a, w, bias=b), None
    post, pre = gemm(a, w, bias=b, act=act_func, preact=True)
    return pre, post


# -------------------------------------------------------------- activations ----
def fused_activation_forward(input, act_func):
    """Elementwise activation (fused_ops/activations.py:212)."""
    x = _A(input)
    y = DeviceArray.empty(x.shape, x.dtype)
    _lib.act_fwd(x.ptr, y.ptr, x.size, _lib.ACT[act_func], x.code, stream())
    return y


def fused_activation_backward(input, output_grad, act_func):
    """act'(input) * output_grad (fused_ops/activations.py:273)."""
    x, dy = _A(input), _A(output_grad)
    _check_float(x, dy)
    dx = DeviceArray.empty(x.shape, x.dtype)
    _lib.act_bwd(x.ptr, dy.ptr, dx.ptr, x.size, _lib.ACT[act_func], x.code, stream())
    return dx


# --------------------------------------------------------------------- norms ----
def fused_layernorm_forward(x, gamma=None, beta=None, eps=1e-5, training=True):
    """x [N,E] -> (y, mean[N], rstd[N]) (fused_ops/layernorm.py:244)."""
    x = _A(x)
    _check_float(x, gamma, beta)
    n, e = x.shape
    y = DeviceArray.empty((n, e), x.dtype)
    mean = DeviceArray.empty((n,), "float32")
    rstd = DeviceArray.empty((n,), "float32")
    _lib.layernorm_fwd(x.ptr, _ptr(gamma), _ptr(beta), y.ptr, mean.ptr, rstd.ptr, n, e, float(eps), x.code, stream())
    return y, mean, rstd


def fused_layernorm_backward(x, mean, inv_var, dy, gamma=None, beta=None, dgamma_out=None, dbeta_out=None,
                             dx_out=None):
    """-> (dx, dgamma, dbeta) (fused_ops/layernorm.py:342). dgamma/dbeta are
    fp32; when `*_out` buffers are given the sums are ADDED into them, and
    `dx_out` (same shape/dtype as x) likewise receives dx ADDED to its contents."""
    x, dy = _A(x), _A(dy)
    _check_float(x, dy, gamma)
    n, e = x.shape
    dx = dx_out if dx_out is not None else DeviceArray.empty((n, e), x.dtype)
    acc = int(dgamma_out is not None or dbeta_out is not None) | (2 if dx_out is not None else 0)
    dg = dgamma_out if dgamma_out is not None else (DeviceArray.empty((e,), "float32") if gamma is not None else None)
    db = dbeta_out if dbeta_out is not None else (DeviceArray.empty((e,), "float32") if beta is not None else None)
    _lib.layernorm_bwd(x.ptr, _A(mean).ptr, _A(inv_var).ptr, dy.ptr, _ptr(gamma), dx.ptr, _ptr(dg), _ptr(db),
                       n, e, int(acc), x.code, stream())
    return dx, dg, db


def fused_rmsnorm_forward(x, gamma=None, eps=1e-5, training=True):
    """x [N,E] -> (y, rstd[N]) (fused_ops/rmsnorm.py:159)."""
    x = _A(x)
    _check_float(x, gamma)
    n, e = x.shape
    y = DeviceArray.empty((n, e), x.dtype)
    rstd = DeviceArray.empty((n,), "float32")
    _lib.rmsnorm_fwd(x.ptr, _ptr(gamma), y.ptr, rstd.ptr, n, e, float(eps), x.code, stream())
    return y, rstd


def fused_rmsnorm_backward(x, rstd, dy, gamma=None, dgamma_out=None, dx_out=None):
    """-> (dx, dgamma) (fused_ops/rmsnorm.py:251); `*_out` buffers are added into."""
    x, dy = _A(x), _A(dy)
    _check_float(x, dy, gamma)
    n, e = x.shape
    dx = dx_out if dx_out is not None else DeviceArray.empty((n, e), x.dtype)
    dg = dgamma_out if dgamma_out is not None else (DeviceArray.empty((e,), "float32") if gamma is not None else None)
    _lib.rmsnorm_bwd(x.ptr, _A(rstd).ptr, dy.ptr, _ptr(gamma), dx.ptr, _ptr(dg), n, e,
                     int(dgamma_out is not None) | (2 if dx_out is not None else 0), x.code, stream())
    return dx, dg


# ------------------------------------------------------------------- softmax ----
def fused_softmax_forward(x):
    """Row softmax over the last axis of x [N,C] (fused_ops/softmax.py:358)."""
    x = _A(x)
    n, c = x.shape
    y = DeviceArray.empty((n, c), x.dtype)
    _lib.softmax_fwd(x.ptr, y.ptr, n, c, x.code, stream())
    return y


def fused_softmax_backward(dy, s):
    """dx = s * (dy - sum(dy*s)) (fused_ops/softmax.py:408)."""
    dy, s = _A(dy), _A(s)
    _check_float(dy, s)
    n, c = s.shape
    dx = DeviceArray.empty((n, c), s.dtype)
    _lib.softmax_bwd(dy.ptr, s.ptr, dx.ptr, n, c, s.code, stream())
    return dx


# ------------------------------------------------------------- cross entropy ----
def fused_cross_entropy_forward(logits, labels, softcap=None, ld=None, reduce=False):
    """logits [N,C], labels int32 [N] -> (loss[N], lse[N]) fp32
    (fused_ops/cross_entropy.py:263). With reduce=True also returns a device
    array (sum of loss, number of valid rows, mean loss) so no host read is needed."""
    logits, labels = _A(logits), _A(labels)
    n, c = logits.shape
    ld = ld or c
    assert labels.dtype == "int32"
    loss = DeviceArray.empty((n,), "float32")
    lse = DeviceArray.empty((n,), "float32")
    tot = DeviceArray.empty((3,), "float32") if reduce else None
    _lib.ce_fwd(logits.ptr, labels.ptr, loss.ptr, lse.ptr, tot.ptr if reduce else None,
                tot.ptr + 4 if reduce else None, tot.ptr + 8 if reduce else None, n, c, ld, float(softcap or 0.0), logits.code, stream())
    if reduce:
        return loss, lse, tot
    return loss, lse


def fused_cross_entropy_forward_backward(logits, labels, softcap=None, ld=None, scale=1.0, scale_dev=None):
    """Forward and gradient in one pass (mt_ce_fwd_grad): returns (loss[N], lse[N], tot) like
    fused_cross_entropy_forward(reduce=True) and OVERWRITES logits with
    (softmax - onehot) * scale * scale_dev / n_valid, the gradient of the mean loss for an
    upstream gradient scale * scale_dev (device scalar, optional)."""
    logits, labels = _A(logits), _A(labels)
    n, c = logits.shape
    ld = ld or c
    assert labels.dtype == "int32"
    loss = DeviceArray.empty((n,), "float32")
    lse = DeviceArray.empty((n,), "float32")
    tot = DeviceArray.empty((3,), "float32")
    _lib.ce_fwd_grad(logits.ptr, labels.ptr, loss.ptr, lse.ptr, tot.ptr, tot.ptr + 4, tot.ptr + 8, float(scale),
                     None if scale_dev is None else _A(scale_dev).ptr, n, c, ld, float(softcap or 0.0), logits.code, stream())
    return loss, lse, tot


def fused_cross_entropy_backward(logits, labels, logsumexp, softcap=None, scale=1.0, ld=None,
                                 scale_dev=None, count_dev=None):
    """(softmax - onehot) * scale written OVER logits, which is returned
    (fused_ops/cross_entropy.py:324). scale_dev / count_dev are optional device
    scalars multiplying / dividing the scale."""
    logits, labels = _A(logits), _A(labels)
    n, c = logits.shape
    ld = ld or c
    _lib.ce_bwd(logits.ptr, labels.ptr, _A(logsumexp).ptr, logits.ptr, float(scale),
                scale_dev if isinstance(scale_dev, (int, type(None))) else _A(scale_dev).ptr,
                count_dev if isinstance(count_dev, (int, type(None))) else _A(count_dev).ptr,
                n, c, ld, float(softcap or 0.0), logits.code, stream())
    return logits


# ----------------------------------------------------------------- embedding ----
def fused_embedding_forward(embeddings, indices):
    """out[..., :] = embeddings[indices] (fused_ops/embedding.py:108)."""
    w, idx = _A(embeddings), _A(indices)
    assert idx.dtype == "int32", "indices must be int32"
    v, d = w.shape
    out = DeviceArray.empty(idx.shape + (d,), w.dtype)
    _lib.embedding_fwd(w.ptr, idx.ptr, out.ptr, idx.size, d, v, w.code, stream())
    return out


def fused_embedding_backward(grad_output, embeddings, indices, out=None):
    """dW[V,D] (fp32) = scatter-add of grad rows (fused_ops/embedding.py:219);
    added into `out` when given."""
    dy, w, idx = _A(grad_output), _A(embeddings), _A(indices)
    v, d = w.shape
    if out is None:
        out = DeviceArray.zeros((v, d), "float32")
    n = idx.size
    scratch = DeviceArray.empty((_lib.embedding_bwd_scratch_bytes(n),), "uint8")
    _lib.embedding_bwd(dy.ptr, idx.ptr, out.ptr, scratch.ptr, n, d, v, dy.code, stream())
    return out


# ----------------------------------------------------------------- attention ----
def _bhsd_strides(a):
    B, H, S, D = a.shape
    return _lib.Strides3(H * S * D, S * D, D)


def _check_self_attention_shapes(Q, K, V):
    """The kernels index K and V with Q's batch and sequence counts and with head h / group, so the
    shapes are checked on the host: q [B,H,S,D], k and v [B,Hkv,S,D] with H a multiple of Hkv
    (Hkv < H is grouped-query attention). Another key length would read out of bounds. Returns Hkv."""
    ok = Q.ndim == 4 and K.ndim == 4 and K.shape == V.shape and K.shape[0] == Q.shape[0] and K.shape[2:] == Q.shape[2:]
    if not ok or K.shape[1] < 1 or Q.shape[1] % K.shape[1] != 0:
        raise NotImplementedError(
            f"self-attention needs q [B,H,S,D] and k, v [B,Hkv,S,D] with H a multiple of Hkv; got {Q.shape}, "
            f"{K.shape}, {V.shape} (another key length, i.e. cross attention, is not part of this path)")
    return K.shape[1]


def fused_sdpa_forward(Q, K, V, attn_mask=None, causal=False, softmax_scale=None, strides=None, out=None,
                       out_strides=None):
    """Q [B,H,S,D], K, V [B,Hkv,S,D] -> (Q, K, V, O, M) with M the per-row log-sum-exp [B,H,S]
    (fused_ops/flash_attention.py:1269; Hkv < H is grouped-query attention, :445-455). `strides`
    (three Strides3) lets callers pass views such as the interleaved qkv projection."""
    if attn_mask is not None:
        raise NotImplementedError("attn_mask is not on the GPT training path; use causal=True/False")
    Q, K, V = _A(Q), _A(K), _A(V)
    _check_float(Q, K, V)
    Hkv = _check_self_attention_shapes(Q, K, V)
    B, H, S, D = Q.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    sq, sk, sv = strides or (_bhsd_strides(Q), _bhsd_strides(K), _bhsd_strides(V))
    O = out if out is not None else DeviceArray.empty((B, H, S, D), Q.dtype)
    so = out_strides or _bhsd_strides(O)
    M = DeviceArray.empty((B, H, S), "float32")
    _lib.attn_fwd_gqa(Q.ptr, K.ptr, V.ptr, O.ptr, M.ptr, sq, sk, sv, so, B, H, Hkv, S, D, scale, int(bool(causal)),
                      Q.code, stream())
    return Q, K, V, O, M


def fused_sdpa_backward(dO, Q, K, V, O, M, attn_mask=None, causal=False, softmax_scale=None, strides=None,
                        out=None, out_strides=None, o_strides=None, do_strides=None):
    """-> (dQ, dK, dV) (fused_ops/flash_attention.py:1441)."""
    if attn_mask is not None:
        raise NotImplementedError("attn_mask is not on the GPT training path")
    dO, Q, K, V, O = _A(dO), _A(Q), _A(K), _A(V), _A(O)
    _check_float(dO, Q, K, V, O)
    Hkv = _check_self_attention_shapes(Q, K, V)
    B, H, S, D = Q.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    sq, sk, sv = strides or (_bhsd_strides(Q), _bhsd_strides(K), _bhsd_strides(V))
    if out is None:
        dQ = DeviceArray.empty((B, H, S, D), Q.dtype)
        dK, dV = (DeviceArray.empty((B, Hkv, S, D), Q.dtype) for _ in range(2))
        sdq, sdk, sdv = _bhsd_strides(dQ), _bhsd_strides(dK), _bhsd_strides(dV)
    else:
        dQ, dK, dV = out
        sdq, sdk, sdv = out_strides
    so = o_strides or _bhsd_strides(O)
    sdo = do_strides or _bhsd_strides(dO)
    delta = DeviceArray.empty((B, H, S), "float32")
    dq_acc = DeviceArray.empty((B * H * S * D,), "float32") if Q.dtype != "float32" else None
    _lib.attn_bwd_gqa(Q.ptr, K.ptr, V.ptr, O.ptr, dO.ptr, _A(M).ptr, dQ.ptr, dK.ptr, dV.ptr, delta.ptr,
                      _ptr(dq_acc), sq, sk, sv, so, sdo, sdq, sdk, sdv, B, H, Hkv, S, D, scale, int(bool(causal)),
                      Q.code, stream())
    return dQ, dK, dV


# ---------------------------------------------------------------------- rope ----
def fused_rope_forward(x, cos, sin):
    """Rotates x [B,L,H,D] IN PLACE; cos/sin fp32 [L,D] or [1,L,D]
    (fused_ops/rope.py:178). Returns (x, cos, sin) like the reference."""
    x = _A(x)
    B, L, H, D = x.shape
    _lib.rope(x.ptr, _A(cos).ptr, _A(sin).ptr, B, L, H, D, 0, x.code, stream())
    return x, cos, sin


def fused_rope_backward(dx, cos, sin):
    """In-place rotation by the negative angle (fused_ops/rope.py:265)."""
    dx = _A(dx)
    B, L, H, D = dx.shape
    _lib.rope(dx.ptr, _A(cos).ptr, _A(sin).ptr, B, L, H, D, 1, dx.code, stream())
    return dx


def fused_rope_rmsnorm_forward(q, k, cos, sin, eps=1e-5):
    """q, k [B,L,H,D] -> (q', k', rstd_q, rstd_k) with x' = rmsnorm(rope(x)) over D, both tensors
    in one launch (fused_rope_forward, fused_ops/rope.py:178, then fused_rmsnorm_forward with
    gamma=None, fused_ops/rmsnorm.py:159, as nanochat_gpt.py:119-124 chains them). Out of place."""
    q, k = _A(q), _A(k)
    _check_float(q, k)
    B, L, H, D = q.shape
    Hk = k.shape[2]
    assert k.shape == (B, L, Hk, D)
    yq, yk = DeviceArray.empty(q.shape, q.dtype), DeviceArray.empty(k.shape, k.dtype)
    rq, rk = DeviceArray.empty((B * L * H,), "float32"), DeviceArray.empty((B * L * Hk,), "float32")
    c, s_ = _A(cos).ptr, _A(sin).ptr
    if Hk == H:      # one launch for both tensors
        _lib.rope_rmsnorm_fwd(q.ptr, k.ptr, yq.ptr, yk.ptr, rq.ptr, rk.ptr, c, s_, B, L, H, D, H * D, H * D, float(eps),
                              q.code, stream())
    else:            # grouped-query heads: k has fewer heads per token
        _lib.rope_rmsnorm_fwd(q.ptr, None, yq.ptr, None, rq.ptr, None, c, s_, B, L, H, D, H * D, H * D, float(eps), q.code, stream())
        _lib.rope_rmsnorm_fwd(k.ptr, None, yk.ptr, None, rk.ptr, None, c, s_, B, L, Hk, D, Hk * D, Hk * D, float(eps), k.code, stream())
    return yq, yk, rq, rk


def fused_rope_rmsnorm_backward(dyq, dyk, yq, yk, rstd_q, rstd_k, cos, sin):
    """Gradients w.r.t. the un-rotated q and k from the gradients of the outputs, the saved outputs
    and rstd (fused_rmsnorm_backward, fused_ops/rmsnorm.py:251, then fused_rope_backward, rope.py:265)."""
    dyq, dyk, yq, yk = _A(dyq), _A(dyk), _A(yq), _A(yk)
    B, L, H, D = yq.shape
    Hk = yk.shape[2]
    dq, dk = DeviceArray.empty(yq.shape, yq.dtype), DeviceArray.empty(yk.shape, yk.dtype)
    c, s_ = _A(cos).ptr, _A(sin).ptr
    if Hk == H:
        _lib.rope_rmsnorm_bwd(dyq.ptr, dyk.ptr, yq.ptr, yk.ptr, _A(rstd_q).ptr, _A(rstd_k).ptr, dq.ptr, dk.ptr,
                              c, s_, B, L, H, D, H * D, H * D, H * D, yq.code, stream())
    else:
        _lib.rope_rmsnorm_bwd(dyq.ptr, None, yq.ptr, None, _A(rstd_q).ptr, None, dq.ptr, None, c, s_, B, L, H, D,
                              H * D, H * D, H * D, yq.code, stream())
        _lib.rope_rmsnorm_bwd(dyk.ptr, None, yk.ptr, None, _A(rstd_k).ptr, None, dk.ptr, None, c, s_, B, L, Hk, D,
                              Hk * D, Hk * D, Hk * D, yk.code, stream())
    return dq, dk


__all__ = [n for n in dir() if n.startswith("fused_")] + ["gemm"]
