"""Differentiable ops of the GPT training step: the `fused=True` branch of the
reference's mytorch/nn/functional/* dispatchers, each op a forward call into
the CUDA library plus a backward closure (same structure as e.g.
mytorch/nn/functional/layers/linear.py:149-236).

Inputs keep their leading dimensions; kernels see them flattened to rows.
"""
import math

from .. import _lib
from .. import fused_ops as K
from ..array import DeviceArray, stream
from ..tensor import Tensor


def _needs_graph(*ts):
    return Tensor.build_graph_enabled() and any(t is not None and t.requires_grad for t in ts)


def _flat2d(arr):
    return arr.reshape(-1, arr.shape[-1])


def _param_grad_gemm(dy2, x2, weight):
    """weight.grad (fp32) += dy2^T @ x2, straight into the accumulation buffer."""
    buf = weight.param_grad_buffer() if weight.is_param else None
    if buf is not None:
        K.gemm(dy2, x2, trans_a=True, out=buf, accumulate=2 if dy2.dtype != "float32" else 1)
    else:
        weight._accumulate(K.gemm(dy2, x2, trans_a=True))


# ---------------------------------------------------------------- linear ----
def _existing_grad(t):
    """The gradient buffer of an activation that already holds another branch's
    gradient (so a kernel can add into it), else None."""
    if t.requires_grad and not t.is_param and t.grad is not None and t.grad.dtype == t.dtype:
        return t.grad
    return None


def _input_grad_gemm(x, g2, w):
    """x.grad (+)= g2 @ w. When another branch has already left its gradient in x.grad (the q, k
    and v projections of one normalised input, say), the sum happens in the GEMM's epilogue
    (C = result + C, read slab by slab) instead of a GEMM into a temporary plus an add pass."""
    have = _existing_grad(x)
    if have is not None and g2.dtype == have.dtype:
        h2 = _flat2d(have)
        K.gemm(g2, w, out=h2, aux=h2, aux_mode=1)
    else:
        x._accumulate(K.gemm(g2, w).reshape(x.shape))


def linear(x, weight, bias=None, auto=False, fused=True, act_func=None, residual=None):
    """y = act(x @ weight^T + bias) (+ residual), weight [out, in]
    (mytorch/nn/functional/layers/linear.py:149-236). No transposed copy of the
    weight is made: the GEMM reads it K-major in place. `residual` (same shape as
    y) is added in the GEMM epilogue: the `x + sublayer(x)` of a transformer block
    (gpt2_trainer/gpt2.py:308-311) without a separate add kernel."""
    x2 = _flat2d(x.data)
    want_pre = act_func is not None and _needs_graph(x, weight, bias)
    res = K.gemm(x2, weight.data, trans_b=True, bias=None if bias is None else bias.data,
                 act=act_func, preact=want_pre,
                 aux=None if residual is None else _flat2d(residual.data), aux_mode=1)
    y2, pre = res if want_pre else (res, None)
    out = Tensor(y2.reshape(*x.shape[:-1], weight.shape[0]))
    if _needs_graph(x, weight, bias, residual):
        def _bw(g):
            if residual is not None and residual.requires_grad:
                residual._accumulate(g)          # the skip connection passes the gradient through
            g2 = _flat2d(g)
            if act_func is not None:
                g2 = K.fused_activation_backward(pre, g2, act_func)
            if weight.requires_grad:
                _param_grad_gemm(g2, x2, weight)
            if bias is not None and bias.requires_grad:
                buf = bias.param_grad_buffer()
                _lib.colsum(g2.ptr, buf.ptr, g2.shape[0], g2.shape[1], g2.code, buf.code, 1, stream())
            if x.requires_grad:
                _input_grad_gemm(x, g2, weight.data)
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<LinearBackward>"
        out._add_parents(x, weight, bias, residual)
    return out


def mlp(x, w1, w2, act_func="gelu", residual=None):
    """act(x @ w1^T) @ w2^T (+ residual): the FeedForward of a block
    (gpt2_trainer/gpt2.py:237-283, bias-free form) as one autograd node. The
    activation is applied in the first GEMM's epilogue, which saves the
    activation's derivative (same tanh) instead of the pre-activation; the backward
    multiplies by it in the epilogue of the dY @ W2 GEMM (mt_gemm_ex aux_mode 5,
    the saved tensor read slab by slab through TMA), so the backward of the
    activation costs no kernel and no transcendental."""
    x2 = _flat2d(x.data)
    graph = _needs_graph(x, w1, w2, residual)
    # relu(u)^2 carries its own derivative: 2*relu(u) = 2*sqrt(h). Nothing extra is stored and the
    # backward GEMM takes the square root of h in its epilogue (aux_mode 6).
    from_output = act_func in ("relu_squared", "relu2")
    if graph and not from_output:
        h, u = K.gemm(x2, w1.data, trans_b=True, act=act_func, preact="grad")      # u = act'(x @ w1^T)
    else:
        h, u = K.gemm(x2, w1.data, trans_b=True, act=act_func), None
    y2 = K.gemm(h, w2.data, trans_b=True, aux=None if residual is None else _flat2d(residual.data), aux_mode=1)
    out = Tensor(y2.reshape(*x.shape[:-1], w2.shape[0]))
    if graph:
        def _bw(g):
            if residual is not None and residual.requires_grad:
                residual._accumulate(g)
            g2 = _flat2d(g)
            if w2.requires_grad:
                _param_grad_gemm(g2, h, w2)
            du = (K.gemm(g2, w2.data, aux=h, aux_mode=6) if from_output                # (dy @ w2) * act'(.), one kernel
                  else K.gemm(g2, w2.data, aux=u, aux_mode=5))
            if w1.requires_grad:
                _param_grad_gemm(du, x2, w1)
            if x.requires_grad:
                _input_grad_gemm(x, du, w1.data)
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<MLPBackward>"
        out._add_parents(x, w1, w2, residual)
    return out


# ------------------------------------------------------------- embedding ----
def embedding(indices, weight, fused=True):
    """weight[indices] (mytorch/nn/functional/layers/embedding.py:11-43)."""
    idx = indices.data if isinstance(indices, Tensor) else DeviceArray.from_numpy(indices, "int32")
    out = Tensor(K.fused_embedding_forward(weight.data, idx))
    if _needs_graph(weight):
        def _bw(g):
            K.fused_embedding_backward(g.reshape(-1, weight.shape[1]), weight.data, idx, out=weight.param_grad_buffer())
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<EmbeddingBackward>"
        out._add_parents(weight)
    return out


def token_position_embedding(indices, wte, wpe):
    """wte[ids] + wpe[arange(T)] in one pass: the Embeddings module of
    gpt2_trainer/gpt2.py:105-119."""
    idx = indices.data if isinstance(indices, Tensor) else DeviceArray.from_numpy(indices, "int32")
    B, T = idx.shape
    V, E = wte.shape
    out_arr = DeviceArray.empty((B, T, E), wte.dtype)
    _lib.embedding_pos_fwd(wte.data.ptr, wpe.data.ptr, idx.ptr, out_arr.ptr, B * T, T, E, V, wte.data.code, stream())
    out = Tensor(out_arr)
    if _needs_graph(wte, wpe):
        def _bw(g):
            if wte.requires_grad:
                K.fused_embedding_backward(g.reshape(-1, E), wte.data, idx, out=wte.param_grad_buffer())
            if wpe.requires_grad:
                _lib.pos_embedding_bwd(g.ptr, wpe.param_grad_buffer().ptr, B, T, E, g.code, stream())
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<EmbeddingsBackward>"
        out._add_parents(wte, wpe)
    return out


# ------------------------------------------------------------------ norms ----
def layernorm(x, weight=None, bias=None, eps=1e-5, training=True, auto=False, fused=True):
    """mytorch/nn/functional/norm/layernorm.py:138-212."""
    x2 = _flat2d(x.data)
    g_arr = None if weight is None else weight.data
    b_arr = None if bias is None else bias.data
    y, mean, rstd = K.fused_layernorm_forward(x2, g_arr, b_arr, eps)
    out = Tensor(y.reshape(x.shape))
    if _needs_graph(x, weight, bias):
        def _bw(g):
            dg = weight.param_grad_buffer() if (weight is not None and weight.requires_grad) else None
            db = bias.param_grad_buffer() if (bias is not None and bias.requires_grad) else None
            have = _existing_grad(x)
            dx, _, _ = K.fused_layernorm_backward(x2, mean, rstd, _flat2d(g), g_arr, None, dgamma_out=dg, dbeta_out=db,
                                                  dx_out=None if have is None else _flat2d(have))
            if x.requires_grad and have is None:
                x._accumulate(dx.reshape(x.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<LayerNormBackward>"
        out._add_parents(x, weight, bias)
    return out


def rmsnorm(x, weight=None, eps=1e-5, training=True, auto=False, fused=True):
    """mytorch/nn/functional/norm/rmsnorm.py:115-189."""
    x2 = _flat2d(x.data)
    g_arr = None if weight is None else weight.data
    y, rstd = K.fused_rmsnorm_forward(x2, g_arr, eps)
    out = Tensor(y.reshape(x.shape))
    if _needs_graph(x, weight):
        def _bw(g):
            dg = weight.param_grad_buffer() if (weight is not None and weight.requires_grad) else None
            have = _existing_grad(x)
            dx, _ = K.fused_rmsnorm_backward(x2, rstd, _flat2d(g), g_arr, dgamma_out=dg,
                                             dx_out=None if have is None else _flat2d(have))
            if x.requires_grad and have is None:
                x._accumulate(dx.reshape(x.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<RMSNormBackward>"
        out._add_parents(x, weight)
    return out


# ------------------------------------------------------------ activations ----
def _activation(x, name, label):
    out = Tensor(K.fused_activation_forward(x.data, name))
    if _needs_graph(x):
        def _bw(g):
            x._accumulate(K.fused_activation_backward(x.data, g, name))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, label
        out._add_parents(x)
    return out


def gelu(x, auto=False, fused=True):
    """tanh-GELU (mytorch/nn/functional/activations/gelu.py:8-95)."""
    return _activation(x, "gelu", "<GELUBackward>")


def relu_squared(x, auto=False, fused=True):
    """relu(x)^2 (mytorch/nn/functional/activations/relu_squared.py:8-80; the
    gradient is 2*relu(x), i.e. the reference's `auto` path)."""
    return _activation(x, "relu_squared", "<ReLUSquaredBackward>")


def relu(x, auto=False, fused=True):
    return _activation(x, "relu", "<ReLUBackward>")


def softmax(x, dim=-1, auto=False, fused=True):
    """Softmax over the last axis (mytorch/nn/functional/activations/softmax.py:15-159)."""
    if dim not in (-1, x.ndim - 1):
        raise NotImplementedError("softmax is implemented over the last axis")
    s = K.fused_softmax_forward(_flat2d(x.data))
    out = Tensor(s.reshape(x.shape))
    if _needs_graph(x):
        def _bw(g):
            x._accumulate(K.fused_softmax_backward(_flat2d(g), s).reshape(x.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<SoftmaxBackward>"
        out._add_parents(x)
    return out


# --------------------------------------------------------- cross entropy ----
def cross_entropy(logits, targets, ignore_index=-100, softcap=None, auto=False, fused=True, fused_backward=False):
    """Mean over valid rows of lse - logit[target]
    (mytorch/nn/functional/losses/cross_entropy.py:107-178). The valid count and
    the upstream gradient stay on the device (the reference reads both back to
    the host, :120 and :144); the backward overwrites the logits buffer, as the
    reference's fused kernel does. Unlike the reference's dispatcher (:178),
    `softcap` is honoured when given.

    fused_backward=True computes the gradient in the forward pass, while each row of logits is
    still in cache (one read and one write of the logits instead of two reads and one write):
    the logits buffer is overwritten ALREADY HERE, so it suits training loops that do not look at
    the logits after the loss. The gradient is pre-multiplied by the upstream value that
    backward() is expected to bring (`Tensor.loss_grad_hint`, the loss scale under mixed
    precision, else 1); if something else arrives it is corrected by one more pass."""
    assert ignore_index == -100, "ignore_index is fixed to -100 like the reference's fused kernel"
    lg = _flat2d(logits.data)
    tg = targets.data if isinstance(targets, Tensor) else DeviceArray.from_numpy(targets, "int32")
    tg = tg.reshape(-1)
    if fused_backward and _needs_graph(logits):
        hint = Tensor.loss_grad_hint
        loss_rows, lse, tot = K.fused_cross_entropy_forward_backward(lg, tg, softcap, scale_dev=hint)
        out = Tensor(DeviceArray(tot.ptr + 8, (), "float32", base=tot))

        def _bw_fused(g):
            expected = hint.ptr if hint is not None else Tensor._unit_grad_ptr
            if g.ptr != expected:      # another upstream gradient than announced: rescale by g / hint
                one = None
                if hint is None:
                    one = DeviceArray.empty((1,), "float32").fill_(1.0)
                _lib.scale_ratio(lg.ptr, lg.size, g.ptr, (hint if hint is not None else one).ptr, lg.code, stream())
            logits._accumulate(lg.reshape(logits.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw_fused, "<CrossEntropyFusedBackward>"
        out._add_parents(logits)
        return out
    loss_rows, lse, tot = K.fused_cross_entropy_forward(lg, tg, softcap, reduce=True)
    out = Tensor(DeviceArray(tot.ptr + 8, (), "float32", base=tot))   # the mean, a device scalar
    if _needs_graph(logits):
        def _bw(g):
            # g is the upstream gradient of the MEAN loss (device scalar, fp32)
            cnt = DeviceArray(tot.ptr + 4, (1,), "float32", base=tot)
            K.fused_cross_entropy_backward(lg, tg, lse, softcap, scale=1.0, scale_dev=g, count_dev=cnt)
            logits._accumulate(lg.reshape(logits.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<CrossEntropyBackward>"
        out._add_parents(logits)
    return out


def lm_head_cross_entropy(x, weight, targets, chunk=8192, softcap=None):
    """mean cross entropy of (x @ weight^T) against targets WITHOUT materialising the
    [rows, vocab] logits: the vocabulary is walked in chunks; each chunk's logits are
    produced by the tensor-core GEMM into one reusable buffer, reduced to a running
    log-sum-exp (forward) or turned into dlogits and fed straight to the dX / dW GEMMs
    (backward, which recomputes the chunk logits). Equivalent to
    cross_entropy(linear(x, weight), targets) (gpt2_trainer/gpt2.py:368 followed by
    mytorch/nn/functional/losses/cross_entropy.py:107-178) with vocab/chunk times less
    logits memory, at the price of one extra lm_head GEMM in the backward."""
    x2 = _flat2d(x.data)
    M, E = x2.shape
    V = weight.shape[0]
    tg = targets.data if isinstance(targets, Tensor) else DeviceArray.from_numpy(targets, "int32")
    tg = tg.reshape(-1)
    chunk = max(8, min(int(chunk), V) // 8 * 8) if V >= 8 else V
    lse = DeviceArray.empty((M,), "float32").fill_(float("-inf"))
    tgt = DeviceArray.zeros((M,), "float32")
    buf = DeviceArray.empty((M, chunk), x2.dtype)
    cap = float(softcap or 0.0)
    for c0 in range(0, V, chunk):
        c1 = min(V, c0 + chunk)
        view = DeviceArray(buf.ptr, (M, c1 - c0), buf.dtype, base=buf)
        K.gemm(x2, weight.data.rows(c0, c1), trans_b=True, out=view)
        _lib.ce_chunk_fwd(view.ptr, tg.ptr, lse.ptr, tgt.ptr, M, c1 - c0, c1 - c0, c0, cap, view.code, stream())
    loss_rows = DeviceArray.empty((M,), "float32")
    tot = DeviceArray.empty((3,), "float32")
    _lib.ce_chunk_finish(lse.ptr, tgt.ptr, tg.ptr, loss_rows.ptr, tot.ptr, tot.ptr + 4, tot.ptr + 8, M, stream())
    out = Tensor(DeviceArray(tot.ptr + 8, (), "float32", base=tot))
    if _needs_graph(x, weight):
        def _bw(g):
            cnt = DeviceArray(tot.ptr + 4, (1,), "float32", base=tot)
            dx32 = DeviceArray.zeros((M, E), "float32") if x.requires_grad else None
            for c0 in range(0, V, chunk):
                c1 = min(V, c0 + chunk)
                view = DeviceArray(buf.ptr, (M, c1 - c0), buf.dtype, base=buf)
                wc = weight.data.rows(c0, c1)
                K.gemm(x2, wc, trans_b=True, out=view)                       # recompute the chunk's logits
                _lib.ce_chunk_bwd(view.ptr, tg.ptr, lse.ptr, view.ptr, 1.0, g.ptr, cnt.ptr, M, c1 - c0, c1 - c0, c0,
                                  cap, view.code, stream())
                if weight.requires_grad:
                    gbuf = weight.param_grad_buffer().rows(c0, c1)
                    K.gemm(view, x2, trans_a=True, out=gbuf, accumulate=2 if view.dtype != "float32" else 1)
                if dx32 is not None:
                    K.gemm(view, wc, out=dx32, accumulate=1)                 # dX += dlogits_c @ W_c (fp32)
            if dx32 is not None:
                x._accumulate(dx32.astype(x.dtype).reshape(x.shape))
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<LMHeadCrossEntropyBackward>"
        out._add_parents(x, weight)
    return out


# -------------------------------------------------------------- attention ----
def scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal=False, softmax_scale=None, enable_gqa=False):
    """q [B,H,S,D], k, v [B,Hkv,S,D] contiguous (mytorch/nn/functional/flash_attention/
    flash_attention.py:20-127); with enable_gqa=True Hkv may divide H and query head h
    attends to key/value head h // (H // Hkv). One backward launch (the reference runs its
    backward kernel twice, :73-91)."""
    if k.shape[1] != q.shape[1] and not enable_gqa:
        # the reference's check (flash_attention.py:43-44): fewer key/value heads need the flag
        raise ValueError(f"q has {q.shape[1]} heads and k has {k.shape[1]}: pass enable_gqa=True for grouped-query attention")
    _, _, _, o, m = K.fused_sdpa_forward(q.data, k.data, v.data, attn_mask, is_causal, softmax_scale)
    out = Tensor(o)
    if _needs_graph(q, k, v):
        def _bw(g):
            dq, dk, dv = K.fused_sdpa_backward(g, q.data, k.data, v.data, o, m, None, is_causal, softmax_scale)
            for t, d in ((q, dq), (k, dk), (v, dv)):
                if t.requires_grad:
                    t._accumulate(d)
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<SDPABackward>"
        out._add_parents(q, k, v)
    return out


def bthd_attention(q, k, v, is_causal=True):
    """Self-attention on q, k, v laid out [B, T, H, D] (what a Linear followed by
    reshape gives, nanochat_trainer/core/nanochat_gpt.py:112-127): heads are
    addressed through strides, so the reference's transpose(1, 2) + contiguous
    copies are not made; the result is [B, T, H*D]."""
    B, T, H, D = q.shape
    Hk = k.shape[2]
    if k.shape != (B, T, Hk, D) or v.shape != k.shape or H % Hk:
        raise NotImplementedError(f"q [B,T,H,D] and k, v [B,T,Hkv,D] with H a multiple of Hkv; got {q.shape}, {k.shape}, {v.shape}")
    st = _lib.Strides3(T * H * D, D, H * D)
    sk_ = _lib.Strides3(T * Hk * D, D, Hk * D)                              # fewer key/value heads per token
    as4 = lambda a, h=H: DeviceArray(a.ptr, (B, h, T, D), a.dtype, base=a)  # logical [B,h,T,D] over [B,T,h,D] memory
    qv, kv, vv = as4(q.data), as4(k.data, Hk), as4(v.data, Hk)
    o_arr = DeviceArray.empty((B, T, H * D), q.dtype)
    ov = as4(o_arr)
    _, _, _, _, m = K.fused_sdpa_forward(qv, kv, vv, None, is_causal, None, strides=(st, sk_, sk_), out=ov, out_strides=st)
    out = Tensor(o_arr)
    if _needs_graph(q, k, v):
        def _bw(g):
            dq = DeviceArray.empty((B, T, H, D), q.dtype)
            dk, dv = (DeviceArray.empty((B, T, Hk, D), q.dtype) for _ in range(2))
            K.fused_sdpa_backward(as4(g), qv, kv, vv, ov, m, None, is_causal, None, strides=(st, sk_, sk_),
                                  out=(as4(dq), as4(dk, Hk), as4(dv, Hk)), out_strides=(st, sk_, sk_), o_strides=st, do_strides=st)
            for t, d in ((q, dq), (k, dk), (v, dv)):
                if t.requires_grad:
                    t._accumulate(d)
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<BTHDAttentionBackward>"
        out._add_parents(q, k, v)
    return out


def qkv_attention(qkv, num_heads, is_causal=True):
    """Causal self-attention straight on the fused projection: qkv [B,T,3E] holds,
    per head, a contiguous [q|k|v] group of 3*D columns — the layout produced by
    `reshape(B,T,H,3D).transpose(1,2).chunk(3)` in gpt2_trainer/gpt2.py:168-177.
    Q, K and V are read in place through strides and the output is written as
    [B,T,E], so none of the reference's transpose/contiguous copies exist."""
    B, T, E3 = qkv.shape
    E = E3 // 3
    D = E // num_heads
    a = qkv.data
    item = a.itemsize
    sin = _lib.Strides3(T * E3, 3 * D, E3)
    qv = DeviceArray(a.ptr, (B, num_heads, T, D), a.dtype, base=a)
    kv = DeviceArray(a.ptr + D * item, (B, num_heads, T, D), a.dtype, base=a)
    vv = DeviceArray(a.ptr + 2 * D * item, (B, num_heads, T, D), a.dtype, base=a)
    o_arr = DeviceArray.empty((B, T, E), a.dtype)
    sout = _lib.Strides3(T * E, D, E)
    ov = DeviceArray(o_arr.ptr, (B, num_heads, T, D), a.dtype, base=o_arr)
    _, _, _, _, m = K.fused_sdpa_forward(qv, kv, vv, None, is_causal, None, strides=(sin, sin, sin), out=ov, out_strides=sout)
    out = Tensor(o_arr)
    if _needs_graph(qkv):
        def _bw(g):
            dqkv = DeviceArray.empty((B, T, E3), a.dtype)
            dqv = DeviceArray(dqkv.ptr, (B, num_heads, T, D), a.dtype, base=dqkv)
            dkv = DeviceArray(dqkv.ptr + D * item, (B, num_heads, T, D), a.dtype, base=dqkv)
            dvv = DeviceArray(dqkv.ptr + 2 * D * item, (B, num_heads, T, D), a.dtype, base=dqkv)
            gv = DeviceArray(g.ptr, (B, num_heads, T, D), a.dtype, base=g)
            K.fused_sdpa_backward(gv, qv, kv, vv, ov, m, None, is_causal, None, strides=(sin, sin, sin),
                                  out=(dqv, dkv, dvv), out_strides=(sin, sin, sin), o_strides=sout, do_strides=sout)
            qkv._accumulate(dqkv)
        out.requires_grad = True
        out.grad_fn, out.grad_fn_name = _bw, "<QKVAttentionBackward>"
        out._add_parents(qkv)
    return out


# ------------------------------------------------------------------- rope ----
def precompute_rotary_cos_sin(head_dim, max_position_embeddings=2048, base=10000, scaling_factor=1.0):
    """cos/sin tables [T, D] fp32 with duplicated halves
    (mytorch/nn/functional/other/rotary_embeddings.py:57-88)."""
    import numpy as np
    every_other = np.arange(0, head_dim, 2, dtype=np.float32)
    inv_freq = (1.0 / (base ** (every_other / head_dim))).astype(np.float32)
    t = np.arange(max_position_embeddings, dtype=np.float32) / scaling_factor
    freqs = t[:, None] @ inv_freq[None, :]
    freqs = np.concatenate([freqs, freqs], axis=-1)
    return (DeviceArray.from_numpy(np.cos(freqs).astype(np.float32)),
            DeviceArray.from_numpy(np.sin(freqs).astype(np.float32)))


def apply_rotary_pos_embed(q, k, cos, sin, unsqueeze_dim=2, auto=False, fused=True):
    """Half-split rotary embedding of q and k [B,T,H,D]
    (mytorch/nn/functional/other/rotary_embeddings.py:111-158). Out of place
    here (the reference rotates in place), so the inputs stay valid."""
    outs = []
    for x in (q, k):
        arr = x.data.copy()
        K.fused_rope_forward(arr, cos, sin)
        o = Tensor(arr)
        if _needs_graph(x):
            def _bw(g, x=x):
                gg = g.copy()
                K.fused_rope_backward(gg, cos, sin)
                x._accumulate(gg)
            o.requires_grad = True
            o.grad_fn, o.grad_fn_name = _bw, "<RopeBackward>"
            o._add_parents(x)
        outs.append(o)
    return outs[0], outs[1]


def rope_qk_norm(q, k, cos, sin, eps=1e-5):
    """norm(rope(q)), norm(rope(k)) for q, k [B,T,H,D]: rotary embedding followed by the
    parameter-free RMSNorm over head_dim (nanochat_trainer/core/nanochat_gpt.py:119-124) as ONE
    autograd node and one kernel per direction. Each tensor is read and written once (the
    separate ops copy, rotate in place and normalise: three passes each way), and only the
    outputs and one rstd per head vector are kept for the backward pass. Head sizes the fused
    kernel does not take (anything but 2..32 16-byte vectors) go through the separate ops."""
    D = q.shape[-1]
    vec = 16 // q.data.itemsize
    if D % vec or (D // vec) not in (2, 4, 8, 16, 32) or q.shape[:2] != k.shape[:2] or k.shape[-1] != D:
        q2, k2 = apply_rotary_pos_embed(q, k, cos, sin)
        return (rmsnorm(q2.reshape(-1, D), eps=eps).reshape(q.shape), rmsnorm(k2.reshape(-1, D), eps=eps).reshape(k.shape))
    yq, yk, rq, rk = K.fused_rope_rmsnorm_forward(q.data, k.data, cos, sin, eps)
    oq, ok = Tensor(yq), Tensor(yk)
    if _needs_graph(q, k):
        # Two outputs, one backward kernel: each output's closure parks its gradient; a graph-only
        # node between the outputs and (q, k) runs after both (it is their parent in the graph) and
        # launches once. An output that received no gradient counts as zero.
        slot = [None, None]

        def _bw_pair(_):
            gq = slot[0] if slot[0] is not None else DeviceArray.zeros(yq.shape, yq.dtype)
            gk = slot[1] if slot[1] is not None else DeviceArray.zeros(yk.shape, yk.dtype)
            dq, dk = K.fused_rope_rmsnorm_backward(gq, gk, yq, yk, rq, rk, cos, sin)
            slot[0] = slot[1] = None
            if q.requires_grad:
                q._accumulate(dq)
            if k.requires_grad:
                k._accumulate(dk)

        pair = Tensor(yq)
        pair.requires_grad = True
        pair.grad_fn, pair.grad_fn_name = _bw_pair, "<RopeQKNormBackward>"
        pair._add_parents(q, k)

        def _park(i):
            def f(g):
                slot[i] = g
            return f
        for i, o in enumerate((oq, ok)):
            o.requires_grad = True
            o.grad_fn, o.grad_fn_name = _park(i), "<RopeQKNormOutput>"
            o._add_parents(pair)
    return oq, ok


def dropout(x, dropout_p=0.0, training=True):
    """Only p = 0 is on the GPT training path (all configs use 0.0)."""
    if dropout_p != 0.0 and training:
        raise NotImplementedError("dropout with p > 0 is outside the GPT training-step path")
    return x
