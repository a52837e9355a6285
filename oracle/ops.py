"""NumPy restatement of the reference's per-op CPU math (forward and backward).

TEST INFRASTRUCTURE: see oracle/__init__.py. Each function cites the reference
file:line it follows (paths relative to the reference project root). All
functions compute in the dtype of their inputs, as the reference does; the
tests feed fp32 (and fp16-rounded fp32 for the half-precision cases).
"""
import numpy as np

SQRT_2_OVER_PI = 0.7978845608  # mytorch/nn/functional/activations/gelu.py:21
GELU_COEFF = 0.044715          # mytorch/nn/functional/activations/gelu.py:22


# --------------------------------------------------------------------------
# LayerNorm  — mytorch/nn/functional/norm/layernorm.py:41-135 (manual_layernorm)
# --------------------------------------------------------------------------
def layernorm_fwd(x, gamma=None, beta=None, eps=1e-5):
    """x [N,E] -> (y, mean[N], rstd[N]); biased variance (np.var)."""
    mean = np.mean(x, axis=-1, keepdims=True)
    var = np.var(x, axis=-1, keepdims=True)
    rstd = np.reciprocal(np.sqrt(var + eps))
    x_hat = (x - mean) * rstd
    y = x_hat * gamma.reshape(1, -1) if gamma is not None else x_hat
    if beta is not None:
        y = y + beta.reshape(1, -1)
    return y, mean[:, 0], rstd[:, 0]


def layernorm_bwd(x, mean, rstd, dy, gamma=None):
    """-> (dx, dgamma, dbeta); layernorm.py:72-115."""
    x_hat = (x - mean[:, None]) * rstd[:, None]
    dgamma = np.sum(dy * x_hat, axis=0)
    dbeta = np.sum(dy, axis=0)
    dxh = dy * gamma if gamma is not None else dy
    m1 = np.mean(dxh, axis=-1, keepdims=True)
    m2 = np.mean(dxh * x_hat, axis=-1, keepdims=True)
    dx = rstd[:, None] * (dxh - m1 - x_hat * m2)
    return dx, dgamma, dbeta


# --------------------------------------------------------------------------
# RMSNorm — mytorch/nn/functional/norm/rmsnorm.py:47-113 (manual_rmsnorm)
# --------------------------------------------------------------------------
def rmsnorm_fwd(x, gamma=None, eps=1e-5):
    ms = np.mean(x * x, axis=-1, keepdims=True)
    rstd = np.reciprocal(np.sqrt(ms + eps))
    x_hat = x * rstd
    y = x_hat * gamma.reshape(1, -1) if gamma is not None else x_hat
    return y, rstd[:, 0]


def rmsnorm_bwd(x, rstd, dy, gamma=None):
    """-> (dx, dgamma); rmsnorm.py:73-98."""
    r = rstd[:, None]
    x_hat = x * r
    dgamma = np.sum(dy * x_hat, axis=0)
    m = dy * gamma if gamma is not None else dy
    s = np.sum(m * x, axis=-1, keepdims=True)
    dx = r * (m - (1.0 / x.shape[-1]) * (r * r * s) * x)
    return dx, dgamma


# --------------------------------------------------------------------------
# Linear — mytorch/nn/functional/layers/linear.py:69-147 (manual_linear);
# weight is [out, in] (mytorch/nn/modules/layers/linear.py:25)
# --------------------------------------------------------------------------
def linear_fwd(x, w, b=None):
    y = x @ w.T
    if b is not None:
        y = y + b
    return y


def linear_bwd(x, w, dy, has_bias=False):
    """-> (dx, dw, db)."""
    dx = dy @ w
    dw = dy.T @ x
    db = dy.sum(axis=0) if has_bias else None
    return dx, dw, db


# --------------------------------------------------------------------------
# GELU (tanh form) — mytorch/nn/functional/activations/gelu.py:8-61
# --------------------------------------------------------------------------
def gelu_fwd(x):
    inner = SQRT_2_OVER_PI * (x + GELU_COEFF * x * x * x)
    return 0.5 * x * (1.0 + np.tanh(inner))


def gelu_bwd(x, dy):
    x2 = x * x
    inner = SQRT_2_OVER_PI * (x + GELU_COEFF * x2 * x)
    t = np.tanh(inner)
    inner_grad = SQRT_2_OVER_PI * (1.0 + 3.0 * GELU_COEFF * x2)
    return 0.5 * (1.0 + t + x * (1 - t * t) * inner_grad) * dy


# --------------------------------------------------------------------------
# ReLU^2 — mytorch/nn/functional/activations/relu_squared.py:8-11
# (auto_relu_squared; the manual variant in the same file returns a zero
# gradient and is not the oracle)
# --------------------------------------------------------------------------
def relu2_fwd(x):
    r = np.maximum(x, 0)
    return r * r


def relu2_bwd(x, dy):
    return 2.0 * np.maximum(x, 0) * dy


# --------------------------------------------------------------------------
# Softmax — mytorch/nn/functional/activations/softmax.py:15-64 (manual_softmax)
# --------------------------------------------------------------------------
def softmax_fwd(x):
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def softmax_bwd(dy, s):
    return s * (dy - np.sum(dy * s, axis=-1, keepdims=True))


# --------------------------------------------------------------------------
# Cross entropy — mytorch/nn/functional/losses/cross_entropy.py:45-103
# (manual_cross_entropy); per-row form follows
# mytorch/nn/functional/fused_ops/cross_entropy.py:263 (loss[N], lse[N])
# --------------------------------------------------------------------------
def cross_entropy_rows(logits, labels, ignore_index=-100):
    """-> (loss[N] f32, lse[N] f32); ignored rows give loss 0."""
    lg = logits.astype(np.float32, copy=False)
    mx = np.max(lg, axis=1, keepdims=True)
    lse = (np.log(np.sum(np.exp(lg - mx), axis=1, keepdims=True)) + mx)[:, 0]
    mask = labels != ignore_index
    safe = np.where(mask, labels, 0)
    loss = (lse - lg[np.arange(lg.shape[0]), safe]) * mask
    return loss.astype(np.float32), lse.astype(np.float32)


def cross_entropy_fwd(logits, labels, ignore_index=-100):
    loss, _ = cross_entropy_rows(logits, labels, ignore_index)
    return loss.sum() / (labels != ignore_index).sum()


def cross_entropy_bwd(logits, labels, grad_output=1.0, ignore_index=-100):
    """d loss_mean / d logits · grad_output; cross_entropy.py:69-88."""
    lg = logits.astype(np.float32, copy=False)
    mask = labels != ignore_index
    g = softmax_fwd(lg)
    safe = np.where(mask, labels, 0)
    g[np.arange(lg.shape[0]), safe] -= 1
    g *= grad_output / mask.sum()
    g *= mask.reshape(-1, 1)
    return g


# --------------------------------------------------------------------------
# Embedding — mytorch/nn/functional/layers/embedding.py:8-10 (auto_embedding:
# Tensor.__getitem__, mytorch/tensor.py:1314-1358, backward np.add.at)
# --------------------------------------------------------------------------
def embedding_fwd(w, idx):
    return w[idx]


def embedding_bwd(dy, idx, num_rows):
    dw = np.zeros((num_rows, dy.shape[-1]), dtype=dy.dtype)
    np.add.at(dw, idx.reshape(-1), dy.reshape(-1, dy.shape[-1]))
    return dw


# --------------------------------------------------------------------------
# Causal attention — the un-fused branch of gpt2_trainer/gpt2.py:187-203:
# scores = q k^T / sqrt(D) + (-inf above the diagonal); softmax; @ v
# --------------------------------------------------------------------------
def attention_fwd(q, k, v, causal=True, scale=None):
    """q,k,v [B,H,S,D] -> (o, p) with p the attention probabilities."""
    D = q.shape[-1]
    scale = (1.0 / np.sqrt(D)) if scale is None else scale
    s = (q @ np.swapaxes(k, -1, -2)) * np.asarray(scale, dtype=q.dtype)
    if causal:
        S, T = s.shape[-2:]
        s = s + np.triu(np.full((S, T), -np.inf, dtype=q.dtype), k=1)
    p = softmax_fwd(s)
    return p @ v, p


def attention_bwd(q, k, v, p, do, scale=None):
    D = q.shape[-1]
    scale = (1.0 / np.sqrt(D)) if scale is None else scale
    dv = np.swapaxes(p, -1, -2) @ do
    dp = do @ np.swapaxes(v, -1, -2)
    ds = softmax_bwd(dp, p) * np.asarray(scale, dtype=q.dtype)
    dq = ds @ k
    dk = np.swapaxes(ds, -1, -2) @ q
    return dq, dk, dv


# --------------------------------------------------------------------------
# RoPE — mytorch/nn/functional/other/rotary_embeddings.py:57-109
# (half-split rotation; cos/sin are [T, D] with the two halves equal)
# --------------------------------------------------------------------------
def rope_cos_sin(head_dim, max_pos, base=10000.0):
    every_other = np.arange(0, head_dim, 2, dtype=np.float32)
    inv_freq = (1.0 / (base ** (every_other / head_dim))).astype(np.float32)
    t = np.arange(max_pos, dtype=np.float32)
    freqs = t[:, None] @ inv_freq[None, :]
    freqs = np.concatenate([freqs, freqs], axis=-1)
    return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)


def _rotate_half(x):
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def rope_fwd(x, cos, sin):
    """x [B,T,H,D]; cos/sin [T,D]."""
    c = cos[None, :, None, :].astype(x.dtype)
    s = sin[None, :, None, :].astype(x.dtype)
    return x * c + _rotate_half(x) * s


def rope_bwd(dy, cos, sin):
    """Transpose of the rotation = rotation by the negative angle."""
    c = cos[None, :, None, :].astype(dy.dtype)
    s = sin[None, :, None, :].astype(dy.dtype)
    return dy * c - _rotate_half(dy) * s


# --------------------------------------------------------------------------
# AdamW — mytorch/optim/optimizers.py:342-371. The decay is applied AFTER the
# Adam update and eps is not bias-corrected.
# --------------------------------------------------------------------------
def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, beta1_pow, beta2_pow):
    """In place on p, m, v (fp32). beta*_pow are the powers AFTER this step's
    multiply (optimizers.py:346-347)."""
    lr_t = lr * (1 - beta2_pow) ** 0.5 / (1 - beta1_pow)
    m *= beta1
    m += (1 - beta1) * g
    v *= beta2
    v += (1 - beta2) * (g ** 2)
    denom = v ** 0.5 + eps
    p -= (lr_t * m / denom).astype(p.dtype)
    if weight_decay != 0.0:
        p[...] = p - lr * weight_decay * p
    return p, m, v


# --------------------------------------------------------------------------
# Gradient clipping — mytorch/accelerate.py:799-856 (single process)
# --------------------------------------------------------------------------
def clip_grad_norm(grads, max_norm=1.0):
    """Scales grads in place; returns the total norm before clipping."""
    sq = 0.0
    for g in grads:
        sq += float(np.sum(g.astype(np.float32) ** 2))
    total = float(np.sqrt(sq))
    coef = max_norm / (total + 1e-6)
    if coef < 1.0:
        for g in grads:
            g *= coef
    return total


class GradScaler:
    """Dynamic loss scale state machine — mytorch/accelerate.py:31-124."""

    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0,
                 backoff_factor=0.5, growth_interval=2000):
        self.scale = init_scale
        self.growth_factor = growth_factor
        self.backoff_factor = backoff_factor
        self.growth_interval = growth_interval
        self.unskipped = 0

    def update(self, found_inf):
        if found_inf:
            self.scale *= self.backoff_factor
            self.unskipped = 0
        else:
            self.unskipped += 1
            if self.unskipped == self.growth_interval:
                self.scale *= self.growth_factor
                self.unskipped = 0
