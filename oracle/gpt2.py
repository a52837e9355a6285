"""NumPy restatement of the reference GPT-2 training step (forward, backward,
AdamW) built from oracle.ops. TEST INFRASTRUCTURE: see oracle/__init__.py.

Wiring follows gpt2_trainer/gpt2.py: Embeddings :88-119 (token + learned
positional), TransformerBlock :285-311 (pre-LayerNorm; block LayerNorms have a
weight and, with use_bias=False, no bias), Attention :120-235 (qkv projection
viewed as [B,T,H,3D] so each head owns a contiguous [q|k|v] column group,
:168-177), FeedForward :237-283 (GELU, 4x), final LayerNorm with weight AND
bias :329-332, lm_head tied to the token embedding :340-347. Parameter names
are the reference state_dict keys (mytorch/nn/modules/base_module.py:220-241).
"""
from dataclasses import dataclass

import numpy as np

from . import ops


@dataclass
class GPT2Config:  # field names follow gpt2_trainer/gpt2.py:12-27
    vocab_size: int = 50257
    max_seq_len: int = 1024
    embed_dim: int = 768
    mlp_ratio: int = 4
    num_blocks: int = 12
    num_heads: int = 12


def init_params(cfg, seed=0, dtype=np.float32):
    """Seeded N(0, 0.02) weights (out_proj: 0.02/sqrt(2L)), LayerNorm weight 1,
    final bias 0 — the distributions of gpt2.py:334-389, drawn from a NumPy
    Generator in state_dict order so that every implementation under test can
    be given identical values."""
    rng = np.random.default_rng(seed)
    E, H = cfg.embed_dim, cfg.embed_dim * cfg.mlp_ratio
    std_o = 0.02 / np.sqrt(2 * cfg.num_blocks)
    p = {}
    p["embeddings.char_embeddings.weight"] = rng.normal(0, 0.02, (cfg.vocab_size, E))
    p["embeddings.position_embeddings.weight"] = rng.normal(0, 0.02, (cfg.max_seq_len, E))
    for i in range(cfg.num_blocks):
        b = f"blocks.{i}."
        p[b + "attention.qkv_proj.weight"] = rng.normal(0, 0.02, (3 * E, E))
        p[b + "attention.out_proj.weight"] = rng.normal(0, std_o, (E, E))
        p[b + "layernorm1.weight"] = np.ones(E)
        p[b + "feedforward.intermediate_dense.weight"] = rng.normal(0, 0.02, (H, E))
        p[b + "feedforward.out_proj.weight"] = rng.normal(0, std_o, (E, H))
        p[b + "layernorm2.weight"] = np.ones(E)
    p["final_layer_norm.weight"] = np.ones(E)
    p["final_layer_norm.bias"] = np.zeros(E)
    return {k: np.ascontiguousarray(v, dtype=dtype) for k, v in p.items()}


def decay_mask(params):
    """Weight decay on >=2-D tensors only (gpt2_trainer/train_gpt2.py:271-281)."""
    return {k: v.ndim >= 2 for k, v in params.items()}


def _split_heads(qkv, B, T, H, D):
    x = qkv.reshape(B, T, H, 3 * D).transpose(0, 2, 1, 3)
    return x[..., :D], x[..., D:2 * D], x[..., 2 * D:]


def _merge_heads(dq, dk, dv):
    B, H, T, D = dq.shape
    x = np.concatenate([dq, dk, dv], axis=-1)          # [B,H,T,3D]
    return x.transpose(0, 2, 1, 3).reshape(B * T, H * 3 * D)


def forward(params, cfg, ids, targets=None):
    """ids [B,T] int -> (loss or None, logits [B*T,V], cache for backward)."""
    B, T = ids.shape
    E, H = cfg.embed_dim, cfg.num_heads
    D = E // H
    wte = params["embeddings.char_embeddings.weight"]
    wpe = params["embeddings.position_embeddings.weight"]
    x = (ops.embedding_fwd(wte, ids) + wpe[None, :T]).reshape(B * T, E)
    cache = {"ids": ids, "blocks": []}
    for i in range(cfg.num_blocks):
        b = f"blocks.{i}."
        c = {"x0": x}
        h1, c["mu1"], c["rs1"] = ops.layernorm_fwd(x, params[b + "layernorm1.weight"])
        c["h1"] = h1
        qkv = ops.linear_fwd(h1, params[b + "attention.qkv_proj.weight"])
        q, k, v = _split_heads(qkv, B, T, H, D)
        o, p = ops.attention_fwd(q, k, v, causal=True)
        c["q"], c["k"], c["v"], c["p"] = q, k, v, p
        a = o.transpose(0, 2, 1, 3).reshape(B * T, E)
        c["a"] = a
        x = x + ops.linear_fwd(a, params[b + "attention.out_proj.weight"])
        c["x1"] = x
        h2, c["mu2"], c["rs2"] = ops.layernorm_fwd(x, params[b + "layernorm2.weight"])
        c["h2"] = h2
        u = ops.linear_fwd(h2, params[b + "feedforward.intermediate_dense.weight"])
        c["u"] = u
        g = ops.gelu_fwd(u)
        c["g"] = g
        x = x + ops.linear_fwd(g, params[b + "feedforward.out_proj.weight"])
        cache["blocks"].append(c)
    cache["xf"] = x
    hf, cache["muf"], cache["rsf"] = ops.layernorm_fwd(
        x, params["final_layer_norm.weight"], params["final_layer_norm.bias"])
    cache["hf"] = hf
    logits = ops.linear_fwd(hf, wte)
    cache["logits"] = logits
    loss = None
    if targets is not None:
        cache["targets"] = targets.reshape(-1)
        loss = ops.cross_entropy_fwd(logits, cache["targets"])
    return loss, logits, cache


def backward(params, cfg, cache, grad_output=1.0):
    """-> dict of gradients keyed like params (tied weight gets both terms)."""
    ids = cache["ids"]
    B, T = ids.shape
    E, H = cfg.embed_dim, cfg.num_heads
    wte = params["embeddings.char_embeddings.weight"]
    grads = {}
    dlogits = ops.cross_entropy_bwd(cache["logits"], cache["targets"], grad_output)
    dlogits = dlogits.astype(wte.dtype, copy=False)
    dhf, dwte, _ = ops.linear_bwd(cache["hf"], wte, dlogits)
    dx, dg, db = ops.layernorm_bwd(cache["xf"], cache["muf"], cache["rsf"], dhf,
                                   params["final_layer_norm.weight"])
    grads["final_layer_norm.weight"], grads["final_layer_norm.bias"] = dg, db
    for i in reversed(range(cfg.num_blocks)):
        b = f"blocks.{i}."
        c = cache["blocks"][i]
        dg_, dw2, _ = ops.linear_bwd(c["g"], params[b + "feedforward.out_proj.weight"], dx)
        grads[b + "feedforward.out_proj.weight"] = dw2
        du = ops.gelu_bwd(c["u"], dg_)
        dh2, dw1, _ = ops.linear_bwd(c["h2"], params[b + "feedforward.intermediate_dense.weight"], du)
        grads[b + "feedforward.intermediate_dense.weight"] = dw1
        dx1, dgam2, _ = ops.layernorm_bwd(c["x1"], c["mu2"], c["rs2"], dh2,
                                          params[b + "layernorm2.weight"])
        grads[b + "layernorm2.weight"] = dgam2
        dx = dx + dx1
        da, dwo, _ = ops.linear_bwd(c["a"], params[b + "attention.out_proj.weight"], dx)
        grads[b + "attention.out_proj.weight"] = dwo
        do = da.reshape(B, T, H, E // H).transpose(0, 2, 1, 3)
        dq, dk, dv = ops.attention_bwd(c["q"], c["k"], c["v"], c["p"], do)
        dqkv = _merge_heads(dq, dk, dv)
        dh1, dwqkv, _ = ops.linear_bwd(c["h1"], params[b + "attention.qkv_proj.weight"], dqkv)
        grads[b + "attention.qkv_proj.weight"] = dwqkv
        dx0, dgam1, _ = ops.layernorm_bwd(c["x0"], c["mu1"], c["rs1"], dh1,
                                          params[b + "layernorm1.weight"])
        grads[b + "layernorm1.weight"] = dgam1
        dx = dx + dx0
    dx3 = dx.reshape(B, T, E)
    grads["embeddings.position_embeddings.weight"] = np.zeros_like(
        params["embeddings.position_embeddings.weight"])
    grads["embeddings.position_embeddings.weight"][:T] = dx3.sum(axis=0)
    grads["embeddings.char_embeddings.weight"] = dwte + ops.embedding_bwd(dx3, ids, wte.shape[0])
    return grads


class AdamW:
    """State + update of mytorch/optim/optimizers.py:288-371 over a param dict,
    two groups as in gpt2_trainer/train_gpt2.py:271-281."""

    def __init__(self, params, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1):
        self.lr, self.beta1, self.beta2, self.eps, self.wd = lr, beta1, beta2, eps, weight_decay
        self.m = {k: np.zeros_like(v) for k, v in params.items()}
        self.v = {k: np.zeros_like(v) for k, v in params.items()}
        self.decay = decay_mask(params)
        self.beta1_pow = 1.0
        self.beta2_pow = 1.0

    def step(self, params, grads):
        self.beta1_pow *= self.beta1
        self.beta2_pow *= self.beta2
        for k, p in params.items():
            ops.adamw_step(p, grads[k], self.m[k], self.v[k], self.lr, self.beta1, self.beta2,
                           self.eps, self.wd if self.decay[k] else 0.0,
                           self.beta1_pow, self.beta2_pow)


def synthetic_batch(rng, batch, ctx, vocab):
    """ids uniform in [0, vocab); targets are the inputs shifted by one."""
    ids = rng.integers(0, vocab, (batch, ctx + 1))
    return ids[:, :-1].astype(np.int32), ids[:, 1:].astype(np.int32)


def train(params, cfg, steps, batch, ctx, data_seed=0, lr=3e-4, betas=(0.9, 0.95),
          weight_decay=0.1, clip=None, vocab=None):
    """Runs `steps` optimizer steps in place on params; returns the losses."""
    opt = AdamW(params, lr, betas[0], betas[1], 1e-8, weight_decay)
    rng = np.random.default_rng(data_seed)
    losses = []
    for _ in range(steps):
        x, y = synthetic_batch(rng, batch, ctx, vocab or cfg.vocab_size)
        loss, _, cache = forward(params, cfg, x, y)
        grads = backward(params, cfg, cache)
        if clip is not None:
            ops.clip_grad_norm(list(grads.values()), clip)
        opt.step(params, grads)
        losses.append(float(loss))
    return losses
