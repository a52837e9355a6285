"""NumPy restatement of the reference nanochat-style GPT training step
(nanochat_trainer/core/nanochat_gpt.py:24-369), multi-head form. TEST
INFRASTRUCTURE: see oracle/__init__.py.

Per block: x + attn(norm(x)), x + mlp(norm(x)) with norm = parameter-free
RMSNorm (:39-43); attention = q/k/v projections (k and v with num_kv_heads heads, :88-90),
rotary embedding then RMSNorm on q and k (:121-124), key/value heads repeated over their
group (:139-141), causal softmax attention, out_proj; mlp = ReLU^2 (4x).
Loss = cross entropy of softcap * tanh(logits / softcap) (:334-349, the
model's stated intent; the reference's CPU dispatcher cannot take a softcap, so
the reference run that pins this file caps the logits with the model's own
inference branch and then applies its plain cross entropy).
"""
from dataclasses import dataclass

import numpy as np

from . import ops


@dataclass
class GPTConfig:
    vocab_size: int = 65536
    max_seq_len: int = 2048
    embed_dim: int = 1280
    mlp_ratio: int = 4
    num_blocks: int = 20
    num_heads: int = 10
    num_kv_heads: int = 0          # 0 = as many as query heads; a divisor of num_heads = grouped-query attention
    rope_base: float = 10000.0
    softcap: float = 15.0


def init_params(cfg, seed=0, dtype=np.float32):
    """Seeded weights in state_dict order. out_proj and lm_head are drawn random
    here (the model zero-initialises them, which would make a parity test blind
    to most of the network)."""
    rng = np.random.default_rng(seed)
    E, Hd = cfg.embed_dim, cfg.embed_dim * cfg.mlp_ratio
    Ekv = (cfg.num_kv_heads or cfg.num_heads) * (E // cfg.num_heads)     # k/v projection width (nanochat_gpt.py:88-90)
    p = {"embeddings.embeddings.weight": rng.normal(0, 0.5, (cfg.vocab_size, E))}
    s = 1.0 / np.sqrt(E)
    for i in range(cfg.num_blocks):
        b = f"blocks.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            p[b + f"attention.{n}.weight"] = rng.normal(0, s, (Ekv if n in ("k_proj", "v_proj") else E, E))
        p[b + "feedforward.intermediate_dense.weight"] = rng.normal(0, s, (Hd, E))
        p[b + "feedforward.out_proj.weight"] = rng.normal(0, 1.0 / np.sqrt(Hd), (E, Hd))
    p["lm_head.weight"] = rng.normal(0, s, (cfg.vocab_size, E))
    return {k: np.ascontiguousarray(v, dtype=dtype) for k, v in p.items()}


def forward(params, cfg, ids, targets):
    B, T = ids.shape
    E, H = cfg.embed_dim, cfg.num_heads
    D = E // H
    Hk = cfg.num_kv_heads or H
    G = H // Hk                                 # query heads per key/value head
    cos, sin = ops.rope_cos_sin(D, T, cfg.rope_base)
    x = params["embeddings.embeddings.weight"][ids].reshape(B * T, E)
    cache = {"ids": ids, "blocks": [], "cos": cos, "sin": sin}
    for i in range(cfg.num_blocks):
        b = f"blocks.{i}."
        c = {"x0": x}
        h1, c["rs1"] = ops.rmsnorm_fwd(x)
        c["h1"] = h1
        q = ops.linear_fwd(h1, params[b + "attention.q_proj.weight"]).reshape(B, T, H, D)
        k = ops.linear_fwd(h1, params[b + "attention.k_proj.weight"]).reshape(B, T, Hk, D)
        v = ops.linear_fwd(h1, params[b + "attention.v_proj.weight"]).reshape(B, T, Hk, D)
        qr, kr = ops.rope_fwd(q, cos, sin), ops.rope_fwd(k, cos, sin)
        c["qr"], c["kr"] = qr.reshape(-1, D), kr.reshape(-1, D)
        qn, c["rsq"] = ops.rmsnorm_fwd(c["qr"])
        kn, c["rsk"] = ops.rmsnorm_fwd(c["kr"])
        qh = qn.reshape(B, T, H, D).transpose(0, 2, 1, 3)
        kh = kn.reshape(B, T, Hk, D).transpose(0, 2, 1, 3)
        vh = v.transpose(0, 2, 1, 3)
        if G > 1:                               # repeat_interleave over the head axis (nanochat_gpt.py:139-141)
            kh, vh = np.repeat(kh, G, axis=1), np.repeat(vh, G, axis=1)
        o, pr = ops.attention_fwd(qh, kh, vh, causal=True)
        c["qh"], c["kh"], c["vh"], c["p"] = qh, kh, vh, pr
        a = o.transpose(0, 2, 1, 3).reshape(B * T, E)
        c["a"] = a
        x = x + ops.linear_fwd(a, params[b + "attention.out_proj.weight"])
        c["x1"] = x
        h2, c["rs2"] = ops.rmsnorm_fwd(x)
        c["h2"] = h2
        u = ops.linear_fwd(h2, params[b + "feedforward.intermediate_dense.weight"])
        c["u"] = u
        g = ops.relu2_fwd(u)
        c["g"] = g
        x = x + ops.linear_fwd(g, params[b + "feedforward.out_proj.weight"])
        cache["blocks"].append(c)
    cache["xf"] = x
    hf, cache["rsf"] = ops.rmsnorm_fwd(x)
    cache["hf"] = hf
    raw = ops.linear_fwd(hf, params["lm_head.weight"])
    cache["raw"] = raw
    capped = cfg.softcap * np.tanh(raw / cfg.softcap)
    cache["capped"] = capped
    cache["targets"] = targets.reshape(-1)
    return ops.cross_entropy_fwd(capped, cache["targets"]), cache


def backward(params, cfg, cache):
    ids = cache["ids"]
    B, T = ids.shape
    E, H = cfg.embed_dim, cfg.num_heads
    D = E // H
    Hk = cfg.num_kv_heads or H
    G = H // Hk
    cos, sin = cache["cos"], cache["sin"]
    grads = {}
    dcap = ops.cross_entropy_bwd(cache["capped"], cache["targets"])
    t = np.tanh(cache["raw"] / cfg.softcap)
    draw = (dcap * (1 - t * t)).astype(cache["raw"].dtype)
    dhf, grads["lm_head.weight"], _ = ops.linear_bwd(cache["hf"], params["lm_head.weight"], draw)
    dx, _ = ops.rmsnorm_bwd(cache["xf"], cache["rsf"], dhf)
    for i in reversed(range(cfg.num_blocks)):
        b = f"blocks.{i}."
        c = cache["blocks"][i]
        dg_, grads[b + "feedforward.out_proj.weight"], _ = ops.linear_bwd(c["g"], params[b + "feedforward.out_proj.weight"], dx)
        du = ops.relu2_bwd(c["u"], dg_)
        dh2, grads[b + "feedforward.intermediate_dense.weight"], _ = ops.linear_bwd(
            c["h2"], params[b + "feedforward.intermediate_dense.weight"], du)
        dx = dx + ops.rmsnorm_bwd(c["x1"], c["rs2"], dh2)[0]
        da, grads[b + "attention.out_proj.weight"], _ = ops.linear_bwd(c["a"], params[b + "attention.out_proj.weight"], dx)
        do = da.reshape(B, T, H, D).transpose(0, 2, 1, 3)
        dqh, dkh, dvh = ops.attention_bwd(c["qh"], c["kh"], c["vh"], c["p"], do)
        if G > 1:                               # a key/value head collects the gradients of its group
            dkh = dkh.reshape(B, Hk, G, T, D).sum(axis=2)
            dvh = dvh.reshape(B, Hk, G, T, D).sum(axis=2)
        dqn = dqh.transpose(0, 2, 1, 3).reshape(-1, D)
        dkn = dkh.transpose(0, 2, 1, 3).reshape(-1, D)
        dqr = ops.rmsnorm_bwd(c["qr"], c["rsq"], dqn)[0].reshape(B, T, H, D)
        dkr = ops.rmsnorm_bwd(c["kr"], c["rsk"], dkn)[0].reshape(B, T, Hk, D)
        dq = ops.rope_bwd(dqr, cos, sin).reshape(B * T, E)
        dk = ops.rope_bwd(dkr, cos, sin).reshape(B * T, Hk * D)
        dv = dvh.transpose(0, 2, 1, 3).reshape(B * T, Hk * D)
        dh1 = 0
        for n, d in (("q_proj", dq), ("k_proj", dk), ("v_proj", dv)):
            dh, grads[b + f"attention.{n}.weight"], _ = ops.linear_bwd(c["h1"], params[b + f"attention.{n}.weight"], d)
            dh1 = dh1 + dh
        dx = dx + ops.rmsnorm_bwd(c["x0"], c["rs1"], dh1)[0]
    grads["embeddings.embeddings.weight"] = ops.embedding_bwd(dx.reshape(B, T, E), ids, cfg.vocab_size)
    return grads
