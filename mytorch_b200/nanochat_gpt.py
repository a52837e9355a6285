"""nanochat-style GPT as wired in the reference
(nanochat_trainer/core/nanochat_gpt.py:24-369): untied token embedding and
lm_head, parameter-free RMSNorm before every sub-layer and at the end, separate
q/k/v projections, rotary embedding THEN parameter-free RMSNorm on q and k
(:121-124), causal attention, ReLU^2 MLP (4x), zero-initialised out_proj and
lm_head (:287-288), loss = cross entropy of tanh-soft-capped logits.

Same config fields, module names and state_dict keys as the reference. Training
path plus cached decoding (`KVCache`, nanochat_trainer/core/cache.py). num_kv_heads may be a
divisor of num_q_heads (grouped-query attention: query head h reads key/value head
h // (num_q_heads // num_kv_heads), nanochat_gpt.py:78-90); the 560M "d20" configuration is
multi-head (10 of each). Cached decoding is built for the multi-head form only.
Unlike the reference's training dispatcher, which drops `softcap` before the
loss is computed (mytorch/nn/functional/losses/cross_entropy.py:178), the cap
is applied, as the model definition intends.
"""
import math
from dataclasses import dataclass

import numpy as np

from . import _lib, nn
from .array import DeviceArray, stream
from .nn import functional as F
from .tensor import Tensor


class KVCache:
    """Preallocated key/value cache [layers][B, H, seq_len, D] with a write position
    (nanochat_trainer/core/cache.py:3-75): update() stores the new rows at [pos, pos+T) of its
    layer, the position advances once per forward pass (after the last layer)."""

    def __init__(self, batch_size, num_heads, seq_len, head_dim, num_layers):
        self.cache_shape = (num_layers, batch_size, num_heads, seq_len, head_dim)
        self.k_cache = self.v_cache = None
        self._pos = 0

    @property
    def pos(self):
        return self._pos

    def reset(self):
        self._pos = 0

    def update(self, k_ptr, v_ptr, strides, n_new, dtype, layer_idx):
        L, B, H, S, D = self.cache_shape
        if self.k_cache is None:
            self.k_cache = DeviceArray.empty(self.cache_shape, dtype)
            self.v_cache = DeviceArray.empty(self.cache_shape, dtype)
        assert self._pos + n_new <= S, "You have filled up your Cache!"
        kc, vc = self.k_cache.rows(layer_idx, layer_idx + 1), self.v_cache.rows(layer_idx, layer_idx + 1)
        sc = _lib.Strides3(H * S * D, S * D, D)
        _lib.kv_append(k_ptr, v_ptr, kc.ptr, vc.ptr, strides, strides, sc, B, H, n_new, self._pos, S, D, kc.code, stream())
        if layer_idx == L - 1:
            self._pos += n_new
            return kc, vc, self._pos
        return kc, vc, self._pos + n_new


@dataclass
class GPTConfig:          # nanochat_gpt.py:24-37
    vocab_size: int = 2 ** 16
    max_seq_len: int = 2048
    embed_dim: int = 1280
    mlp_ratio: int = 4
    num_blocks: int = 20
    num_q_heads: int = 10
    num_kv_heads: int = 10
    dropout_p: float = 0.0
    use_fused_ops: bool = True
    use_bias: bool = False
    rope_base: float = 10000
    softcap: float = 15.0


def norm(x, training=True):
    """parameter-free RMSNorm (nanochat_gpt.py:39-43)."""
    return F.rmsnorm(x, weight=None, training=training)


class Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embeddings = nn.Embedding(config.vocab_size, config.embed_dim)

    def forward(self, input_ids):
        return self.embeddings(input_ids)


class Attention(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        assert config.num_kv_heads <= config.num_q_heads and config.num_q_heads % config.num_kv_heads == 0, \
            "Q Heads must be divisible by KV Heads"
        self.embed_dim, self.num_heads = config.embed_dim, config.num_q_heads
        self.num_kv_heads = config.num_kv_heads
        self.head_dim = config.embed_dim // config.num_q_heads
        # fewer key/value heads than query heads = grouped-query attention (nanochat_gpt.py:78-90)
        self.q_proj = nn.Linear(self.embed_dim, self.num_heads * self.head_dim, bias=config.use_bias)
        self.k_proj = nn.Linear(self.embed_dim, self.num_kv_heads * self.head_dim, bias=config.use_bias)
        self.v_proj = nn.Linear(self.embed_dim, self.num_kv_heads * self.head_dim, bias=config.use_bias)
        self.out_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)

    def forward(self, x, cos_sin, residual=None, cache=None, layer_idx=None):
        B, T, E = x.shape
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        q = self.q_proj(x).reshape(B, T, H, D)
        k = self.k_proj(x).reshape(B, T, Hk, D)
        v = self.v_proj(x).reshape(B, T, Hk, D)
        cos, sin = cos_sin
        q, k = F.rope_qk_norm(q, k, cos, sin)                    # rotary first, then QK-norm over head_dim: one kernel
        if cache is not None:
            # inference: new keys/values join the cache; the prompt (empty cache) attends causally
            # among its own tokens, later tokens see everything cached (nanochat_gpt.py:126-160)
            past = cache.pos
            sin3 = _lib.Strides3(T * H * D, D, H * D)               # q [B, T, H, D] as (batch, head, row)
            skv3 = _lib.Strides3(T * Hk * D, D, Hk * D)             # k, v [B, T, Hk, D]: the cache holds Hk heads
            kc, vc, kv_len = cache.update(k.data.ptr, v.data.ptr, skv3, T, k.data.dtype, layer_idx)
            if past == 0:
                out = F.bthd_attention(q, k, v, is_causal=True)
            else:
                S = cache.cache_shape[3]
                o = DeviceArray.empty((B, T, E), q.data.dtype)
                _lib.attn_decode_gqa(q.data.ptr, kc.ptr, vc.ptr, o.ptr, sin3, _lib.Strides3(Hk * S * D, S * D, D),
                                     _lib.Strides3(T * E, D, E), B, H, Hk, T, kv_len, D, float(D) ** -0.5, past,
                                     q.data.code, stream())
                out = Tensor(o)
        else:
            out = F.bthd_attention(q, k, v, is_causal=True)       # [B, T, E], heads read in place
        return F.linear(out, self.out_proj.weight, self.out_proj.bias, residual=residual)


class FeedForward(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = config.embed_dim * config.mlp_ratio
        self.intermediate_dense = nn.Linear(config.embed_dim, hidden, bias=config.use_bias, act_func="relu_squared")
        self.out_proj = nn.Linear(hidden, config.embed_dim, bias=config.use_bias)

    def forward(self, x, residual=None):
        if self.intermediate_dense.bias is None and self.out_proj.bias is None:
            return F.mlp(x, self.intermediate_dense.weight, self.out_proj.weight, "relu_squared", residual=residual)
        return F.linear(self.intermediate_dense(x), self.out_proj.weight, self.out_proj.bias, residual=residual)


class TransformerBlock(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.attention = Attention(config, layer_idx)
        self.feedforward = FeedForward(config)

    def forward(self, x, cos_sin, cache=None, layer_idx=None):
        # the skip connections are added in the epilogue of each sublayer's last GEMM
        x = self.attention(norm(x), cos_sin, residual=x, cache=cache, layer_idx=layer_idx)
        x = self.feedforward(norm(x), residual=x)
        return x


def _init_weights(module):      # nanochat_gpt.py:352-369
    if isinstance(module, nn.Linear):
        fan_out, fan_in = module.weight.shape
        std = 1.0 / math.sqrt(fan_in) * min(1.0, math.sqrt(fan_out / fan_in))
        nn.init.normal_(module.weight, mean=0.0, std=std)
        if module.bias is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, mean=0.0, std=0.02)


class GPT(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embeddings = Embeddings(config)
        self.blocks = nn.ModuleList([TransformerBlock(config, i) for i in range(config.num_blocks)])
        self.lm_head = nn.Linear(config.embed_dim, config.vocab_size, bias=config.use_bias)
        self.apply(_init_weights)
        for name, param in self.named_parameters():
            if ("out_proj" in name) or ("lm_head" in name):
                nn.init.zeros_(param)
        self.cos, self.sin = F.precompute_rotary_cos_sin(config.embed_dim // config.num_q_heads,
                                                         config.max_seq_len, config.rope_base)
        self._gradient_checkpointing_enabled = False
        # How forward(input_ids, target_ids) produces the loss. "logits": (logits, loss) as the
        # reference returns them. "fused": the loss writes the gradient of the logits over them in
        # its forward pass (one read and one write of the [tokens, vocab] tensor) and None is
        # returned in their place. "chunked": lm_head and loss walk the vocabulary in chunks and
        # the logits are never held (F.lm_head_cross_entropy); None is returned in their place.
        self.loss_mode = "logits"
        self.loss_chunk = 8192

    def enable_gradient_checkpointing(self):
        """Recompute each block in the backward pass (nanochat_gpt.py:318-322)."""
        self._gradient_checkpointing_enabled = True

    def forward(self, input_ids, target_ids=None, cache=None):
        B, T = input_ids.shape
        past = cache.pos if cache is not None else 0
        assert past + T <= self.config.max_seq_len, "sequence longer than the rotary table"
        cos, sin = self.cos.rows(past, past + T), self.sin.rows(past, past + T)   # positions continue after the cache
        x = self.embeddings(input_ids)
        for layer_idx, block in enumerate(self.blocks):
            if cache is not None:
                x = block(x, (cos, sin), cache=cache, layer_idx=layer_idx)
                continue
            if self._gradient_checkpointing_enabled and self.training and x.requires_grad:
                from .utils.checkpoint import checkpoint
                x = checkpoint(block, x, (cos, sin))
            else:
                x = block(x, (cos, sin))
        x = norm(x)
        if target_ids is not None and self.loss_mode == "chunked" and self.lm_head.bias is None:
            return None, F.lm_head_cross_entropy(x, self.lm_head.weight, target_ids, chunk=self.loss_chunk,
                                                 softcap=self.config.softcap)
        logits = self.lm_head(x)
        if target_ids is None:
            # inference branch (nanochat_gpt.py:334-340): soft-capped logits, plus the cache if one was given
            if self.config.softcap and not self.training:
                arr = logits.data
                _lib.softcap(arr.ptr, arr.ptr, arr.size, float(self.config.softcap), arr.code, stream())
            return (logits,) if cache is None else (logits, cache)
        if self.loss_mode == "fused":
            return None, F.cross_entropy(logits, target_ids, softcap=self.config.softcap, fused_backward=True)
        loss = F.cross_entropy(logits, target_ids, softcap=self.config.softcap)
        return logits, loss

    def generate(self, input_ids, max_new_tokens, temperature=1.0, top_k=None, seed=None):
        """Cached autoregressive sampling for one batch of equally long prompts: the prompt fills a
        KVCache, then one token per step (temperature 0 = arg-max)."""
        from .tensor import no_grad
        cfg = self.config
        rng = np.random.default_rng(seed)
        ids = np.asarray(input_ids.numpy() if isinstance(input_ids, Tensor) else input_ids, dtype=np.int32)
        cache = KVCache(ids.shape[0], cfg.num_kv_heads, cfg.max_seq_len, cfg.embed_dim // cfg.num_q_heads, cfg.num_blocks)
        was_training = self.training
        self.eval()
        feed = ids
        with no_grad():
            for _ in range(max_new_tokens):
                logits, cache = self.forward(Tensor(feed), None, cache=cache)
                last = logits.numpy()[:, -1, :].astype(np.float64)
                if temperature == 0:
                    nxt = last.argmax(-1)
                else:
                    last = last / temperature
                    if top_k is not None:
                        kth = np.sort(last, -1)[:, -top_k][:, None]
                        last = np.where(last < kth, -np.inf, last)
                    p = np.exp(last - last.max(-1, keepdims=True))
                    p /= p.sum(-1, keepdims=True)
                    nxt = np.array([rng.choice(p.shape[-1], p=row) for row in p])
                ids = np.concatenate([ids, nxt[:, None].astype(np.int32)], axis=1)
                feed = ids[:, -1:]
        if was_training:
            self.train()
        return ids
