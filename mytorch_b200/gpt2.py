"""GPT-2 as wired in the reference (gpt2_trainer/gpt2.py:88-390): learned token
and position embeddings, pre-LayerNorm blocks (attention + GELU MLP, 4x), final
LayerNorm, lm_head tied to the token embedding. Same config fields, module
names and state_dict keys, so checkpoints move between the two.

Only the training path is here (no KV cache). The attention module reads the
per-head interleaved [q|k|v] projection in place (see F.qkv_attention) and the
embedding pair is one kernel; everything else is the same sequence of ops.
"""
from dataclasses import dataclass

import numpy as np

from . import _lib, nn
from .array import DeviceArray, stream
from .nn import functional as F
from .tensor import Tensor


@dataclass
class GPT2Config:          # gpt2_trainer/gpt2.py:12-27
    vocab_size: int = 50257
    max_seq_len: int = 1024
    embed_dim: int = 768
    mlp_ratio: int = 4
    num_blocks: int = 12
    num_heads: int = 12
    mlp_dropout_p: float = 0.0
    attn_dropout_p: float = 0.0
    use_bias: bool = False
    use_layernorm_weight: bool = True
    use_full_auto: bool = False
    use_fused_ops: bool = True


class Cache:
    """Key/value cache of the inference step (gpt2_trainer/gpt2.py:29-86): per layer one
    preallocated ring [B, H, max_seq_len, D] for keys and one for values. `update` appends the new
    rows in place; when the ring is full the oldest row is overwritten, which is the reference's
    drop-the-oldest policy without its concatenate and slice copies (attention does not depend on
    the order in which the cached keys are stored)."""

    def __init__(self, config):
        self.max_seq_len = config.max_seq_len
        self.key_cache = [None] * config.num_blocks
        self.value_cache = [None] * config.num_blocks
        self._appended = [0] * config.num_blocks

    def __repr__(self):
        return f"DynamicCache(Num_Layers: {len(self.key_cache)} | Cached Tokens: {self.get_seq_len()})"

    def get_seq_len(self, layer_idx=0):
        return min(self._appended[layer_idx], self.max_seq_len)

    def update(self, k_ptr, v_ptr, strides, batch, heads, n_new, head_dim, dtype, layer_idx):
        """Appends n_new rows read through (ptr, strides) and returns (keys, values, rows held)."""
        if self.key_cache[layer_idx] is None:
            shape = (batch, heads, self.max_seq_len, head_dim)
            self.key_cache[layer_idx] = DeviceArray.empty(shape, dtype)
            self.value_cache[layer_idx] = DeviceArray.empty(shape, dtype)
        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]
        assert kc.shape[0] == batch and kc.dtype == dtype, "cache was created for another batch size or dtype"
        sc = _lib.Strides3(heads * self.max_seq_len * head_dim, self.max_seq_len * head_dim, head_dim)
        _lib.kv_append(k_ptr, v_ptr, kc.ptr, vc.ptr, strides, strides, sc, batch, heads, n_new,
                       self._appended[layer_idx] % self.max_seq_len, self.max_seq_len, head_dim, kc.code, stream())
        self._appended[layer_idx] += n_new
        return kc, vc, self.get_seq_len(layer_idx)


class Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.char_embeddings = nn.Embedding(config.vocab_size, config.embed_dim)
        self.position_embeddings = nn.Embedding(config.max_seq_len, config.embed_dim)

    def forward(self, input_ids, past_length=0):
        if past_length == 0:
            return F.token_position_embedding(input_ids, self.char_embeddings.weight, self.position_embeddings.weight)
        # decoding: positions continue after the cached tokens (gpt2.py:115-117); inference only
        B, T = input_ids.shape
        E = self.config.embed_dim
        assert past_length + T <= self.config.max_seq_len, "position table exhausted"
        x = F.embedding(input_ids, self.char_embeddings.weight).data
        pos = self.position_embeddings.weight.data.rows(past_length, past_length + T)
        _lib.add_rowvec(x.ptr, pos.ptr, x.ptr, B, T * E, x.code, stream())
        return Tensor(x)


class Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.embed_dim % config.num_heads == 0
        self.embed_dim, self.num_heads = config.embed_dim, config.num_heads
        self.head_dim = config.embed_dim // config.num_heads
        self.qkv_proj = nn.Linear(self.embed_dim, 3 * self.embed_dim, bias=config.use_bias)
        self.out_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)
        self.proj_drop = nn.Dropout(config.attn_dropout_p)

    def forward(self, x, residual=None, cache=None, layer_idx=None):
        qkv = self.qkv_proj(x)                                   # [B, T, 3E], per-head [q|k|v]
        if cache is not None and layer_idx is not None:
            out = self._cached_attention(qkv, cache, layer_idx)
        else:
            out = F.qkv_attention(qkv, self.num_heads, is_causal=True)  # [B, T, E]
        # the block's skip connection is added in the projection's GEMM epilogue
        out = F.linear(out, self.out_proj.weight, self.out_proj.bias, residual=residual)
        return self.proj_drop(out)


    def _cached_attention(self, qkv, cache, layer_idx):
        """gpt2.py:179-215: the new keys/values join the cache; an empty cache means this call is
        the prompt (causal attention among its tokens), otherwise the new queries see every cached
        key. Inference only (no graph is recorded)."""
        B, T, _ = qkv.shape
        H, D, E = self.num_heads, self.head_dim, self.embed_dim
        arr = qkv.data
        sin = _lib.Strides3(T * 3 * E, 3 * D, 3 * E)               # q/k/v of head h start at h*3D (+0, +D, +2D)
        past = cache.get_seq_len(layer_idx)
        kc, vc, kv_len = cache.update(arr.ptr + D * arr.itemsize, arr.ptr + 2 * D * arr.itemsize, sin, B, H, T, D,
                                      arr.dtype, layer_idx)
        if past == 0:
            return F.qkv_attention(qkv.detach(), H, is_causal=True)
        out = DeviceArray.empty((B, T, E), arr.dtype)
        sc = _lib.Strides3(H * cache.max_seq_len * D, cache.max_seq_len * D, D)
        _lib.attn_decode(arr.ptr, kc.ptr, vc.ptr, out.ptr, sin, sc, _lib.Strides3(T * E, D, E), B, H, T, kv_len, D,
                         float(D) ** -0.5, -1, arr.code, stream())
        return Tensor(out)


class FeedForward(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = config.embed_dim * config.mlp_ratio
        self.intermediate_dense = nn.Linear(config.embed_dim, hidden, bias=config.use_bias, act_func="gelu")
        self.intermediate_dropout = nn.Dropout(config.mlp_dropout_p)
        self.out_proj = nn.Linear(hidden, config.embed_dim, bias=config.use_bias)
        self.output_dropout = nn.Dropout(config.mlp_dropout_p)

    def forward(self, x, residual=None):
        if self.intermediate_dense.bias is None and self.out_proj.bias is None:
            # bias-free (the GPT-2 configuration): one fused node, activation and its
            # derivative live in GEMM epilogues, skip connection added in the last one
            return F.mlp(x, self.intermediate_dense.weight, self.out_proj.weight, "gelu", residual=residual)
        h = self.intermediate_dropout(self.intermediate_dense(x))
        return self.output_dropout(F.linear(h, self.out_proj.weight, self.out_proj.bias, residual=residual))


class TransformerBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = Attention(config)
        self.layernorm1 = nn.LayerNorm(config.embed_dim, weight=config.use_layernorm_weight, bias=config.use_bias)
        self.feedforward = FeedForward(config)
        self.layernorm2 = nn.LayerNorm(config.embed_dim, weight=config.use_layernorm_weight, bias=config.use_bias)

    def forward(self, x, cache=None, layer_idx=None):
        # The skip connections are added in the epilogue of each sublayer's last GEMM.
        x = self.attention(self.layernorm1(x), residual=x, cache=cache, layer_idx=layer_idx)
        x = self.feedforward(self.layernorm2(x), residual=x)
        return x


def _init_weights(module):     # gpt2_trainer/gpt2.py:376-389
    if isinstance(module, nn.Linear):
        nn.init.normal_(module.weight, mean=0.0, std=0.02)
        if module.bias is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, mean=0.0, std=0.02)
    elif isinstance(module, nn.LayerNorm):
        if module.weight is not None:
            nn.init.ones_(module.weight)
        if module.bias is not None:
            nn.init.zeros_(module.bias)


class GPT2(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embeddings = Embeddings(config)
        self.blocks = nn.ModuleList([TransformerBlock(config) for _ in range(config.num_blocks)])
        self.final_layer_norm = nn.LayerNorm(config.embed_dim, weight=config.use_layernorm_weight)
        self.lm_head = nn.Linear(config.embed_dim, config.vocab_size, bias=config.use_bias)
        self.apply(_init_weights)
        for name, param in self.named_parameters():
            if "out_proj" in name:
                nn.init.normal_(param, mean=0.0, std=0.02 / np.sqrt(2 * config.num_blocks))
        self.lm_head.weight = self.embeddings.char_embeddings.weight      # weight tying (:340-347)
        self._gradient_checkpointing_enabled = False

    def enable_gradient_checkpointing(self):
        """Recompute every transformer block in the backward pass instead of keeping its
        activations (gpt2.py:349-365)."""
        self._gradient_checkpointing_enabled = True

    def forward(self, x, cache=None):
        """Logits; with a `Cache`, (logits, cache) as in gpt2.py:352-374."""
        from .utils.checkpoint import checkpoint
        past_length = cache.get_seq_len() if cache is not None else 0
        x = self.embeddings(x, past_length)
        for layer_idx, block in enumerate(self.blocks):
            if cache is not None:
                x = block(x, cache=cache, layer_idx=layer_idx)
            elif self._gradient_checkpointing_enabled and self.training and x.requires_grad:
                x = checkpoint(block, x)
            else:
                x = block(x)
        x = self.final_layer_norm(x)
        logits = self.lm_head(x)
        return logits if cache is None else (logits, cache)

    def generate(self, input_ids, max_new_tokens, temperature=1.0, top_k=None, use_cache=True, seed=None):
        """Autoregressive sampling as in gpt2_trainer/inference_gpt2.py:137-174: the prompt fills
        the cache, then one token per step; temperature-scaled softmax (optionally restricted to
        the top_k logits), one draw per sequence on the host; temperature 0 takes the arg-max."""
        from .tensor import no_grad
        rng = np.random.default_rng(seed)
        ids = np.asarray(input_ids.numpy() if isinstance(input_ids, Tensor) else input_ids, dtype=np.int32)
        cache = Cache(self.config) if use_cache else None
        feed = ids
        with no_grad():
            for _ in range(max_new_tokens):
                out = self.forward(Tensor(feed), cache=cache)
                logits = out[0] if use_cache else out
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
                feed = ids[:, -1:] if use_cache else ids[:, -self.config.max_seq_len:]
        return ids
