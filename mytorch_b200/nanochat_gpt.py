"""nanochat-style GPT as wired in the reference
(nanochat_trainer/core/nanochat_gpt.py:24-369): untied token embedding and
lm_head, parameter-free RMSNorm before every sub-layer and at the end, separate
q/k/v projections, rotary embedding THEN parameter-free RMSNorm on q and k
(:121-124), causal attention, ReLU^2 MLP (4x), zero-initialised out_proj and
lm_head (:287-288), loss = cross entropy of tanh-soft-capped logits.

Same config fields, module names and state_dict keys as the reference. Training
path only (no KV cache). Multi-head attention (num_kv_heads == num_q_heads, the
560M "d20" configuration); grouped-query attention is not on this path.
Unlike the reference's training dispatcher, which drops `softcap` before the
loss is computed (mytorch/nn/functional/losses/cross_entropy.py:178), the cap
is applied, as the model definition intends.
"""
import math
from dataclasses import dataclass

from . import nn
from .array import DeviceArray
from .nn import functional as F
from .tensor import Tensor


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
        if config.num_kv_heads != config.num_q_heads:
            raise NotImplementedError("grouped-query attention is outside the training path built here")
        self.embed_dim, self.num_heads = config.embed_dim, config.num_q_heads
        self.head_dim = config.embed_dim // config.num_q_heads
        self.q_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)
        self.k_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)
        self.v_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)
        self.out_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)

    def forward(self, x, cos_sin):
        B, T, E = x.shape
        H, D = self.num_heads, self.head_dim
        q = self.q_proj(x).reshape(B, T, H, D)
        k = self.k_proj(x).reshape(B, T, H, D)
        v = self.v_proj(x).reshape(B, T, H, D)
        cos, sin = cos_sin
        q, k = F.apply_rotary_pos_embed(q, k, cos, sin)          # rotary first ...
        q = norm(q.reshape(B * T * H, D)).reshape(B, T, H, D)     # ... then QK-norm over head_dim
        k = norm(k.reshape(B * T * H, D)).reshape(B, T, H, D)
        out = F.bthd_attention(q, k, v, is_causal=True)           # [B, T, E], heads read in place
        return self.out_proj(out)


class FeedForward(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = config.embed_dim * config.mlp_ratio
        self.intermediate_dense = nn.Linear(config.embed_dim, hidden, bias=config.use_bias, act_func="relu_squared")
        self.out_proj = nn.Linear(hidden, config.embed_dim, bias=config.use_bias)

    def forward(self, x):
        if self.intermediate_dense.bias is None and self.out_proj.bias is None:
            return F.mlp(x, self.intermediate_dense.weight, self.out_proj.weight, "relu_squared")
        return self.out_proj(self.intermediate_dense(x))


class TransformerBlock(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.attention = Attention(config, layer_idx)
        self.feedforward = FeedForward(config)

    def forward(self, x, cos_sin):
        x = x + self.attention(norm(x), cos_sin)
        x = x + self.feedforward(norm(x))
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

    def enable_gradient_checkpointing(self):
        """Recompute each block in the backward pass (nanochat_gpt.py:318-322)."""
        self._gradient_checkpointing_enabled = True

    def forward(self, input_ids, target_ids=None):
        B, T = input_ids.shape
        assert T <= self.config.max_seq_len, "sequence longer than the rotary table"
        cos = DeviceArray(self.cos.ptr, (T, self.cos.shape[1]), "float32", base=self.cos)
        sin = DeviceArray(self.sin.ptr, (T, self.sin.shape[1]), "float32", base=self.sin)
        x = self.embeddings(input_ids)
        for block in self.blocks:
            if self._gradient_checkpointing_enabled and self.training and x.requires_grad:
                from .utils.checkpoint import checkpoint
                x = checkpoint(block, x, (cos, sin))
            else:
                x = block(x, (cos, sin))
        x = norm(x)
        logits = self.lm_head(x)
        if target_ids is None:
            return (logits,)
        loss = F.cross_entropy(logits, target_ids, softcap=self.config.softcap)
        return logits, loss
