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

from . import nn
from .nn import functional as F


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


class Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.char_embeddings = nn.Embedding(config.vocab_size, config.embed_dim)
        self.position_embeddings = nn.Embedding(config.max_seq_len, config.embed_dim)

    def forward(self, input_ids, past_length=0):
        assert past_length == 0, "the KV-cache path is outside the training step"
        return F.token_position_embedding(input_ids, self.char_embeddings.weight, self.position_embeddings.weight)


class Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.embed_dim % config.num_heads == 0
        self.embed_dim, self.num_heads = config.embed_dim, config.num_heads
        self.head_dim = config.embed_dim // config.num_heads
        self.qkv_proj = nn.Linear(self.embed_dim, 3 * self.embed_dim, bias=config.use_bias)
        self.out_proj = nn.Linear(self.embed_dim, self.embed_dim, bias=config.use_bias)
        self.proj_drop = nn.Dropout(config.attn_dropout_p)

    def forward(self, x, residual=None):
        qkv = self.qkv_proj(x)                                   # [B, T, 3E], per-head [q|k|v]
        out = F.qkv_attention(qkv, self.num_heads, is_causal=True)  # [B, T, E]
        # the block's skip connection is added in the projection's GEMM epilogue
        out = F.linear(out, self.out_proj.weight, self.out_proj.bias, residual=residual)
        return self.proj_drop(out)


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

    def forward(self, x):
        # The skip connections stay separate adds: fusing them into the projection GEMM's
        # epilogue (residual=x) is supported but measured slower on B200 at these shapes.
        x = x + self.attention(self.layernorm1(x))
        x = x + self.feedforward(self.layernorm2(x))
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

    def forward(self, x):
        from .utils.checkpoint import checkpoint
        x = self.embeddings(x)
        for block in self.blocks:
            if self._gradient_checkpointing_enabled and self.training and x.requires_grad:
                x = checkpoint(block, x)
            else:
                x = block(x)
        x = self.final_layer_norm(x)
        return self.lm_head(x)
