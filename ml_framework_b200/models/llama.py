"""Llama-style decoder: RMSNorm, RoPE, GQA attention, SwiGLU MLP, untied LM head.

Presets: 8 B (32 layers, d 4096, 32 query / 8 KV heads of 128, FFN 14336, vocab 128256,
RoPE theta 500000, seq 4096) for the tensor-parallel training and serving configurations and
13 B (40 layers, d 5120, 40 heads, FFN 13824, vocab 32000) for the pipeline configuration.
Tensor-parallel construction is in :mod:`ml_framework_b200.parallel.tensor_parallel`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..nn.layers import Embedding, RMSNorm, SelfAttention, SwiGLUMLP
from ..ops import functional as Fm


@dataclass
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    d_ff: int = 14336
    vocab_size: int = 128256
    max_seq: int = 4096
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    vocab_multiple: int = 128
    activation_checkpointing: bool = False

    @property
    def padded_vocab(self) -> int:
        m = self.vocab_multiple
        return (self.vocab_size + m - 1) // m * m

    def num_params(self) -> int:
        d, f = self.d_model, self.d_ff
        qkv = d * (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        per_layer = qkv + self.n_heads * self.head_dim * d + 3 * d * f + 2 * d
        return self.n_layers * per_layer + 2 * self.padded_vocab * d + d

    def flops_per_token(self, seq: Optional[int] = None) -> float:
        s = seq or self.max_seq
        d, f = self.d_model, self.d_ff
        qkv = d * (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        dense = 2 * (qkv + self.n_heads * self.head_dim * d + 3 * d * f) * self.n_layers + 2 * d * self.padded_vocab
        attn = 2 * 2 * s * self.n_heads * self.head_dim * self.n_layers / 2
        return 3.0 * (dense + attn)

    @classmethod
    def llama_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def llama_13b(cls) -> "LlamaConfig":
        return cls(n_layers=40, d_model=5120, n_heads=40, n_kv_heads=40, d_ff=13824, vocab_size=32000)

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, d_ff=512, vocab_size=1000, max_seq=256)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype=None, device=None):
        super().__init__()
        out_std = cfg.init_std / (2 * cfg.n_layers) ** 0.5
        self.norm1 = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        self.attn = SelfAttention(cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, bias=False,
                                  rope_theta=cfg.rope_theta, dtype=dtype, device=device, init_std=cfg.init_std,
                                  out_init_std=out_std)
        self.norm2 = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        self.mlp = SwiGLUMLP(cfg.d_model, cfg.d_ff, dtype, device, cfg.init_std, out_std)

    def forward(self, x, positions=None):
        h, skip = self.norm1.with_skip(x)
        x = self.attn(h, residual=skip, positions=positions)
        h, skip = self.norm2.with_skip(x)
        x = self.mlp(h, residual=skip)
        return x


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = Embedding(cfg.padded_vocab, cfg.d_model, 0, dtype=dtype, device=device, init_std=cfg.init_std)
        self.blocks = nn.ModuleList([LlamaBlock(cfg, dtype, device) for _ in range(cfg.n_layers)])
        self.norm_f = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        self.lm_head = nn.Parameter(torch.empty(cfg.padded_vocab, cfg.d_model, dtype=dtype, device=device)
                                    .normal_(0, cfg.init_std))

    def hidden(self, ids):
        x = self.embed(ids)
        for blk in self.blocks:
            if self.cfg.activation_checkpointing and torch.is_grad_enabled():
                from ..checkpoint.activation import checkpoint
                x = checkpoint(blk, x)
            else:
                x = blk(x)
        return self.norm_f(x)

    def forward(self, ids, targets=None, loss_scale=None):
        h = self.hidden(ids)
        if targets is None:
            return torch.nn.functional.linear(h, self.lm_head)[..., :self.cfg.vocab_size]
        return Fm.lm_head_loss(h, self.lm_head, targets, self.cfg.vocab_size, loss_scale)
