"""GPT-style decoder (pre-LayerNorm, learned position embedding, tanh-GELU MLP, tied LM head).

The 1.3 B preset is the FSDP benchmark configuration: 24 layers, d_model 2048, 16 heads of
128, FFN 8192, vocab 50257 (padded to a multiple of 128 for the tensor-core tiles), seq 2048.
The reference ships no model definitions; its Linear / Module containers are what these
blocks are built from (src/MLFramework/Modules/Linear.cs:9, src/MLFramework/NN/Module.cs:10).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..nn.layers import Embedding, GeluMLP, LayerNorm, SelfAttention
from ..ops import functional as Fm


@dataclass
class GPTConfig:
    n_layers: int = 24
    d_model: int = 2048
    n_heads: int = 16
    d_ff: int = 8192
    vocab_size: int = 50257
    max_seq: int = 2048
    init_std: float = 0.02
    vocab_multiple: int = 128
    tie_embeddings: bool = True
    activation_checkpointing: bool = False

    @property
    def padded_vocab(self) -> int:
        m = self.vocab_multiple
        return (self.vocab_size + m - 1) // m * m

    def num_params(self) -> int:
        d, f = self.d_model, self.d_ff
        per_layer = 4 * d * d + 4 * d + 2 * d * f + f + d + 4 * d
        return self.n_layers * per_layer + self.padded_vocab * d + self.max_seq * d + 2 * d

    def flops_per_token(self, seq: Optional[int] = None) -> float:
        """Training FLOPs per token (forward + backward = 3x forward), causal attention counted at half."""
        s = seq or self.max_seq
        d, f = self.d_model, self.d_ff
        dense = 2 * (4 * d * d + 2 * d * f) * self.n_layers + 2 * d * self.padded_vocab
        attn = 2 * 2 * s * d * self.n_layers / 2
        return 3.0 * (dense + attn)

    @classmethod
    def gpt_1_3b(cls) -> "GPTConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "GPTConfig":
        return cls(n_layers=2, d_model=256, n_heads=2, d_ff=1024, vocab_size=1000, max_seq=256)


class GPTBlock(nn.Module):
    def __init__(self, cfg: GPTConfig, dtype=None, device=None):
        super().__init__()
        out_std = cfg.init_std / (2 * cfg.n_layers) ** 0.5
        self.ln1 = LayerNorm(cfg.d_model, dtype=dtype, device=device)
        self.attn = SelfAttention(cfg.d_model, cfg.n_heads, bias=True, dtype=dtype, device=device,
                                  init_std=cfg.init_std, out_init_std=out_std)
        self.ln2 = LayerNorm(cfg.d_model, dtype=dtype, device=device)
        self.mlp = GeluMLP(cfg.d_model, cfg.d_ff, dtype=dtype, device=device, init_std=cfg.init_std,
                           out_init_std=out_std)

    def forward(self, x):
        h, skip = self.ln1.with_skip(x)
        x = self.attn(h, residual=skip)
        h, skip = self.ln2.with_skip(x)
        x = self.mlp(h, residual=skip)
        return x


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = Embedding(cfg.padded_vocab, cfg.d_model, cfg.max_seq, dtype=dtype, device=device,
                               init_std=cfg.init_std)
        self.blocks = nn.ModuleList([GPTBlock(cfg, dtype, device) for _ in range(cfg.n_layers)])
        self.ln_f = LayerNorm(cfg.d_model, dtype=dtype, device=device)
        if not cfg.tie_embeddings:
            self.lm_head = nn.Parameter(torch.empty(cfg.padded_vocab, cfg.d_model, dtype=dtype, device=device)
                                        .normal_(0, cfg.init_std))
        else:
            self.lm_head = None

    @property
    def head_weight(self) -> torch.Tensor:
        return self.embed.weight if self.lm_head is None else self.lm_head

    def hidden(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.embed(ids)
        for blk in self.blocks:
            if self.cfg.activation_checkpointing and torch.is_grad_enabled():
                from ..checkpoint.activation import checkpoint
                x = checkpoint(blk, x)
            else:
                x = blk(x)
        return self.ln_f(x)

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None,
                loss_scale: Optional[torch.Tensor] = None):
        """Returns mean token cross-entropy when ``targets`` is given, else logits ``[B, S, vocab]``."""
        h = self.hidden(ids)
        if targets is None:
            return torch.nn.functional.linear(h, self.head_weight)[..., :self.cfg.vocab_size]
        return Fm.lm_head_loss(h, self.head_weight, targets, self.cfg.vocab_size, loss_scale)
