"""Plain PyTorch baseline of the GPT 1.3 B FSDP configuration: torch.nn modules, cuBLAS matmuls,
SDPA (flash) attention, torch.distributed FSDP (NCCL) full-shard bf16, torch AdamW (fused) and
torch's dynamic GradScaler (``ShardedGradScaler`` under FSDP). None of this repository's kernels or engine are on this path; it is the
"torch.distributed NCCL + cuBLAS implementation of the identical config" the numbers are
compared with.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d, h, f):
        super().__init__()
        self.h = h
        self.ln1 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d)
        self.fc1 = nn.Linear(d, f)
        self.fc2 = nn.Linear(f, d)

    def forward(self, x):
        B, S, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.h, D // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class TorchGPT(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.padded_vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg.d_model, cfg.n_heads, cfg.d_ff) for _ in range(cfg.n_layers)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)

    def forward(self, ids, targets):
        B, S = ids.shape
        x = self.wte(ids) + self.wpe(torch.arange(S, device=ids.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.view(-1))


def build(cfg, dev, world, mb, S):
    model = TorchGPT(cfg).to(dev).to(torch.bfloat16)
    n_params = sum(p.numel() for p in model.parameters())
    if world > 1:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy, MixedPrecision
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy
        model = FSDP(model, sharding_strategy=ShardingStrategy.FULL_SHARD, auto_wrap_policy=ModuleWrapPolicy({Block}),
                     device_id=dev, use_orig_params=True,
                     mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    if world > 1:
        from torch.distributed.fsdp.sharded_grad_scaler import ShardedGradScaler
        scaler = ShardedGradScaler(init_scale=65536.0)
    else:
        scaler = torch.amp.GradScaler("cuda", init_scale=65536.0)

    def step(ids, tgt):
        opt.zero_grad(set_to_none=True)
        loss = model(ids, tgt)
        scaler.scale(loss).backward()
        scaler.step(opt)          # unscale + overflow check + skip-or-apply
        scaler.update()
        return loss.detach()
    return step, n_params
