"""Plain PyTorch baseline of the GPT 1.3 B FSDP configuration: torch.nn modules, cuBLAS matmuls,
SDPA (flash) attention, torch.distributed FSDP (NCCL) full-shard bf16, torch AdamW (fused) with a
dynamic loss scaler built from torch's own pieces: the overflow test is one ``_foreach_norm`` over the
gradients (all-reduced under FSDP), the unscale and the skip-on-overflow happen inside the fused AdamW
kernel through its ``grad_scale`` / ``found_inf`` inputs (the route ``torch.amp.GradScaler`` takes with
fused optimizers; its own unscale kernel does not accept bf16 gradients), and the scale is updated on
the device by ``torch._amp_update_scale_``. None of this repository's kernels or engine are on this path; it is the
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
    scale = torch.full((), 65536.0, device=dev)
    growth_tracker = torch.full((), 0, dtype=torch.int32, device=dev)

    def step(ids, tgt):
        opt.zero_grad(set_to_none=True)
        loss = model(ids, tgt)
        (loss * scale).backward()
        grads = [p.grad for p in model.parameters() if p.grad is not None]
        norms = torch.stack(torch._foreach_norm(grads)) if grads else torch.zeros(1, device=dev)
        found_inf = (~torch.isfinite(norms.float().sum())).float()
        if world > 1:
            torch.distributed.all_reduce(found_inf, op=torch.distributed.ReduceOp.MAX)
        opt.grad_scale, opt.found_inf = scale, found_inf      # fused AdamW unscales in-kernel and skips on overflow
        opt.step()
        torch._amp_update_scale_(scale, growth_tracker, found_inf, 2.0, 0.5, 2000)
        return loss.detach()
    return step, n_params
