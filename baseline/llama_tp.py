"""Plain torch.distributed + cuBLAS + SDPA tensor-parallel Llama training step (Megatron-style column / row
parallel linears, all-reduce after each row-parallel linear, vocab-parallel head with an all-gather of the
logits), bf16 parameters, fused torch AdamW. The comparison arm for the tensor-parallel configuration;
none of this package's kernels run here."""
import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

GROUP = None        # tensor-parallel process group (None = the default group); set by the pipeline arm


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        dist.all_reduce(x, group=GROUP)
        return x

    @staticmethod
    def backward(ctx, g):
        return g


class _CopyIn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        dist.all_reduce(g, group=GROUP)
        return g


def _rope(x, theta):
    T, H, D = x.shape[-3:]
    pos = torch.arange(T, device=x.device, dtype=torch.float32)
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = pos[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), -1).flatten(-2).to(x.dtype)


class Block(nn.Module):
    def __init__(self, c, W, dev):
        super().__init__()
        d, D = c["d_model"], c["head_dim"]
        self.hq, self.hkv, self.D, self.theta = c["n_heads"] // W, c["n_kv_heads"] // W, D, c.get("rope_theta", 500000.0)
        kw = dict(device=dev, dtype=torch.bfloat16)
        self.n1 = nn.RMSNorm(d, eps=c.get("norm_eps", 1e-5), **kw)
        self.n2 = nn.RMSNorm(d, eps=c.get("norm_eps", 1e-5), **kw)
        self.qkv = nn.Linear(d, (self.hq + 2 * self.hkv) * D, bias=False, **kw)
        self.o = nn.Linear(self.hq * D, d, bias=False, **kw)
        self.gu = nn.Linear(d, 2 * c["d_ff"] // W, bias=False, **kw)
        self.down = nn.Linear(c["d_ff"] // W, d, bias=False, **kw)

    def forward(self, x):
        B, S, _ = x.shape
        h = self.qkv(_CopyIn.apply(self.n1(x)))
        q, k, v = h.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], -1)
        q = _rope(q.view(B, S, self.hq, self.D), self.theta).transpose(1, 2)
        k = _rope(k.view(B, S, self.hkv, self.D), self.theta).transpose(1, 2)
        v = v.view(B, S, self.hkv, self.D).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.hq != self.hkv)
        x = x + _AllReduce.apply(self.o(a.transpose(1, 2).reshape(B, S, -1)))
        g, u = self.gu(_CopyIn.apply(self.n2(x))).chunk(2, -1)
        return x + _AllReduce.apply(self.down(F.silu(g) * u))


class Model(nn.Module):
    def __init__(self, c, W, rank, dev):
        super().__init__()
        V = (c["vocab_size"] + 127) // 128 * 128
        self.Vl, self.rank, self.W = V // W, rank, W
        kw = dict(device=dev, dtype=torch.bfloat16)
        self.embed = nn.Embedding(self.Vl, c["d_model"], **kw)
        self.blocks = nn.ModuleList([Block(c, W, dev) for _ in range(c["n_layers"])])
        self.nf = nn.RMSNorm(c["d_model"], eps=c.get("norm_eps", 1e-5), **kw)
        self.head = nn.Linear(c["d_model"], self.Vl, bias=False, **kw)

    def forward(self, ids, tgt):
        lo = self.rank * self.Vl
        mask = (ids >= lo) & (ids < lo + self.Vl)
        x = self.embed((ids - lo).clamp(0, self.Vl - 1)) * mask[..., None]
        x = _AllReduce.apply(x)
        for b in self.blocks:
            x = b(x)
        logits = self.head(_CopyIn.apply(self.nf(x))).float()                  # [B, S, V / W]
        # vocab-parallel cross entropy: max and sum-exp reduced over the group
        m = logits.detach().amax(-1)
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=GROUP)
        se = (logits - m[..., None]).exp().sum(-1)
        se = _AllReduce.apply(se)
        tmask = (tgt >= lo) & (tgt < lo + self.Vl)
        tl = logits.gather(-1, (tgt - lo).clamp(0, self.Vl - 1)[..., None])[..., 0] * tmask
        tl = _AllReduce.apply(tl)
        return (m + se.log() - tl).mean()


def init_weights(model, c):
    """Embedding and head N(0, 0.02); every linear N(0, 2 / (fan_in + fan_out)) over its FULL (unsharded) shape --
    the initialisation of the package's tensor-parallel layers, so that the loss curves of the two arms are
    comparable (with 0.02 everywhere this model memorises the fixed synthetic batch within three AdamW steps)."""
    d, D = c["d_model"], c["head_dim"]
    full = {"qkv": (d, (c["n_heads"] + 2 * c["n_kv_heads"]) * D), "o": (c["n_heads"] * D, d), "gu": (d, 2 * c["d_ff"]),
            "down": (c["d_ff"], d)}
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if prm.dim() < 2:
                continue
            kind = name.split(".")[-2]
            if kind in full:
                prm.normal_(0.0, math.sqrt(2.0 / sum(full[kind])))
            else:
                prm.normal_(0.0, 0.02)


def build(cfg, dev, ids, tgt):
    W, rank = dist.get_world_size(), dist.get_rank()
    model = Model(cfg, W, rank, dev)
    init_weights(model, cfg)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    n_params = sum(p.numel() for p in model.parameters()) * W

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(ids, tgt)
        loss.backward()
        opt.step()
        return loss
    return step, n_params
