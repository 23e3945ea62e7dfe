"""Tensor-parallel (optionally sequence-parallel) Llama: query heads, KV heads, FFN columns and
the vocabulary are split over the TP group; with sequence parallelism the residual stream,
RMSNorms and residual adds run on ``[T/W, d]`` token shards and every linear pair is
all-gather->GEMM ... GEMM->reduce-scatter (the fused kernels of the TP layers).

Per-rank shapes for the 8 B model at TP 8: QKV ``[4096 -> 768]`` (4 query + 1 key + 1 value head of
128), o ``[512 -> 4096]``, gate+up ``[4096 -> 3584]``, down ``[1792 -> 4096]``, head ``[4096 -> 16032]``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..nn.layers import RMSNorm
from ..ops import functional as Fm
from ..parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, TPContext, VocabParallelEmbedding, gather_tokens, vocab_parallel_lm_loss)
from .llama import LlamaConfig


class LlamaBlockTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, sequence_parallel: bool, dtype=None, device=None, idx: int = 0):
        super().__init__()
        W = tp.world
        if cfg.n_heads % W or cfg.n_kv_heads % W or cfg.d_ff % W:
            raise ValueError("heads, kv heads and d_ff must be divisible by the tensor-parallel size")
        self.cfg, self.tp, self.sp = cfg, tp, sequence_parallel
        self.hq, self.hkv = cfg.n_heads // W, cfg.n_kv_heads // W
        qkv_out = (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim
        self.norm1 = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        self.qkv = ColumnParallelLinear(cfg.d_model, qkv_out, False, False, sequence_parallel, tp, dtype, device, f"l{idx}.qkv")
        self.o = RowParallelLinear(cfg.n_heads * cfg.head_dim, cfg.d_model, False, True, sequence_parallel, tp, dtype, device, f"l{idx}.o")
        self.norm2 = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        self.gate_up = ColumnParallelLinear(cfg.d_model, 2 * cfg.d_ff, False, False, sequence_parallel, tp, dtype, device, f"l{idx}.gu")
        self.down = RowParallelLinear(cfg.d_ff, cfg.d_model, False, True, sequence_parallel, tp, dtype, device, f"l{idx}.down")

    def forward(self, x, B: int, S: int):
        """x: [T, d] (replicated) or [T/W, d] (sequence parallel) with T = B*S."""
        n1, skip = self.norm1.with_skip(x)
        h = self.qkv(n1)                                              # [T, (hq + 2 hkv) * D]
        a = Fm.attention_packed(h, B, S, self.hq, self.hkv, self.cfg.head_dim, True, self.cfg.rope_theta)
        x = self.o(a, residual=skip)
        n2, x = self.norm2.with_skip(x)
        gu = self.gate_up(n2)                                         # local (gate, up) pairs
        if Fm._native(gu):
            from ..ops import native
            hid = _SwiGLU.apply(gu)
        else:
            hid = (torch.nn.functional.silu(gu[..., 0::2].float()) * gu[..., 1::2].float()).to(gu.dtype)
        return self.down(hid, residual=x)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        from ..ops import native
        ctx.save_for_backward(gu)
        return native.swiglu_fwd(gu, interleaved=True)

    @staticmethod
    def backward(ctx, d):
        from ..ops import native
        (gu,) = ctx.saved_tensors
        return native.swiglu_bwd(d.contiguous(), gu, interleaved=True)


class LlamaTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, sequence_parallel: bool = True, dtype=None, device=None):
        super().__init__()
        self.cfg, self.tp, self.sp = cfg, tp, sequence_parallel
        self.embed = VocabParallelEmbedding(cfg.padded_vocab, cfg.d_model, tp, dtype, device, cfg.init_std,
                                            local_multiple=128 if tp.world > 1 else 1)
        self.blocks = nn.ModuleList([LlamaBlockTP(cfg, tp, sequence_parallel, dtype, device, i) for i in range(cfg.n_layers)])
        self.norm_f = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device)
        Vl = self.embed.local_v        # whole 128-column tiles per rank; columns past the vocabulary are masked in the loss
        self.lm_head = nn.Parameter(torch.empty(Vl, cfg.d_model, dtype=dtype, device=device).normal_(0, cfg.init_std))

    def replicated_parameters(self):
        """Parameters every TP rank holds a full copy of (their gradients must be summed over the
        TP group when the activations they saw were token shards)."""
        return [p for n, p in self.named_parameters() if "norm" in n]

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None, loss_scale=None):
        B, S = ids.shape
        sp = self.sp and self.tp.world > 1
        x = self.embed(ids, sequence_parallel=sp).reshape(-1, self.cfg.d_model)     # [T, d], or the token shard [T/W, d]
        for blk in self.blocks:
            x = blk(x, B, S)
        x = self.norm_f(x)
        if targets is None:
            return gather_tokens(x, self.tp) if sp else x
        return vocab_parallel_lm_loss(x, self.lm_head, targets, self.tp, self.cfg.vocab_size, loss_scale,
                                      sequence_parallel=sp, key="lm_head")

    def sync_replicated_grads(self):
        """Sum gradients of replicated parameters over the TP group (sequence-parallel mode): each rank saw its token
        shard only. One all-reduce over the concatenated gradients instead of one per norm."""
        if not (self.sp and self.tp.world > 1):
            return
        from ..dist.process_group import ReduceOp
        gs = []
        for p in self.replicated_parameters():
            g = getattr(p, "main_grad", None) if getattr(p, "_main_grad_started", False) else p.grad
            if g is not None:
                gs.append(g)
        if not gs:
            return
        flat = torch.cat([g.reshape(-1).float() for g in gs])
        self.tp.pg.all_reduce(flat, ReduceOp.SUM)
        off = 0
        for g in gs:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
