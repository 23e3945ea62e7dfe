"""Paged attention as a layer of its own: projections, rotary embedding, KV-cache write and attention over the block
table for both phases, for models that are not driven by the bundled executor.

Reference: src/MLFramework/Inference/PagedAttention/Layers/PagedAttentionLayer.cs:244-389 (``Forward`` with a phase
argument: prefill computes attention over the prompt and stores K / V page by page; decode appends one token and
attends to every cached token through the block table), Phases/PrefillOrchestrator.cs:31-78,
Phases/DecodeOrchestrator.cs, Kernels/IPagedAttentionKernel.cs. On bf16 CUDA tensors with head dimension 128 the
hand-written kernels run (``rope_kv_write``, the tcgen05 prefill kernel, the paged decode kernel); anything else
evaluates the same mathematics in PyTorch (``ops/reference.py``).
"""
from __future__ import annotations

import enum
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import native, reference
from ..ops.gemm import gemm
from .kv_cache import KVCacheBlockManager


class AttentionPhase(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class PagedAttentionLayer(nn.Module):
    """``forward(x, seq_ids, phase)``.

    prefill: ``x`` is ``[sum(n_i), d_model]``, the new tokens of the sequences in ``seq_ids`` concatenated
    (``n_tokens[i]`` each); a sequence may already have cached tokens (chunked prefill): its new queries attend to
    the cached prefix and, causally, to the chunk. decode: ``x`` is ``[len(seq_ids), d_model]``, one new token per
    sequence. Block allocation happens here (``KVCacheBlockManager.append_tokens``); the caller frees sequences.
    """

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: Optional[int] = None, head_dim: Optional[int] = None,
                 rope_theta: Optional[float] = 500000.0, layer_index: int = 0, bias: bool = False, dtype=None, device=None):
        super().__init__()
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads or n_heads
        if n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.head_dim = head_dim or d_model // n_heads
        self.rope_theta, self.layer_index = rope_theta, layer_index
        qkv_out = (n_heads + 2 * self.n_kv_heads) * self.head_dim
        self.qkv = nn.Linear(d_model, qkv_out, bias=bias, dtype=dtype, device=device)
        self.proj = nn.Linear(n_heads * self.head_dim, d_model, bias=bias, dtype=dtype, device=device)

    def _native(self, x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and self.head_dim == 128

    def _split(self, qkv: torch.Tensor):
        T, D, hq, hkv = qkv.shape[0], self.head_dim, self.n_heads, self.n_kv_heads
        return (qkv[:, :hq * D].view(T, hq, D), qkv[:, hq * D:(hq + hkv) * D].view(T, hkv, D), qkv[:, (hq + hkv) * D:].view(T, hkv, D))

    def forward(self, x: torch.Tensor, kv: KVCacheBlockManager, seq_ids: Sequence[int], phase: AttentionPhase,
                n_tokens: Optional[Sequence[int]] = None) -> torch.Tensor:
        cache = kv.caches[self.layer_index]
        dev, D = x.device, self.head_dim
        if phase == AttentionPhase.DECODE:
            n_tokens = [1] * len(seq_ids)
        elif n_tokens is None:
            if len(seq_ids) != 1:
                raise ValueError("prefill of several sequences needs n_tokens")
            n_tokens = [x.shape[0]]
        if sum(n_tokens) != x.shape[0]:
            raise ValueError(f"x has {x.shape[0]} rows, n_tokens sum to {sum(n_tokens)}")
        starts = [kv.get_sequence_length(s) for s in seq_ids]
        slot_list, pos_list = [], []
        for s, n, st in zip(seq_ids, n_tokens, starts):
            slots, _ = kv.append_tokens(s, n)
            if slots is None:
                raise MemoryError(f"KV cache exhausted for sequence {s}")
            slot_list.append(slots)
            pos_list.append(torch.arange(st, st + n, dtype=torch.int64))
        slots = torch.cat(slot_list).to(dev)
        positions = torch.cat(pos_list).to(dev)
        nat = self._native(x)
        if nat:
            qkv = gemm(x, self.qkv.weight, bias=self.qkv.bias)
            q, k, v = self._split(qkv)
            if self.rope_theta is not None:
                native.rope_kv_write_(qkv, positions, slots, cache, self.n_heads, self.n_kv_heads, self.rope_theta)
            else:
                native.kv_cache_write(cache, k, v, slots)
        else:
            qkv = F.linear(x, self.qkv.weight, self.qkv.bias)
            q, k, v = self._split(qkv)
            if self.rope_theta is not None:
                q = reference.rope_ref(q, positions, self.rope_theta).to(x.dtype)
                k = reference.rope_ref(k, positions, self.rope_theta).to(x.dtype)
            flat = cache.view(-1, 2, kv.block_size, self.n_kv_heads, D)
            flat[slots // kv.block_size, 0, slots % kv.block_size] = k.to(cache.dtype)
            flat[slots // kv.block_size, 1, slots % kv.block_size] = v.to(cache.dtype)
        max_blocks = max(kv.blocks_needed(st + n) for st, n in zip(starts, n_tokens))
        table, lens = kv.build_tables(list(seq_ids), max_blocks, dev)
        if phase == AttentionPhase.DECODE:
            if nat:
                a = native.paged_decode(q, cache, table, lens, int(max(st + 1 for st in starts)))
            else:
                a = reference.paged_attention_ref(q.float(), cache.float(), table, lens).to(x.dtype)
        else:
            outs, off = [], 0
            for i, (n, st) in enumerate(zip(n_tokens, starts)):
                qi = q[off:off + n]
                total = st + n
                if nat and st == 0:
                    o, _ = native.flash_fwd(qi, k[off:off + n], v[off:off + n], 1, n, causal=True, want_lse=False)
                elif nat and kv.block_size == 16:
                    o = native.flash_fwd_paged(qi, cache, table[i:i + 1], 1, n, total, causal=True)    # pages read in the kernel
                elif nat:
                    kk, vv = native.kv_gather(cache, table[i], total)
                    o = native.flash_fwd_prefix(qi, kk, vv, 1, n, total, causal=True)
                else:
                    nb = kv.blocks_needed(total)
                    c = cache[table[i, :nb].long()]
                    kk = c[:, 0].reshape(-1, self.n_kv_heads, D)[:total]
                    vv = c[:, 1].reshape(-1, self.n_kv_heads, D)[:total]
                    o, _ = reference.attention_ref(qi[None].float(), kk[None].float(), vv[None].float(), causal=True, start_pos=st)
                    o = o[0].to(x.dtype)
                outs.append(o)
                off += n
            a = torch.cat(outs) if len(outs) > 1 else outs[0]
        a2 = a.reshape(x.shape[0], self.n_heads * D)
        if nat:
            return gemm(a2.contiguous(), self.proj.weight, bias=self.proj.bias)
        return F.linear(a2, self.proj.weight, self.proj.bias)
