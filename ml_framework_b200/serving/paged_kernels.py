"""The paged-attention kernel interface over contiguous K / V, and the prefill / decode orchestrators.

Reference (src/MLFramework/Inference/PagedAttention/): Kernels/IPagedAttentionKernel.cs:11-33
(``ComputePagedAttention(query[B,Q,H,D], cachedKeys[B,C,H,D], cachedValues[B,C,H,D], phase, scale)``),
Kernels/StandardPagedAttentionKernel.cs:21-257 (QK^T, scale, causal mask with ``startPos = C - Q`` in the decode phase,
max-subtracted softmax, PV), Kernels/CudaPagedAttentionKernel.cs (a stub that throws), Phases/PrefillOrchestrator.cs
(PrefillAllocateBlocks :31-52, ComputePrefillAttention :62, BatchPrefill :84), Phases/DecodeOrchestrator.cs
(AllocateDecodeBlock :30-55, ComputeDecodeAttention :64, BatchDecode :85).

The production path of this package reads K / V through the block table inside its CUDA kernels
(:mod:`ml_framework_b200.serving.paged_attention_layer`); this interface is the reference's "already gathered" form and
the oracle the GPU kernels are checked against.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .kv_cache import KVCacheBlockManager
from .paged_attention_layer import AttentionPhase, PagedAttentionLayer


class PagedAttentionKernel:
    name = "abstract"

    def compute_paged_attention(self, query: torch.Tensor, cached_keys: torch.Tensor, cached_values: torch.Tensor,
                                phase: AttentionPhase = AttentionPhase.DECODE, scale: Optional[float] = None) -> torch.Tensor:
        raise NotImplementedError

    @staticmethod
    def _check(q, k, v):
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
            raise ValueError("query, keys and values are [batch, tokens, heads, head_dim]")
        if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
            raise ValueError(f"shapes do not agree: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
        if q.shape[2] % k.shape[2]:
            raise ValueError(f"{q.shape[2]} query heads are not a multiple of {k.shape[2]} key / value heads")


class StandardPagedAttentionKernel(PagedAttentionKernel):
    """fp32 statement of the operator, step by step."""
    name = "standard"

    @staticmethod
    def matmul_query_key(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
        """[B, Q, H, D] x [B, C, Hkv, D] -> scores [B, H, Q, C] (key heads repeated for grouped queries)."""
        rep = q.shape[2] // k.shape[2]
        kk = k.repeat_interleave(rep, 2) if rep > 1 else k
        return torch.einsum("bqhd,bchd->bhqc", q.float(), kk.float())

    @staticmethod
    def scale_tensor(t: torch.Tensor, s: float) -> torch.Tensor:
        return t * s

    @staticmethod
    def apply_causal_mask(scores: torch.Tensor, start_pos: int) -> torch.Tensor:
        """Query ``i`` sees keys ``<= start_pos + i``."""
        Q, C = scores.shape[-2:]
        keep = torch.arange(C, device=scores.device)[None, :] <= (start_pos + torch.arange(Q, device=scores.device))[:, None]
        return scores.masked_fill(~keep, float("-inf"))

    @staticmethod
    def softmax(scores: torch.Tensor) -> torch.Tensor:
        m = scores.amax(-1, keepdim=True)
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        e = torch.exp(scores - m)
        return e / e.sum(-1, keepdim=True).clamp_min(1e-30)

    @staticmethod
    def matmul_weight_value(w: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        rep = w.shape[1] // v.shape[2]
        vv = v.repeat_interleave(rep, 2) if rep > 1 else v
        return torch.einsum("bhqc,bchd->bqhd", w, vv.float())

    def compute_paged_attention(self, query, cached_keys, cached_values, phase=AttentionPhase.DECODE, scale=None):
        self._check(query, cached_keys, cached_values)
        Q, C, D = query.shape[1], cached_keys.shape[1], query.shape[3]
        s = self.scale_tensor(self.matmul_query_key(query, cached_keys), scale if scale is not None else 1.0 / math.sqrt(D))
        if (phase == AttentionPhase.DECODE and C > Q) or (phase == AttentionPhase.PREFILL and Q > 1):
            s = self.apply_causal_mask(s, C - Q)
        return self.matmul_weight_value(self.softmax(s), cached_values).to(query.dtype)


class FusedPagedAttentionKernel(PagedAttentionKernel):
    """One fused call: this package's tensor-core attention on bf16 CUDA tensors with head dimension 128 (contiguous
    K / V, cached prefix of any length), PyTorch's fused attention elsewhere. Same contract as the standard kernel."""
    name = "fused"

    def compute_paged_attention(self, query, cached_keys, cached_values, phase=AttentionPhase.DECODE, scale=None):
        self._check(query, cached_keys, cached_values)
        B, Q, H, D = query.shape
        C = cached_keys.shape[1]
        causal = (phase == AttentionPhase.DECODE and C > Q) or (phase == AttentionPhase.PREFILL and Q > 1)
        if query.is_cuda and query.dtype == torch.bfloat16 and D == 128 and scale is None and causal and Q >= 16:
            from ..ops import native
            outs = [native.flash_fwd_prefix(query[b].contiguous(), cached_keys[b].contiguous(), cached_values[b].contiguous(), 1, Q, C, causal=True)
                    for b in range(B)]
            return torch.stack(outs)
        rep = H // cached_keys.shape[2]
        k = cached_keys.repeat_interleave(rep, 2) if rep > 1 else cached_keys
        v = cached_values.repeat_interleave(rep, 2) if rep > 1 else cached_values
        mask = None
        if causal:
            mask = torch.arange(C, device=query.device)[None, :] <= (C - Q + torch.arange(Q, device=query.device))[:, None]
        o = torch.nn.functional.scaled_dot_product_attention(query.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask, scale=scale)
        return o.transpose(1, 2)


def create_kernel(name: str = "auto", device: Optional[torch.device] = None) -> PagedAttentionKernel:
    if name == "standard":
        return StandardPagedAttentionKernel()
    if name in ("fused", "cuda"):
        return FusedPagedAttentionKernel()
    if name == "auto":
        return FusedPagedAttentionKernel() if device is not None and torch.device(device).type == "cuda" else StandardPagedAttentionKernel()
    raise KeyError(f"unknown kernel {name!r}")


# ------------------------------------------------------------------ orchestrators
class PrefillOrchestrator:
    """Prompt processing for one layer stack: reserves the prompt's blocks up front (all or nothing), then runs the
    layers' attention over the prompt, optionally in chunks."""

    def __init__(self, kv: KVCacheBlockManager, chunk_size: Optional[int] = None):
        self.kv, self.chunk_size = kv, chunk_size

    def blocks_for(self, prompt_len: int) -> int:
        return self.kv.blocks_needed(prompt_len)

    def can_prefill(self, prompt_len: int) -> bool:
        return self.kv.has_available_blocks(self.blocks_for(prompt_len))

    def prefill_allocate_blocks(self, seq_id: int, prompt_len: int) -> bool:
        """True when the cache has room for the whole prompt (blocks themselves are taken as tokens are appended)."""
        if prompt_len <= 0:
            raise ValueError("prompt must not be empty")
        return self.can_prefill(prompt_len)

    def compute_prefill_attention(self, layer: PagedAttentionLayer, hidden: torch.Tensor, seq_id: int) -> torch.Tensor:
        """``hidden`` [tokens, d_model] of ONE sequence; chunked when a chunk size is set."""
        n = hidden.shape[0]
        if not self.chunk_size or n <= self.chunk_size:
            return layer(hidden, self.kv, [seq_id], AttentionPhase.PREFILL)
        outs = [layer(hidden[i:i + self.chunk_size], self.kv, [seq_id], AttentionPhase.PREFILL) for i in range(0, n, self.chunk_size)]
        return torch.cat(outs)

    def batch_prefill(self, layer: PagedAttentionLayer, hidden: Sequence[torch.Tensor], seq_ids: Sequence[int]) -> List[torch.Tensor]:
        """First chunks of several sequences in one layer call; results split back per sequence."""
        if len(hidden) != len(seq_ids):
            raise ValueError("one hidden tensor per sequence")
        lens = [h.shape[0] for h in hidden]
        if not self.kv.has_available_blocks(sum(self.blocks_for(n) for n in lens)):
            raise MemoryError("KV cache cannot hold the batch's prompts")
        out = layer(torch.cat(list(hidden)), self.kv, list(seq_ids), AttentionPhase.PREFILL, n_tokens=lens)
        return list(out.split(lens))


class DecodeOrchestrator:
    """One new token per sequence: the last block is reused while it has room, else a block is taken."""

    def __init__(self, kv: KVCacheBlockManager):
        self.kv = kv

    def needs_new_block(self, seq_id: int) -> bool:
        return self.kv.get_sequence_length(seq_id) % self.kv.block_size == 0

    def allocate_decode_block(self, seq_id: int) -> bool:
        """True when the next token of the sequence has a slot (room in its last block, or a free block)."""
        return (not self.needs_new_block(seq_id)) or self.kv.has_available_blocks(1)

    def compute_decode_attention(self, layer: PagedAttentionLayer, hidden: torch.Tensor, seq_id: int) -> torch.Tensor:
        if hidden.shape[0] != 1:
            raise ValueError("decode takes one token")
        return layer(hidden, self.kv, [seq_id], AttentionPhase.DECODE)

    def batch_decode(self, layer: PagedAttentionLayer, hidden: torch.Tensor, seq_ids: Sequence[int]) -> torch.Tensor:
        if hidden.shape[0] != len(seq_ids):
            raise ValueError("one token per sequence")
        need = sum(1 for s in seq_ids if self.needs_new_block(s))
        if need and not self.kv.has_available_blocks(need):
            raise MemoryError("KV cache cannot take the batch's next tokens")
        return layer(hidden, self.kv, list(seq_ids), AttentionPhase.DECODE)
