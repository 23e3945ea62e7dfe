"""Context (sequence) parallel attention: the sequence is sharded over a process group.

The reference framework shards batch (DDP), parameters (FSDP), weights (tensor parallel) and
layers (pipeline) but always keeps a whole sequence on one device
(src/MLFramework/Distributed, src/MLFramework/Inference/PagedAttention). This module adds the
missing axis for sequences that do not fit one GPU's activations:

* ``ring_attention``: every rank keeps its query shard; key/value shards travel once round
  the ring, the partial results merge through their log-sum-exp, so the full score matrix
  never exists. Backward sends each key/value shard round again with its gradient
  accumulators, which arrive home holding every rank's contribution.
* ``ulysses_attention``: two all-to-alls swap the sharded axis from sequence to heads, so
  each rank runs ordinary attention over the full sequence for ``H / W`` heads.

Token positions travel with the shards, so the causal mask is right for the contiguous and
for the zig-zag layout (rank ``r`` holds chunks ``r`` and ``2W-1-r`` of ``2W``, which gives
every rank the same amount of unmasked work).

Ring transfers are paired send/receive batches, so no rank blocks on a send that its peer
has not yet matched. The block arithmetic is written with torch operators in fp32: on a GPU
the products run on the library GEMM; the point of this module is the communication pattern
and its gradients.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch

__all__ = [
    "local_positions", "shard_sequence", "unshard_sequence",
    "ring_attention", "ulysses_attention", "context_parallel_attention",
    "ContextParallelAttention",
]


# ------------------------------------------------------------------ sequence layouts
def local_positions(rank: int, world: int, seq_len: int, zigzag: bool = False) -> torch.Tensor:
    """Global token positions (int64, ascending within a chunk) that ``rank`` holds."""
    parts = 2 * world if zigzag else world
    if seq_len % parts != 0:
        raise ValueError(f"sequence length {seq_len} is not divisible by {parts}")
    c = seq_len // parts
    if not zigzag:
        return torch.arange(rank * c, (rank + 1) * c)
    hi = 2 * world - 1 - rank
    return torch.cat([torch.arange(rank * c, (rank + 1) * c), torch.arange(hi * c, (hi + 1) * c)])


def shard_sequence(x: torch.Tensor, rank: int, world: int, dim: int = 1, zigzag: bool = False) -> torch.Tensor:
    """This rank's slice of ``x`` along the sequence axis ``dim``."""
    pos = local_positions(rank, world, x.shape[dim], zigzag).to(x.device)
    return x.index_select(dim, pos).contiguous()


def unshard_sequence(shards, dim: int = 1, zigzag: bool = False) -> torch.Tensor:
    """Inverse of ``shard_sequence`` given every rank's shard in rank order."""
    world = len(shards)
    full = torch.cat(list(shards), dim=dim)
    if not zigzag:
        return full
    seq = full.shape[dim]
    order = torch.cat([local_positions(r, world, seq, True) for r in range(world)])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(seq)
    return full.index_select(dim, inv.to(full.device))


# ------------------------------------------------------------------ block arithmetic
def _expand_kv(k: torch.Tensor, rep: int) -> torch.Tensor:
    # [B, Sk, Hkv, D] -> [B, Hq, Sk, D] (fp32)
    return k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)


def _scores(qf, kf, scale, q_pos, k_pos, causal):
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(k_pos[None, :] > q_pos[:, None], float("-inf"))
    return s


def _block_forward(qf, k, v, scale, q_pos, k_pos, causal) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of the local queries against one key/value shard.

    Returns (o [B, H, Sq, D] normalised within the block, lse [B, H, Sq]); a row that sees
    nothing in this block has lse = -inf and o = 0.
    """
    rep = qf.shape[1] // k.shape[2]
    s = _scores(qf, _expand_kv(k, rep), scale, q_pos, k_pos, causal)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    return torch.matmul(p, _expand_kv(v, rep)), lse


def _merge(o, lse, o_b, lse_b):
    """Combine two partial attention results over disjoint key sets."""
    new = torch.logaddexp(lse, lse_b)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    w_a = torch.exp(lse - safe)[..., None]
    w_b = torch.exp(lse_b - safe)[..., None]
    return o * w_a + o_b * w_b, new


def _block_backward(qf, k, v, dof, lse, delta, scale, q_pos, k_pos, causal):
    """Gradient contributions of one key/value shard: (dq [B,H,Sq,D], dk, dv [B,Sk,Hkv,D])."""
    B, H, Sq, D = qf.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    kf, vf = _expand_kv(k, rep), _expand_kv(v, rep)
    s = _scores(qf, kf, scale, q_pos, k_pos, causal)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe[..., None])
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    Sk = k.shape[1]
    dk = dk.view(B, Hkv, rep, Sk, D).sum(2).permute(0, 2, 1, 3)
    dv = dv.view(B, Hkv, rep, Sk, D).sum(2).permute(0, 2, 1, 3)
    return dq, dk, dv


def _may_skip(q_pos, k_pos, causal) -> bool:
    return bool(causal and int(k_pos.min()) > int(q_pos.max()))


# ------------------------------------------------------------------ ring transfers
def _start_ring(pg, send: torch.Tensor):
    """Post one hop of the ring (to rank+1, from rank-1); returns (works, receive buffer)."""
    W, r = pg.world_size, pg.rank
    recv = torch.empty_like(send)
    works = pg.batch_isend_irecv([("send", send.contiguous(), (r + 1) % W), ("recv", recv, (r - 1) % W)])
    return works, recv


def _finish(works):
    for w in works:
        w.wait()


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pg, causal, scale, zigzag, seq_len):
        W, r = pg.world_size, pg.rank
        dev = q.device
        q_pos = local_positions(r, W, seq_len, zigzag).to(dev)
        qf = q.float().permute(0, 2, 1, 3)
        B, H, Sq, D = qf.shape
        o = torch.zeros(B, H, Sq, D, dtype=torch.float32, device=dev)
        lse = torch.full((B, H, Sq), float("-inf"), dtype=torch.float32, device=dev)
        kv = torch.stack([k, v]).contiguous()
        for step in range(W):
            src = (r - step) % W
            pending = _start_ring(pg, kv) if step + 1 < W else None   # next shard flies during the math
            k_pos = local_positions(src, W, seq_len, zigzag).to(dev)
            if not _may_skip(q_pos, k_pos, causal):
                o_b, lse_b = _block_forward(qf, kv[0], kv[1], scale, q_pos, k_pos, causal)
                o, lse = _merge(o, lse, o_b, lse_b)
            if pending is not None:
                _finish(pending[0])
                kv = pending[1]
        out = o.permute(0, 2, 1, 3).to(q.dtype).contiguous()
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.pg, ctx.causal, ctx.scale, ctx.zigzag, ctx.seq_len = pg, causal, scale, zigzag, seq_len
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        pg, causal, scale, zigzag, seq_len = ctx.pg, ctx.causal, ctx.scale, ctx.zigzag, ctx.seq_len
        W, r = pg.world_size, pg.rank
        dev = q.device
        q_pos = local_positions(r, W, seq_len, zigzag).to(dev)
        qf = q.float().permute(0, 2, 1, 3)
        dof = dout.float().permute(0, 2, 1, 3)
        delta = (dof * out.float().permute(0, 2, 1, 3)).sum(-1)
        dq = torch.zeros_like(qf)
        # the travelling bundle: [k, v, dk, dv] of one shard, fp32 so the sums do not round per hop
        bundle = torch.stack([k.float(), v.float(), torch.zeros_like(k, dtype=torch.float32),
                              torch.zeros_like(v, dtype=torch.float32)]).contiguous()
        for step in range(W):
            src = (r - step) % W
            k_pos = local_positions(src, W, seq_len, zigzag).to(dev)
            if not _may_skip(q_pos, k_pos, causal):
                dq_b, dk_b, dv_b = _block_backward(qf, bundle[0], bundle[1], dof, lse, delta, scale,
                                                   q_pos, k_pos, causal)
                dq += dq_b
                bundle[2] += dk_b
                bundle[3] += dv_b
            works, recv = _start_ring(pg, bundle)
            _finish(works)
            bundle = recv
        # after W hops the bundle that started here is back, carrying every rank's dk and dv
        return (dq.permute(0, 2, 1, 3).to(q.dtype), bundle[2].to(k.dtype), bundle[3].to(v.dtype),
                None, None, None, None, None)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pg, *, causal: bool = True,
                   scale: Optional[float] = None, zigzag: bool = False) -> torch.Tensor:
    """Attention over a sequence sharded on ``pg``.

    q [B, S/W, Hq, D] and k, v [B, S/W, Hkv, D] are this rank's shards (``shard_sequence``
    layout); the result is the matching shard of full attention. Differentiable in q, k, v.
    """
    if q.shape[1] != k.shape[1] or k.shape != v.shape:
        raise ValueError("ring_attention: q, k and v must hold the same sequence shard")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError("ring_attention: query heads must be a multiple of key/value heads")
    W = pg.world_size
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _RingAttention.apply(q, k, v, pg, bool(causal), float(scale), bool(zigzag), q.shape[1] * W)


# ------------------------------------------------------------------ Ulysses (all-to-all)
class _SeqToHeads(torch.autograd.Function):
    """[B, S/W, H, D] sharded by sequence -> [B, S, H/W, D] sharded by heads."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _seq_to_heads(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g.contiguous(), ctx.pg), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _heads_to_seq(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g.contiguous(), ctx.pg), None


def _seq_to_heads(x, pg):
    W = pg.world_size
    B, Sl, H, D = x.shape
    if H % W != 0:
        raise ValueError(f"ulysses: {H} heads are not divisible by {W} ranks")
    send = x.view(B, Sl, W, H // W, D).permute(2, 0, 1, 3, 4).reshape(W * B, Sl, H // W, D)
    got = pg.all_to_all(send)                      # chunk j: sequence shard j, my heads
    return got.view(W, B, Sl, H // W, D).permute(1, 0, 2, 3, 4).reshape(B, W * Sl, H // W, D)


def _heads_to_seq(x, pg):
    W = pg.world_size
    B, S, Hl, D = x.shape
    Sl = S // W
    send = x.view(B, W, Sl, Hl, D).permute(1, 0, 2, 3, 4).reshape(W * B, Sl, Hl, D)
    got = pg.all_to_all(send)                      # chunk j: my sequence shard, head group j
    return got.view(W, B, Sl, Hl, D).permute(1, 2, 0, 3, 4).reshape(B, Sl, W * Hl, D)


def _full_attention(q, k, v, causal, scale):
    from ..ops.reference import attention_ref
    return attention_ref(q, k, v, causal=causal, scale=scale)[0].to(q.dtype)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pg, *, causal: bool = True,
                      scale: Optional[float] = None,
                      attn_fn: Optional[Callable] = None) -> torch.Tensor:
    """Attention over a contiguously sharded sequence by swapping to head sharding and back.

    Needs both head counts divisible by the group size. ``attn_fn(q, k, v, causal, scale)``
    runs on the full sequence with ``H / W`` heads; the default is the fp32 reference.
    """
    fn = attn_fn or _full_attention
    qh, kh, vh = (_SeqToHeads.apply(t.contiguous(), pg) for t in (q, k, v))
    oh = fn(qh, kh, vh, causal, scale)
    return _HeadsToSeq.apply(oh.contiguous(), pg)


# ------------------------------------------------------------------ dispatcher and module
def context_parallel_attention(q, k, v, pg, *, mode: str = "ring", causal: bool = True,
                               scale: Optional[float] = None, zigzag: bool = False):
    """``mode`` "ring" (any head count, optional zig-zag balance) or "ulysses" (heads % W == 0)."""
    if pg is None or pg.world_size == 1:
        return _full_attention(q, k, v, causal, scale)
    if mode == "ring":
        return ring_attention(q, k, v, pg, causal=causal, scale=scale, zigzag=zigzag)
    if mode == "ulysses":
        if zigzag:
            raise ValueError("ulysses mode needs the contiguous layout")
        return ulysses_attention(q, k, v, pg, causal=causal, scale=scale)
    raise ValueError(f"unknown context-parallel mode {mode!r}")


class ContextParallelAttention(torch.nn.Module):
    """Self-attention block (fused QKV projection, output projection) over a sharded sequence.

    ``forward(x)`` takes this rank's [B, S/W, hidden] shard. Weights are replicated: their
    gradients are partial sums over the local tokens and need the usual data-parallel
    all-reduce over the same group.
    """

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: Optional[int] = None, pg=None,
                 mode: str = "ring", causal: bool = True, zigzag: bool = False, bias: bool = False):
        super().__init__()
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads or n_heads
        if hidden % n_heads != 0:
            raise ValueError("hidden size must be divisible by the head count")
        self.head_dim = hidden // n_heads
        self.pg, self.mode, self.causal, self.zigzag = pg, mode, causal, zigzag
        self.qkv = torch.nn.Linear(hidden, (n_heads + 2 * self.n_kv_heads) * self.head_dim, bias=bias)
        self.proj = torch.nn.Linear(hidden, hidden, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, Sl, _ = x.shape
        hq, hk, d = self.n_heads, self.n_kv_heads, self.head_dim
        q, k, v = self.qkv(x).split([hq * d, hk * d, hk * d], dim=-1)
        o = context_parallel_attention(q.reshape(B, Sl, hq, d), k.reshape(B, Sl, hk, d), v.reshape(B, Sl, hk, d),
                                       self.pg, mode=self.mode, causal=self.causal, zigzag=self.zigzag)
        return self.proj(o.reshape(B, Sl, hq * d))
