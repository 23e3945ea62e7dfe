"""Software all-reduce algorithms over point-to-point exchanges, and the optimiser that picks one.

Reference: src/MLFramework/Communication/Optimizations/AlgorithmSelector.cs:24-62 names recursive doubling (tiny
messages), Rabenseifner (medium), ring (large) and tree (very large, latency-tolerant) and selects by message size and
world size; CommunicationOptimizer.cs:40 ``AllReduceOptimized`` applies the choice; the reference implements only the
ring (Distributed/RingAllReduce.cs). Here all four run over the process-group facade's paired send / receive, so they
work on any back-end (gloo on CPU, NCCL p2p) and serve as the oracle and the fall-back for the in-kernel one-shot /
two-shot NVLink collectives, which are what a B200 node uses when its ranks can map each other's memory.

World sizes that are not a power of two use the usual fold: the first ``2 * (W - P)`` ranks pair up (odd ranks hand
their data to the even neighbour and sit out), the remaining ``P`` ranks run the power-of-two schedule, and the result
is handed back.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .fault_tolerance import AlgorithmSelector, CollectiveAlgorithm, RingAllReduce
from .process_group import ReduceOp


def _combine(dst: torch.Tensor, src: torch.Tensor, op: ReduceOp):
    if op in (ReduceOp.SUM, ReduceOp.AVG):
        dst.add_(src)
    elif op == ReduceOp.MAX:
        torch.maximum(dst, src, out=dst)
    elif op == ReduceOp.MIN:
        torch.minimum(dst, src, out=dst)
    else:
        dst.mul_(src)


def _exchange(pg, send: Optional[torch.Tensor], recv: Optional[torch.Tensor], peer: int):
    """Paired transfer with one peer; both directions are posted before either is waited for."""
    ops = []
    if send is not None:
        ops.append(("send", send.contiguous(), peer))
    if recv is not None:
        ops.append(("recv", recv, peer))
    for w in pg.batch_isend_irecv(ops):
        w.wait()


def _pow2_below(w: int) -> int:
    p = 1
    while p * 2 <= w:
        p *= 2
    return p


class _Folded:
    """Maps a world of any size onto a power-of-two core. ``core_rank`` is ``None`` for ranks that sit out."""

    def __init__(self, pg):
        self.pg, self.W, self.r = pg, pg.world_size, pg.rank
        self.P = _pow2_below(self.W)
        self.extra = self.W - self.P
        if self.r < 2 * self.extra:
            self.core_rank = self.r // 2 if self.r % 2 == 0 else None
        else:
            self.core_rank = self.r - self.extra

    def to_world(self, core: int) -> int:
        return 2 * core if core < self.extra else core + self.extra

    def fold_in(self, flat: torch.Tensor, op: ReduceOp):
        if self.r < 2 * self.extra:
            if self.r % 2:
                _exchange(self.pg, flat, None, self.r - 1)
            else:
                buf = torch.empty_like(flat)
                _exchange(self.pg, None, buf, self.r + 1)
                _combine(flat, buf, op)

    def fold_out(self, flat: torch.Tensor):
        if self.r < 2 * self.extra:
            if self.r % 2:
                _exchange(self.pg, None, flat, self.r - 1)
            else:
                _exchange(self.pg, flat, None, self.r + 1)


class _Base:
    algorithm: CollectiveAlgorithm

    def __init__(self, pg):
        self.pg = pg
        self.steps = 0                 # exchanges this rank took part in during the last call
        self.bytes_sent = 0

    def _note(self, t: Optional[torch.Tensor]):
        self.steps += 1
        if t is not None:
            self.bytes_sent += t.numel() * t.element_size()

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        self.steps = self.bytes_sent = 0
        if self.pg.world_size == 1:
            return t
        flat = t.contiguous().view(-1)
        self._run(flat, op)
        if op == ReduceOp.AVG:
            flat.div_(self.pg.world_size)
        if flat.data_ptr() != t.data_ptr():
            t.copy_(flat.view_as(t))
        return t

    def _run(self, flat: torch.Tensor, op: ReduceOp):
        raise NotImplementedError


class RecursiveDoublingAllReduce(_Base):
    """log2(P) rounds; in round k a rank swaps its WHOLE vector with the partner at distance 2^k and combines. Fewest
    rounds, most bytes: for messages of a few KB where latency is everything."""
    algorithm = CollectiveAlgorithm.RECURSIVE_DOUBLING

    def _run(self, flat, op):
        f = _Folded(self.pg)
        f.fold_in(flat, op)
        if f.core_rank is not None:
            buf = torch.empty_like(flat)
            d = 1
            while d < f.P:
                peer = f.to_world(f.core_rank ^ d)
                _exchange(self.pg, flat.clone(), buf, peer)
                self._note(flat)
                _combine(flat, buf, op)
                d *= 2
        f.fold_out(flat)


class RabenseifnerAllReduce(_Base):
    """Reduce-scatter by recursive halving (each round sends half of what the rank still owns), then all-gather by
    recursive doubling: 2 log2(P) rounds and 2 (P-1)/P of the vector sent per rank, the bandwidth optimum."""
    algorithm = CollectiveAlgorithm.RABENSEIFNER

    def _run(self, flat, op):
        f = _Folded(self.pg)
        f.fold_in(flat, op)
        if f.core_rank is not None:
            n, P, c = flat.numel(), f.P, f.core_rank
            lo, hi = 0, n                           # the range this rank is still responsible for
            d = P // 2
            path: List[Tuple[int, int, int, int, int]] = []
            while d >= 1:
                mid = lo + (hi - lo) // 2
                peer = f.to_world(c ^ d)
                keep_low = (c & d) == 0
                k_lo, k_hi = (lo, mid) if keep_low else (mid, hi)
                s_lo, s_hi = (mid, hi) if keep_low else (lo, mid)
                buf = torch.empty(k_hi - k_lo, dtype=flat.dtype, device=flat.device)
                _exchange(self.pg, flat[s_lo:s_hi].clone(), buf, peer)
                self._note(flat[s_lo:s_hi])
                _combine(flat[k_lo:k_hi], buf, op)
                path.append((peer, k_lo, k_hi, s_lo, s_hi))
                lo, hi = k_lo, k_hi
                d //= 2
            for peer, k_lo, k_hi, s_lo, s_hi in reversed(path):       # all-gather: undo the halving
                buf = torch.empty(s_hi - s_lo, dtype=flat.dtype, device=flat.device)
                _exchange(self.pg, flat[k_lo:k_hi].clone(), buf, peer)
                self._note(flat[k_lo:k_hi])
                flat[s_lo:s_hi].copy_(buf)
        f.fold_out(flat)


class TreeAllReduce(_Base):
    """Binomial-tree reduce to rank 0, binomial-tree broadcast back: 2 log2(W) rounds, any world size, and only one
    message in flight per rank - the gentlest schedule for a congested or high-latency fabric."""
    algorithm = CollectiveAlgorithm.TREE

    def _run(self, flat, op):
        W, r = self.pg.world_size, self.pg.rank
        buf = torch.empty_like(flat)
        d = 1
        while d < W:                                 # reduce
            if r % (2 * d) == d:
                _exchange(self.pg, flat, None, r - d)
                self._note(flat)
                break
            if r % (2 * d) == 0 and r + d < W:
                _exchange(self.pg, None, buf, r + d)
                self._note(None)
                _combine(flat, buf, op)
            d *= 2
        top = 1
        while top < W:
            top *= 2
        d = top // 2
        while d >= 1:                                # broadcast
            if r % (2 * d) == 0 and r + d < W:
                _exchange(self.pg, flat, None, r + d)
                self._note(flat)
            elif r % (2 * d) == d:
                _exchange(self.pg, None, flat, r - d)
                self._note(None)
            d //= 2


class _Ring(_Base):
    algorithm = CollectiveAlgorithm.RING

    def all_reduce(self, t, op=ReduceOp.SUM):
        return RingAllReduce(self.pg).all_reduce(t, op)


_SOFTWARE = {CollectiveAlgorithm.RECURSIVE_DOUBLING: RecursiveDoublingAllReduce, CollectiveAlgorithm.RABENSEIFNER: RabenseifnerAllReduce,
             CollectiveAlgorithm.TREE: TreeAllReduce, CollectiveAlgorithm.RING: _Ring}


def all_reduce_with(pg, t: torch.Tensor, algorithm: CollectiveAlgorithm, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
    """All-reduce by a named algorithm; ``ONE_SHOT`` / ``TWO_SHOT`` mean the back-end's own collective."""
    cls = _SOFTWARE.get(algorithm)
    if cls is None:
        pg.all_reduce(t, op)
        return t
    return cls(pg).all_reduce(t, op)


class CommunicationOptimizer:
    """``all_reduce_optimized`` picks the algorithm for the message (``AlgorithmSelector``) and keeps a count of its
    choices; ``all_reduce_many`` packs small tensors of one dtype into flat buckets first, so that a list of bias-sized
    gradients costs one collective instead of one each."""

    def __init__(self, pg, selector: Optional[AlgorithmSelector] = None, native_collectives: bool = True, bucket_bytes: int = 25 << 20):
        self.pg, self.native, self.bucket_bytes = pg, native_collectives, bucket_bytes
        self.selector = selector or AlgorithmSelector(nvswitch=native_collectives)
        self.choices: Dict[str, int] = {}

    def all_reduce_optimized(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        alg = self.selector.select_all_reduce(t.numel() * t.element_size(), self.pg.world_size)
        self.choices[alg.value] = self.choices.get(alg.value, 0) + 1
        return all_reduce_with(self.pg, t, alg, op)

    def all_reduce_many(self, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.SUM) -> int:
        """In place; returns the number of collectives issued."""
        by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
        for t in tensors:
            by_dtype.setdefault(t.dtype, []).append(t)
        n = 0
        for dt, ts in by_dtype.items():
            bucket: List[torch.Tensor] = []
            size = 0

            def flush():
                nonlocal bucket, size, n
                if not bucket:
                    return
                if len(bucket) == 1:
                    self.all_reduce_optimized(bucket[0], op)
                else:
                    flat = torch.cat([b.reshape(-1) for b in bucket])
                    self.all_reduce_optimized(flat, op)
                    off = 0
                    for b in bucket:
                        b.copy_(flat[off:off + b.numel()].view_as(b))
                        off += b.numel()
                n += 1
                bucket, size = [], 0
            for t in ts:
                nb = t.numel() * t.element_size()
                if size and size + nb > self.bucket_bytes:
                    flush()
                bucket.append(t)
                size += nb
            flush()
        return n
