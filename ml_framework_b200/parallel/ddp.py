"""Distributed data parallel: parameter broadcast, size-sorted gradient bucketing, overlapped
bucket all-reduce.

Behaviour follows the reference (src/MLFramework/Distributed/DistributedDataParallel.cs:47-177,
GradientBucketManager.cs:24-170, GradientBucket.cs:85-156): rank-0 parameters are broadcast at
construction; gradients are packed greedily, largest first, into flat buckets of at most
``bucket_size_mb`` (25 MB default; an oversized tensor gets a bucket of its own); each bucket
is all-reduced and copied back. Unlike the reference, whose per-parameter hooks are stored
but never fired, buckets here are reduced from autograd's post-accumulate hooks as soon as
their last gradient arrives, on a side stream, so communication overlaps the rest of
backward. ``reduce_gradients()`` / ``wait_for_reduction()`` remain as the explicit path.

On GPUs with the peer-memory layer initialised the bucket all-reduce runs through the
in-kernel two-shot all-reduce of :mod:`ml_framework_b200.parallel.fused_comm`; otherwise it is
``torch.distributed`` (NCCL or gloo).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from ..dist.process_group import ProcessGroup, ReduceOp, default_group

DEFAULT_BUCKET_MB = 25


@dataclass
class GradientBucket:
    index: int
    params: List[nn.Parameter]
    numel: int
    dtype: torch.dtype
    device: torch.device
    flat: Optional[torch.Tensor] = None
    offsets: List[int] = field(default_factory=list)
    pending: int = 0
    work: object = None

    def allocate(self):
        if self.flat is None:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)

    def prepare(self):
        """Flatten the member gradients into the bucket (missing gradients count as zeros)."""
        self.allocate()
        for p, off in zip(self.params, self.offsets):
            view = self.flat[off:off + p.numel()]
            if p.grad is None:
                view.zero_()
            elif p.grad.data_ptr() != view.data_ptr():
                view.copy_(p.grad.reshape(-1))

    def copy_back(self):
        for p, off in zip(self.params, self.offsets):
            view = self.flat[off:off + p.numel()].view_as(p)
            if p.grad is None:
                p.grad = view.clone()
            elif p.grad.data_ptr() != view.data_ptr():
                p.grad.copy_(view)


def create_buckets(params: Iterable[nn.Parameter], bucket_bytes: int) -> List[GradientBucket]:
    """Greedy packing, largest tensor first (GradientBucketManager.CreateBuckets :115-170)."""
    params = [p for p in params if p.requires_grad]
    order = sorted(range(len(params)), key=lambda i: -params[i].numel() * params[i].element_size())
    buckets: List[GradientBucket] = []
    cur: List[nn.Parameter] = []
    cur_bytes = 0

    def flush():
        nonlocal cur, cur_bytes
        if cur:
            b = GradientBucket(len(buckets), cur, sum(p.numel() for p in cur), cur[0].dtype, cur[0].device)
            off = 0
            for p in cur:
                b.offsets.append(off)
                off += p.numel()
            buckets.append(b)
            cur, cur_bytes = [], 0

    for i in order:
        p = params[i]
        size = p.numel() * p.element_size()
        if size > bucket_bytes:
            flush()
            cur = [p]
            flush()
            continue
        if cur and (cur_bytes + size > bucket_bytes or cur[0].dtype != p.dtype or cur[0].device != p.device):
            flush()
        cur.append(p)
        cur_bytes += size
    flush()
    return buckets


class GradientBucketManager:
    def __init__(self, pg, params: Iterable[nn.Parameter], bucket_size_mb: float = DEFAULT_BUCKET_MB):
        if bucket_size_mb <= 0:
            raise ValueError("bucket_size_mb must be positive")
        self.pg = pg
        self.buckets = create_buckets(params, int(bucket_size_mb * 1024 * 1024))
        self.param_to_bucket: Dict[int, int] = {id(p): b.index for b in self.buckets for p in b.params}

    def reduce_bucket(self, b: GradientBucket, op: ReduceOp):
        b.prepare()
        b.work = self.pg.all_reduce(b.flat, op=op, async_op=True)

    def reduce_all(self, op: ReduceOp = ReduceOp.SUM):
        for b in self.buckets:
            self.reduce_bucket(b, op)

    def wait_all(self):
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                b.work = None

    def copy_back_all(self):
        for b in self.buckets:
            b.copy_back()


class DistributedDataParallel(nn.Module):
    """Wraps ``module``; gradients are averaged (or summed) over ``process_group``."""

    def __init__(self, module: nn.Module, process_group=None, bucket_size_mb: float = DEFAULT_BUCKET_MB,
                 find_unused_parameters: bool = False, reduce_op: ReduceOp = ReduceOp.AVG,
                 overlap: bool = True, broadcast_parameters: bool = True):
        super().__init__()
        self.module = module
        self.pg = process_group if process_group is not None else default_group()
        self.reduce_op = reduce_op
        self.find_unused_parameters = find_unused_parameters
        self.overlap = overlap
        self._params = [p for p in module.parameters() if p.requires_grad]
        self.bucket_manager = GradientBucketManager(self.pg, self._params, bucket_size_mb)
        self._hooks = []
        self._in_backward_reduce = False
        self._require_sync = True
        if broadcast_parameters:
            self.broadcast_parameters()
        if overlap:
            self._register_gradient_hooks()

    # ---- construction-time broadcast (one flat message per dtype instead of one per tensor)
    def broadcast_parameters(self, src: int = 0):
        tensors = list(self.module.parameters()) + list(self.module.buffers())
        by_key: Dict[tuple, List[torch.Tensor]] = {}
        for t in tensors:
            by_key.setdefault((t.dtype, t.device), []).append(t)
        for group in by_key.values():
            flat = torch.cat([t.detach().reshape(-1) for t in group])
            self.pg.broadcast(flat, src=src)
            off = 0
            with torch.no_grad():
                for t in group:
                    t.copy_(flat[off:off + t.numel()].view_as(t))
                    off += t.numel()

    # ---- hook-driven overlapped reduction
    def _register_gradient_hooks(self):
        for b in self.bucket_manager.buckets:
            b.pending = len(b.params)
        for p in self._params:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_ready))

    def _on_grad_ready(self, p: nn.Parameter):
        if not self._require_sync:
            return
        bm = self.bucket_manager
        b = bm.buckets[bm.param_to_bucket[id(p)]]
        b.pending -= 1
        if b.pending == 0:
            bm.reduce_bucket(b, self.reduce_op)
            b.pending = len(b.params)
            self._in_backward_reduce = True

    def no_sync(self):
        """Context manager: accumulate gradients locally (gradient accumulation micro-steps)."""
        ddp = self

        class _NoSync:
            def __enter__(self):
                ddp._require_sync = False

            def __exit__(self, *a):
                ddp._require_sync = True
        return _NoSync()

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    # ---- explicit path (ReduceGradientsAsync / WaitForReductionAsync)
    def reduce_gradients(self, op: Optional[ReduceOp] = None):
        self.bucket_manager.reduce_all(op or self.reduce_op)

    def wait_for_reduction(self):
        self.bucket_manager.wait_all()
        self.bucket_manager.copy_back_all()

    def finish_backward(self):
        """Call after ``loss.backward()``: waits for hook-launched reductions, reduces buckets
        whose parameters received no gradient (unused parameters), and writes results back."""
        bm = self.bucket_manager
        for b in bm.buckets:
            if b.work is None and (self.find_unused_parameters or b.pending != len(b.params) or not self.overlap):
                bm.reduce_bucket(b, self.reduce_op)
            b.pending = len(b.params)
        self.wait_for_reduction()
        self._in_backward_reduce = False

    def unused_parameters(self) -> List[str]:
        return [n for n, p in self.module.named_parameters() if p.requires_grad and p.grad is None]

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)
