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

On CUDA with more than one rank and ``fused_comm=True`` the bucket buffers live in symmetric
(peer-mapped) memory and a bucket is reduced by ONE launch of the two-shot all-reduce kernel that
synchronises with the peers inside the kernel, scales by 1/W and checks the result for overflow
(``SymmetricMemory.all_reduce_two_shot_sync``, ``csrc/symm/symm_mem.cu``), on a communication
stream, as soon as the bucket's last gradient has been queued; otherwise it is
``torch.distributed`` (NCCL or gloo). ``FlatGradReducer`` is the same hook-driven reduction over a
flat gradient buffer whose kernels write ``main_grad`` views directly (the training engine's path).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from ..dist.process_group import ReduceOp, default_group

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
    reduced: bool = False            # a reduction was launched for this bucket in the current step
    symm_buf: object = None          # SymmBuffer behind ``flat`` on the fused path

    def allocate(self, symm=None):
        if self.flat is None:
            if symm is not None:
                padded = (self.numel + 7) // 8 * 8
                self.symm_buf = symm.alloc(padded * self.flat_elem_size())
                self.flat = self.symm_buf.view(self.dtype, padded)
                self.flat.zero_()
            else:
                self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)

    def flat_elem_size(self) -> int:
        return torch.empty(0, dtype=self.dtype).element_size()

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
        """Write the reduced values to ``p.grad``. A parameter without a gradient gets the bucket view
        itself, so that later steps accumulate in place and neither copy is needed again."""
        for p, off in zip(self.params, self.offsets):
            view = self.flat[off:off + p.numel()].view_as(p)
            if p.grad is None:
                p.grad = view
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


class _StreamWork:
    """Completion handle of a launch on a side stream: ``wait`` orders the current stream after it."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)

    def is_completed(self) -> bool:
        return bool(self.event.query())


def fused_comm_possible(pg, device, fused_comm: bool, dtype=torch.bfloat16) -> bool:
    """The in-kernel path needs CUDA, 2..8 ranks, bf16 gradients and a NCCL / gloo group to exchange handles."""
    return bool(fused_comm and pg is not None and 1 < pg.world_size <= 8 and torch.device(device).type == "cuda"
                and dtype == torch.bfloat16 and not getattr(pg, "is_fake", False))


class GradientBucketManager:
    def __init__(self, pg, params: Iterable[nn.Parameter], bucket_size_mb: float = DEFAULT_BUCKET_MB, symm=None,
                 flag=None):
        if bucket_size_mb <= 0:
            raise ValueError("bucket_size_mb must be positive")
        self.pg = pg
        self.buckets = create_buckets(params, int(bucket_size_mb * 1024 * 1024))
        self.param_to_bucket: Dict[int, int] = {id(p): b.index for b in self.buckets for p in b.params}
        self.symm = symm                      # SymmetricMemory when the fused path is active
        self.flag = flag                      # overflow flag in symmetric memory (optional)
        self.comm_stream = torch.cuda.Stream(device=self.buckets[0].device) if (symm is not None and self.buckets) else None
        if symm is not None:
            # collective allocations: same order on every rank
            for b in self.buckets:
                b.allocate(symm)

    def reduce_bucket(self, b: GradientBucket, op: ReduceOp):
        b.prepare()
        b.reduced = True
        if self.symm is not None and b.symm_buf is not None and op in (ReduceOp.SUM, ReduceOp.AVG):
            cs = self.comm_stream
            cs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cs):
                self.symm.all_reduce_two_shot_sync(b.symm_buf, b.flat.numel(), scale=1.0 / self.symm.world if op == ReduceOp.AVG else 1.0,
                                                   flag=self.flag, key="ddp", max_ctas=32)
                ev = torch.cuda.Event()
                ev.record(cs)
            b.work = _StreamWork(ev)
            return
        b.work = self.pg.all_reduce(b.flat, op=op, async_op=True)

    def reduce_all(self, op: ReduceOp = ReduceOp.SUM):
        for b in self.buckets:
            self.reduce_bucket(b, op)

    def wait_all(self) -> List[GradientBucket]:
        """Waits for the reductions launched this step; returns the buckets that had one."""
        done = []
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                b.work = None
            if b.reduced:
                done.append(b)
        return done

    def copy_back_all(self, only: Optional[List[GradientBucket]] = None):
        for b in (self.buckets if only is None else only):
            if b.flat is not None:
                b.copy_back()
            b.reduced = False


class DistributedDataParallel(nn.Module):
    """Wraps ``module``; gradients are averaged (or summed) over ``process_group``."""

    def __init__(self, module: nn.Module, process_group=None, bucket_size_mb: float = DEFAULT_BUCKET_MB,
                 find_unused_parameters: bool = False, reduce_op: ReduceOp = ReduceOp.AVG,
                 overlap: bool = True, broadcast_parameters: bool = True, fused_comm: bool = True):
        super().__init__()
        self.module = module
        self.pg = process_group if process_group is not None else default_group()
        self.reduce_op = reduce_op
        self.find_unused_parameters = find_unused_parameters
        self.overlap = overlap
        self._params = [p for p in module.parameters() if p.requires_grad]
        symm = None
        if self._params and fused_comm_possible(self.pg, self._params[0].device, fused_comm, self._params[0].dtype) \
                and all(p.dtype == torch.bfloat16 for p in self._params):
            from ..dist.symm import SymmetricMemory
            symm = SymmetricMemory(self.pg, self._params[0].device)
        self.symm = symm
        self.bucket_manager = GradientBucketManager(self.pg, self._params, bucket_size_mb, symm=symm)
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
        """Waits for the reductions of this step and writes back the buckets that were reduced (a bucket
        that was not reduced, e.g. under ``no_sync``, keeps its local gradients)."""
        self.bucket_manager.copy_back_all(self.bucket_manager.wait_all())

    def finish_backward(self):
        """Call after ``loss.backward()``: waits for hook-launched reductions, reduces the buckets the
        hooks did not (no overlap, or parameters that received no gradient), and writes results
        back. Inside ``no_sync()`` it does nothing: gradients stay local until a synchronised step."""
        bm = self.bucket_manager
        if not self._require_sync:
            for b in bm.buckets:
                b.pending = len(b.params)
            return
        for b in bm.buckets:
            if not b.reduced:
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


class FlatGradReducer:
    """Hook-driven all-reduce of a flat gradient buffer (``FlatParams.grad``) in contiguous buckets.

    The weight-gradient kernels write ``main_grad`` views of the flat buffer and then call the
    parameter's ``grad_ready`` callback (see :mod:`ml_framework_b200.ops.functional`); a bucket is a
    contiguous range of that buffer (parameters in registration order, at most ``bucket_size_mb``), and it
    is reduced as soon as its last parameter reports ready, while the rest of backward runs. On the
    fused path the flat buffer lives in symmetric memory and each bucket is one launch of the in-kernel
    two-shot all-reduce (scale 1/W and the overflow check included, every rank's overflow flag raised
    by whoever sees a non-finite sum); otherwise buckets are ``torch.distributed`` all-reduces.

    Reference: GradientBucketManager.cs:81-170 (hook -> bucket ready -> async all-reduce),
    GradientBucket.cs:112-126.
    """

    def __init__(self, flat, pg, bucket_size_mb: float = DEFAULT_BUCKET_MB, symm=None, symm_buf=None, flag=None,
                 average: bool = True):
        self.flat, self.pg, self.symm, self.symm_buf, self.flag = flat, pg, symm, symm_buf, flag
        self.world = pg.world_size if pg is not None else 1
        self.average = average
        limit = int(bucket_size_mb * 1024 * 1024)
        esz = flat.grad.element_size()
        self.ranges: List[tuple] = []            # (lo, hi) element ranges of the flat gradient buffer
        self.members: List[List[nn.Parameter]] = []
        cur, lo = [], 0
        for i, (p, off) in enumerate(zip(flat.params, flat.offsets)):
            end = flat.offsets[i + 1] if i + 1 < len(flat.params) else flat.numel
            if cur and (end - lo) * esz > limit:
                self.ranges.append((lo, off))
                self.members.append(cur)
                cur, lo = [], off
            cur.append(p)
        if cur:
            self.ranges.append((lo, flat.numel))
            self.members.append(cur)
        self.bucket_of = {id(p): k for k, ms in enumerate(self.members) for p in ms}
        self.pending = [len(ms) for ms in self.members]
        self.launched = [False] * len(self.members)
        self.works: List[object] = []
        self.enabled = True
        # A parameter used more than once in the model (a tied embedding / head) reports ready once per
        # use. The first step only counts the reports per parameter; from the second step on a
        # parameter is complete when it has reported that many times.
        self.expected: Optional[Dict[int, int]] = None
        self.counts: Dict[int, int] = {}
        self.comm_stream = torch.cuda.Stream(device=flat.device) if flat.device.type == "cuda" else None
        for p in flat.params:
            p.grad_ready = self._on_ready

    # ---- hooks
    def _on_ready(self, p):
        if not self.enabled or self.world == 1:
            return
        n = self.counts.get(id(p), 0) + 1
        self.counts[id(p)] = n
        if self.expected is None or n != self.expected.get(id(p), 0):
            return
        k = self.bucket_of[id(p)]
        self.pending[k] -= 1
        if self.pending[k] == 0 and not self.launched[k]:
            self._launch(k)

    def _launch(self, k: int):
        lo, hi = self.ranges[k]
        self.launched[k] = True
        g = self.flat.grad
        scale = 1.0 / self.world if self.average else 1.0
        if self.symm is not None:
            cs = self.comm_stream
            cs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cs):
                self.symm.all_reduce_two_shot_sync(self.symm_buf, hi - lo, scale=scale, flag=self.flag,
                                                   offset_bytes=lo * g.element_size(), key="ddp", max_ctas=32)
                ev = torch.cuda.Event()
                ev.record(cs)
            self.works.append(_StreamWork(ev))
        else:
            view = g[lo:hi]
            w = self.pg.all_reduce(view, op=ReduceOp.SUM, async_op=True)
            self.works.append((w, view, scale))

    def finish(self):
        """After backward (and after gradients that arrived through autograd were folded into the flat
        buffer): reduces the buckets no hook completed, in bucket order, then waits for all of them."""
        if self.world > 1 and self.enabled:
            for k in range(len(self.ranges)):
                if not self.launched[k]:
                    self._launch(k)
            for w in self.works:
                if isinstance(w, tuple):
                    w[0].wait()
                    if w[2] != 1.0:
                        w[1].mul_(w[2])
                else:
                    w.wait()
        self.works = []
        if self.expected is None and self.counts:
            self.expected = dict(self.counts)
        self.counts = {}
        self.pending = [len(ms) for ms in self.members]
        self.launched = [False] * len(self.members)
