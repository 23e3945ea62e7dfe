"""Request-level dynamic batching.

Reference: src/MLFramework/Serving/DynamicBatcher.cs:35-113 (bounded queue -> batch builder -> user batch
processor -> response scatterer), BatchingConfiguration.cs:8-86 (MaxBatchSize 32, MaxWaitTime 5 ms,
PreferBatchSize 16, MaxQueueSize 100, TimeoutStrategy DispatchPartial / WaitForFull / Adaptive),
BatchBuilder.cs, BoundedRequestQueue.cs, ResponseScatterer.cs, BatchingMetrics.cs, TensorOperations.cs
(pad / stack helpers, PaddingStrategy).

One dispatcher thread forms batches; callers block on a future (``process``) or get the future
(``submit``). The batch processor receives a list of requests and returns a list of responses of the same
length (for tensors, use ``stack_padded`` / ``unstack``).
"""
from __future__ import annotations

import enum
import queue
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable, Generic, List, Optional, Sequence, Tuple, TypeVar

import torch

TReq = TypeVar("TReq")
TResp = TypeVar("TResp")


class TimeoutStrategy(enum.Enum):
    DISPATCH_PARTIAL = "dispatch_partial"   # send whatever is there when the wait expires
    WAIT_FOR_FULL = "wait_for_full"         # only full batches (or on shutdown)
    ADAPTIVE = "adaptive"                   # wait shrinks when the queue is deep, grows when it is shallow


class PaddingStrategy(enum.Enum):
    POST = "post"
    PRE = "pre"


@dataclass
class BatchingConfiguration:
    max_batch_size: int = 32
    max_wait_time_s: float = 0.005
    prefer_batch_size: int = 16
    max_queue_size: int = 100
    timeout_strategy: TimeoutStrategy = TimeoutStrategy.DISPATCH_PARTIAL

    def validate(self):
        if not (0 < self.prefer_batch_size <= self.max_batch_size):
            raise ValueError("0 < prefer_batch_size <= max_batch_size required")
        if self.max_queue_size < self.max_batch_size:
            raise ValueError("max_queue_size must be at least max_batch_size")
        if self.max_wait_time_s < 0:
            raise ValueError("max_wait_time_s must be non-negative")


class QueueFullError(RuntimeError):
    pass


@dataclass
class BatchingMetrics:
    batches: int = 0
    requests: int = 0
    rejected: int = 0
    failed_batches: int = 0
    total_wait_s: float = 0.0
    total_process_s: float = 0.0
    size_histogram: dict = field(default_factory=dict)

    def record(self, size: int, wait_s: float, proc_s: float):
        self.batches += 1
        self.requests += size
        self.total_wait_s += wait_s
        self.total_process_s += proc_s
        self.size_histogram[size] = self.size_histogram.get(size, 0) + 1

    @property
    def mean_batch_size(self) -> float:
        return self.requests / self.batches if self.batches else 0.0


def stack_padded(tensors: Sequence[torch.Tensor], pad_value: float = 0, strategy: PaddingStrategy = PaddingStrategy.POST,
                 multiple_of: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stacks tensors that differ in their first dimension; returns (batch, lengths)."""
    L = max(t.shape[0] for t in tensors)
    L = (L + multiple_of - 1) // multiple_of * multiple_of
    out = tensors[0].new_full((len(tensors), L) + tuple(tensors[0].shape[1:]), pad_value)
    for i, t in enumerate(tensors):
        if strategy == PaddingStrategy.POST:
            out[i, :t.shape[0]] = t
        else:
            out[i, L - t.shape[0]:] = t
    return out, torch.tensor([t.shape[0] for t in tensors])


def unstack(batch: torch.Tensor, lengths: Optional[torch.Tensor] = None, strategy: PaddingStrategy = PaddingStrategy.POST) -> List[torch.Tensor]:
    if lengths is None:
        return list(batch.unbind(0))
    L = batch.shape[1]
    return [batch[i, :int(n)] if strategy == PaddingStrategy.POST else batch[i, L - int(n):] for i, n in enumerate(lengths)]


class DynamicBatcher(Generic[TReq, TResp]):
    def __init__(self, processor: Callable[[List[TReq]], Sequence[TResp]], config: Optional[BatchingConfiguration] = None):
        self.cfg = config or BatchingConfiguration()
        self.cfg.validate()
        self.processor = processor
        self._q: "queue.Queue[Tuple[TReq, Future, float]]" = queue.Queue(self.cfg.max_queue_size)
        self.metrics = BatchingMetrics()
        self._stop = threading.Event()
        self._wait = self.cfg.max_wait_time_s
        self._t = threading.Thread(target=self._loop, daemon=True, name="mlf-batcher")
        self._t.start()

    def submit(self, request: TReq) -> Future:
        if self._stop.is_set():
            raise RuntimeError("batcher is shut down")
        f: Future = Future()
        try:
            self._q.put_nowait((request, f, time.perf_counter()))
        except queue.Full:
            self.metrics.rejected += 1
            raise QueueFullError(f"request queue full ({self.cfg.max_queue_size})")
        return f

    def process(self, request: TReq, timeout: Optional[float] = None) -> TResp:
        return self.submit(request).result(timeout)

    def _collect(self) -> List[Tuple[TReq, Future, float]]:
        cfg = self.cfg
        try:
            first = self._q.get(timeout=0.05)
        except queue.Empty:
            return []
        items = [first]
        deadline = time.perf_counter() + self._wait
        while len(items) < cfg.max_batch_size:
            remaining = deadline - time.perf_counter()
            if cfg.timeout_strategy == TimeoutStrategy.WAIT_FOR_FULL:
                if self._stop.is_set():
                    break
                remaining = 0.01
            elif remaining <= 0:
                break
            elif len(items) >= cfg.prefer_batch_size and self._q.empty():
                break                                            # preferred size reached and nothing queued: go
            try:
                items.append(self._q.get(timeout=remaining))
            except queue.Empty:
                if cfg.timeout_strategy != TimeoutStrategy.WAIT_FOR_FULL:
                    break
        if cfg.timeout_strategy == TimeoutStrategy.ADAPTIVE:
            depth = self._q.qsize()
            if depth > cfg.prefer_batch_size:
                self._wait = max(cfg.max_wait_time_s * 0.1, self._wait * 0.5)
            elif len(items) < cfg.prefer_batch_size:
                self._wait = min(cfg.max_wait_time_s * 4, self._wait * 1.25)
        return items

    def _loop(self):
        while not (self._stop.is_set() and self._q.empty()):
            items = self._collect()
            if not items:
                continue
            t0 = time.perf_counter()
            wait = sum(t0 - t for _, _, t in items) / len(items)
            try:
                out = self.processor([r for r, _, _ in items])
                if len(out) != len(items):
                    raise RuntimeError(f"batch processor returned {len(out)} responses for {len(items)} requests")
                for (_, f, _), o in zip(items, out):       # scatter
                    f.set_result(o)
            except BaseException as e:
                self.metrics.failed_batches += 1
                for _, f, _ in items:
                    if not f.done():
                        f.set_exception(e)
            self.metrics.record(len(items), wait, time.perf_counter() - t0)

    def shutdown(self, timeout: float = 5.0):
        self._stop.set()
        self._t.join(timeout)
