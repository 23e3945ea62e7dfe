"""Data-pipeline pieces around the loader: policies, device-side transforms, stream sharing,
prefetching iterable datasets, loader statistics, pinned host memory.

Reference: src/MLFramework/Data/{ErrorPolicy.cs, DynamicBatchStrategy.cs, InterpolationMode.cs,
IGpuTransform.cs, GpuNormalizeTransform.cs, GpuResizeTransform.cs, StreamReplicator.cs:12-128,
OptimizedIterableDataset.cs:12-149, DataLoaderStatistics.cs, ConsoleErrorLogger.cs,
WorkerPoolFactory.cs} and Data/Memory/{PinningStrategy.cs:9-170, PinnedBuffer.cs:12-186,
PinnedMemoryAllocator.cs:12-242, PinnedMemoryHelper.cs}.

Pinned memory here is page-locked host memory as CUDA sees it (``torch`` pins through the CUDA
runtime), which is what lets a host-to-device copy run asynchronously from a copy stream; with
no GPU the same objects work on pageable memory and say so.
"""
from __future__ import annotations

import enum
import math
import sys
import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "ErrorPolicy", "ErrorPolicyHandler", "DynamicBatchStrategy", "InterpolationMode", "GpuTransform",
    "GpuNormalizeTransform", "GpuResizeTransform", "lanczos_resize", "StreamReplicator", "OptimizedIterableDataset",
    "QueueStatistics", "PrefetchStatistics", "DataLoaderStatistics", "StatisticsTracker", "ConsoleErrorLogger",
    "WorkerPoolFactory", "PinningStrategy", "PinningStrategySelector", "PinnedBuffer", "PinnedMemoryAllocator",
    "pin", "pin_and_copy",
]


# ------------------------------------------------------------------ policies
class ErrorPolicy(enum.Enum):
    FAIL_FAST = "fail_fast"      # the first error ends the epoch
    CONTINUE = "continue"        # record it, skip the item, go on
    RESTART = "restart"          # retry the item (a restarted worker) up to a limit, then fail
    IGNORE = "ignore"            # skip silently


class DynamicBatchStrategy(enum.Enum):
    PAD_TO_MAX = "pad_to_max"    # every batch padded to the longest sequence of the data set
    BUCKET = "bucket"            # sequences grouped by length, padded to the bucket's bound
    DYNAMIC = "dynamic"          # batches filled up to a token budget, padded to their own longest


class ErrorPolicyHandler:
    """Applies an ``ErrorPolicy`` around a per-item function: ``run(fn, item)`` returns ``(ok, value)``."""

    def __init__(self, policy: ErrorPolicy = ErrorPolicy.FAIL_FAST, max_restarts: int = 3, logger: Optional["ConsoleErrorLogger"] = None):
        self.policy, self.max_restarts, self.logger = policy, max_restarts, logger
        self.errors: List[Tuple[Any, BaseException]] = []
        self.skipped = self.restarts = 0

    def run(self, fn: Callable[[Any], Any], item) -> Tuple[bool, Any]:
        attempts = 0
        while True:
            try:
                return True, fn(item)
            except Exception as e:                       # noqa: BLE001 - the policy decides what an error means
                if self.policy is ErrorPolicy.FAIL_FAST:
                    raise
                if self.policy is ErrorPolicy.RESTART and attempts < self.max_restarts:
                    attempts += 1
                    self.restarts += 1
                    continue
                if self.policy is ErrorPolicy.RESTART:
                    raise RuntimeError(f"item failed {attempts + 1} times: {e}") from e
                self.skipped += 1
                if self.policy is ErrorPolicy.CONTINUE:
                    self.errors.append((item, e))
                    if self.logger is not None:
                        self.logger.log_error(f"skipping item after error: {e}", e)
                return False, None

    def map(self, fn: Callable[[Any], Any], items: Iterable) -> Iterator:
        for it in items:
            ok, v = self.run(fn, it)
            if ok:
                yield v


class ConsoleErrorLogger:
    """Timestamped lines on a stream (standard error by default), with counts per level."""

    def __init__(self, stream=None, prefix: str = "data", clock: Callable[[], float] = time.time):
        self._s, self.prefix, self._clock = stream, prefix, clock
        self.counts: Dict[str, int] = {"error": 0, "warning": 0, "info": 0}
        self._lock = threading.Lock()

    def _emit(self, level: str, message: str, error: Optional[BaseException] = None, worker_id: Optional[int] = None):
        stamp = time.strftime("%Y-%m-%d %H:%M:%S", time.gmtime(self._clock()))
        who = f" worker {worker_id}" if worker_id is not None else ""
        tail = f" ({type(error).__name__}: {error})" if error is not None else ""
        with self._lock:
            self.counts[level] += 1
            print(f"[{stamp}] [{self.prefix}{who}] {level.upper()}: {message}{tail}", file=self._s or sys.stderr)

    def log_error(self, message: str, error: Optional[BaseException] = None, worker_id: Optional[int] = None):
        self._emit("error", message, error, worker_id)

    def log_warning(self, message: str, worker_id: Optional[int] = None):
        self._emit("warning", message, None, worker_id)

    def log_info(self, message: str, worker_id: Optional[int] = None):
        self._emit("info", message, None, worker_id)


# ------------------------------------------------------------------ device-side transforms
class InterpolationMode(enum.Enum):
    NEAREST = "nearest"
    BILINEAR = "bilinear"
    BICUBIC = "bicubic"
    LANCZOS = "lanczos"


def _lanczos_matrix(n_in: int, n_out: int, a: int, device, dtype) -> torch.Tensor:
    """[n_out, n_in] resampling weights of the Lanczos-``a`` kernel: widened when shrinking (so that it
    also low-passes), samples beyond the border folded onto the border sample, rows normalised to sum 1."""
    scale = n_in / n_out
    stretch = max(scale, 1.0)
    reach = int(math.ceil(a * stretch)) + 1
    centers = (torch.arange(n_out, device=device, dtype=torch.float64) + 0.5) * scale - 0.5
    ext = torch.arange(-reach, n_in + reach, device=device, dtype=torch.float64)
    x = (ext[None, :] - centers[:, None]) / stretch
    w = torch.where(x.abs() < a, torch.sinc(x) * torch.sinc(x / a), torch.zeros_like(x))
    idx = ext.clamp(0, n_in - 1).long()
    m = torch.zeros(n_out, n_in, device=device, dtype=torch.float64).index_add_(1, idx, w)
    return (m / m.sum(dim=1, keepdim=True)).to(dtype)


def lanczos_resize(x: torch.Tensor, size: Tuple[int, int], a: int = 3) -> torch.Tensor:
    """Separable Lanczos resampling of [..., H, W] to ``size`` = (height, width): two small matrix products."""
    h, w = x.shape[-2:]
    wh = _lanczos_matrix(h, size[0], a, x.device, x.dtype)
    ww = _lanczos_matrix(w, size[1], a, x.device, x.dtype)
    return wh @ x @ ww.transpose(0, 1)


class GpuTransform:
    """A transform that does its arithmetic on a chosen GPU: the input is moved there (asynchronously
    when it is pinned) and the result stays there. Without a GPU it runs where the input is."""

    def __init__(self, device_id: int = 0):
        self._device_id = device_id

    @property
    def gpu_available(self) -> bool:
        return torch.cuda.is_available() and self._device_id < torch.cuda.device_count()

    @property
    def gpu_device(self) -> int:
        return self._device_id

    def set_gpu_device(self, device_id: int) -> None:
        if device_id < 0:
            raise ValueError("the device id cannot be negative")
        self._device_id = device_id

    def _place(self, x: torch.Tensor) -> torch.Tensor:
        if self.gpu_available and (not x.is_cuda or x.device.index != self._device_id):
            return x.to(f"cuda:{self._device_id}", non_blocking=True)
        return x

    def apply(self, x):
        raise NotImplementedError

    def __call__(self, x):
        return self.apply(x)


class GpuNormalizeTransform(GpuTransform):
    """``(x - mean) / std`` per channel of [C, H, W] or [N, C, H, W]."""

    def __init__(self, mean: Sequence[float], std: Sequence[float], device_id: int = 0):
        super().__init__(device_id)
        if len(mean) != len(std) or not len(mean):
            raise ValueError("mean and std need one value per channel")
        if any(s == 0 for s in std):
            raise ValueError("std must be non-zero")
        self.mean, self.std = torch.tensor(mean, dtype=torch.float32), torch.tensor(std, dtype=torch.float32)

    def apply(self, x):
        if not isinstance(x, torch.Tensor):
            raise TypeError(f"expected a tensor, got {type(x).__name__}")
        x = self._place(x)
        if not x.is_floating_point():
            x = x.float()
        c = x.shape[-3] if x.dim() >= 3 else x.shape[0]
        if c != self.mean.numel():
            raise ValueError(f"the input has {c} channels, the transform {self.mean.numel()}")
        shape = (-1, 1, 1) if x.dim() >= 3 else (-1,)
        m, s = self.mean.to(x.device, x.dtype).view(shape), self.std.to(x.device, x.dtype).view(shape)
        return (x - m) / s


class GpuResizeTransform(GpuTransform):
    """Resizes [C, H, W] or [N, C, H, W] to ``height`` x ``width``."""

    def __init__(self, width: int, height: int, mode: InterpolationMode = InterpolationMode.BILINEAR, device_id: int = 0):
        super().__init__(device_id)
        if width <= 0 or height <= 0:
            raise ValueError("width and height must be positive")
        self.width, self.height, self.mode = width, height, mode

    def apply(self, x):
        if not isinstance(x, torch.Tensor) or x.dim() not in (3, 4):
            raise TypeError("expected a [C, H, W] or [N, C, H, W] tensor")
        x = self._place(x)
        if not x.is_floating_point():
            x = x.float()
        if self.mode is InterpolationMode.LANCZOS:
            return lanczos_resize(x, (self.height, self.width))
        batched = x.dim() == 4
        align = False if self.mode in (InterpolationMode.BILINEAR, InterpolationMode.BICUBIC) else None
        y = F.interpolate(x if batched else x[None], size=(self.height, self.width), mode=self.mode.value, align_corners=align)
        return y if batched else y[0]


# ------------------------------------------------------------------ one stream, several readers
class StreamReplicator:
    """Splits one stream among ``num_replicas`` readers: reader ``r`` sees items ``r, r + n, r + 2n, ...``.
    Readers advance independently (each in its own worker thread): items read ahead for the others are
    buffered per reader, at most ``max_buffered`` each, beyond which the fast reader waits."""

    def __init__(self, source: Iterable, num_replicas: int, max_buffered: int = 1024):
        if source is None:
            raise ValueError("the source stream is required")
        if num_replicas <= 0:
            raise ValueError("the number of replicas must be positive")
        self._it, self.num_replicas, self.max_buffered = iter(source), num_replicas, max_buffered
        self._buf: List[Deque] = [deque() for _ in range(num_replicas)]
        self._cv = threading.Condition()
        self._pos = 0
        self._done = False
        self._taken = [False] * num_replicas

    def get_replica_stream(self, replica_id: int) -> Iterator:
        if not 0 <= replica_id < self.num_replicas:
            raise IndexError(f"replica {replica_id} of {self.num_replicas}")
        if self._taken[replica_id]:
            raise RuntimeError(f"replica {replica_id} has already been handed out")
        self._taken[replica_id] = True
        return self._reader(replica_id)

    def _reader(self, r: int) -> Iterator:
        while True:
            with self._cv:
                while not self._buf[r]:
                    if self._done:
                        return
                    target = self._pos % self.num_replicas
                    if target != r and len(self._buf[target]) >= self.max_buffered:
                        self._cv.wait(0.05)                  # let the slow reader drain
                        continue
                    try:
                        item = next(self._it)
                    except StopIteration:
                        self._done = True
                        self._cv.notify_all()
                        return
                    self._buf[target].append(item)
                    self._pos += 1
                item = self._buf[r].popleft()
                self._cv.notify_all()
            yield item


class OptimizedIterableDataset:
    """An iterable data set read by a background thread into a bounded buffer, with an optional
    per-item transform and batch assembly on that thread (OptimizedIterableDataset.cs:12-149)."""

    _END = object()

    def __init__(self, source_factory: Callable[[], Iterable], buffer_size: int = 64, transform: Optional[Callable] = None,
                 batch_size: Optional[int] = None, collate: Optional[Callable[[List], Any]] = None):
        if buffer_size <= 0:
            raise ValueError("the buffer size must be positive")
        if batch_size is not None and batch_size <= 0:
            raise ValueError("the batch size must be positive")
        self._factory, self.buffer_size, self.transform = source_factory, buffer_size, transform
        self.batch_size, self.collate = batch_size, collate or (lambda items: items)
        self.items_read = 0
        self._epoch = 0

    def reset(self) -> None:
        """The next iteration starts the source afresh (it always does; this counts epochs)."""
        self._epoch += 1

    def __iter__(self) -> Iterator:
        buf: Deque = deque()
        cv = threading.Condition()
        state = {"stop": False, "error": None}

        def produce():
            try:
                pending: List = []
                for item in self._factory():
                    if self.transform is not None:
                        item = self.transform(item)
                    self.items_read += 1
                    if self.batch_size is not None:
                        pending.append(item)
                        if len(pending) < self.batch_size:
                            continue
                        item, pending = self.collate(pending), []
                    with cv:
                        while len(buf) >= self.buffer_size and not state["stop"]:
                            cv.wait(0.05)
                        if state["stop"]:
                            return
                        buf.append(item)
                        cv.notify_all()
                if pending:
                    with cv:
                        buf.append(self.collate(pending))
            except BaseException as e:                    # noqa: BLE001 - re-raised on the consumer's thread
                state["error"] = e
            finally:
                with cv:
                    buf.append(self._END)
                    cv.notify_all()

        t = threading.Thread(target=produce, name="mlf-iterable-prefetch", daemon=True)
        t.start()
        try:
            while True:
                with cv:
                    while not buf:
                        cv.wait(0.05)
                    item = buf.popleft()
                    cv.notify_all()
                if item is self._END:
                    if state["error"] is not None:
                        raise state["error"]
                    return
                yield item
        finally:
            with cv:
                state["stop"] = True
                cv.notify_all()
            t.join(timeout=5)


# ------------------------------------------------------------------ loader statistics
@dataclass
class QueueStatistics:
    capacity: int = 0
    average_depth: float = 0.0
    max_depth: int = 0
    producer_waits: int = 0
    consumer_waits: int = 0


@dataclass
class PrefetchStatistics:
    hits: int = 0                   # batches that were ready when asked for
    misses: int = 0                 # the consumer had to wait

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0


@dataclass(frozen=True)
class DataLoaderStatistics:
    batches_loaded: int
    total_samples: int
    average_batch_time_ms: float
    throughput_samples_per_second: float
    queue_statistics: Optional[QueueStatistics] = None
    prefetch_statistics: Optional[PrefetchStatistics] = None

    def __str__(self):
        s = (f"{self.batches_loaded} batches, {self.total_samples} samples, {self.average_batch_time_ms:.2f} ms/batch, "
             f"{self.throughput_samples_per_second:.1f} samples/s")
        if self.prefetch_statistics is not None:
            s += f", prefetch hit rate {self.prefetch_statistics.hit_rate * 100:.0f} %"
        if self.queue_statistics is not None:
            s += f", queue depth {self.queue_statistics.average_depth:.1f}/{self.queue_statistics.capacity}"
        return s


class StatisticsTracker:
    """Wraps any iterable of batches and measures it: ``for batch in tracker.track(loader)``; a batch that
    arrives within ``ready_threshold_ms`` counts as a prefetch hit."""

    def __init__(self, batch_size_of: Optional[Callable[[Any], int]] = None, ready_threshold_ms: float = 1.0,
                 clock: Callable[[], float] = time.perf_counter):
        self._size = batch_size_of or self._guess
        self._thr, self._clock = ready_threshold_ms, clock
        self.batches = self.samples = 0
        self.wait_ms = 0.0
        self.prefetch = PrefetchStatistics()
        self._t_first: Optional[float] = None
        self._t_last: Optional[float] = None

    @staticmethod
    def _guess(batch) -> int:
        if isinstance(batch, torch.Tensor):
            return batch.shape[0] if batch.dim() else 1
        if isinstance(batch, dict):
            return StatisticsTracker._guess(next(iter(batch.values())))
        if isinstance(batch, (tuple, list)) and batch:
            return StatisticsTracker._guess(batch[0]) if isinstance(batch[0], (torch.Tensor, dict, tuple, list)) else len(batch)
        return 1

    def track(self, batches: Iterable) -> Iterator:
        it = iter(batches)
        while True:
            t0 = self._clock()
            self._t_first = t0 if self._t_first is None else self._t_first
            try:
                b = next(it)
            except StopIteration:
                return
            now = self._clock()
            waited = (now - t0) * 1e3
            self.wait_ms += waited
            self.batches += 1
            self.samples += self._size(b)
            if waited <= self._thr:
                self.prefetch.hits += 1
            else:
                self.prefetch.misses += 1
            self._t_last = now
            yield b

    def statistics(self, queue: Optional[QueueStatistics] = None) -> DataLoaderStatistics:
        span = (self._t_last - self._t_first) if self.batches and self._t_last > self._t_first else 0.0
        return DataLoaderStatistics(self.batches, self.samples, self.wait_ms / self.batches if self.batches else 0.0,
                                    self.samples / span if span > 0 else 0.0, queue, self.prefetch)


class WorkerPoolFactory:
    """Worker pools sized for the job (WorkerPoolFactory.cs): by hand, from the CPU count, or for one
    of the usual workloads."""

    @staticmethod
    def create(fn, num_workers: int, **kw):
        from .workers import WorkerPool
        return WorkerPool(fn, num_workers=num_workers, **kw)

    @staticmethod
    def optimal_worker_count(reserve: int = 1, cap: int = 32) -> int:
        import os
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        return max(1, min(cap, n - reserve))

    @classmethod
    def create_for_cpu_bound(cls, fn, **kw):
        return cls.create(fn, cls.optimal_worker_count(), **kw)

    @classmethod
    def create_for_io_bound(cls, fn, **kw):
        return cls.create(fn, min(64, 4 * cls.optimal_worker_count()), **kw)


# ------------------------------------------------------------------ pinned host memory
class PinningStrategy(enum.IntEnum):
    NONE = 0             # too small to matter: pageable memory
    PIN_IN_PLACE = 1     # page-lock the tensor's own storage (the reference's GC-handle pinning)
    ALLOCATE_PINNED = 2  # a fresh page-locked buffer, copy into it
    PINNED_POOL = 3      # a recycled page-locked buffer from a pool


class PinningStrategySelector:
    SMALL_BUFFER_SIZE_THRESHOLD_BYTES = 1024
    LARGE_BUFFER_SIZE_THRESHOLD_BYTES = 1024 * 1024
    HIGH_REUSE_THRESHOLD_COUNT = 10

    @classmethod
    def select_strategy(cls, numel: int, dtype: torch.dtype, expected_reuses: int) -> PinningStrategy:
        if numel <= 0:
            raise ValueError("the buffer size must be greater than zero")
        return cls.select_strategy_by_byte_size(numel * torch.empty((), dtype=dtype).element_size(), expected_reuses)

    @classmethod
    def select_strategy_by_byte_size(cls, byte_size: int, expected_reuses: int) -> PinningStrategy:
        if byte_size <= 0:
            raise ValueError("the byte size must be greater than zero")
        if expected_reuses < 0:
            raise ValueError("the expected number of reuses cannot be negative")
        if byte_size < cls.SMALL_BUFFER_SIZE_THRESHOLD_BYTES:
            return PinningStrategy.NONE
        if expected_reuses >= cls.HIGH_REUSE_THRESHOLD_COUNT:
            return PinningStrategy.PINNED_POOL
        if byte_size >= cls.LARGE_BUFFER_SIZE_THRESHOLD_BYTES:
            return PinningStrategy.ALLOCATE_PINNED
        return PinningStrategy.PIN_IN_PLACE

    @classmethod
    def create_pinned_memory(cls, t: torch.Tensor, strategy: PinningStrategy, pool=None) -> Optional["PinnedBuffer"]:
        if strategy is PinningStrategy.NONE:
            return None
        if strategy is PinningStrategy.PIN_IN_PLACE:
            return pin(t)
        if strategy is PinningStrategy.ALLOCATE_PINNED:
            return pin_and_copy(t)
        if strategy is PinningStrategy.PINNED_POOL:
            if pool is None:
                raise ValueError("the pool strategy needs a pool")
            buf = PinnedBuffer(pool.get(t.shape, t.dtype), pool=pool)
            buf.copy_from(t)
            return buf
        raise ValueError(f"unknown pinning strategy {strategy!r}")


class PinnedBuffer:
    """A host tensor that is page-locked where that is possible, with the copies a staging buffer needs."""

    def __init__(self, tensor: torch.Tensor, pool=None):
        self._t: Optional[torch.Tensor] = tensor
        self._pool = pool

    @classmethod
    def allocate(cls, length: int, dtype: torch.dtype = torch.float32) -> "PinnedBuffer":
        if length <= 0:
            raise ValueError("the length must be positive")
        return cls(torch.empty(length, dtype=dtype, pin_memory=torch.cuda.is_available()))

    def _alive(self) -> torch.Tensor:
        if self._t is None:
            raise RuntimeError("the buffer has been released")
        return self._t

    @property
    def tensor(self) -> torch.Tensor:
        return self._alive()

    @property
    def length(self) -> int:
        return self._alive().numel()

    @property
    def is_pinned(self) -> bool:
        return self._t is not None and self._t.is_pinned()

    @property
    def pointer(self) -> int:
        return self._alive().data_ptr()

    def copy_from(self, source: torch.Tensor, source_offset: int = 0) -> None:
        t = self._alive()
        src = source.reshape(-1)[source_offset:]
        if src.numel() < t.numel():
            raise ValueError(f"the source holds {src.numel()} elements from offset {source_offset}, the buffer {t.numel()}")
        t.view(-1).copy_(src[:t.numel()])

    def copy_to(self, destination: torch.Tensor, destination_offset: int = 0) -> None:
        t = self._alive()
        dst = destination.view(-1)[destination_offset:]
        if dst.numel() < t.numel():
            raise ValueError(f"the destination has room for {dst.numel()} elements, the buffer holds {t.numel()}")
        dst[:t.numel()].copy_(t.view(-1), non_blocking=self.is_pinned)

    def to_device(self, device, stream: Optional["torch.cuda.Stream"] = None) -> torch.Tensor:
        """Host-to-device copy, asynchronous when the buffer is pinned (on ``stream`` when given)."""
        t = self._alive()
        if stream is not None:
            with torch.cuda.stream(stream):
                return t.to(device, non_blocking=self.is_pinned)
        return t.to(device, non_blocking=self.is_pinned)

    def fill(self, value) -> None:
        self._alive().fill_(value)

    def release(self) -> None:
        """Gives the memory back (to its pool when it came from one)."""
        if self._t is not None and self._pool is not None:
            self._pool.put(self._t)
        self._t = None

    unpin = release

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.release()


def pin(t: torch.Tensor) -> PinnedBuffer:
    """Page-locks a CPU tensor (torch makes a pinned copy that shares nothing with ``t``; without a GPU the
    tensor is wrapped as it is)."""
    if t.is_cuda:
        raise ValueError("only host tensors can be pinned")
    return PinnedBuffer(t.pin_memory() if torch.cuda.is_available() else t)


def pin_and_copy(t: torch.Tensor) -> PinnedBuffer:
    buf = PinnedBuffer(torch.empty(t.shape, dtype=t.dtype, pin_memory=torch.cuda.is_available()))
    buf.tensor.copy_(t)
    return buf


class PinnedMemoryAllocator:
    """Hands out page-locked byte buffers and keeps count (PinnedMemoryAllocator.cs:12-242). Falls back to
    pageable memory when pinning is not possible unless ``force_pinned``."""

    def __init__(self, force_pinned: bool = False):
        self.is_pinned_memory_supported = torch.cuda.is_available()
        if force_pinned and not self.is_pinned_memory_supported:
            raise RuntimeError("pinned memory was demanded but no CUDA runtime is available to pin with")
        self._live: Dict[int, PinnedBuffer] = {}
        self._lock = threading.Lock()
        self.total_allocated_bytes = 0

    def allocate(self, size: int) -> PinnedBuffer:
        if size <= 0:
            raise ValueError("the size must be positive")
        buf = PinnedBuffer(torch.empty(size, dtype=torch.uint8, pin_memory=self.is_pinned_memory_supported))
        with self._lock:
            self._live[buf.pointer] = buf
            self.total_allocated_bytes += size
        return buf

    def free(self, buf: PinnedBuffer) -> None:
        with self._lock:
            found = self._live.pop(buf.pointer if buf._t is not None else -1, None)
            if found is None:
                raise KeyError("the buffer does not belong to this allocator (or was freed already)")
            self.total_allocated_bytes -= found.length
        found.release()

    @property
    def live_buffers(self) -> int:
        return len(self._live)

    @staticmethod
    def copy_to_pinned_memory(buf: PinnedBuffer, data: bytes, offset: int = 0, length: Optional[int] = None) -> None:
        n = len(data) - offset if length is None else length
        if offset < 0 or n < 0 or offset + n > len(data) or n > buf.length:
            raise ValueError("offset / length outside the data or larger than the buffer")
        buf.tensor[:n].copy_(torch.frombuffer(bytearray(data[offset:offset + n]), dtype=torch.uint8))

    @staticmethod
    def copy_from_pinned_memory(buf: PinnedBuffer, length: int, offset: int = 0) -> bytes:
        if offset < 0 or length < 0 or offset + length > buf.length:
            raise ValueError("offset / length outside the buffer")
        return bytes(buf.tensor[offset:offset + length].tolist())

    def dispose(self) -> None:
        with self._lock:
            live, self._live = list(self._live.values()), {}
            self.total_allocated_bytes = 0
        for b in live:
            b.release()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()
