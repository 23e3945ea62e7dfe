"""Datasets, collation, multi-worker data loader with prefetch into pinned memory.

Reference: src/MLFramework/Data/DataLoader.cs, AdvancedDataLoader.cs, DataLoaderConfig.cs (presets +
builder), datasets (map-style / iterable / array / list / in-memory), Collate/*, WorkerPool.cs with crash
detection / recovery / timeouts / error aggregation (WorkerCrashDetector.cs, WorkerRecoveryService.cs,
WorkerTimeoutTracker.cs, ErrorAggregator.cs), SharedQueue.cs, SimplePrefetchStrategy.cs, pinned-memory
pool (Data/Memory/Pinned*.cs), and the pools project (src/Data/*.cs: ArrayPool, TensorPool, PrefetchBuffer).

Design: worker *threads* produce collated CPU batches into a bounded queue (tensor collation and file
reads release the GIL); the consumer side copies each batch into a recycled pinned staging buffer and
issues the host-to-device copy on a side stream one batch ahead, so the training stream never waits for
PCIe. A worker that raises is restarted up to ``max_worker_restarts`` times; its batch is retried;
errors are aggregated and surface when the limit is exceeded. A batch that takes longer than
``worker_timeout_s`` raises ``TimeoutError``.
"""
from __future__ import annotations

import queue
import threading
import time
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .samplers import BatchSampler, RandomSampler, SequentialSampler


# ------------------------------------------------------------------ datasets
class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, i: int):
        raise NotImplementedError


class IterableDataset:
    def __iter__(self):
        raise NotImplementedError


class TensorDataset(Dataset):
    def __init__(self, *tensors: torch.Tensor):
        if not tensors or any(t.shape[0] != tensors[0].shape[0] for t in tensors):
            raise ValueError("tensors must share their first dimension")
        self.tensors = tensors

    def __len__(self):
        return self.tensors[0].shape[0]

    def __getitem__(self, i):
        return tuple(t[i] for t in self.tensors)


class ListDataset(Dataset):
    def __init__(self, items: Sequence[Any]):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


class SyntheticTokenDataset(Dataset):
    """Uniform random token ids of a fixed sequence length (the benchmark's data), generated per index
    from a counter-based seed so every rank and every epoch can reproduce item ``i``."""

    def __init__(self, n_items: int, seq_len: int, vocab: int, seed: int = 0):
        self.n, self.seq_len, self.vocab, self.seed = n_items, seq_len, vocab, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        t = torch.randint(0, self.vocab, (self.seq_len + 1,), generator=g)
        return t[:-1], t[1:]


class ArrayDataset(Dataset):
    """Row ``i`` of one or several NumPy arrays (shared first dimension), as tensors that alias the arrays."""

    def __init__(self, *arrays):
        import numpy as np
        self.arrays = [np.ascontiguousarray(a) for a in arrays]
        if not self.arrays or any(a.shape[0] != self.arrays[0].shape[0] for a in self.arrays):
            raise ValueError("arrays must share their first dimension")

    def __len__(self):
        return self.arrays[0].shape[0]

    def __getitem__(self, i):
        out = tuple(torch.from_numpy(a[i]) if a[i].ndim else torch.tensor(a[i]) for a in self.arrays)
        return out if len(out) > 1 else out[0]


class InMemoryDataset(Dataset):
    """Materialises another dataset (map-style or iterable) once, optionally through ``transform``; later epochs read
    the cached items."""

    def __init__(self, source, transform: Optional[Callable[[Any], Any]] = None, limit: Optional[int] = None):
        it = (source[i] for i in range(len(source))) if hasattr(source, "__getitem__") and hasattr(source, "__len__") else iter(source)
        self.items = []
        for k, x in enumerate(it):
            if limit is not None and k >= limit:
                break
            self.items.append(transform(x) if transform is not None else x)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


# ------------------------------------------------------------------ collate
def stack_collate(items: Sequence[torch.Tensor]) -> torch.Tensor:
    """Tensors of one shape stacked along a new first dimension; anything else is an error (no silent lists)."""
    if not items or not all(isinstance(t, torch.Tensor) for t in items):
        raise TypeError("stack_collate takes tensors")
    if any(t.shape != items[0].shape for t in items):
        raise ValueError(f"shapes differ: {sorted({tuple(t.shape) for t in items})}")
    return torch.stack(list(items), 0)


def dict_collate(items: Sequence[Dict[str, Any]], per_key: Optional[Dict[str, Callable]] = None) -> Dict[str, Any]:
    """Dictionaries with the same keys, collated key by key (``per_key`` overrides the default for a key)."""
    keys = list(items[0])
    if any(list(it) != keys for it in items):
        raise KeyError("samples disagree on their keys")
    per_key = per_key or {}
    return {k: per_key.get(k, default_collate)([it[k] for it in items]) for k in keys}


def default_collate(items: Sequence[Any]):
    x = items[0]
    if isinstance(x, torch.Tensor):
        return torch.stack(list(items), 0)
    if isinstance(x, (int, float)):
        return torch.tensor(list(items))
    if isinstance(x, (tuple, list)):
        return type(x)(default_collate([it[k] for it in items]) for k in range(len(x)))
    if isinstance(x, dict):
        return {k: default_collate([it[k] for it in items]) for k in x}
    return list(items)


def pad_collate(pad_value: int = 0, multiple_of: int = 8):
    """Pads 1-D sequences to the batch maximum rounded up to ``multiple_of`` (8 keeps bf16 rows 16-byte aligned)."""
    def fn(items: Sequence[torch.Tensor]):
        L = max(t.shape[0] for t in items)
        L = (L + multiple_of - 1) // multiple_of * multiple_of
        out = torch.full((len(items), L), pad_value, dtype=items[0].dtype)
        lens = torch.tensor([t.shape[0] for t in items])
        for i, t in enumerate(items):
            out[i, :t.shape[0]] = t
        return out, lens
    return fn


# ------------------------------------------------------------------ pinned staging
class PinnedMemoryPool:
    """Recycles pinned host buffers by (shape, dtype); pinning is expensive, reuse is free."""

    def __init__(self, max_per_key: int = 4):
        self._free: Dict[Tuple, List[torch.Tensor]] = defaultdict(list)
        self.max_per_key = max_per_key
        self._lock = threading.Lock()
        self.allocations = self.reuses = 0
        self._pin = torch.cuda.is_available()

    def get(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        with self._lock:
            if self._free[key]:
                self.reuses += 1
                return self._free[key].pop()
            self.allocations += 1
        return torch.empty(shape, dtype=dtype, pin_memory=self._pin)

    def put(self, t: torch.Tensor):
        key = (tuple(t.shape), t.dtype)
        with self._lock:
            if len(self._free[key]) < self.max_per_key:
                self._free[key].append(t)


def _map_tensors(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (tuple, list)):
        return type(obj)(_map_tensors(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    return obj


# ------------------------------------------------------------------ errors
@dataclass
class WorkerError:
    worker_id: int
    batch_index: int
    error: BaseException
    time: float = field(default_factory=time.time)


class ErrorAggregator:
    def __init__(self):
        self.errors: List[WorkerError] = []
        self._lock = threading.Lock()

    def add(self, e: WorkerError):
        with self._lock:
            self.errors.append(e)

    def summary(self) -> str:
        by = defaultdict(int)
        for e in self.errors:
            by[type(e.error).__name__] += 1
        return ", ".join(f"{k} x{v}" for k, v in by.items()) or "no errors"


class DataLoaderError(RuntimeError):
    pass


# ------------------------------------------------------------------ config
@dataclass
class DataLoaderConfig:
    batch_size: int = 1
    shuffle: bool = False
    drop_last: bool = False
    num_workers: int = 0
    prefetch_batches: int = 2
    pin_memory: bool = True
    device: Optional[str] = None           # e.g. "cuda:0": batches arrive on the device
    worker_timeout_s: float = 60.0
    max_worker_restarts: int = 3
    seed: int = 0

    def validate(self):
        if self.batch_size <= 0 or self.num_workers < 0 or self.prefetch_batches <= 0:
            raise ValueError("batch_size > 0, num_workers >= 0 and prefetch_batches > 0 required")

    @staticmethod
    def for_cpu_bound(workers: int = 8):
        return DataLoaderConfig(num_workers=workers, prefetch_batches=4)

    @staticmethod
    def for_gpu_training(batch_size: int, device: str = "cuda:0"):
        return DataLoaderConfig(batch_size=batch_size, shuffle=True, drop_last=True, num_workers=4, prefetch_batches=3, device=device)

    @staticmethod
    def for_debugging():
        return DataLoaderConfig(num_workers=0, prefetch_batches=1, pin_memory=False)


class DataLoaderConfigBuilder:
    def __init__(self):
        self._c = DataLoaderConfig()

    def batch_size(self, n): self._c.batch_size = n; return self
    def shuffle(self, b=True): self._c.shuffle = b; return self
    def workers(self, n): self._c.num_workers = n; return self
    def prefetch(self, n): self._c.prefetch_batches = n; return self
    def device(self, d): self._c.device = d; return self
    def drop_last(self, b=True): self._c.drop_last = b; return self

    def build(self):
        self._c.validate()
        return self._c


# ------------------------------------------------------------------ loader
class DataLoader:
    def __init__(self, dataset, config: Optional[DataLoaderConfig] = None, sampler=None, batch_sampler=None,
                 collate_fn: Callable = default_collate, transform: Optional[Callable] = None, **kw):
        self.ds = dataset
        self.cfg = config or DataLoaderConfig(**kw)
        self.cfg.validate()
        self.collate, self.transform = collate_fn, transform
        self.iterable = not hasattr(dataset, "__getitem__")
        if not self.iterable:
            if batch_sampler is None:
                if sampler is None:
                    sampler = RandomSampler(len(dataset), seed=self.cfg.seed) if self.cfg.shuffle else SequentialSampler(len(dataset))
                batch_sampler = BatchSampler(sampler, self.cfg.batch_size, self.cfg.drop_last)
        self.batch_sampler = batch_sampler
        self.errors = ErrorAggregator()
        self.pool = PinnedMemoryPool()
        self.worker_restarts = 0
        self.batches_served = 0
        self.wait_seconds = 0.0

    def __len__(self):
        return len(self.batch_sampler)

    def set_epoch(self, epoch: int):
        s = getattr(self.batch_sampler, "sampler", None)
        if hasattr(s, "set_epoch"):
            s.set_epoch(epoch)

    # ---- batch production
    def _make(self, indices: Sequence[int]):
        items = [self.ds[i] for i in indices]
        if self.transform is not None:
            items = [self.transform(it) for it in items]
        return self.collate(items)

    def _iter_batches_sync(self) -> Iterator[Any]:
        if self.iterable:
            buf = []
            for it in self.ds:
                buf.append(self.transform(it) if self.transform else it)
                if len(buf) == self.cfg.batch_size:
                    yield self.collate(buf)
                    buf = []
            if buf and not self.cfg.drop_last:
                yield self.collate(buf)
        else:
            for idx in self.batch_sampler:
                yield self._make(idx)

    def _iter_batches_workers(self) -> Iterator[Any]:
        cfg = self.cfg
        plan = list(self.batch_sampler)
        tasks: "queue.Queue[Optional[Tuple[int, Sequence[int]]]]" = queue.Queue()
        for i, idx in enumerate(plan):
            tasks.put((i, idx))
        results: Dict[int, Any] = {}
        cond = threading.Condition()
        stop = threading.Event()
        window = cfg.prefetch_batches + cfg.num_workers
        next_needed = [0]

        def worker(wid: int):
            while not stop.is_set():
                with cond:                                     # do not run further ahead than the window
                    while not stop.is_set() and tasks.qsize() and tasks.queue[0][0] >= next_needed[0] + window:
                        cond.wait(0.05)
                try:
                    task = tasks.get_nowait()
                except queue.Empty:
                    return
                i, idx = task
                attempts = 0
                while True:
                    try:
                        out = self._make(idx)
                        break
                    except BaseException as e:                 # worker "crash": record, restart, retry the batch
                        self.errors.add(WorkerError(wid, i, e))
                        attempts += 1
                        with cond:
                            self.worker_restarts += 1
                            over = self.worker_restarts > cfg.max_worker_restarts
                        if over:
                            out = DataLoaderError(f"batch {i} failed after {attempts} attempts; errors: {self.errors.summary()}")
                            out.__cause__ = e
                            break
                with cond:
                    results[i] = out
                    cond.notify_all()

        threads = [threading.Thread(target=worker, args=(w,), daemon=True, name=f"mlf-data-{w}") for w in range(cfg.num_workers)]
        for t in threads:
            t.start()
        try:
            for i in range(len(plan)):
                t0 = time.perf_counter()
                with cond:
                    next_needed[0] = i
                    cond.notify_all()
                    while i not in results:
                        if not cond.wait(cfg.worker_timeout_s):
                            raise TimeoutError(f"batch {i} not produced within {cfg.worker_timeout_s} s")
                    out = results.pop(i)
                self.wait_seconds += time.perf_counter() - t0
                if isinstance(out, BaseException):
                    raise out
                yield out
        finally:
            stop.set()
            with cond:
                cond.notify_all()
            for t in threads:
                t.join(timeout=1.0)

    # ---- device staging: copy batch k+1 while batch k is consumed
    def _stage(self, batch, stream):
        pinned = []

        def to_dev(t: torch.Tensor):
            if self.cfg.pin_memory and not t.is_pinned():
                p = self.pool.get(t.shape, t.dtype)
                p.copy_(t)
                pinned.append(p)
                t = p
            return t.to(self.cfg.device, non_blocking=True)
        with torch.cuda.stream(stream):
            out = _map_tensors(batch, to_dev)
            ev = torch.cuda.Event()
            ev.record(stream)
        return out, ev, pinned

    def __iter__(self):
        src = self._iter_batches_workers() if (self.cfg.num_workers > 0 and not self.iterable) else self._iter_batches_sync()
        on_device = self.cfg.device is not None and str(self.cfg.device).startswith("cuda") and torch.cuda.is_available()
        if not on_device:
            for b in src:
                self.batches_served += 1
                yield b if self.cfg.device is None else _map_tensors(b, lambda t: t.to(self.cfg.device))
            return
        stream = torch.cuda.Stream(self.cfg.device)
        pending = None
        for b in src:
            staged = self._stage(b, stream)
            if pending is not None:
                out, ev, pinned = pending
                torch.cuda.current_stream().wait_event(ev)
                self.batches_served += 1
                yield out
                ev.synchronize()
                for p in pinned:
                    self.pool.put(p)
            pending = staged
        if pending is not None:
            out, ev, pinned = pending
            torch.cuda.current_stream().wait_event(ev)
            self.batches_served += 1
            yield out
            ev.synchronize()
            for p in pinned:
                self.pool.put(p)

    def metrics(self) -> Dict[str, float]:
        return {"batches": self.batches_served, "wait_seconds": self.wait_seconds, "worker_restarts": self.worker_restarts,
                "errors": len(self.errors.errors), "pinned_allocations": self.pool.allocations, "pinned_reuses": self.pool.reuses}


class AdvancedDataLoader(DataLoader):
    """The same loader for ``async`` programs: ``async for batch in loader`` and ``await loader.next_batch_async()``
    hand the blocking wait for the next batch to a helper thread, so an event loop that also serves requests keeps
    running while workers fill the queue (reference: src/MLFramework/Data/AdvancedDataLoader.cs, async enumerators)."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self._it: Optional[Iterator[Any]] = None
        self._done = object()

    def reset(self):
        self._it = None

    def _next_blocking(self):
        if self._it is None:
            self._it = iter(self)
        try:
            return next(self._it)
        except StopIteration:
            self._it = None
            return self._done

    async def next_batch_async(self):
        """The next batch, or ``None`` at the end of the epoch (the following call starts the next epoch)."""
        import asyncio
        b = await asyncio.get_running_loop().run_in_executor(None, self._next_blocking)
        return None if b is self._done else b

    def __aiter__(self):
        self._it = None
        return self

    async def __anext__(self):
        b = await self.next_batch_async()
        if b is None:
            raise StopAsyncIteration
        return b
