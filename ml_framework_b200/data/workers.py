"""Building blocks of the input pipeline as parts of their own: queues, prefetch, worker pool, supervision, pools.

The loader in :mod:`ml_framework_b200.data.loader` has its worker handling built in; these are the reference's separate
components for programs that assemble their own pipeline:

* ``SharedQueue`` - bounded multi-producer / multi-consumer queue with time-outs, batch operations, completion and
  statistics (src/MLFramework/Data/SharedQueue.cs:33-336, src/Data/SharedQueue.cs);
* ``PrefetchBuffer`` / ``SimplePrefetchStrategy`` - keeps N items pulled ahead of the consumer
  (Data/SimplePrefetchStrategy.cs:32-349, src/Data/PrefetchBuffer.cs);
* ``WorkerPool`` - worker threads that apply a function to submitted tasks, results in submission order or as they
  finish, with per-worker context (Data/WorkerPool.cs, Data/Worker/{WorkerPool,OptimizedWorkerPool,WorkerContext}.cs);
* ``WorkerCrashDetector`` (heartbeats and dead threads), ``WorkerRecoveryService`` (bounded restarts with back-off),
  ``WorkerTimeoutTracker`` (operations that run too long) (WorkerCrashDetector.cs, WorkerRecoveryService.cs,
  WorkerTimeoutTracker.cs);
* ``ObjectPool`` / ``ArrayPool`` / ``TensorPool`` / ``PoolManager`` with statistics (src/Data/{ObjectPool,ArrayPool,
  TensorPool,PoolManager,PoolStatistics}.cs).

Threads, not processes: tensor collation, decoding and file reads release the interpreter lock, and a thread's
output needs no serialisation on its way to the pinned staging buffers.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, Generic, Iterable, Iterator, List, Optional, Tuple, TypeVar

import numpy as np
import torch

T = TypeVar("T")


class QueueClosed(RuntimeError):
    """Raised by a blocking ``dequeue`` once the queue is complete and empty, and by ``enqueue`` after completion."""


@dataclass
class QueueStatistics:
    enqueued: int = 0
    dequeued: int = 0
    max_size: int = 0
    producer_wait_s: float = 0.0
    consumer_wait_s: float = 0.0
    capacity: int = 0
    size: int = 0

    @property
    def average_producer_wait_ms(self) -> float:
        return 1e3 * self.producer_wait_s / self.enqueued if self.enqueued else 0.0

    @property
    def average_consumer_wait_ms(self) -> float:
        return 1e3 * self.consumer_wait_s / self.dequeued if self.dequeued else 0.0


class SharedQueue(Generic[T]):
    def __init__(self, capacity: int, enable_statistics: bool = True):
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.capacity = capacity
        self._q: Deque[T] = deque()
        self._lock = threading.Lock()
        self._not_full = threading.Condition(self._lock)
        self._not_empty = threading.Condition(self._lock)
        self._complete = False
        self._shutdown = False
        self._stats = QueueStatistics(capacity=capacity) if enable_statistics else None

    def __len__(self) -> int:
        with self._lock:
            return len(self._q)

    @property
    def is_completed(self) -> bool:
        with self._lock:
            return self._complete and not self._q

    def _put(self, item: T, timeout: Optional[float]) -> bool:
        t0 = time.perf_counter()
        with self._not_full:
            if self._complete:
                raise QueueClosed("queue is complete: no more items accepted")
            end = None if timeout is None else t0 + timeout
            while len(self._q) >= self.capacity:
                if self._complete:
                    raise QueueClosed("queue was completed while waiting for room")
                rest = None if end is None else end - time.perf_counter()
                if rest is not None and rest <= 0:
                    return False
                self._not_full.wait(rest)
            self._q.append(item)
            if self._stats is not None:
                self._stats.enqueued += 1
                self._stats.max_size = max(self._stats.max_size, len(self._q))
                self._stats.producer_wait_s += time.perf_counter() - t0
            self._not_empty.notify()
            return True

    def enqueue(self, item: T):
        self._put(item, None)

    def try_enqueue(self, item: T, timeout_ms: int = 0) -> bool:
        return self._put(item, timeout_ms / 1e3)

    def _get(self, timeout: Optional[float]) -> Tuple[bool, Optional[T]]:
        t0 = time.perf_counter()
        with self._not_empty:
            end = None if timeout is None else t0 + timeout
            while not self._q:
                if self._complete:
                    if timeout is None:
                        raise QueueClosed("queue is complete and empty")
                    return False, None
                rest = None if end is None else end - time.perf_counter()
                if rest is not None and rest <= 0:
                    return False, None
                self._not_empty.wait(rest)
            item = self._q.popleft()
            if self._stats is not None:
                self._stats.dequeued += 1
                self._stats.consumer_wait_s += time.perf_counter() - t0
            self._not_full.notify()
            return True, item

    def dequeue(self) -> T:
        return self._get(None)[1]

    def try_dequeue(self, timeout_ms: int = 0) -> Tuple[bool, Optional[T]]:
        return self._get(timeout_ms / 1e3)

    def try_peek(self) -> Tuple[bool, Optional[T]]:
        with self._lock:
            return (True, self._q[0]) if self._q else (False, None)

    def enqueue_batch(self, items: Iterable[T]):
        for it in items:
            self.enqueue(it)

    def dequeue_batch(self, batch_size: int, timeout_ms: int) -> List[T]:
        """Up to ``batch_size`` items; waits at most ``timeout_ms`` in total and returns what it has by then."""
        out: List[T] = []
        end = time.perf_counter() + timeout_ms / 1e3
        while len(out) < batch_size:
            ok, it = self._get(max(0.0, end - time.perf_counter()))
            if not ok:
                break
            out.append(it)
        return out

    def complete_adding(self):
        with self._lock:
            self._complete = True
            self._not_empty.notify_all()
            self._not_full.notify_all()

    def wait_for_completion(self, timeout: Optional[float] = None) -> bool:
        """Blocks until the queue is complete AND drained."""
        end = None if timeout is None else time.perf_counter() + timeout
        with self._not_full:
            while not (self._complete and not self._q):
                rest = None if end is None else end - time.perf_counter()
                if rest is not None and rest <= 0:
                    return False
                self._not_full.wait(0.05 if rest is None else min(rest, 0.05))
            return True

    def shutdown(self):
        """Completes the queue and discards what is in it."""
        with self._lock:
            self._complete = self._shutdown = True
            self._q.clear()
            self._not_empty.notify_all()
            self._not_full.notify_all()

    def statistics(self) -> QueueStatistics:
        with self._lock:
            if self._stats is None:
                return QueueStatistics(capacity=self.capacity, size=len(self._q))
            s = QueueStatistics(**{**self._stats.__dict__})
            s.size = len(self._q)
            return s

    def __iter__(self) -> Iterator[T]:
        while True:
            try:
                yield self.dequeue()
            except QueueClosed:
                return

    def __repr__(self):
        s = self.statistics()
        return f"SharedQueue(size={s.size}/{self.capacity}, in={s.enqueued}, out={s.dequeued}, complete={self._complete})"


# ------------------------------------------------------------------ prefetch
@dataclass
class PrefetchStatistics:
    requests: int = 0
    hits: int = 0             # served from the buffer without waiting for the source
    misses: int = 0
    prefetched: int = 0

    @property
    def hit_rate(self) -> float:
        return self.hits / self.requests if self.requests else 0.0


class PrefetchBuffer(Generic[T]):
    def __init__(self, capacity: int):
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.capacity = capacity
        self._d: Deque[T] = deque()

    def __len__(self):
        return len(self._d)

    @property
    def is_full(self) -> bool:
        return len(self._d) >= self.capacity

    def add(self, item: T):
        if self.is_full:
            raise OverflowError("prefetch buffer is full")
        self._d.append(item)

    def get_next(self) -> T:
        if not self._d:
            raise IndexError("prefetch buffer is empty")
        return self._d.popleft()

    def try_get(self) -> Tuple[bool, Optional[T]]:
        return (True, self._d.popleft()) if self._d else (False, None)

    def peek(self) -> T:
        if not self._d:
            raise IndexError("prefetch buffer is empty")
        return self._d[0]

    def try_peek(self) -> Tuple[bool, Optional[T]]:
        return (True, self._d[0]) if self._d else (False, None)

    def clear(self):
        self._d.clear()

    def __repr__(self):
        return f"PrefetchBuffer({len(self._d)}/{self.capacity})"


class SimplePrefetchStrategy(Generic[T]):
    """Keeps up to ``prefetch_count`` items from ``source`` in a local buffer, topped up without blocking after every
    ``get_next``; ``get_next`` only waits on the source when the buffer is empty."""

    def __init__(self, source: SharedQueue, prefetch_count: int):
        self.source, self.buffer = source, PrefetchBuffer(prefetch_count)
        self._stats = PrefetchStatistics()
        self._lock = threading.Lock()

    def prefetch(self, count: Optional[int] = None) -> int:
        n = 0
        with self._lock:
            want = self.buffer.capacity - len(self.buffer) if count is None else min(count, self.buffer.capacity - len(self.buffer))
            while n < want:
                ok, it = self.source.try_dequeue(0)
                if not ok:
                    break
                self.buffer.add(it)
                n += 1
            self._stats.prefetched += n
        return n

    def get_next(self, timeout_ms: Optional[int] = None) -> T:
        with self._lock:
            self._stats.requests += 1
            ok, it = self.buffer.try_get()
            if ok:
                self._stats.hits += 1
        if not ok:
            with self._lock:
                self._stats.misses += 1
            if timeout_ms is None:
                it = self.source.dequeue()
            else:
                ok, it = self.source.try_dequeue(timeout_ms)
                if not ok:
                    raise TimeoutError(f"no item within {timeout_ms} ms")
        self.prefetch()
        return it

    def reset(self):
        with self._lock:
            self.buffer.clear()
            self._stats = PrefetchStatistics()

    def statistics(self) -> PrefetchStatistics:
        with self._lock:
            return PrefetchStatistics(**self._stats.__dict__)


# ------------------------------------------------------------------ supervision
class WorkerCrashDetector:
    """A worker is reported crashed when its thread ended without unregistering, or when it sent no heartbeat for
    ``heartbeat_timeout_s``. ``on_crash(worker_id, reason)`` runs on the monitor thread, once per crash."""

    def __init__(self, heartbeat_timeout_s: float = 30.0, check_interval_s: float = 1.0):
        self.heartbeat_timeout_s, self.check_interval_s = heartbeat_timeout_s, check_interval_s
        self._w: Dict[int, Tuple[Optional[threading.Thread], float]] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None
        self.on_crash: List[Callable[[int, str], None]] = []
        self.crashes: List[Tuple[int, str]] = []

    def register_worker(self, worker_id: int, thread: Optional[threading.Thread] = None):
        with self._lock:
            self._w[worker_id] = (thread, time.monotonic())

    def unregister_worker(self, worker_id: int):
        with self._lock:
            self._w.pop(worker_id, None)

    def update_heartbeat(self, worker_id: int):
        with self._lock:
            if worker_id in self._w:
                self._w[worker_id] = (self._w[worker_id][0], time.monotonic())

    def registered_worker_count(self) -> int:
        with self._lock:
            return len(self._w)

    def time_since_last_heartbeat(self, worker_id: int) -> Optional[float]:
        with self._lock:
            e = self._w.get(worker_id)
            return None if e is None else time.monotonic() - e[1]

    def check_now(self) -> List[Tuple[int, str]]:
        now, found = time.monotonic(), []
        with self._lock:
            for wid, (th, beat) in list(self._w.items()):
                if th is not None and th.ident is not None and not th.is_alive():
                    found.append((wid, "thread ended"))
                elif now - beat > self.heartbeat_timeout_s:
                    found.append((wid, f"no heartbeat for {now - beat:.1f} s"))
            for wid, _ in found:
                del self._w[wid]
        for wid, why in found:
            self.crashes.append((wid, why))
            for cb in self.on_crash:
                cb(wid, why)
        return found

    def start_monitoring(self):
        if self._t is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.wait(self.check_interval_s):
                self.check_now()
        self._t = threading.Thread(target=loop, daemon=True, name="mlf-crash-detector")
        self._t.start()

    def stop_monitoring(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2.0)
            self._t = None


class WorkerRecoveryService:
    """Bounded restarts per worker. ``try_restart(worker_id, start_fn)`` waits ``restart_delay_s * backoff**(n-1)``
    before the n-th retry, calls ``start_fn(worker_id)``, and marks the worker failed for good once its retries are
    used up or ``start_fn`` itself raises on the last one."""

    def __init__(self, max_retries: int = 3, restart_delay_s: float = 0.0, backoff: float = 2.0, sleep: Callable[[float], None] = time.sleep):
        if max_retries < 0:
            raise ValueError("max_retries must be non-negative")
        self.max_retries, self.restart_delay_s, self.backoff, self._sleep = max_retries, restart_delay_s, backoff, sleep
        self._retries: Dict[int, int] = {}
        self._failed: set = set()
        self._lock = threading.Lock()
        self.history: List[Tuple[int, int, bool, str]] = []      # worker, attempt, ok, message

    def can_restart(self, worker_id: int) -> bool:
        with self._lock:
            return worker_id not in self._failed and self._retries.get(worker_id, 0) < self.max_retries

    def try_restart(self, worker_id: int, start_fn: Callable[[int], None]) -> bool:
        with self._lock:
            if worker_id in self._failed:
                return False
            n = self._retries.get(worker_id, 0)
            if n >= self.max_retries:
                self._failed.add(worker_id)
                self.history.append((worker_id, n, False, "retries exhausted"))
                return False
            self._retries[worker_id] = n = n + 1
        delay = self.restart_delay_s * self.backoff ** (n - 1)
        if delay > 0:
            self._sleep(delay)
        try:
            start_fn(worker_id)
        except Exception as e:           # noqa: BLE001 - a failed restart is recorded, the caller decides what next
            with self._lock:
                self.history.append((worker_id, n, False, str(e)))
                if n >= self.max_retries:
                    self._failed.add(worker_id)
            return False
        with self._lock:
            self.history.append((worker_id, n, True, ""))
        return True

    def mark_worker_failed(self, worker_id: int):
        with self._lock:
            self._failed.add(worker_id)

    def retry_count(self, worker_id: int) -> int:
        with self._lock:
            return self._retries.get(worker_id, 0)

    def remaining_retries(self, worker_id: int) -> int:
        with self._lock:
            return 0 if worker_id in self._failed else max(0, self.max_retries - self._retries.get(worker_id, 0))

    def is_worker_failed(self, worker_id: int) -> bool:
        with self._lock:
            return worker_id in self._failed

    def failed_workers(self) -> List[int]:
        with self._lock:
            return sorted(self._failed)

    def failed_worker_count(self) -> int:
        return len(self.failed_workers())

    def reset_worker(self, worker_id: int):
        with self._lock:
            self._retries.pop(worker_id, None)
            self._failed.discard(worker_id)

    def reset_all(self):
        with self._lock:
            self._retries.clear()
            self._failed.clear()

    def recovery_summary(self) -> str:
        with self._lock:
            ok = sum(1 for h in self.history if h[2])
            return (f"{len(self._retries)} workers restarted ({ok} successful restarts, {len(self.history) - ok} failed attempts), "
                    f"{len(self._failed)} failed for good: {sorted(self._failed)}")


class WorkerTimeoutTracker:
    """Start / end marks per worker operation; an operation that runs longer than ``timeout_s`` is reported once
    through ``on_timeout(worker_id, elapsed_s)``."""

    def __init__(self, timeout_s: float = 60.0, check_interval_s: float = 1.0):
        self.timeout_s, self.check_interval_s = timeout_s, check_interval_s
        self._start: Dict[int, float] = {}
        self._reported: set = set()
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None
        self.on_timeout: List[Callable[[int, float], None]] = []

    def start_operation(self, worker_id: int):
        with self._lock:
            self._start[worker_id] = time.monotonic()
            self._reported.discard(worker_id)

    def end_operation(self, worker_id: int) -> Optional[float]:
        with self._lock:
            t0 = self._start.pop(worker_id, None)
            self._reported.discard(worker_id)
            return None if t0 is None else time.monotonic() - t0

    def elapsed(self, worker_id: int) -> Optional[float]:
        with self._lock:
            t0 = self._start.get(worker_id)
            return None if t0 is None else time.monotonic() - t0

    def active_worker_count(self) -> int:
        with self._lock:
            return len(self._start)

    def is_tracking(self, worker_id: int) -> bool:
        with self._lock:
            return worker_id in self._start

    def check_now(self) -> List[Tuple[int, float]]:
        now, late = time.monotonic(), []
        with self._lock:
            for wid, t0 in self._start.items():
                if now - t0 > self.timeout_s and wid not in self._reported:
                    self._reported.add(wid)
                    late.append((wid, now - t0))
        for wid, el in late:
            for cb in self.on_timeout:
                cb(wid, el)
        return late

    def start_monitoring(self):
        if self._t is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.wait(self.check_interval_s):
                self.check_now()
        self._t = threading.Thread(target=loop, daemon=True, name="mlf-timeout-tracker")
        self._t.start()

    def stop_monitoring(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2.0)
            self._t = None

    def clear_all(self):
        with self._lock:
            self._start.clear()
            self._reported.clear()

    def tracking_summary(self) -> str:
        with self._lock:
            now = time.monotonic()
            parts = [f"worker {w}: {now - t:.2f} s" for w, t in sorted(self._start.items())]
        return f"{len(parts)} operations in flight" + (": " + ", ".join(parts) if parts else "")


# ------------------------------------------------------------------ worker pool
@dataclass
class WorkerContext:
    worker_id: int
    num_workers: int
    seed: int
    state: Dict[str, Any] = field(default_factory=dict)


class WorkerPool:
    """``num_workers`` threads apply ``fn(task, context)`` to submitted tasks. ``results()`` yields results in
    submission order (``ordered=True``) or as they finish. A task whose function raises is retried on a restarted
    worker while the recovery service allows; afterwards the error is delivered in place of the result and raised by
    ``results()``."""

    def __init__(self, fn: Callable[[Any, WorkerContext], Any], num_workers: int = 4, queue_capacity: int = 64, seed: int = 0,
                 init_fn: Optional[Callable[[WorkerContext], None]] = None, recovery: Optional[WorkerRecoveryService] = None,
                 crash_detector: Optional[WorkerCrashDetector] = None, timeouts: Optional[WorkerTimeoutTracker] = None):
        if num_workers <= 0:
            raise ValueError("num_workers must be positive")
        self.fn, self.num_workers, self.seed, self.init_fn = fn, num_workers, seed, init_fn
        self.tasks: SharedQueue = SharedQueue(queue_capacity)
        self.recovery = recovery or WorkerRecoveryService(max_retries=2)
        self.crash_detector, self.timeouts = crash_detector, timeouts
        self._done: Dict[int, Tuple[bool, Any]] = {}
        self._cv = threading.Condition()
        self._submitted = 0
        self._delivered = 0
        self._threads: Dict[int, threading.Thread] = {}
        self._started = False
        self.completed_by_worker: Dict[int, int] = {}

    def start(self):
        if self._started:
            return
        self._started = True
        for w in range(self.num_workers):
            self._spawn(w)

    def _spawn(self, wid: int):
        t = threading.Thread(target=self._run, args=(wid,), daemon=True, name=f"mlf-worker-{wid}")
        self._threads[wid] = t
        if self.crash_detector is not None:
            self.crash_detector.register_worker(wid, t)
        t.start()

    def _run(self, wid: int):
        ctx = WorkerContext(wid, self.num_workers, self.seed + wid)
        if self.init_fn is not None:
            self.init_fn(ctx)
        while True:
            try:
                seq, task, attempt = self.tasks.dequeue()
            except QueueClosed:
                break
            if self.crash_detector is not None:
                self.crash_detector.update_heartbeat(wid)
            if self.timeouts is not None:
                self.timeouts.start_operation(wid)
            try:
                res = (True, self.fn(task, ctx))
            except Exception as e:       # noqa: BLE001 - delivered to the consumer or retried
                res = (False, e)
            finally:
                if self.timeouts is not None:
                    self.timeouts.end_operation(wid)
            if not res[0] and self.recovery.try_restart(wid, lambda _w: None):
                # the "restart" of a thread worker is a fresh context; the task goes back to the queue
                ctx = WorkerContext(wid, self.num_workers, self.seed + wid)
                if self.init_fn is not None:
                    self.init_fn(ctx)
                try:
                    self.tasks.enqueue((seq, task, attempt + 1))
                    continue
                except QueueClosed:
                    pass
            with self._cv:
                self._done[seq] = res
                self.completed_by_worker[wid] = self.completed_by_worker.get(wid, 0) + 1
                self._cv.notify_all()
        if self.crash_detector is not None:
            self.crash_detector.unregister_worker(wid)

    def submit(self, task: Any) -> int:
        if not self._started:
            self.start()
        with self._cv:
            seq = self._submitted
            self._submitted += 1
        self.tasks.enqueue((seq, task, 0))
        return seq

    def map(self, tasks: Iterable[Any], ordered: bool = True) -> Iterator[Any]:
        n = 0
        for t in tasks:
            self.submit(t)
            n += 1
        yield from self.results(n, ordered)

    def results(self, count: int, ordered: bool = True, timeout_s: Optional[float] = None) -> Iterator[Any]:
        for _ in range(count):
            with self._cv:
                end = None if timeout_s is None else time.monotonic() + timeout_s
                while True:
                    key = self._delivered if ordered else next(iter(self._done), None)
                    if key is not None and key in self._done:
                        ok, val = self._done.pop(key)
                        self._delivered += 1
                        break
                    rest = None if end is None else end - time.monotonic()
                    if rest is not None and rest <= 0:
                        raise TimeoutError(f"no result within {timeout_s} s")
                    self._cv.wait(rest)
            if not ok:
                raise val
            yield val

    def shutdown(self, wait: bool = True):
        self.tasks.complete_adding()
        if wait:
            for t in self._threads.values():
                t.join(timeout=5.0)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.shutdown()


# ------------------------------------------------------------------ pools
@dataclass
class PoolStatistics:
    rents: int = 0
    returns: int = 0
    created: int = 0
    discarded: int = 0
    available: int = 0

    @property
    def hit_rate(self) -> float:
        return 1.0 - self.created / self.rents if self.rents else 0.0


class ObjectPool(Generic[T]):
    def __init__(self, factory: Callable[[], T], reset: Optional[Callable[[T], None]] = None, max_size: int = 64, initial: int = 0):
        self._factory, self._reset, self.max_size = factory, reset, max_size
        self._free: List[T] = []
        self._lock = threading.Lock()
        self._s = PoolStatistics()
        for _ in range(initial):
            self._free.append(factory())
            self._s.created += 1

    def rent(self) -> T:
        with self._lock:
            self._s.rents += 1
            if self._free:
                return self._free.pop()
            self._s.created += 1
        return self._factory()

    def give_back(self, obj: T):
        if self._reset is not None:
            self._reset(obj)
        with self._lock:
            self._s.returns += 1
            if len(self._free) < self.max_size:
                self._free.append(obj)
            else:
                self._s.discarded += 1

    def clear(self):
        with self._lock:
            self._free.clear()

    def statistics(self) -> PoolStatistics:
        with self._lock:
            s = PoolStatistics(**self._s.__dict__)
            s.available = len(self._free)
            return s


def _bucket(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


class ArrayPool:
    """NumPy arrays by power-of-two length bucket; ``rent(n)`` returns a view of exactly ``n`` elements."""

    def __init__(self, dtype=np.float32, max_per_bucket: int = 8):
        self.dtype, self.max_per_bucket = np.dtype(dtype), max_per_bucket
        self._free: Dict[int, List[np.ndarray]] = {}
        self._lock = threading.Lock()
        self._s = PoolStatistics()

    def rent(self, n: int, clear: bool = False) -> np.ndarray:
        b = _bucket(n)
        with self._lock:
            self._s.rents += 1
            lst = self._free.get(b)
            base = lst.pop() if lst else None
            if base is None:
                self._s.created += 1
        if base is None:
            base = np.empty(b, self.dtype)
        v = base[:n]
        if clear:
            v.fill(0)
        return v

    def give_back(self, a: np.ndarray):
        base = a.base if a.base is not None else a
        b = base.shape[0]
        with self._lock:
            self._s.returns += 1
            if base.ndim != 1 or b != _bucket(b) or base.dtype != self.dtype:
                self._s.discarded += 1
                return
            lst = self._free.setdefault(b, [])
            if len(lst) < self.max_per_bucket:
                lst.append(base)
            else:
                self._s.discarded += 1

    def statistics(self) -> PoolStatistics:
        with self._lock:
            s = PoolStatistics(**self._s.__dict__)
            s.available = sum(len(v) for v in self._free.values())
            return s


class TensorPool:
    """Tensors by (shape, dtype, device, pinned); what the loader's staging path uses for batches of fixed shape."""

    def __init__(self, max_per_key: int = 4):
        self.max_per_key = max_per_key
        self._free: Dict[tuple, List[torch.Tensor]] = {}
        self._lock = threading.Lock()
        self._s = PoolStatistics()

    @staticmethod
    def _key(shape, dtype, device, pinned):
        return (tuple(shape), dtype, str(device), bool(pinned))

    def rent(self, shape, dtype=torch.float32, device="cpu", pinned: bool = False) -> torch.Tensor:
        k = self._key(shape, dtype, device, pinned)
        with self._lock:
            self._s.rents += 1
            lst = self._free.get(k)
            if lst:
                return lst.pop()
            self._s.created += 1
        return torch.empty(tuple(shape), dtype=dtype, device=device, pin_memory=pinned and torch.cuda.is_available())

    def give_back(self, t: torch.Tensor, pinned: bool = False):
        k = self._key(t.shape, t.dtype, t.device, pinned)
        with self._lock:
            self._s.returns += 1
            lst = self._free.setdefault(k, [])
            if len(lst) < self.max_per_key:
                lst.append(t)
            else:
                self._s.discarded += 1

    def clear(self):
        with self._lock:
            self._free.clear()

    def statistics(self) -> PoolStatistics:
        with self._lock:
            s = PoolStatistics(**self._s.__dict__)
            s.available = sum(len(v) for v in self._free.values())
            return s


class PoolManager:
    """Named pools with one report."""

    def __init__(self):
        self._pools: Dict[str, Any] = {}
        self._lock = threading.Lock()

    def register(self, name: str, pool) -> Any:
        with self._lock:
            if name in self._pools:
                raise KeyError(f"pool {name!r} already registered")
            self._pools[name] = pool
        return pool

    def get(self, name: str):
        with self._lock:
            return self._pools[name]

    def get_or_create(self, name: str, factory: Callable[[], Any]):
        with self._lock:
            if name not in self._pools:
                self._pools[name] = factory()
            return self._pools[name]

    def remove(self, name: str) -> bool:
        with self._lock:
            return self._pools.pop(name, None) is not None

    def names(self) -> List[str]:
        with self._lock:
            return sorted(self._pools)

    def statistics(self) -> Dict[str, PoolStatistics]:
        with self._lock:
            return {k: p.statistics() for k, p in self._pools.items()}

    def clear_all(self):
        with self._lock:
            for p in self._pools.values():
                if hasattr(p, "clear"):
                    p.clear()

    def report(self) -> str:
        return "\n".join(f"{k}: {s.rents} rents, {s.created} created, {s.available} available, hit rate {s.hit_rate:.0%}"
                         for k, s in sorted(self.statistics().items()))
