"""Event system, collectors and scalar logging.

Reference: src/MLFramework.Visualization/Events/EventSystem.cs (pub-sub), typed events (ScalarMetric,
Histogram, ProfilingStart / End, MemoryAllocation, TensorOperation: Events/*Event.cs), synchronous and
asynchronous collectors with buffers, flush strategies and back-pressure (Collection/EventCollector.cs,
AsyncEventCollector.cs, EventBuffer.cs, Configuration/EventCollectorConfig.cs:6-135), scalar logger with
smoothing / resampling (Scalars/ScalarLogger.cs, ScalarSeries.cs, Smoothing/*), storage back-ends
(Storage/IStorageBackend.cs, FileStorageBackend.cs, EventFileWriter.cs / Reader.cs).
"""
from __future__ import annotations

import enum
import json
import os
import threading
import time
from collections import defaultdict, deque
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple


class EventType(enum.Enum):
    SCALAR = "scalar"
    HISTOGRAM = "histogram"
    PROFILING_START = "profiling_start"
    PROFILING_END = "profiling_end"
    MEMORY_ALLOCATION = "memory_allocation"
    TENSOR_OPERATION = "tensor_operation"
    TEXT = "text"
    HYPERPARAMETERS = "hparams"
    GRAPH = "graph"
    IMAGE = "image"


@dataclass
class Event:
    type: EventType
    name: str
    step: int = 0
    value: Any = None
    wall_time: float = field(default_factory=time.time)
    metadata: Dict[str, Any] = field(default_factory=dict)

    def to_json(self) -> str:
        d = asdict(self)
        d["type"] = self.type.value
        return json.dumps(d, default=lambda o: o.tolist() if hasattr(o, "tolist") else str(o))

    @staticmethod
    def from_json(s: str) -> "Event":
        d = json.loads(s)
        d["type"] = EventType(d["type"])
        return Event(**d)


class EventFactory:
    @staticmethod
    def scalar(name, value, step=0, **md): return Event(EventType.SCALAR, name, step, float(value), metadata=md)
    @staticmethod
    def histogram(name, values, step=0, **md): return Event(EventType.HISTOGRAM, name, step, list(map(float, values)), metadata=md)
    @staticmethod
    def profiling_start(name, step=0, **md): return Event(EventType.PROFILING_START, name, step, time.perf_counter_ns(), metadata=md)
    @staticmethod
    def profiling_end(name, step=0, duration_ns=0, **md): return Event(EventType.PROFILING_END, name, step, duration_ns, metadata=md)
    @staticmethod
    def memory(name, nbytes, step=0, **md): return Event(EventType.MEMORY_ALLOCATION, name, step, int(nbytes), metadata=md)
    @staticmethod
    def tensor_op(name, shapes, step=0, **md): return Event(EventType.TENSOR_OPERATION, name, step, [list(s) for s in shapes], metadata=md)


class EventSystem:
    """Publish / subscribe by event type (or to everything with ``None``)."""

    def __init__(self):
        self._subs: Dict[Optional[EventType], List[Callable[[Event], None]]] = defaultdict(list)
        self._lock = threading.Lock()
        self.published = 0

    def subscribe(self, fn: Callable[[Event], None], type: Optional[EventType] = None) -> Callable[[], None]:
        with self._lock:
            self._subs[type].append(fn)

        def unsubscribe():
            with self._lock:
                if fn in self._subs[type]:
                    self._subs[type].remove(fn)
        return unsubscribe

    def publish(self, e: Event):
        with self._lock:
            subs = list(self._subs[e.type]) + list(self._subs[None])
            self.published += 1
        for fn in subs:
            fn(e)


# ------------------------------------------------------------------ storage
class StorageBackend:
    def write(self, events: Sequence[Event]):
        raise NotImplementedError

    def flush(self):
        pass

    def close(self):
        pass


class MemoryStorageBackend(StorageBackend):
    def __init__(self):
        self.events: List[Event] = []

    def write(self, events):
        self.events.extend(events)


class FileStorageBackend(StorageBackend):
    """One JSON event per line; ``read`` is the matching reader."""

    def __init__(self, log_dir: str, prefix: str = "events"):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, f"{prefix}.{int(time.time())}.{os.getpid()}.jsonl")
        self._f = open(self.path, "a")
        self._lock = threading.Lock()

    def write(self, events):
        with self._lock:
            for e in events:
                self._f.write(e.to_json() + "\n")

    def flush(self):
        with self._lock:
            self._f.flush()

    def close(self):
        with self._lock:
            self._f.close()

    @staticmethod
    def read(path: str) -> List[Event]:
        with open(path) as f:
            return [Event.from_json(l) for l in f if l.strip()]


def storage_backend(kind: str, **kw) -> StorageBackend:
    if kind == "memory":
        return MemoryStorageBackend()
    if kind == "file":
        return FileStorageBackend(**kw)
    raise KeyError(f"unknown storage backend {kind!r}")


# ------------------------------------------------------------------ collectors
class BackpressureStrategy(enum.Enum):
    DROP_OLDEST = "drop_oldest"
    DROP_NEWEST = "drop_newest"
    BLOCK = "block"


@dataclass
class EventCollectorConfig:
    buffer_capacity: int = 1000
    flush_batch: int = 100
    flush_interval_s: float = 1.0
    backpressure: BackpressureStrategy = BackpressureStrategy.DROP_OLDEST


class EventCollector:
    """Synchronous: buffers events and writes them to the back-end when the batch size is reached."""

    def __init__(self, backend: StorageBackend, config: Optional[EventCollectorConfig] = None):
        self.backend, self.cfg = backend, config or EventCollectorConfig()
        self._buf: Deque[Event] = deque()
        self._lock = threading.Lock()
        self.dropped = 0

    def collect(self, e: Event):
        with self._lock:
            if len(self._buf) >= self.cfg.buffer_capacity:
                if self.cfg.backpressure == BackpressureStrategy.DROP_NEWEST:
                    self.dropped += 1
                    return
                if self.cfg.backpressure == BackpressureStrategy.DROP_OLDEST:
                    self._buf.popleft()
                    self.dropped += 1
                else:
                    self._flush_locked()
            self._buf.append(e)
            if len(self._buf) >= self.cfg.flush_batch:
                self._flush_locked()

    def _flush_locked(self):
        if self._buf:
            self.backend.write(list(self._buf))
            self._buf.clear()

    def flush(self):
        with self._lock:
            self._flush_locked()
        self.backend.flush()

    def close(self):
        self.flush()
        self.backend.close()


class AsyncEventCollector(EventCollector):
    """A background thread drains the buffer every ``flush_interval_s`` so logging never blocks a step."""

    def __init__(self, backend, config=None):
        super().__init__(backend, config)
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._loop, daemon=True, name="mlf-events")
        self._t.start()

    def collect(self, e: Event):
        with self._lock:
            if len(self._buf) >= self.cfg.buffer_capacity:
                if self.cfg.backpressure == BackpressureStrategy.DROP_NEWEST:
                    self.dropped += 1
                    return
                self._buf.popleft()
                self.dropped += 1
            self._buf.append(e)

    def _loop(self):
        while not self._stop.wait(self.cfg.flush_interval_s):
            self.flush()

    def close(self):
        self._stop.set()
        self._t.join(timeout=2.0)
        super().close()


# ------------------------------------------------------------------ scalars
class ScalarSeries:
    def __init__(self, name: str):
        self.name = name
        self.steps: List[int] = []
        self.values: List[float] = []

    def add(self, step: int, v: float):
        self.steps.append(step)
        self.values.append(float(v))

    def ema(self, alpha: float = 0.6) -> List[float]:
        """TensorBoard-style debiased exponential smoothing (``alpha`` = weight of history)."""
        out, last, n = [], 0.0, 0
        for v in self.values:
            last = last * alpha + (1 - alpha) * v
            n += 1
            out.append(last / (1 - alpha ** n))
        return out

    def moving_average(self, window: int) -> List[float]:
        out, s, q = [], 0.0, deque()
        for v in self.values:
            q.append(v)
            s += v
            if len(q) > window:
                s -= q.popleft()
            out.append(s / len(q))
        return out

    def resample(self, n_points: int) -> Tuple[List[int], List[float]]:
        if len(self.values) <= n_points:
            return list(self.steps), list(self.values)
        idx = [round(i * (len(self.values) - 1) / (n_points - 1)) for i in range(n_points)]
        return [self.steps[i] for i in idx], [self.values[i] for i in idx]

    def stats(self) -> Dict[str, float]:
        v = self.values
        return {"count": len(v), "min": min(v), "max": max(v), "mean": sum(v) / len(v), "last": v[-1]} if v else {"count": 0}


class ScalarLogger:
    def __init__(self, events: Optional[EventSystem] = None):
        self.series: Dict[str, ScalarSeries] = {}
        self.events = events

    def log(self, name: str, value: float, step: int):
        self.series.setdefault(name, ScalarSeries(name)).add(step, value)
        if self.events is not None:
            self.events.publish(EventFactory.scalar(name, value, step))

    def get(self, name: str) -> ScalarSeries:
        return self.series[name]
