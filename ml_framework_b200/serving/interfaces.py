"""Serving-side interfaces and small utilities: tokenizers, the executor contract, request tracking, batch building.

Reference: src/MLFramework/Inference/ITokenizer.cs:6-20, IModelExecutor.cs:8-16, Serving/RequestTracker.cs,
Serving/{BatchBuilder.cs, BoundedRequestQueue.cs, ResponseScatterer.cs} (pieces of the dynamic batcher),
Inference/ContinuousBatching/API/{SchedulerStatus.cs, SchedulerStatistics.cs}.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, Generic, List, Optional, Protocol, Sequence, Tuple, TypeVar, runtime_checkable

T = TypeVar("T")
R = TypeVar("R")


@runtime_checkable
class Tokenizer(Protocol):
    def encode(self, text: str) -> List[int]: ...
    def decode(self, ids: Sequence[int]) -> str: ...


@runtime_checkable
class ModelExecutor(Protocol):
    """One scheduler iteration: given the batch, return one new token per request id."""
    def execute_batch(self, batch) -> Dict[int, int]: ...


class ByteTokenizer:
    """UTF-8 bytes as token ids (offset by the special tokens): lossless for any text, vocabulary of 256 + specials."""

    def __init__(self, bos_id: Optional[int] = 1, eos_id: int = 2, pad_id: int = 0):
        self.bos_id, self.eos_id, self.pad_id = bos_id, eos_id, pad_id
        self.offset = 3
        self.vocab_size = 256 + self.offset

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = False) -> List[int]:
        ids = [b + self.offset for b in text.encode("utf-8")]
        if add_bos and self.bos_id is not None:
            ids.insert(0, self.bos_id)
        if add_eos:
            ids.append(self.eos_id)
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i - self.offset for i in ids if i >= self.offset).decode("utf-8", errors="replace")


class WhitespaceTokenizer:
    """Words split on whitespace with a vocabulary that grows on ``encode`` (or is fixed with ``freeze``); for tests
    and examples that want readable tokens."""

    def __init__(self, unk_id: int = 1, eos_id: int = 2):
        self.unk_id, self.eos_id = unk_id, eos_id
        self._w2i: Dict[str, int] = {}
        self._i2w: Dict[int, str] = {}
        self._next = 3
        self._frozen = False

    def freeze(self):
        self._frozen = True

    @property
    def vocab_size(self) -> int:
        return self._next

    def encode(self, text: str) -> List[int]:
        out = []
        for w in text.split():
            i = self._w2i.get(w)
            if i is None:
                if self._frozen:
                    i = self.unk_id
                else:
                    i = self._w2i[w] = self._next
                    self._i2w[i] = w
                    self._next += 1
            out.append(i)
        return out

    def decode(self, ids: Sequence[int]) -> str:
        return " ".join(self._i2w.get(i, "<unk>") for i in ids if i != self.eos_id)


# ------------------------------------------------------------------ request tracking
@dataclass
class TrackedRequest:
    request_id: str
    model: str
    started: float
    finished: Optional[float] = None
    ok: Optional[bool] = None
    error: str = ""

    @property
    def duration_s(self) -> Optional[float]:
        return None if self.finished is None else self.finished - self.started


class RequestTracker:
    """In-flight and recently finished requests by id; counts per model; what a drain or a rollback decision reads."""

    def __init__(self, history: int = 1000, clock: Callable[[], float] = time.monotonic):
        self._live: Dict[str, TrackedRequest] = {}
        self._done: Deque[TrackedRequest] = deque(maxlen=history)
        self._lock = threading.Lock()
        self._clock = clock
        self._idle = threading.Condition(self._lock)

    def start(self, request_id: str, model: str = "") -> TrackedRequest:
        with self._lock:
            if request_id in self._live:
                raise KeyError(f"request {request_id!r} is already in flight")
            r = self._live[request_id] = TrackedRequest(request_id, model, self._clock())
            return r

    def finish(self, request_id: str, ok: bool = True, error: str = "") -> TrackedRequest:
        with self._lock:
            r = self._live.pop(request_id, None)
            if r is None:
                raise KeyError(f"request {request_id!r} is not in flight")
            r.finished, r.ok, r.error = self._clock(), ok, error
            self._done.append(r)
            if not self._live:
                self._idle.notify_all()
            return r

    def in_flight(self, model: Optional[str] = None) -> int:
        with self._lock:
            return sum(1 for r in self._live.values() if model is None or r.model == model)

    def oldest_age_s(self) -> float:
        with self._lock:
            return max((self._clock() - r.started for r in self._live.values()), default=0.0)

    def wait_idle(self, timeout_s: Optional[float] = None) -> bool:
        with self._idle:
            return self._idle.wait_for(lambda: not self._live, timeout_s)

    def statistics(self, model: Optional[str] = None) -> Dict[str, float]:
        with self._lock:
            done = [r for r in self._done if model is None or r.model == model]
        n = len(done)
        bad = sum(1 for r in done if not r.ok)
        d = sorted(r.duration_s for r in done)
        return {"finished": n, "failed": bad, "error_rate": bad / n if n else 0.0, "mean_s": sum(d) / n if n else 0.0,
                "p99_s": d[min(n - 1, int(0.99 * n))] if n else 0.0}


# ------------------------------------------------------------------ dynamic-batcher pieces as parts of their own
class BoundedRequestQueue(Generic[T]):
    def __init__(self, max_size: int):
        if max_size <= 0:
            raise ValueError("max_size must be positive")
        self.max_size = max_size
        self._q: Deque[Tuple[T, float]] = deque()
        self._cv = threading.Condition()

    def __len__(self):
        with self._cv:
            return len(self._q)

    def try_enqueue(self, item: T) -> bool:
        with self._cv:
            if len(self._q) >= self.max_size:
                return False
            self._q.append((item, time.monotonic()))
            self._cv.notify()
            return True

    def take(self, max_items: int, wait_s: float) -> List[Tuple[T, float]]:
        """Up to ``max_items`` with their arrival times; waits at most ``wait_s`` for the first one."""
        with self._cv:
            if not self._q:
                self._cv.wait(wait_s)
            out = []
            while self._q and len(out) < max_items:
                out.append(self._q.popleft())
            return out


class BatchBuilder(Generic[T]):
    """Collects a batch: returns when ``max_batch_size`` items are in hand, or ``max_wait_s`` after the FIRST item
    arrived (a partial batch), whichever comes first; with ``prefer_batch_size`` a batch of at least that size is
    dispatched without waiting for more."""

    def __init__(self, queue: BoundedRequestQueue, max_batch_size: int = 32, max_wait_s: float = 0.005, prefer_batch_size: Optional[int] = None):
        self.q, self.max_batch_size, self.max_wait_s = queue, max_batch_size, max_wait_s
        self.prefer = prefer_batch_size or max_batch_size

    def build(self, idle_wait_s: float = 0.05) -> List[T]:
        first = self.q.take(self.max_batch_size, idle_wait_s)
        if not first:
            return []
        items = list(first)
        deadline = first[0][1] + self.max_wait_s
        while len(items) < self.prefer:
            rest = deadline - time.monotonic()
            if rest <= 0:
                break
            more = self.q.take(self.max_batch_size - len(items), rest)
            if not more:
                break
            items += more
        return [x for x, _ in items]


class ResponseScatterer(Generic[R]):
    """Hands the responses of a processed batch back to the waiters, in request order; a count mismatch or a processor
    error fails every waiter of the batch."""

    @staticmethod
    def scatter(futures: Sequence, responses: Sequence[R]):
        if len(futures) != len(responses):
            err = ValueError(f"processor returned {len(responses)} responses for {len(futures)} requests")
            for f in futures:
                f.set_exception(err)
            raise err
        for f, r in zip(futures, responses):
            f.set_result(r)

    @staticmethod
    def fail_all(futures: Sequence, error: BaseException):
        for f in futures:
            if not f.done():
                f.set_exception(error)


@dataclass
class SchedulerStatus:
    queued: int
    running: int
    iterations: int
    utilization: float
    is_running: bool = True


@dataclass
class SchedulerStatistics:
    completed_requests: int = 0
    tokens_generated: int = 0
    mean_iteration_ms: float = 0.0
    p50_iteration_ms: float = 0.0
    p99_iteration_ms: float = 0.0
    mean_batch_utilization: float = 0.0
    errors: int = 0

    @staticmethod
    def from_snapshot(s: Dict[str, Any]) -> "SchedulerStatistics":
        return SchedulerStatistics(int(s.get("requests_completed", s.get("completed", 0))), int(s.get("tokens_generated", s.get("tokens", 0))),
                                   float(s.get("iteration_ms_mean", 0.0)), float(s.get("iteration_ms_p50", 0.0)), float(s.get("iteration_ms_p99", 0.0)),
                                   float(s.get("batch_utilization_mean", s.get("mean_batch_utilization", 0.0))), int(s.get("errors", 0)))
