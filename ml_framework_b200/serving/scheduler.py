"""Continuous-batching scheduler: request queue, capacity and KV-cache accounting, batch manager,
completion detection, metrics, the scheduler loop and its client API.

The iteration is the reference's (src/MLFramework/Inference/ContinuousBatching/Scheduler/
ContinuousBatchScheduler.cs:114-276): remove completed requests -> admit new ones while slots
and KV blocks last -> ``executor.execute_batch(batch)`` -> append one token per request ->
completion check (Cancelled > MaxTokens > EOS > StopString > Length, CompletionDetector.cs:29-63)
-> resolve futures and release KV blocks -> record metrics. Defaults mirror the reference's
configuration classes (SchedulerConfiguration.cs:6-27, BatchConstraints.cs:6-21,
CapacityConstraints.cs:11-34, CompletionConfiguration.cs:6-25, KVCacheConfiguration.cs:6-32,
PrefillConfiguration.cs:6-25). Where the reference disagrees with itself (EOS id 0 in
BatchManager.cs:10 vs 2 in CompletionConfiguration.cs:19) the configurable
``CompletionConfiguration.eos_token_id`` (default 2) is the single source.

The scheduler survives executor failures: the failing iteration's requests are failed or
retried and the loop continues (ContinuousBatchScheduler.cs:197-201).
"""
from __future__ import annotations

import collections
import enum
import heapq
import itertools
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from .kv_cache import KVCacheBlockManager


# ------------------------------------------------------------------ models
class Priority(enum.IntEnum):
    LOW = 0
    NORMAL = 1
    HIGH = 2
    URGENT = 3


class CompletionReason(enum.Enum):
    EOS = "eos"
    MAX_TOKENS = "max_tokens"
    CANCELLED = "cancelled"
    LENGTH = "length"
    STOP_STRING = "stop_string"
    TIMEOUT = "timeout"
    ERROR = "error"


class RequestState(enum.Enum):
    QUEUED = "queued"
    PREFILL = "prefill"
    DECODE = "decode"
    DONE = "done"


_ids = itertools.count(1)


@dataclass
class Request:
    prompt_tokens: List[int]
    max_tokens: int = 256
    priority: Priority = Priority.NORMAL
    prompt: str = ""
    stop_strings: Sequence[str] = ()
    id: int = field(default_factory=lambda: next(_ids))
    generated: List[int] = field(default_factory=list)
    state: RequestState = RequestState.QUEUED
    cancelled: bool = False
    future: Future = field(default_factory=Future)
    enqueue_time: float = 0.0
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    prefilled: int = 0                 # prompt tokens already in the KV cache
    text: str = ""

    @property
    def total_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.generated)


@dataclass
class RequestResult:
    request_id: int
    tokens: List[int]
    reason: CompletionReason
    text: str = ""
    ttft_s: Optional[float] = None
    latency_s: Optional[float] = None
    error: Optional[str] = None


@dataclass
class Batch:
    requests: List[Request]
    prefill: List[Request] = field(default_factory=list)
    decode: List[Request] = field(default_factory=list)


@dataclass
class BatchOutput:
    generated_tokens: Dict[int, int]      # request id -> next token


# ------------------------------------------------------------------ configuration
@dataclass
class SchedulerConfiguration:
    iteration_timeout_ms: float = 1000.0
    max_idle_iterations: int = 10
    min_iterations_per_second: int = 30
    enable_adaptive_batching: bool = True
    warmup_iterations: int = 5
    target_utilization: float = 0.85
    max_batch_size: int = 32
    idle_sleep_s: float = 0.001


@dataclass
class BatchConstraints:
    max_batch_size: int = 32
    max_memory_bytes: int = 16 << 30
    min_batch_size: int = 4
    max_sequence_length: int = 4096
    max_prefills_per_iteration: int = 4


@dataclass
class CapacityConstraints:
    max_batch_size: int = 32
    max_memory_bytes: int = 16 << 30
    memory_per_slot_bytes: int = 512 << 20
    max_concurrent_requests: int = 64
    buffer_ratio: float = 0.1


@dataclass
class CompletionConfiguration:
    eos_token_id: int = 2
    default_max_tokens: int = 256
    stop_strings: Sequence[str] = ()
    max_response_length: int = 4096
    enable_early_stopping: bool = True


@dataclass
class KVCacheConfiguration:
    page_size_tokens: int = 16
    initial_pages: int = 16
    max_pages_per_request: int = 256
    target_utilization: float = 0.85
    enable_compaction: bool = True
    max_batch_size: int = 64


@dataclass
class PrefillConfiguration:
    chunk_size: int = 512
    max_batch_prefill: int = 8
    max_prefill_memory_bytes: int = 4 << 30
    prompt_cache_entries: int = 100
    prompt_cache_ttl_s: float = 300.0


# ------------------------------------------------------------------ queue
class RequestQueue:
    """Four priority levels, FIFO inside a level (RequestQueue.cs:60-193)."""

    def __init__(self, max_size: int = 10000):
        self._heap: List[tuple] = []
        self._seq = itertools.count()
        self._lock = threading.Lock()
        self.max_size = max_size

    def enqueue(self, req: Request):
        with self._lock:
            if len(self._heap) >= self.max_size:
                raise OverflowError("request queue is full")
            req.enqueue_time = req.enqueue_time or time.time()
            heapq.heappush(self._heap, (-int(req.priority), next(self._seq), req))

    def dequeue(self) -> Optional[Request]:
        with self._lock:
            while self._heap:
                _, _, r = heapq.heappop(self._heap)
                if not r.cancelled:
                    return r
                self._finish_cancelled(r)
        return None

    @staticmethod
    def _finish_cancelled(r: Request):
        if not r.future.done():
            r.future.set_result(RequestResult(r.id, [], CompletionReason.CANCELLED))

    def get_requests(self, max_count: int, admit: Callable[[Request], bool]) -> List[Request]:
        """Pops up to ``max_count`` requests in priority order for which ``admit`` (memory check)
        returns True; the first request that does not fit stays at the head (no starvation)."""
        out = []
        with self._lock:
            while self._heap and len(out) < max_count:
                _, _, r = self._heap[0]
                if r.cancelled:
                    heapq.heappop(self._heap)
                    self._finish_cancelled(r)
                    continue
                if not admit(r):
                    break
                heapq.heappop(self._heap)
                out.append(r)
        return out

    def mark_cancelled(self, request_id: int) -> bool:
        with self._lock:
            for _, _, r in self._heap:
                if r.id == request_id:
                    r.cancelled = True
                    return True
        return False

    def __len__(self):
        return len(self._heap)


# ------------------------------------------------------------------ capacity
class CapacityManager:
    """Slot and memory accounting with a safety buffer (CapacityManager.cs:40-214)."""

    def __init__(self, c: Optional[CapacityConstraints] = None, bytes_per_token: int = 0):
        self.c = c or CapacityConstraints()
        self.bytes_per_token = bytes_per_token
        self._alloc: Dict[int, int] = {}

    @property
    def usable_memory(self) -> int:
        return int(self.c.max_memory_bytes * (1.0 - self.c.buffer_ratio))

    def estimate_required_memory(self, req: Request) -> int:
        if self.bytes_per_token:
            return (len(req.prompt_tokens) + req.max_tokens) * self.bytes_per_token
        return min(self.c.memory_per_slot_bytes, (len(req.prompt_tokens) + req.max_tokens) * 1024)

    def try_allocate(self, req: Request) -> bool:
        need = self.estimate_required_memory(req)
        if len(self._alloc) >= min(self.c.max_batch_size, self.c.max_concurrent_requests):
            return False
        if sum(self._alloc.values()) + need > self.usable_memory:
            return False
        self._alloc[req.id] = need
        return True

    def release(self, request_id: int):
        self._alloc.pop(request_id, None)

    def can_fit_batch(self, reqs: Sequence[Request]) -> bool:
        return (len(self._alloc) + len(reqs) <= self.c.max_batch_size and
                sum(self._alloc.values()) + sum(self.estimate_required_memory(r) for r in reqs) <= self.usable_memory)

    @property
    def utilization(self) -> float:
        return sum(self._alloc.values()) / max(1, self.usable_memory)

    @property
    def active_slots(self) -> int:
        return len(self._alloc)


class PagedAttentionScheduler:
    """Block-level admission control (src/MLFramework/Inference/Scheduling/PagedAttentionScheduler.cs:34-138):
    admit when blocks needed <= free - reserved; back-pressure above 0.8 pressure."""

    def __init__(self, manager: KVCacheBlockManager, reserved_blocks: int = 0, backpressure_threshold: float = 0.8):
        self.m, self.reserved, self.threshold = manager, reserved_blocks, backpressure_threshold

    def can_admit(self, prompt_tokens: int, max_new_tokens: int = 0) -> bool:
        need = self.m.blocks_needed(prompt_tokens + max_new_tokens)
        return need <= self.m.free_blocks - self.reserved

    def memory_pressure(self) -> float:
        return 1.0 - self.m.free_blocks / self.m.total_blocks

    def should_apply_backpressure(self) -> bool:
        return self.memory_pressure() >= self.threshold

    def recommended_max_sequence_length(self, active: int) -> int:
        free = max(0, self.m.free_blocks - self.reserved)
        return (free // max(1, active)) * self.m.block_size


# ------------------------------------------------------------------ completion
class CompletionDetector:
    def __init__(self, cfg: Optional[CompletionConfiguration] = None, detokenize: Optional[Callable[[List[int]], str]] = None):
        self.cfg = cfg or CompletionConfiguration()
        self.detok = detokenize

    def check(self, req: Request) -> Optional[CompletionReason]:
        if req.cancelled:
            return CompletionReason.CANCELLED
        if len(req.generated) >= req.max_tokens:
            return CompletionReason.MAX_TOKENS
        if req.generated and req.generated[-1] == self.cfg.eos_token_id and self.cfg.enable_early_stopping:
            return CompletionReason.EOS
        stops = list(req.stop_strings) + list(self.cfg.stop_strings)
        if stops and self.detok is not None:
            text = self.detok(req.generated)
            if any(s and s in text for s in stops):
                return CompletionReason.STOP_STRING
        if req.total_tokens >= self.cfg.max_response_length:
            return CompletionReason.LENGTH
        return None


# ------------------------------------------------------------------ metrics
class CircularBuffer:
    def __init__(self, capacity: int):
        self._d: Deque = collections.deque(maxlen=capacity)

    def add(self, x):
        self._d.append(x)

    def values(self):
        return list(self._d)

    def __len__(self):
        return len(self._d)


class SlidingWindowCounter:
    def __init__(self, window_s: float = 60.0, clock=time.time):
        self.window, self.clock, self._ev = window_s, clock, collections.deque()

    def add(self, n: float = 1.0):
        self._ev.append((self.clock(), n))
        self._trim()

    def _trim(self):
        t = self.clock() - self.window
        while self._ev and self._ev[0][0] < t:
            self._ev.popleft()

    def total(self) -> float:
        self._trim()
        return sum(n for _, n in self._ev)

    def rate(self) -> float:
        return self.total() / self.window


def _pct(xs: List[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


class SchedulerMetricsCollector:
    def __init__(self, capacity: int = 10000):
        self.iter_ms, self.batch_sizes = CircularBuffer(capacity), CircularBuffer(capacity)
        self.ttft, self.latency, self.tokens_per_req = CircularBuffer(capacity), CircularBuffer(capacity), CircularBuffer(capacity)
        self.utilization = CircularBuffer(capacity)
        self.tokens = SlidingWindowCounter()
        self.errors: Dict[str, int] = {}
        self.completed = 0
        self.total_tokens = 0
        self.decode_time_s = 0.0
        self.reasons: Dict[str, int] = {}

    def record_iteration(self, ms: float, batch_size: int, new_tokens: int):
        self.iter_ms.add(ms)
        self.batch_sizes.add(batch_size)
        self.tokens.add(new_tokens)
        self.total_tokens += new_tokens
        self.decode_time_s += ms / 1e3

    def record_request_completion(self, res: RequestResult):
        self.completed += 1
        self.reasons[res.reason.value] = self.reasons.get(res.reason.value, 0) + 1
        if res.ttft_s is not None:
            self.ttft.add(res.ttft_s)
        if res.latency_s is not None:
            self.latency.add(res.latency_s)
        self.tokens_per_req.add(len(res.tokens))

    def record_batch_utilization(self, used: int, capacity: int):
        """Share of the batch slots an iteration filled (SchedulerMetricsCollector.RecordBatchUtilization)."""
        self.utilization.add(used / capacity if capacity > 0 else 0.0)

    def record_error(self, kind: str):
        self.errors[kind] = self.errors.get(kind, 0) + 1

    def snapshot(self) -> Dict:
        it = self.iter_ms.values()
        return {"iterations": len(it), "iteration_ms_p50": _pct(it, 0.5), "iteration_ms_p99": _pct(it, 0.99),
                "mean_batch": (sum(self.batch_sizes.values()) / len(self.batch_sizes)) if len(self.batch_sizes) else 0.0,
                "mean_batch_utilization": (sum(self.utilization.values()) / len(self.utilization)) if len(self.utilization) else 0.0,
                "completed": self.completed, "total_tokens": self.total_tokens,
                "decode_tokens_per_s": self.total_tokens / self.decode_time_s if self.decode_time_s else 0.0,
                "ttft_p50_s": _pct(self.ttft.values(), 0.5), "ttft_p99_s": _pct(self.ttft.values(), 0.99),
                "latency_p50_s": _pct(self.latency.values(), 0.5), "errors": dict(self.errors), "reasons": dict(self.reasons)}


# ------------------------------------------------------------------ batch manager
class BatchManager:
    """Keeps the running batch: drops finished requests, admits queued ones under slot, memory and
    KV-block limits, splits the batch into prefill and decode work (BatchManager.cs:52-255)."""

    def __init__(self, queue: RequestQueue, capacity: CapacityManager, kv: Optional[KVCacheBlockManager],
                 constraints: Optional[BatchConstraints] = None, admission: Optional[PagedAttentionScheduler] = None):
        self.queue, self.capacity, self.kv = queue, capacity, kv
        self.c = constraints or BatchConstraints()
        self.admission = admission or (PagedAttentionScheduler(kv) if kv is not None else None)
        self.running: List[Request] = []

    def has_capacity(self) -> bool:
        return len(self.running) < self.c.max_batch_size

    def remove_completed(self, done: Sequence[Request]):
        ids = {r.id for r in done}
        self.running = [r for r in self.running if r.id not in ids]
        for r in done:
            self.capacity.release(r.id)
            if self.kv is not None:
                self.kv.free_sequence_blocks(r.id)

    def _admit(self, r: Request) -> bool:
        if len(r.prompt_tokens) + r.max_tokens > self.c.max_sequence_length:
            r.max_tokens = max(1, self.c.max_sequence_length - len(r.prompt_tokens))
        if self.admission is not None and not self.admission.can_admit(len(r.prompt_tokens), r.max_tokens):
            return False
        return self.capacity.try_allocate(r)

    def add_new_requests(self) -> List[Request]:
        slots = self.c.max_batch_size - len(self.running)
        if slots <= 0:
            return []
        new = self.queue.get_requests(slots, self._admit)
        for r in new:
            r.state = RequestState.PREFILL
        self.running.extend(new)
        return new

    def prepare_next_iteration(self) -> Batch:
        self.add_new_requests()
        prefill = [r for r in self.running if r.state == RequestState.PREFILL][: self.c.max_prefills_per_iteration]
        decode = [r for r in self.running if r.state == RequestState.DECODE]
        return Batch(prefill + decode, prefill, decode)


# ------------------------------------------------------------------ scheduler
class ContinuousBatchScheduler:
    """``executor.execute_batch(batch) -> BatchOutput`` is called once per iteration with the
    prefill and decode requests of that iteration."""

    def __init__(self, executor, kv: Optional[KVCacheBlockManager] = None, config: Optional[SchedulerConfiguration] = None,
                 constraints: Optional[BatchConstraints] = None, capacity: Optional[CapacityConstraints] = None,
                 completion: Optional[CompletionConfiguration] = None, detokenize=None, clock=time.time):
        self.cfg = config or SchedulerConfiguration()
        self.executor, self.kv, self.clock = executor, kv, clock
        self.queue = RequestQueue()
        cons = constraints or BatchConstraints(max_batch_size=self.cfg.max_batch_size)
        cap = capacity or CapacityConstraints(max_batch_size=cons.max_batch_size, max_concurrent_requests=max(64, cons.max_batch_size))
        self.capacity = CapacityManager(cap)
        self.batch_manager = BatchManager(self.queue, self.capacity, kv, cons)
        self.detector = CompletionDetector(completion, detokenize)
        self.metrics = SchedulerMetricsCollector()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.iterations = 0
        self.warmup_done = 0              # iterations spent warming up the executor before the loop serves
        self.timed_out_iterations = 0

    # ---- API
    def enqueue(self, req: Request) -> Future:
        req.enqueue_time = self.clock()
        self.queue.enqueue(req)
        return req.future

    def cancel(self, request_id: int) -> bool:
        if self.queue.mark_cancelled(request_id):
            return True
        for r in self.batch_manager.running:
            if r.id == request_id:
                r.cancelled = True
                return True
        return False

    def start(self):
        if self._thread is not None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self, timeout_s: float = 10.0):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout_s)
            self._thread = None

    def warm_up(self) -> int:
        """Runs ``warmup_iterations`` iterations of the executor's own warm-up work (``executor.warm_up(i)``, e.g.
        capturing the decode graphs of the first batch buckets) before requests are served; executors without a
        warm-up hook skip this. ContinuousBatchScheduler.cs:143-175 counts the first iterations of its loop as
        warm-up and keeps them out of the idle accounting."""
        fn = getattr(self.executor, "warm_up", None)
        n = 0
        for i in range(self.cfg.warmup_iterations if fn is not None else 0):
            if self._stop.is_set():
                break
            try:
                fn(i)
            except Exception as e:  # noqa: BLE001
                self.metrics.record_error(f"Warmup{type(e).__name__}")
                break
            n += 1
        self.warmup_done = n
        return n

    def _loop(self):
        idle = 0
        self.warm_up()
        while not self._stop.is_set():
            did = self.execute_iteration()
            if did:
                idle = 0
            else:
                idle += 1
                time.sleep(self.cfg.idle_sleep_s * min(idle, self.cfg.max_idle_iterations))

    # ---- one iteration
    def execute_iteration(self) -> bool:
        if getattr(self, "_skip_admission_once", False):
            self._skip_admission_once = False
            bm = self.batch_manager
            prefill = [r for r in bm.running if r.state == RequestState.PREFILL][: bm.c.max_prefills_per_iteration]
            decode = [r for r in bm.running if r.state == RequestState.DECODE]
            batch = Batch(prefill + decode, prefill, decode)
        else:
            batch = self.batch_manager.prepare_next_iteration()
        if not batch.requests:
            return False
        t0 = self.clock()
        try:
            out = self.executor.execute_batch(batch)
        except Exception as e:  # noqa: BLE001 - the scheduler must survive executor failures
            self.metrics.record_error(type(e).__name__)
            self._fail(batch.requests, str(e))
            return True
        now = self.clock()
        if self.cfg.iteration_timeout_ms > 0 and (now - t0) * 1e3 > self.cfg.iteration_timeout_ms:
            # The iteration ran past its budget (SchedulerConfiguration.IterationTimeoutMs; the reference cancels the
            # iteration's token, ContinuousBatchScheduler.cs:155-160). A device step cannot be cancelled half way, so
            # its tokens are kept, the overrun is recorded, and the next iteration admits no new prefill work.
            self.timed_out_iterations += 1
            self.metrics.record_error("IterationTimeout")
            self._skip_admission_once = True
        done = []
        for r in batch.requests:
            tok = out.generated_tokens.get(r.id)
            if r.state == RequestState.PREFILL and r.prefilled >= len(r.prompt_tokens):
                r.state = RequestState.DECODE
            if tok is not None:
                r.generated.append(int(tok))
                if r.first_token_time is None:
                    r.first_token_time = now
                    r.state = RequestState.DECODE
            reason = self.detector.check(r)
            if reason is not None:
                done.append((r, reason))
        for r, reason in done:
            self._complete(r, reason, now)
        self.batch_manager.remove_completed([r for r, _ in done])
        self.iterations += 1
        self.metrics.record_iteration((now - t0) * 1e3, len(batch.requests), len(out.generated_tokens))
        self.metrics.record_batch_utilization(len(batch.requests), self.batch_manager.c.max_batch_size)
        return True

    def _complete(self, r: Request, reason: CompletionReason, now: float, error: Optional[str] = None):
        r.state, r.finish_time = RequestState.DONE, now
        res = RequestResult(r.id, list(r.generated), reason, self.detector.detok(r.generated) if self.detector.detok else "",
                            (r.first_token_time - r.enqueue_time) if r.first_token_time else None, now - r.enqueue_time, error)
        self.metrics.record_request_completion(res)
        if not r.future.done():
            r.future.set_result(res)

    def _fail(self, reqs: Sequence[Request], msg: str):
        now = self.clock()
        for r in reqs:
            self._complete(r, CompletionReason.ERROR, now, msg)
        self.batch_manager.remove_completed(list(reqs))

    def run_until_idle(self, max_iterations: int = 1_000_000):
        n = 0
        while n < max_iterations and (len(self.queue) or self.batch_manager.running):
            if not self.execute_iteration():
                break
            n += 1
        return n


# ------------------------------------------------------------------ prefill handler
class PrefillHandler:
    """Chunked prefill with a prompt cache (PrefillHandler.cs:40-223): prompts longer than
    ``chunk_size`` are fed to the executor chunk by chunk; identical prompts reuse cached state."""

    def __init__(self, cfg: Optional[PrefillConfiguration] = None, clock=time.time):
        self.cfg, self.clock = cfg or PrefillConfiguration(), clock
        self._cache: "collections.OrderedDict[tuple, tuple]" = collections.OrderedDict()

    def needs_prefill(self, r: Request) -> bool:
        return r.prefilled < len(r.prompt_tokens)

    def next_chunk(self, r: Request) -> List[int]:
        a = r.prefilled
        return r.prompt_tokens[a:a + self.cfg.chunk_size]

    def estimate_prefill_memory(self, r: Request, bytes_per_token: int) -> int:
        return len(r.prompt_tokens) * bytes_per_token

    def cache_lookup(self, tokens: Sequence[int]):
        k = tuple(tokens)
        e = self._cache.get(k)
        if e is None:
            return None
        value, t = e
        if self.clock() - t > self.cfg.prompt_cache_ttl_s:
            del self._cache[k]
            return None
        self._cache.move_to_end(k)
        return value

    def cache_store(self, tokens: Sequence[int], value):
        self._cache[tuple(tokens)] = (value, self.clock())
        while len(self._cache) > self.cfg.prompt_cache_entries:
            self._cache.popitem(last=False)


# ------------------------------------------------------------------ client
@dataclass
class GenerationOptions:
    stop_strings: Sequence[str] = ()
    temperature: float = 0.0


class ContinuousBatchSchedulerClient:
    """``generate_text(prompt, max_tokens)`` facade (API/ContinuousBatchSchedulerClient.cs:18-264)."""

    def __init__(self, scheduler: ContinuousBatchScheduler, tokenizer):
        self.s, self.tok = scheduler, tokenizer

    def submit(self, prompt: str, max_tokens: int = 256, priority: Priority = Priority.NORMAL,
               options: Optional[GenerationOptions] = None) -> Request:
        ids = self.tok.encode(prompt)
        r = Request(ids, max_tokens, priority, prompt, (options or GenerationOptions()).stop_strings)
        self.s.enqueue(r)
        return r

    def generate_text(self, prompt: str, max_tokens: int = 256, priority: Priority = Priority.NORMAL,
                      options: Optional[GenerationOptions] = None, timeout_s: Optional[float] = None) -> RequestResult:
        r = self.submit(prompt, max_tokens, priority, options)
        res = r.future.result(timeout_s)
        res.text = self.tok.decode(res.tokens)
        return res

    def generate_batch(self, prompts: Sequence[str], max_tokens: int = 256, timeout_s: Optional[float] = None) -> List[RequestResult]:
        reqs = [self.submit(p, max_tokens) for p in prompts]
        return [r.future.result(timeout_s) for r in reqs]

    def cancel(self, request_id: int) -> bool:
        return self.s.cancel(request_id)

    def status(self) -> Dict:
        return {"queued": len(self.s.queue), "running": len(self.s.batch_manager.running), "iterations": self.s.iterations,
                "utilization": self.s.capacity.utilization}

    def statistics(self) -> Dict:
        return self.s.metrics.snapshot()

    def estimate_wait_time_s(self) -> float:
        snap = self.s.metrics.snapshot()
        per_iter = snap["iteration_ms_p50"] / 1e3 or 0.01
        return len(self.s.queue) / max(1, self.s.batch_manager.c.max_batch_size) * per_iter * 64
