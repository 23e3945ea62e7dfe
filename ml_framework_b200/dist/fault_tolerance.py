"""Communication fault tolerance, algorithm selection, profiling and group helpers.

* ``FaultTolerantCommunication`` wraps any process group: every collective runs under a timeout
  and a retry loop driven by an error -> strategy table
  (src/MLFramework/Communication/FaultTolerance/FaultTolerantCommunication.cs:67-138,
  ErrorRecoveryManager.cs:60-139: Timeout -> Retry, RankMismatch -> Abort, IOError -> Retry).
* ``TimeoutManager`` (TimeoutManager.cs:33-90), ``HealthMonitor`` (heartbeat table: Healthy ->
  Unresponsive after 30 s -> Failed after 60 s, HealthMonitor.cs:40-155).
* ``AlgorithmSelector`` keeps the reference's size thresholds (AlgorithmSelector.cs:24-65) for
  switched fabrics that need them, and adds the NVSwitch rule used here: every peer is one hop, so
  small messages go one-shot (each rank reads all peers) and large ones two-shot (reduce-scatter +
  all-gather); ring / tree depth buys nothing.
* ``RingAllReduce`` / ``ChunkManager``: the reference's software ring over send/recv
  (src/MLFramework/Distributed/RingAllReduce.cs:30-217, ChunkManager.cs:124-145), kept as an
  executable statement of the schedule and for backends without collectives.
* ``CommunicationProfiler`` (Optimizations/CommunicationProfiler.cs:40-146), ``NCCLConfig``
  (Backends/NCCLConfig.cs:59-154), process-group helpers (ProcessGroupHelpers.cs:15-74),
  ``ComputeCommunicationOverlap`` and ``CommunicationOperationQueue`` (Communication/Async/*.cs).

All failure handling is host-side; nothing here ever asks a GPU to fault or hang.
"""
from __future__ import annotations

import enum
import os
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .process_group import CommunicationError, CommunicationTimeout, RankMismatchError, ReduceOp


class ErrorSeverity(enum.Enum):
    LOW = 1
    MEDIUM = 2
    HIGH = 3
    CRITICAL = 4


class RecoveryStrategy(enum.Enum):
    RETRY = "retry"
    FALLBACK_TO_DIFFERENT_BACKEND = "fallback_backend"
    USE_DIFFERENT_ALGORITHM = "different_algorithm"
    ABORT = "abort"


@dataclass
class CommunicationConfig:
    """src/MLFramework/Distributed/Communication/CommunicationConfig.cs:6-36."""
    timeout_ms: int = 300_000
    enable_logging: bool = False
    use_pinned_memory: bool = True
    max_retries: int = 3
    retry_delay_ms: int = 100

    def validate(self):
        if self.timeout_ms <= 0 or self.max_retries < 0 or self.retry_delay_ms < 0:
            raise ValueError("invalid communication configuration")


@dataclass
class ErrorRecord:
    op: str
    error: str
    strategy: RecoveryStrategy
    time: float


class ErrorRecoveryManager:
    def __init__(self):
        self.strategies: Dict[type, RecoveryStrategy] = {
            CommunicationTimeout: RecoveryStrategy.RETRY, TimeoutError: RecoveryStrategy.RETRY,
            RankMismatchError: RecoveryStrategy.ABORT, IOError: RecoveryStrategy.RETRY, OSError: RecoveryStrategy.RETRY,
            CommunicationError: RecoveryStrategy.RETRY,
        }
        self.history: List[ErrorRecord] = []

    def register(self, exc_type: type, strategy: RecoveryStrategy):
        self.strategies[exc_type] = strategy

    def handle_error(self, op: str, e: BaseException) -> RecoveryStrategy:
        strat = RecoveryStrategy.ABORT
        for t in type(e).__mro__:
            if t in self.strategies:
                strat = self.strategies[t]
                break
        self.history.append(ErrorRecord(op, repr(e), strat, time.time()))
        return strat

    def get_statistics(self) -> Dict:
        by: Dict[str, int] = {}
        for r in self.history:
            by[r.strategy.value] = by.get(r.strategy.value, 0) + 1
        return {"total_errors": len(self.history), "by_strategy": by}


class TimeoutManager:
    def __init__(self, clock=time.time):
        self.clock = clock
        self._deadlines: Dict[int, float] = {}
        self._next = 0

    def start_timeout(self, seconds: float) -> int:
        self._next += 1
        self._deadlines[self._next] = self.clock() + seconds
        return self._next

    def cancel_timeout(self, handle: int):
        self._deadlines.pop(handle, None)

    def extend_timeout(self, handle: int, seconds: float):
        if handle in self._deadlines:
            self._deadlines[handle] += seconds

    def is_expired(self, handle: int) -> bool:
        return handle in self._deadlines and self.clock() > self._deadlines[handle]


class RankHealth(enum.Enum):
    HEALTHY = "healthy"
    UNRESPONSIVE = "unresponsive"
    FAILED = "failed"


class HealthMonitor:
    def __init__(self, world_size: int, unresponsive_after_s: float = 30.0, failed_after_s: float = 60.0, clock=time.time):
        self.world_size, self.t_unresp, self.t_fail, self.clock = world_size, unresponsive_after_s, failed_after_s, clock
        now = clock()
        self.last: Dict[int, float] = {r: now for r in range(world_size)}

    def update_heartbeat(self, rank: int):
        if not (0 <= rank < self.world_size):
            raise ValueError("rank out of range")
        self.last[rank] = self.clock()

    def status(self, rank: int) -> RankHealth:
        age = self.clock() - self.last[rank]
        if age >= self.t_fail:
            return RankHealth.FAILED
        return RankHealth.UNRESPONSIVE if age >= self.t_unresp else RankHealth.HEALTHY

    def get_healthy_ranks(self) -> List[int]:
        return [r for r in range(self.world_size) if self.status(r) == RankHealth.HEALTHY]

    def get_failed_ranks(self) -> List[int]:
        return [r for r in range(self.world_size) if self.status(r) == RankHealth.FAILED]


class FaultTolerantCommunication:
    """Decorator: ``ft.all_reduce(t)`` = retry/timeout-guarded ``pg.all_reduce(t)``."""

    _OPS = ("all_reduce", "broadcast", "reduce", "all_gather", "reduce_scatter", "barrier", "send", "recv",
            "all_gather_into", "all_gather_object", "broadcast_object")

    def __init__(self, pg, config: Optional[CommunicationConfig] = None, recovery: Optional[ErrorRecoveryManager] = None,
                 sleep: Callable[[float], None] = time.sleep, fallback=None):
        self.pg, self.cfg = pg, config or CommunicationConfig()
        self.cfg.validate()
        self.recovery, self.sleep, self.fallback = recovery or ErrorRecoveryManager(), sleep, fallback
        self.retries = 0

    @property
    def rank(self): return self.pg.rank
    @property
    def world_size(self): return self.pg.world_size

    def execute_with_retry(self, op: str, fn: Callable):
        attempt = 0
        while True:
            try:
                return self._with_timeout(fn)
            except BaseException as e:  # noqa: BLE001
                strat = self.recovery.handle_error(op, e)
                if strat == RecoveryStrategy.FALLBACK_TO_DIFFERENT_BACKEND and self.fallback is not None:
                    return getattr(self.fallback, op)
                if strat != RecoveryStrategy.RETRY or attempt >= self.cfg.max_retries:
                    raise
                attempt += 1
                self.retries += 1
                self.sleep(self.cfg.retry_delay_ms / 1e3)

    def _with_timeout(self, fn: Callable):
        box: Dict[str, object] = {}

        def run():
            try:
                box["r"] = fn()
            except BaseException as e:  # noqa: BLE001
                box["e"] = e
        t = threading.Thread(target=run, daemon=True)
        t.start()
        t.join(self.cfg.timeout_ms / 1e3)
        if t.is_alive():
            raise CommunicationTimeout(f"operation exceeded {self.cfg.timeout_ms} ms")
        if "e" in box:
            raise box["e"]  # type: ignore
        return box.get("r")

    def __getattr__(self, name):
        if name in self._OPS:
            target = getattr(self.pg, name)
            return lambda *a, **k: self.execute_with_retry(name, lambda: target(*a, **k))
        return getattr(self.pg, name)


# ------------------------------------------------------------------ algorithm selection
class CollectiveAlgorithm(enum.Enum):
    RECURSIVE_DOUBLING = "recursive_doubling"
    RABENSEIFNER = "rabenseifner"
    RING = "ring"
    TREE = "tree"
    ONE_SHOT = "one_shot"
    TWO_SHOT = "two_shot"


class AlgorithmSelector:
    def __init__(self, nvswitch: bool = True, one_shot_max_bytes: int = 4 << 20):
        self.nvswitch, self.one_shot_max = nvswitch, one_shot_max_bytes

    def select_all_reduce(self, nbytes: int, world: int) -> CollectiveAlgorithm:
        if self.nvswitch:
            return CollectiveAlgorithm.ONE_SHOT if nbytes <= self.one_shot_max else CollectiveAlgorithm.TWO_SHOT
        if nbytes < 4 * 1024 and world <= 8:
            return CollectiveAlgorithm.RECURSIVE_DOUBLING
        if nbytes < 1024 * 1024 and world <= 16:
            return CollectiveAlgorithm.RABENSEIFNER
        return CollectiveAlgorithm.RING if nbytes < 16 * 1024 * 1024 else CollectiveAlgorithm.TREE

    def select_all_gather(self, nbytes: int, world: int) -> CollectiveAlgorithm:
        return CollectiveAlgorithm.ONE_SHOT if self.nvswitch else CollectiveAlgorithm.RING

    def select_reduce_scatter(self, nbytes: int, world: int) -> CollectiveAlgorithm:
        return CollectiveAlgorithm.ONE_SHOT if self.nvswitch else CollectiveAlgorithm.RABENSEIFNER


# ------------------------------------------------------------------ software ring
class ChunkManager:
    """Even split; the first ``N mod W`` chunks get one extra element."""

    def __init__(self, numel: int, world: int):
        base, extra = divmod(numel, world)
        self.sizes = [base + (1 if i < extra else 0) for i in range(world)]
        self.offsets = [sum(self.sizes[:i]) for i in range(world)]

    def chunk(self, t: torch.Tensor, i: int) -> torch.Tensor:
        return t.view(-1)[self.offsets[i]:self.offsets[i] + self.sizes[i]]


class RingAllReduce:
    """Reduce-scatter (W-1 steps) then all-gather (W-1 steps) over send/recv."""

    def __init__(self, pg):
        self.pg = pg

    def _swap(self, out: torch.Tensor, dst: int, buf: torch.Tensor, src: int):
        """Send to the next rank and receive from the previous one with both transfers posted before either is waited
        for: every rank of the ring sends at the same moment, so a blocking send would wait for a receive that its
        peer only posts after its own send."""
        for w in self.pg.batch_isend_irecv([("send", out, dst), ("recv", buf, src)]):
            w.wait()

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        W, r = self.pg.world_size, self.pg.rank
        if W == 1:
            return t
        flat = t.contiguous().view(-1)
        cm = ChunkManager(flat.numel(), W)
        nxt, prv = (r + 1) % W, (r - 1) % W
        for step in range(W - 1):                 # reduce-scatter
            si, ri = (r - step) % W, (r - step - 1) % W
            buf = torch.empty_like(cm.chunk(flat, ri))
            self._swap(cm.chunk(flat, si).clone(), nxt, buf, prv)
            c = cm.chunk(flat, ri)
            if op in (ReduceOp.SUM, ReduceOp.AVG):
                c.add_(buf)
            elif op == ReduceOp.MAX:
                torch.maximum(c, buf, out=c)
            elif op == ReduceOp.MIN:
                torch.minimum(c, buf, out=c)
            else:
                c.mul_(buf)
        for step in range(W - 1):                 # all-gather
            si, ri = (r + 1 - step) % W, (r - step) % W
            buf = torch.empty_like(cm.chunk(flat, ri))
            self._swap(cm.chunk(flat, si).clone(), nxt, buf, prv)
            cm.chunk(flat, ri).copy_(buf)
        if op == ReduceOp.AVG:
            flat.div_(W)
        if flat.data_ptr() != t.data_ptr():
            t.copy_(flat.view_as(t))
        return t


# ------------------------------------------------------------------ profiling / config / helpers
@dataclass
class _OpStat:
    count: int = 0
    bytes: int = 0
    seconds: float = 0.0


class CommunicationProfiler:
    def __init__(self):
        self.stats: Dict[str, _OpStat] = {}

    def profile(self, op: str, nbytes: int, fn: Callable, algorithm: str = ""):
        t0 = time.perf_counter()
        r = fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        s = self.stats.setdefault(f"{op}:{algorithm}" if algorithm else op, _OpStat())
        s.count += 1
        s.bytes += nbytes
        s.seconds += time.perf_counter() - t0
        return r

    def get_statistics(self) -> Dict[str, Dict]:
        return {k: {"count": s.count, "bytes": s.bytes, "seconds": s.seconds,
                    "GBps": s.bytes / s.seconds / 1e9 if s.seconds else 0.0} for k, s in self.stats.items()}


@dataclass
class NCCLConfig:
    algorithm: str = ""            # "", "Ring", "Tree", "NVLS"
    tree_threshold_bytes: int = 1 << 20
    num_channels: int = 0
    buffer_size: int = 4 << 20
    timeout_ms: int = 300_000
    debug: str = ""
    blocking_wait: bool = False

    def apply(self, env=os.environ):
        if self.debug:
            env["NCCL_DEBUG"] = self.debug
        if self.buffer_size:
            env["NCCL_BUFFSIZE"] = str(self.buffer_size)
        if self.num_channels:
            env["NCCL_NCHANNELS"] = str(self.num_channels)
        if self.blocking_wait:
            env["NCCL_BLOCKING_WAIT"] = "1"
        if self.algorithm:
            env["NCCL_ALGO"] = self.algorithm
        return env

    @classmethod
    def create_default(cls): return cls()
    @classmethod
    def create_high_performance(cls): return cls(num_channels=32, buffer_size=16 << 20)
    @classmethod
    def create_debug(cls): return cls(debug="INFO", blocking_wait=True)


def create_split_groups(world_size: int, group_size: int) -> List[List[int]]:
    if world_size % group_size:
        raise ValueError("world size must be divisible by the group size")
    return [list(range(i, i + group_size)) for i in range(0, world_size, group_size)]


def create_pipeline_groups(world_size: int, num_stages: int) -> List[List[int]]:
    """Ranks r, r + W/p, r + 2W/p, ... form one pipeline."""
    if world_size % num_stages:
        raise ValueError("world size must be divisible by the number of stages")
    per = world_size // num_stages
    return [[r + s * per for s in range(num_stages)] for r in range(per)]


def create_data_parallel_groups(world_size: int, model_parallel_size: int) -> List[List[int]]:
    if world_size % model_parallel_size:
        raise ValueError("world size must be divisible by the model-parallel size")
    return [list(range(i, world_size, model_parallel_size)) for i in range(model_parallel_size)]


class ProcessGroupManager:
    """Named sub-groups (src/MLFramework/Communication/ProcessGroupManager.cs:68-104)."""

    def __init__(self, base):
        self.base, self.groups = base, {}

    def create_group(self, name: str, ranks: Sequence[int]):
        if name in self.groups:
            raise ValueError(f"group {name!r} exists")
        self.groups[name] = self.base.new_subgroup(list(ranks)) if hasattr(self.base, "new_subgroup") else list(ranks)
        return self.groups[name]

    def get_group(self, name: str):
        return self.groups[name]


class PinnedMemoryManager:
    """Pool of page-locked host buffers with a byte cap (Optimizations/PinnedMemoryManager.cs:31-42: 1 GB)."""

    def __init__(self, cap_bytes: int = 1 << 30):
        self.cap, self.used, self._free = cap_bytes, 0, {}

    def get(self, nbytes: int) -> torch.Tensor:
        pool = self._free.get(nbytes)
        if pool:
            return pool.pop()
        if self.used + nbytes > self.cap:
            raise MemoryError("pinned memory cap exceeded")
        self.used += nbytes
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=torch.cuda.is_available())

    def put(self, buf: torch.Tensor):
        self._free.setdefault(buf.numel(), []).append(buf)


class CommunicationOperationQueue:
    def __init__(self):
        self._ops: List = []

    def enqueue(self, work):
        self._ops.append(work)
        return work

    def wait_for_all(self):
        for w in self._ops:
            w.wait()
        self._ops = []

    def wait_for_any(self):
        while self._ops:
            for i, w in enumerate(self._ops):
                if w.is_completed():
                    w.wait()
                    return self._ops.pop(i)
            time.sleep(0.0005)
        return None


class ComputeCommunicationOverlap:
    """Start a collective, run compute, then wait (Communication/Async/ComputeCommunicationOverlap.cs:17-65)."""

    def __init__(self, pg):
        self.pg = pg

    def compute_while_communicating(self, tensor: torch.Tensor, compute: Callable, op: ReduceOp = ReduceOp.SUM):
        work = self.pg.all_reduce(tensor, op, async_op=True)
        result = compute()
        work.wait()
        return result, tensor

    def pipeline(self, tensors: Sequence[torch.Tensor], compute: Callable[[int], object], op: ReduceOp = ReduceOp.SUM):
        out, work = [], None
        for i, t in enumerate(tensors):
            nxt = self.pg.all_reduce(t, op, async_op=True)
            out.append(compute(i))
            if work is not None:
                work.wait()
            work = nxt
        if work is not None:
            work.wait()
        return out
