"""Operational side of model versioning: loading and warm-up with load records, health checks, guarded swaps with drain
and automatic rollback, lineage (tags, parent versions), metric samples over time with alert subscriptions.

Reference (src/MLFramework/ModelVersioning/): ModelVersionManager.cs:31-197 (LoadVersion, UnloadVersion, WarmUpVersion,
GetLoadInfo), ModelHotSwapper.cs:35-391 (SwapVersion, RollbackVersion, CheckVersionHealth, DrainVersion, GetSwapStatus,
in-flight counters), ModelRegistry.cs:73-198 (TagModel, SetParentModel, state listing), VersionMonitor.cs:42-178
(RecordMetric, GetMetrics, CompareVersions, alert subscriptions), and the records VersionLoadInfo, HealthCheckResult,
SwapResult / SwapState / SwapStatus, RollbackResult, MetricSample, MetricDelta, MetricComparison, VersionAlert,
AlertSeverity, AlertType, TimeRange.
"""
from __future__ import annotations

import enum
import threading
import time
from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, Iterable, List, Optional, Tuple

from .deployment import ModelHotSwapper, ModelMetadata, ModelRegistry


# ------------------------------------------------------------------ loading
@dataclass
class VersionLoadInfo:
    model: str
    version: str
    loaded_at: float
    load_seconds: float
    memory_bytes: int
    warmed_up: bool = False
    warmup_seconds: float = 0.0
    warmup_requests: int = 0
    source: str = ""


def _memory_of(obj: Any) -> int:
    try:
        import torch
        if isinstance(obj, torch.nn.Module):
            seen, n = set(), 0
            for t in list(obj.parameters()) + list(obj.buffers()):
                if id(t) not in seen:
                    seen.add(id(t))
                    n += t.numel() * t.element_size()
            return n
    except Exception:       # noqa: BLE001
        pass
    return 0


class VersionLoader:
    """``load_version(name, version, loader)`` runs ``loader()`` (which builds or reads the model), registers the result
    and records how long it took and how much memory it holds; ``warm_up_version`` pushes sample inputs through it so
    that the first real request does not pay for lazy initialisation (kernel loading, graph capture, allocator growth)."""

    def __init__(self, registry: Optional[ModelRegistry] = None, clock: Callable[[], float] = time.time):
        self.reg = registry or ModelRegistry()
        self._info: Dict[Tuple[str, str], VersionLoadInfo] = {}
        self._lock = threading.Lock()
        self._clock = clock

    def load_version(self, name: str, version: str, loader: Callable[[], Any], source: str = "", **tags) -> VersionLoadInfo:
        with self._lock:
            if (name, version) in self._info:
                raise ValueError(f"{name}:{version} is already loaded")
        t0 = time.perf_counter()
        model = loader()
        dt = time.perf_counter() - t0
        self.reg.register(model, ModelMetadata(name, version, tags=dict(tags)))
        info = VersionLoadInfo(name, version, self._clock(), dt, _memory_of(model), source=source)
        with self._lock:
            self._info[(name, version)] = info
        return info

    def unload_version(self, name: str, version: str):
        with self._lock:
            if (name, version) not in self._info:
                raise KeyError(f"{name}:{version} is not loaded")
            del self._info[(name, version)]
        self.reg.unregister(name, version)

    def is_version_loaded(self, name: str, version: str) -> bool:
        with self._lock:
            return (name, version) in self._info

    def loaded_versions(self, name: str) -> List[str]:
        with self._lock:
            return sorted(v for (n, v) in self._info if n == name)

    def warm_up_version(self, name: str, version: str, samples: Iterable[Any], run: Optional[Callable[[Any, Any], Any]] = None) -> VersionLoadInfo:
        info = self.get_load_info(name, version)
        model = self.reg.get(name, version)
        call = run or (lambda m, x: m(x))
        t0, n = time.perf_counter(), 0
        for x in samples:
            call(model, x)
            n += 1
        info.warmed_up, info.warmup_seconds, info.warmup_requests = n > 0, time.perf_counter() - t0, n
        return info

    def get_load_info(self, name: str, version: str) -> VersionLoadInfo:
        with self._lock:
            if (name, version) not in self._info:
                raise KeyError(f"{name}:{version} is not loaded")
            return self._info[(name, version)]

    def total_memory_bytes(self) -> int:
        with self._lock:
            return sum(i.memory_bytes for i in self._info.values())


# ------------------------------------------------------------------ lineage
class ModelLineage:
    """Tags (``"stable"``, ``"candidate"`` ... -> one version each per model) and parent links (fine-tuned from)."""

    def __init__(self):
        self._tags: Dict[Tuple[str, str], str] = {}
        self._parent: Dict[Tuple[str, str], Tuple[str, str]] = {}

    def tag(self, name: str, version: str, tag: str):
        if not tag:
            raise ValueError("tag must not be empty")
        self._tags[(name, tag)] = version

    def resolve(self, name: str, tag: str) -> Optional[str]:
        return self._tags.get((name, tag))

    def tags_of(self, name: str, version: str) -> List[str]:
        return sorted(t for (n, t), v in self._tags.items() if n == name and v == version)

    def untag(self, name: str, tag: str) -> bool:
        return self._tags.pop((name, tag), None) is not None

    def set_parent(self, name: str, version: str, parent_name: str, parent_version: str):
        node, cur = (name, version), (parent_name, parent_version)
        while cur is not None:
            if cur == node:
                raise ValueError("a version cannot descend from itself")
            cur = self._parent.get(cur)
        self._parent[node] = (parent_name, parent_version)

    def parent(self, name: str, version: str) -> Optional[Tuple[str, str]]:
        return self._parent.get((name, version))

    def ancestry(self, name: str, version: str) -> List[Tuple[str, str]]:
        out, cur = [], self._parent.get((name, version))
        while cur is not None:
            out.append(cur)
            cur = self._parent.get(cur)
        return out

    def children(self, name: str, version: str) -> List[Tuple[str, str]]:
        return sorted(k for k, p in self._parent.items() if p == (name, version))


# ------------------------------------------------------------------ metrics over time and alerts
class AlertSeverity(enum.Enum):
    INFO = 0
    WARNING = 1
    CRITICAL = 2


class AlertType(enum.Enum):
    HIGH_ERROR_RATE = "high_error_rate"
    HIGH_LATENCY = "high_latency"
    LOW_THROUGHPUT = "low_throughput"
    MEMORY_EXCEEDED = "memory_exceeded"
    ANOMALY = "anomaly"


@dataclass
class MetricSample:
    timestamp: float
    latency_ms: float
    success: bool = True
    memory_mb: float = 0.0
    custom: Dict[str, float] = field(default_factory=dict)


@dataclass
class TimeRange:
    start: float = 0.0
    end: float = float("inf")

    def contains(self, t: float) -> bool:
        return self.start <= t <= self.end


@dataclass
class VersionMetrics:
    model: str
    version: str
    total_requests: int = 0
    error_rate: float = 0.0
    latency_mean_ms: float = 0.0
    latency_p50_ms: float = 0.0
    latency_p95_ms: float = 0.0
    latency_p99_ms: float = 0.0
    throughput_rps: float = 0.0
    memory_mean_mb: float = 0.0


@dataclass
class MetricDelta:
    metric: str
    v1: float
    v2: float
    lower_is_better: bool = True

    @property
    def absolute(self) -> float:
        return self.v2 - self.v1

    @property
    def relative(self) -> float:
        if self.v1:
            return (self.v2 - self.v1) / abs(self.v1)
        return 0.0 if self.v2 == 0 else float("inf") * (1 if self.v2 > 0 else -1)      # from zero: any change is unbounded

    @property
    def improved(self) -> bool:
        return self.absolute < 0 if self.lower_is_better else self.absolute > 0


@dataclass
class MetricComparison:
    model: str
    v1: str
    v2: str
    deltas: Dict[str, MetricDelta]

    def regressions(self, tolerance: float = 0.05) -> List[str]:
        return sorted(k for k, d in self.deltas.items() if not d.improved and abs(d.relative) > tolerance)

    @property
    def v2_is_better(self) -> bool:
        return sum(d.improved for d in self.deltas.values()) > len(self.deltas) / 2


@dataclass
class VersionAlert:
    model: str
    version: str
    type: AlertType
    severity: AlertSeverity
    message: str
    value: float
    threshold: float
    timestamp: float = field(default_factory=time.time)


def _pct(s: List[float], q: float) -> float:
    if not s:
        return 0.0
    pos = q * (len(s) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (pos - lo)


class TimedVersionMonitor:
    """Samples with timestamps (bounded per version), metrics over a time range, version comparison with deltas, and
    alerts pushed to subscribers. An alert of one type for one version is raised again only after ``cooldown_s``."""

    def __init__(self, max_samples: int = 10_000, error_rate_threshold: float = 0.05, latency_p99_ms_threshold: float = 1000.0,
                 memory_mb_threshold: Optional[float] = None, min_samples: int = 20, cooldown_s: float = 60.0, clock: Callable[[], float] = time.time):
        self.max_samples, self.min_samples, self.cooldown_s, self._clock = max_samples, min_samples, cooldown_s, clock
        self.thr_err, self.thr_lat, self.thr_mem = error_rate_threshold, latency_p99_ms_threshold, memory_mb_threshold
        self._s: Dict[Tuple[str, str], Deque[MetricSample]] = defaultdict(lambda: deque(maxlen=max_samples))
        self._subs: List[Callable[[VersionAlert], None]] = []
        self._last_alert: Dict[Tuple[str, str, AlertType], float] = {}
        self.alerts: List[VersionAlert] = []
        self._lock = threading.Lock()

    def subscribe_to_alerts(self, cb: Callable[[VersionAlert], None]):
        self._subs.append(cb)

    def unsubscribe_from_alerts(self, cb: Callable[[VersionAlert], None]) -> bool:
        if cb in self._subs:
            self._subs.remove(cb)
            return True
        return False

    def record_metric(self, model: str, version: str, sample: MetricSample):
        with self._lock:
            self._s[(model, version)].append(sample)
        self._check(model, version)

    def record(self, model: str, version: str, latency_ms: float, success: bool = True, memory_mb: float = 0.0, **custom):
        self.record_metric(model, version, MetricSample(self._clock(), latency_ms, success, memory_mb, dict(custom)))

    def get_metrics(self, model: str, version: str, time_range: Optional[TimeRange] = None) -> VersionMetrics:
        with self._lock:
            ss = [s for s in self._s.get((model, version), ()) if time_range is None or time_range.contains(s.timestamp)]
        m = VersionMetrics(model, version, len(ss))
        if not ss:
            return m
        lat = sorted(s.latency_ms for s in ss)
        m.error_rate = sum(1 for s in ss if not s.success) / len(ss)
        m.latency_mean_ms, m.latency_p50_ms, m.latency_p95_ms, m.latency_p99_ms = sum(lat) / len(lat), _pct(lat, 0.5), _pct(lat, 0.95), _pct(lat, 0.99)
        span = ss[-1].timestamp - ss[0].timestamp
        m.throughput_rps = (len(ss) - 1) / span if span > 0 else 0.0
        m.memory_mean_mb = sum(s.memory_mb for s in ss) / len(ss)
        return m

    def compare_versions(self, model: str, v1: str, v2: str, time_range: Optional[TimeRange] = None) -> MetricComparison:
        a, b = self.get_metrics(model, v1, time_range), self.get_metrics(model, v2, time_range)
        d = {"error_rate": MetricDelta("error_rate", a.error_rate, b.error_rate), "latency_mean_ms": MetricDelta("latency_mean_ms", a.latency_mean_ms, b.latency_mean_ms),
             "latency_p99_ms": MetricDelta("latency_p99_ms", a.latency_p99_ms, b.latency_p99_ms),
             "throughput_rps": MetricDelta("throughput_rps", a.throughput_rps, b.throughput_rps, lower_is_better=False),
             "memory_mean_mb": MetricDelta("memory_mean_mb", a.memory_mean_mb, b.memory_mean_mb)}
        return MetricComparison(model, v1, v2, d)

    def clear_metrics(self, model: str, version: str):
        with self._lock:
            self._s.pop((model, version), None)

    def _raise(self, model, version, type_, sev, msg, value, thr):
        now = self._clock()
        k = (model, version, type_)
        if now - self._last_alert.get(k, -1e30) < self.cooldown_s:
            return
        self._last_alert[k] = now
        a = VersionAlert(model, version, type_, sev, msg, value, thr, now)
        self.alerts.append(a)
        for cb in list(self._subs):
            cb(a)

    def _check(self, model: str, version: str):
        m = self.get_metrics(model, version)
        if m.total_requests < self.min_samples:
            return
        if m.error_rate > self.thr_err:
            sev = AlertSeverity.CRITICAL if m.error_rate > 2 * self.thr_err else AlertSeverity.WARNING
            self._raise(model, version, AlertType.HIGH_ERROR_RATE, sev, f"error rate {m.error_rate:.1%} above {self.thr_err:.1%}", m.error_rate, self.thr_err)
        if m.latency_p99_ms > self.thr_lat:
            sev = AlertSeverity.CRITICAL if m.latency_p99_ms > 2 * self.thr_lat else AlertSeverity.WARNING
            self._raise(model, version, AlertType.HIGH_LATENCY, sev, f"p99 latency {m.latency_p99_ms:.0f} ms above {self.thr_lat:.0f} ms", m.latency_p99_ms, self.thr_lat)
        if self.thr_mem is not None and m.memory_mean_mb > self.thr_mem:
            self._raise(model, version, AlertType.MEMORY_EXCEEDED, AlertSeverity.WARNING, f"memory {m.memory_mean_mb:.0f} MB above {self.thr_mem:.0f} MB", m.memory_mean_mb, self.thr_mem)


# ------------------------------------------------------------------ guarded swap
class SwapState(enum.Enum):
    IDLE = "idle"
    HEALTH_CHECK = "health_check"
    SWAPPING = "swapping"
    DRAINING = "draining"
    COMPLETED = "completed"
    FAILED = "failed"
    ROLLED_BACK = "rolled_back"


@dataclass
class HealthCheckResult:
    healthy: bool
    model: str
    version: str
    checks: Dict[str, bool] = field(default_factory=dict)
    message: str = ""


@dataclass
class SwapResult:
    success: bool
    model: str
    from_version: Optional[str]
    to_version: str
    drained: bool = False
    duration_s: float = 0.0
    message: str = ""


@dataclass
class RollbackResult:
    success: bool
    model: str
    from_version: Optional[str]
    to_version: Optional[str]
    message: str = ""


@dataclass
class SwapStatus:
    model: str
    state: SwapState
    active_version: Optional[str]
    target_version: Optional[str] = None
    in_flight: Dict[str, int] = field(default_factory=dict)


class GuardedVersionSwapper:
    """Swap with pre-checks and a way back: the target must be loaded and healthy (optionally probed with a canary
    call), traffic moves at once, the old version drains within a timeout; if the canary fails AFTER the switch the
    previous version is restored."""

    def __init__(self, swapper: ModelHotSwapper, loader: Optional[VersionLoader] = None, monitor: Optional[TimedVersionMonitor] = None,
                 max_error_rate: float = 0.1, max_p99_ms: Optional[float] = None):
        self.sw, self.loader, self.mon = swapper, loader, monitor
        self.max_error_rate, self.max_p99_ms = max_error_rate, max_p99_ms
        self._state: Dict[str, SwapState] = defaultdict(lambda: SwapState.IDLE)
        self._target: Dict[str, Optional[str]] = {}
        self._inflight: Dict[Tuple[str, str], int] = defaultdict(int)
        self._lock = threading.Lock()
        self.log: List[SwapResult] = []

    # ---- in-flight accounting for callers that do not go through ``serve``
    def increment_in_flight(self, model: str, version: str):
        with self._lock:
            self._inflight[(model, version)] += 1

    def decrement_in_flight(self, model: str, version: str):
        with self._lock:
            if self._inflight[(model, version)] <= 0:
                raise ValueError(f"{model}:{version} has no request in flight")
            self._inflight[(model, version)] -= 1

    def check_version_health(self, model: str, version: str, canary: Optional[Callable[[Any], bool]] = None) -> HealthCheckResult:
        checks: Dict[str, bool] = {}
        try:
            obj = self.sw.reg.get(model, version)
            checks["registered"] = True
        except KeyError:
            return HealthCheckResult(False, model, version, {"registered": False}, "version is not registered")
        if self.loader is not None:
            checks["loaded"] = self.loader.is_version_loaded(model, version)
        if self.mon is not None:
            m = self.mon.get_metrics(model, version)
            if m.total_requests:
                checks["error_rate"] = m.error_rate <= self.max_error_rate
                if self.max_p99_ms is not None:
                    checks["latency"] = m.latency_p99_ms <= self.max_p99_ms
        if canary is not None:
            try:
                checks["canary"] = bool(canary(obj))
            except Exception as e:       # noqa: BLE001 - a canary that raises is a failed check
                checks["canary"] = False
                return HealthCheckResult(False, model, version, checks, f"canary raised: {e}")
        bad = [k for k, ok in checks.items() if not ok]
        return HealthCheckResult(not bad, model, version, checks, "" if not bad else "failed: " + ", ".join(bad))

    def drain_version(self, model: str, version: str, timeout_s: float = 30.0) -> bool:
        end = time.monotonic() + timeout_s
        if not self.sw.refs.wait_idle(f"{model}:{version}", timeout_s):
            return False
        while True:
            with self._lock:
                if self._inflight[(model, version)] == 0:
                    return True
            if time.monotonic() >= end:
                return False
            time.sleep(0.005)

    def swap_version(self, model: str, to_version: str, canary: Optional[Callable[[Any], bool]] = None, drain_timeout_s: float = 30.0) -> SwapResult:
        t0 = time.perf_counter()
        old = self.sw.active.get(model)
        self._target[model] = to_version
        self._state[model] = SwapState.HEALTH_CHECK
        h = self.check_version_health(model, to_version, canary)
        if not h.healthy:
            self._state[model] = SwapState.FAILED
            r = SwapResult(False, model, old, to_version, message=h.message)
            self.log.append(r)
            return r
        self._state[model] = SwapState.SWAPPING
        self.sw.activate(model, to_version)
        drained = True
        if old is not None and old != to_version:
            self._state[model] = SwapState.DRAINING
            drained = self.drain_version(model, old, drain_timeout_s)
        if canary is not None:                                   # once more, on the live path
            after = self.check_version_health(model, to_version, canary)
            if not after.healthy and old is not None:
                self.sw.activate(model, old)
                self._state[model] = SwapState.ROLLED_BACK
                r = SwapResult(False, model, old, to_version, drained, time.perf_counter() - t0, "rolled back: " + after.message)
                self.log.append(r)
                return r
        self._state[model] = SwapState.COMPLETED
        r = SwapResult(True, model, old, to_version, drained, time.perf_counter() - t0, "" if drained else "old version still had requests at the drain deadline")
        self.log.append(r)
        return r

    def rollback_version(self, model: str, target_version: Optional[str] = None) -> RollbackResult:
        cur = self.sw.active.get(model)
        if target_version is None:
            hist = self.sw.history[model]
            target_version = next((v for v in reversed(hist[:-1]) if v != cur), None)
        if target_version is None:
            return RollbackResult(False, model, cur, None, "no earlier version to go back to")
        try:
            self.sw.reg.get(model, target_version)
        except KeyError:
            return RollbackResult(False, model, cur, target_version, "target version is not registered")
        self.sw.activate(model, target_version)
        self._state[model] = SwapState.ROLLED_BACK
        return RollbackResult(True, model, cur, target_version)

    def get_swap_status(self, model: str) -> SwapStatus:
        with self._lock:
            infl = {v: n for (m, v), n in self._inflight.items() if m == model and n}
        return SwapStatus(model, self._state[model], self.sw.active.get(model), self._target.get(model), infl)
