"""Metric collection and exporters (console, Prometheus text format, StatsD lines).

Reference: src/MLFramework/Data/Metrics/MetricsCollector.cs, PerformanceCounter.cs, PrometheusExporter.cs,
StatsDExporter.cs, ConsoleExporter.cs, MetricsReporter.cs; scheduler metrics with circular buffers and
sliding-window counters (src/MLFramework/Inference/ContinuousBatching/Metrics/*).
"""
from __future__ import annotations

import socket
import threading
import time
from collections import deque
from typing import Callable, Deque, Dict, List, Optional, Tuple


class CircularBuffer:
    def __init__(self, capacity: int):
        self._d: Deque[float] = deque(maxlen=capacity)

    def add(self, v: float):
        self._d.append(v)

    def values(self) -> List[float]:
        return list(self._d)

    def mean(self) -> float:
        return sum(self._d) / len(self._d) if self._d else 0.0

    def percentile(self, q: float) -> float:
        from .profiler import percentile
        return percentile(sorted(self._d), q)


class SlidingWindowCounter:
    def __init__(self, window_s: float = 60.0, clock: Callable[[], float] = time.monotonic):
        self.window, self._clock = window_s, clock
        self._ev: Deque[Tuple[float, float]] = deque()

    def add(self, n: float = 1.0):
        self._ev.append((self._clock(), n))
        self._trim()

    def _trim(self):
        t = self._clock() - self.window
        while self._ev and self._ev[0][0] < t:
            self._ev.popleft()

    def total(self) -> float:
        self._trim()
        return sum(n for _, n in self._ev)

    def rate(self) -> float:
        return self.total() / self.window


class MetricsCollector:
    def __init__(self):
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.timings: Dict[str, CircularBuffer] = {}
        self._lock = threading.Lock()

    def inc(self, name: str, n: float = 1.0):
        with self._lock:
            self.counters[name] = self.counters.get(name, 0.0) + n

    def gauge(self, name: str, v: float):
        with self._lock:
            self.gauges[name] = v

    def timing(self, name: str, seconds: float):
        with self._lock:
            self.timings.setdefault(name, CircularBuffer(1024)).add(seconds)

    def time(self, name: str):
        col = self

        class _T:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *a):
                col.timing(name, time.perf_counter() - self.t0)
        return _T()

    def snapshot(self) -> Dict[str, Dict[str, float]]:
        with self._lock:
            return {"counters": dict(self.counters), "gauges": dict(self.gauges),
                    "timings": {k: {"count": len(v.values()), "mean": v.mean(), "p50": v.percentile(50), "p99": v.percentile(99)}
                                for k, v in self.timings.items()}}


class PerformanceCounter:
    """One named duration series: count, total, min, max, mean and the last value
    (src/MLFramework/Data/Metrics/PerformanceCounter.cs)."""

    def __init__(self, name: str):
        self.name = name
        self.count, self.total_s, self.min_s, self.max_s, self.last_s = 0, 0.0, float("inf"), 0.0, 0.0
        self._lock = threading.Lock()

    def record(self, seconds: float):
        with self._lock:
            self.count += 1
            self.total_s += seconds
            self.min_s, self.max_s, self.last_s = min(self.min_s, seconds), max(self.max_s, seconds), seconds

    @property
    def mean_s(self) -> float:
        return self.total_s / self.count if self.count else 0.0

    def reset(self):
        with self._lock:
            self.count, self.total_s, self.min_s, self.max_s, self.last_s = 0, 0.0, float("inf"), 0.0, 0.0

    def as_dict(self) -> Dict[str, float]:
        return {"count": self.count, "total_s": self.total_s, "mean_s": self.mean_s, "min_s": self.min_s if self.count else 0.0,
                "max_s": self.max_s, "last_s": self.last_s}


class ProfilingScope:
    """``with ProfilingScope(counter_or_collector, name):`` records the block's wall time on exit, also when it raises
    (src/MLFramework/Data/Metrics/ProfilingScope.cs)."""

    def __init__(self, sink, name: Optional[str] = None):
        self.sink, self.name = sink, name
        self.elapsed_s = 0.0

    def __enter__(self):
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.elapsed_s = time.perf_counter() - self._t0
        if isinstance(self.sink, PerformanceCounter):
            self.sink.record(self.elapsed_s)
        else:
            self.sink.timing(self.name or "scope", self.elapsed_s)
        return False


class DataLoadingMetrics:
    """The input pipeline's own numbers: time per stage (fetch, collate, transfer), batches and samples served, the
    consumer's wait, queue depth, and whether the trainer or the loader is the bottleneck
    (src/MLFramework/Data/Metrics/DataLoadingMetrics.cs)."""
    STAGES = ("fetch", "collate", "transfer", "wait")

    def __init__(self):
        self.stages = {k: PerformanceCounter(k) for k in self.STAGES}
        self.batches = self.samples = 0
        self.queue_depth = CircularBuffer(256)
        self._t0 = time.perf_counter()

    def scope(self, stage: str) -> ProfilingScope:
        return ProfilingScope(self.stages[stage])

    def record_batch(self, n_samples: int, queue_depth: Optional[int] = None):
        self.batches += 1
        self.samples += n_samples
        if queue_depth is not None:
            self.queue_depth.add(queue_depth)

    def samples_per_second(self) -> float:
        dt = time.perf_counter() - self._t0
        return self.samples / dt if dt > 0 else 0.0

    def wait_fraction(self) -> float:
        """Share of the elapsed time the consumer spent waiting for a batch."""
        dt = time.perf_counter() - self._t0
        return min(1.0, self.stages["wait"].total_s / dt) if dt > 0 else 0.0

    def bottleneck(self) -> str:
        if self.wait_fraction() > 0.1:
            busy = {k: c.total_s for k, c in self.stages.items() if k != "wait"}
            return "loader:" + max(busy, key=busy.get) if any(busy.values()) else "loader"
        return "consumer"

    def snapshot(self) -> Dict[str, object]:
        return {"batches": self.batches, "samples": self.samples, "samples_per_second": self.samples_per_second(),
                "wait_fraction": self.wait_fraction(), "mean_queue_depth": self.queue_depth.mean(), "bottleneck": self.bottleneck(),
                "stages": {k: c.as_dict() for k, c in self.stages.items()}}

    def publish(self, collector: "MetricsCollector", prefix: str = "data"):
        collector.gauge(f"{prefix}.samples_per_second", self.samples_per_second())
        collector.gauge(f"{prefix}.wait_fraction", self.wait_fraction())
        collector.inc(f"{prefix}.batches", 0)
        collector.counters[f"{prefix}.batches"] = float(self.batches)
        for k, c in self.stages.items():
            collector.gauge(f"{prefix}.{k}_mean_ms", c.mean_s * 1e3)


def _prom_name(n: str) -> str:
    return "".join(c if c.isalnum() else "_" for c in n)


class PrometheusExporter:
    def __init__(self, prefix: str = "mlf"):
        self.prefix = prefix

    def render(self, snap: Dict[str, Dict]) -> str:
        out = []
        for k, v in snap["counters"].items():
            n = f"{self.prefix}_{_prom_name(k)}_total"
            out += [f"# TYPE {n} counter", f"{n} {v}"]
        for k, v in snap["gauges"].items():
            n = f"{self.prefix}_{_prom_name(k)}"
            out += [f"# TYPE {n} gauge", f"{n} {v}"]
        for k, t in snap["timings"].items():
            n = f"{self.prefix}_{_prom_name(k)}_seconds"
            out += [f"# TYPE {n} summary", f'{n}{{quantile="0.5"}} {t["p50"]}', f'{n}{{quantile="0.99"}} {t["p99"]}', f"{n}_count {t['count']}"]
        return "\n".join(out) + "\n"


class StatsDExporter:
    def __init__(self, host: str = "127.0.0.1", port: int = 8125, prefix: str = "mlf", send: Optional[Callable[[bytes], None]] = None):
        self.prefix = prefix
        if send is None:
            sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
            send = lambda b: sock.sendto(b, (host, port))
        self._send = send

    def lines(self, snap) -> List[str]:
        out = [f"{self.prefix}.{k}:{v}|c" for k, v in snap["counters"].items()]
        out += [f"{self.prefix}.{k}:{v}|g" for k, v in snap["gauges"].items()]
        out += [f"{self.prefix}.{k}:{t['mean'] * 1e3:.3f}|ms" for k, t in snap["timings"].items()]
        return out

    def export(self, snap):
        for l in self.lines(snap):
            self._send(l.encode())


class ConsoleExporter:
    def export(self, snap, printer: Callable[[str], None] = print):
        for sect in ("counters", "gauges"):
            for k, v in snap[sect].items():
                printer(f"[{sect[:-1]}] {k} = {v}")
        for k, t in snap["timings"].items():
            printer(f"[timing] {k}: n={t['count']} mean={t['mean'] * 1e3:.3f} ms p99={t['p99'] * 1e3:.3f} ms")


class MetricsReporter:
    def __init__(self, collector: MetricsCollector, exporters: List, interval_s: float = 10.0):
        self.col, self.exporters, self.interval = collector, exporters, interval_s
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None

    def report_once(self):
        snap = self.col.snapshot()
        for e in self.exporters:
            e.export(snap) if hasattr(e, "export") else e.render(snap)

    def start(self):
        def loop():
            while not self._stop.wait(self.interval):
                self.report_once()
        self._t = threading.Thread(target=loop, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=2.0)
