"""Benchmarking for the mobile runtime: runner with memory / energy monitors, scope profiler, exporters, comparator.

Reference: src/MobileRuntime/Benchmarking/{BenchmarkRunner.cs:19-173, Profiler.cs:17-134, Monitoring/MemoryMonitor.cs,
Monitoring/EnergyMonitor.cs (sampling threads, snapshots), Export/BenchmarkExporter.cs:12-119 (JSON, CSV, Markdown,
HTML), Comparison/PerformanceComparator.cs:11-46, Models/*}. The energy monitor integrates the board power NVML
reports for the GPU the model runs on (read-only; ``power_reader`` is injectable), the memory monitor samples the
process's resident set and the device allocator.
"""
from __future__ import annotations

import csv
import html
import io
import json
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch


@dataclass
class MemorySnapshot:
    samples: int = 0
    start_bytes: int = 0
    peak_bytes: int = 0
    end_bytes: int = 0
    device_peak_bytes: int = 0

    @property
    def growth_bytes(self) -> int:
        return self.end_bytes - self.start_bytes


@dataclass
class EnergySnapshot:
    samples: int = 0
    duration_s: float = 0.0
    energy_joules: float = 0.0
    average_power_w: float = 0.0
    peak_power_w: float = 0.0


class _Sampler:
    def __init__(self, interval_ms: int):
        self.interval_s = interval_ms / 1e3
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None

    def _sample(self):
        raise NotImplementedError

    def start_monitoring(self):
        if self._t is not None:
            return
        self._stop.clear()
        self._sample()

        def loop():
            while not self._stop.wait(self.interval_s):
                self._sample()
        self._t = threading.Thread(target=loop, daemon=True, name=f"mlf-{type(self).__name__}")
        self._t.start()

    def stop_monitoring(self):
        if self._t is None:
            return
        self._stop.set()
        self._t.join(timeout=2.0)
        self._t = None
        self._sample()


def _rss() -> int:
    try:
        import psutil
        return int(psutil.Process().memory_info().rss)
    except Exception:       # noqa: BLE001 - no psutil: host memory is reported as zero
        return 0


class MemoryMonitor(_Sampler):
    def __init__(self, sample_interval_ms: int = 100, device: Optional[str] = None, reader: Callable[[], int] = _rss):
        super().__init__(sample_interval_ms)
        self.device, self._read = device, reader
        self.reset()

    def _sample(self):
        v = self._read()
        with self._lock:
            if self._s.samples == 0:
                self._s.start_bytes = v
            self._s.samples += 1
            self._s.peak_bytes = max(self._s.peak_bytes, v)
            self._s.end_bytes = v
            if self.device is not None and self.device.startswith("cuda") and torch.cuda.is_available():
                self._s.device_peak_bytes = max(self._s.device_peak_bytes, torch.cuda.max_memory_allocated(self.device))

    def snapshot(self) -> MemorySnapshot:
        with self._lock:
            return MemorySnapshot(**asdict(self._s))

    def reset(self):
        self._lock = getattr(self, "_lock", threading.Lock())
        with self._lock:
            self._s = MemorySnapshot()


def nvml_power_reader(device_index: int = 0) -> Optional[Callable[[], float]]:
    """A function returning the board power in watts, or ``None`` without NVML. Reads only."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        pynvml.nvmlDeviceGetPowerUsage(h)
        return lambda: pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
    except Exception:       # noqa: BLE001
        return None


class EnergyMonitor(_Sampler):
    """Trapezoidal integral of sampled power. Without a power source every figure is zero (``available`` is False)."""

    def __init__(self, sample_interval_ms: int = 100, power_reader: Optional[Callable[[], float]] = None, clock: Callable[[], float] = time.perf_counter):
        super().__init__(sample_interval_ms)
        self._read = power_reader if power_reader is not None else nvml_power_reader()
        self._clock = clock
        self._lock = threading.Lock()
        self.reset()

    @property
    def available(self) -> bool:
        return self._read is not None

    def _sample(self):
        if self._read is None:
            return
        p, t = float(self._read()), self._clock()
        with self._lock:
            if self._last is not None:
                dt = t - self._last[0]
                self._s.energy_joules += 0.5 * (p + self._last[1]) * dt
                self._s.duration_s += dt
            self._last = (t, p)
            self._s.samples += 1
            self._s.peak_power_w = max(self._s.peak_power_w, p)

    def snapshot(self) -> EnergySnapshot:
        with self._lock:
            s = EnergySnapshot(**asdict(self._s))
        s.average_power_w = s.energy_joules / s.duration_s if s.duration_s > 0 else (self._last[1] if self._last else 0.0)
        return s

    def reset(self):
        with self._lock:
            self._s, self._last = EnergySnapshot(), None


# ------------------------------------------------------------------ benchmark runner
@dataclass
class BenchmarkConfig:
    name: str
    fn: Callable[[], Any]
    iterations: int = 10
    warmup: int = 2


@dataclass
class BenchmarkResult:
    name: str
    iterations: int
    times_ms: List[float]
    memory: MemorySnapshot = field(default_factory=MemorySnapshot)
    energy: EnergySnapshot = field(default_factory=EnergySnapshot)

    @property
    def mean_ms(self) -> float: return sum(self.times_ms) / len(self.times_ms)
    @property
    def min_ms(self) -> float: return min(self.times_ms)
    @property
    def max_ms(self) -> float: return max(self.times_ms)
    @property
    def median_ms(self) -> float:
        s = sorted(self.times_ms)
        n = len(s)
        return s[n // 2] if n % 2 else 0.5 * (s[n // 2 - 1] + s[n // 2])
    @property
    def std_ms(self) -> float:
        m = self.mean_ms
        return (sum((t - m) ** 2 for t in self.times_ms) / len(self.times_ms)) ** 0.5
    @property
    def energy_per_iteration_j(self) -> float:
        return self.energy.energy_joules / self.iterations if self.iterations else 0.0

    def row(self) -> Dict[str, Any]:
        return {"name": self.name, "iterations": self.iterations, "mean_ms": self.mean_ms, "median_ms": self.median_ms, "min_ms": self.min_ms,
                "max_ms": self.max_ms, "std_ms": self.std_ms, "peak_memory_bytes": self.memory.peak_bytes, "memory_growth_bytes": self.memory.growth_bytes,
                "device_peak_bytes": self.memory.device_peak_bytes, "energy_j": self.energy.energy_joules, "avg_power_w": self.energy.average_power_w}


@dataclass
class BenchmarkSummary:
    total_benchmarks: int
    total_time_ms: float
    fastest: str
    slowest: str


@dataclass
class BenchmarkResults:
    suite: str
    results: List[BenchmarkResult] = field(default_factory=list)

    def summary(self) -> BenchmarkSummary:
        if not self.results:
            return BenchmarkSummary(0, 0.0, "", "")
        return BenchmarkSummary(len(self.results), sum(sum(r.times_ms) for r in self.results),
                                min(self.results, key=lambda r: r.mean_ms).name, max(self.results, key=lambda r: r.mean_ms).name)

    def by_name(self) -> Dict[str, BenchmarkResult]:
        return {r.name: r for r in self.results}


class BenchmarkRunner:
    def __init__(self, memory_monitor: Optional[MemoryMonitor] = None, energy_monitor: Optional[EnergyMonitor] = None, sync: Optional[Callable[[], None]] = None):
        """``sync`` is called before every clock reading (``torch.cuda.synchronize`` for a model on a GPU)."""
        self.memory, self.energy, self.sync = memory_monitor, energy_monitor, sync
        self._results = BenchmarkResults("default")

    def run_benchmark(self, name: str, fn: Callable[[], Any], iterations: int = 10, warmup: int = 2) -> BenchmarkResult:
        if iterations <= 0:
            raise ValueError("iterations must be positive")
        for _ in range(warmup):
            fn()
        for m in (self.memory, self.energy):
            if m is not None:
                m.reset()
                m.start_monitoring()
        times = []
        try:
            for _ in range(iterations):
                if self.sync:
                    self.sync()
                t0 = time.perf_counter()
                fn()
                if self.sync:
                    self.sync()
                times.append((time.perf_counter() - t0) * 1e3)
        finally:
            for m in (self.memory, self.energy):
                if m is not None:
                    m.stop_monitoring()
        r = BenchmarkResult(name, iterations, times, self.memory.snapshot() if self.memory else MemorySnapshot(),
                            self.energy.snapshot() if self.energy else EnergySnapshot())
        self._results.results.append(r)
        return r

    def run_benchmark_suite(self, suite_name: str, *benchmarks: BenchmarkConfig) -> BenchmarkResults:
        out = BenchmarkResults(suite_name)
        for b in benchmarks:
            out.results.append(self.run_benchmark(b.name, b.fn, b.iterations, b.warmup))
        return out

    def results(self) -> BenchmarkResults:
        return self._results

    def reset(self):
        self._results = BenchmarkResults("default")

    def export_results(self, path: str, fmt: str = "json"):
        BenchmarkExporter.export(self._results, path, fmt)


# ------------------------------------------------------------------ scope profiler
@dataclass
class ProfileEntry:
    name: str
    depth: int
    calls: int = 0
    total_ms: float = 0.0
    min_ms: float = float("inf")
    max_ms: float = 0.0

    @property
    def mean_ms(self) -> float:
        return self.total_ms / self.calls if self.calls else 0.0


@dataclass
class ProfileReport:
    entries: List[ProfileEntry]
    total_ms: float

    def by_name(self) -> Dict[str, ProfileEntry]:
        return {e.name: e for e in self.entries}


class ProfileScope:
    def __init__(self, profiler: "Profiler", name: str):
        self._p, self.name = profiler, name

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self._p.end_scope()
        return False


class Profiler:
    """Nested named scopes; an entry's name is its path (``outer/inner``), so the same name under two parents stays
    apart."""

    def __init__(self, clock: Callable[[], float] = time.perf_counter):
        self._clock = clock
        self.reset()

    def begin_scope(self, name: str) -> ProfileScope:
        path = (self._stack[-1][0] + "/" if self._stack else "") + name
        self._stack.append((path, self._clock()))
        return ProfileScope(self, name)

    def end_scope(self):
        if not self._stack:
            raise RuntimeError("no scope is open")
        path, t0 = self._stack.pop()
        ms = (self._clock() - t0) * 1e3
        e = self._entries.setdefault(path, ProfileEntry(path, path.count("/")))
        e.calls += 1
        e.total_ms += ms
        e.min_ms, e.max_ms = min(e.min_ms, ms), max(e.max_ms, ms)

    def profile(self, name: str, fn: Callable[[], Any]):
        with self.begin_scope(name):
            return fn()

    def report(self) -> ProfileReport:
        es = sorted(self._entries.values(), key=lambda e: e.name)
        return ProfileReport(es, sum(e.total_ms for e in es if e.depth == 0))

    def reset(self):
        self._stack: List[tuple] = []
        self._entries: Dict[str, ProfileEntry] = {}

    def render(self) -> str:
        r = self.report()
        lines = [f"profile: {r.total_ms:.3f} ms in top-level scopes"]
        for e in r.entries:
            share = e.total_ms / r.total_ms if r.total_ms else 0.0
            lines.append(f"{'  ' * e.depth}{e.name.rsplit('/', 1)[-1]}: {e.calls} calls, {e.total_ms:.3f} ms total, {e.mean_ms:.3f} ms mean ({share:.0%})")
        return "\n".join(lines)

    def export_report(self, path: str, fmt: str = "json"):
        BenchmarkExporter.export_profile(self.report(), path, fmt)


# ------------------------------------------------------------------ exporters
class BenchmarkExporter:
    FORMATS = ("json", "csv", "markdown", "html")

    @classmethod
    def render(cls, results: BenchmarkResults, fmt: str = "json") -> str:
        rows = [r.row() for r in results.results]
        if fmt == "json":
            return json.dumps({"suite": results.suite, "summary": asdict(results.summary()), "results": rows}, indent=1)
        cols = list(rows[0]) if rows else ["name"]
        if fmt == "csv":
            buf = io.StringIO()
            w = csv.DictWriter(buf, fieldnames=cols)
            w.writeheader()
            w.writerows(rows)
            return buf.getvalue()
        f = lambda v: f"{v:.3f}" if isinstance(v, float) else str(v)      # noqa: E731
        if fmt == "markdown":
            out = [f"# {results.suite}", "", "| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
            out += ["| " + " | ".join(f(r[c]) for c in cols) + " |" for r in rows]
            return "\n".join(out) + "\n"
        if fmt == "html":
            head = "".join(f"<th>{html.escape(c)}</th>" for c in cols)
            body = "".join("<tr>" + "".join(f"<td>{html.escape(f(r[c]))}</td>" for c in cols) + "</tr>" for r in rows)
            return f"<html><body><h1>{html.escape(results.suite)}</h1><table><tr>{head}</tr>{body}</table></body></html>"
        raise ValueError(f"unknown format {fmt!r}; one of {cls.FORMATS}")

    @classmethod
    def export(cls, results: BenchmarkResults, path: str, fmt: str = "json"):
        with open(path, "w") as fh:
            fh.write(cls.render(results, fmt))

    @classmethod
    def export_profile(cls, report: ProfileReport, path: str, fmt: str = "json"):
        rows = [{"name": e.name, "depth": e.depth, "calls": e.calls, "total_ms": e.total_ms, "mean_ms": e.mean_ms, "min_ms": e.min_ms, "max_ms": e.max_ms}
                for e in report.entries]
        if fmt == "json":
            text = json.dumps({"total_ms": report.total_ms, "entries": rows}, indent=1)
        elif fmt == "csv":
            buf = io.StringIO()
            w = csv.DictWriter(buf, fieldnames=list(rows[0]) if rows else ["name"])
            w.writeheader()
            w.writerows(rows)
            text = buf.getvalue()
        else:
            raise ValueError(f"unknown format {fmt!r}")
        with open(path, "w") as fh:
            fh.write(text)


# ------------------------------------------------------------------ comparison
@dataclass
class ComparisonEntry:
    name: str
    baseline_ms: float
    current_ms: float

    @property
    def change(self) -> float:
        return self.current_ms / self.baseline_ms - 1.0 if self.baseline_ms > 0 else 0.0

    @property
    def speedup(self) -> float:
        return self.baseline_ms / self.current_ms if self.current_ms > 0 else 0.0


@dataclass
class ComparisonReport:
    entries: List[ComparisonEntry]
    only_in_baseline: List[str]
    only_in_current: List[str]
    threshold: float

    def regressions(self) -> List[ComparisonEntry]:
        return [e for e in self.entries if e.change > self.threshold]

    def improvements(self) -> List[ComparisonEntry]:
        return [e for e in self.entries if e.change < -self.threshold]


class PerformanceComparator:
    def __init__(self, threshold: float = 0.05):
        self.threshold = threshold

    def _cmp(self, a: Dict[str, float], b: Dict[str, float]) -> ComparisonReport:
        return ComparisonReport([ComparisonEntry(k, a[k], b[k]) for k in a if k in b], sorted(set(a) - set(b)), sorted(set(b) - set(a)), self.threshold)

    def compare(self, baseline: BenchmarkResults, current: BenchmarkResults) -> ComparisonReport:
        return self._cmp({r.name: r.median_ms for r in baseline.results}, {r.name: r.median_ms for r in current.results})

    def compare_profiles(self, baseline: ProfileReport, current: ProfileReport) -> ComparisonReport:
        return self._cmp({e.name: e.mean_ms for e in baseline.entries}, {e.name: e.mean_ms for e in current.entries})
