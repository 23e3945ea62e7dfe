"""Profilers: hierarchical host timing, CUDA-event kernel timing, memory, GPU utilisation.

Reference: src/MLFramework.Visualization/Profiling/Profiler.cs:77-238 (scopes, parent scopes, instants,
percentiles), Memory/MemoryProfiler.cs + GCMonitor.cs, GPU/GPUUtilizationTracker.cs with vendor trackers
(the CUDA tracker there simulates its readings; this one reads NVML, read-only), data-pipeline
PerformanceCounter / ProfilingScope (src/MLFramework/Data/Metrics/*).
"""
from __future__ import annotations

import contextlib
import gc
import threading
import time
from collections import defaultdict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


def percentile(sorted_vals: List[float], q: float) -> float:
    if not sorted_vals:
        return 0.0
    k = (len(sorted_vals) - 1) * q / 100.0
    lo, hi = int(k), min(int(k) + 1, len(sorted_vals) - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (k - lo)


@dataclass
class ProfileResult:
    name: str
    count: int
    total_ns: int
    min_ns: int
    max_ns: int
    p50_ns: float
    p95_ns: float
    p99_ns: float
    parent: Optional[str] = None

    @property
    def mean_ns(self) -> float:
        return self.total_ns / self.count if self.count else 0.0


class Profiler:
    """``with prof.scope("fwd"):`` nests; durations are host nanoseconds. With ``cuda=True`` a scope is
    bracketed by CUDA events on the current stream and resolved at ``results()`` (no sync in the hot loop)."""

    def __init__(self, enabled: bool = True, cuda: bool = False):
        self.enabled, self.cuda = enabled, cuda and torch.cuda.is_available()
        self._dur: Dict[str, List[int]] = defaultdict(list)
        self._parent: Dict[str, Optional[str]] = {}
        self._stack = threading.local()
        self._pending: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self.instants: List[Tuple[str, int]] = []

    def _st(self) -> List[str]:
        if not hasattr(self._stack, "s"):
            self._stack.s = []
        return self._stack.s

    @contextlib.contextmanager
    def scope(self, name: str):
        if not self.enabled:
            yield
            return
        st = self._st()
        self._parent.setdefault(name, st[-1] if st else None)
        st.append(name)
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        t0 = time.perf_counter_ns()
        try:
            yield
        finally:
            if self.cuda:
                b.record()
                self._pending.append((name, a, b))
            else:
                self._dur[name].append(time.perf_counter_ns() - t0)
            st.pop()

    def record_instant(self, name: str):
        self.instants.append((name, time.perf_counter_ns()))

    def _resolve(self):
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self._dur[name].append(int(a.elapsed_time(b) * 1e6))
            self._pending.clear()

    def result(self, name: str) -> ProfileResult:
        self._resolve()
        d = sorted(self._dur[name])
        return ProfileResult(name, len(d), sum(d), d[0] if d else 0, d[-1] if d else 0, percentile(d, 50), percentile(d, 95),
                             percentile(d, 99), self._parent.get(name))

    def results(self) -> Dict[str, ProfileResult]:
        self._resolve()
        return {n: self.result(n) for n in self._dur}

    def report(self) -> str:
        rows = sorted(self.results().values(), key=lambda r: -r.total_ns)
        return "\n".join(f"{r.name:32s} n={r.count:5d} total={r.total_ns / 1e6:9.3f} ms  p50={r.p50_ns / 1e3:9.1f} us  p99={r.p99_ns / 1e3:9.1f} us"
                         + (f"  (in {r.parent})" if r.parent else "") for r in rows)

    def reset(self):
        self._dur.clear()
        self._pending.clear()
        self.instants.clear()


class MemoryProfiler:
    def __init__(self):
        self.snapshots: List[Dict[str, float]] = []

    def snapshot(self, tag: str = "") -> Dict[str, float]:
        s = {"tag": tag, "time": time.time(), "py_objects": len(gc.get_objects())}
        if torch.cuda.is_available():
            s.update(allocated=torch.cuda.memory_allocated(), reserved=torch.cuda.memory_reserved(), peak=torch.cuda.max_memory_allocated())
        try:
            import psutil
            s["host_rss"] = psutil.Process().memory_info().rss
        except Exception:
            pass
        self.snapshots.append(s)
        return s

    def delta(self, key: str = "allocated") -> float:
        if len(self.snapshots) < 2:
            return 0.0
        return self.snapshots[-1].get(key, 0) - self.snapshots[0].get(key, 0)


class GCMonitor:
    def __init__(self):
        self.collections = 0
        self.pause_ns = 0
        self._t0 = 0

    def _cb(self, phase, info):
        if phase == "start":
            self._t0 = time.perf_counter_ns()
        else:
            self.collections += 1
            self.pause_ns += time.perf_counter_ns() - self._t0

    def start(self):
        gc.callbacks.append(self._cb)

    def stop(self):
        if self._cb in gc.callbacks:
            gc.callbacks.remove(self._cb)


class GpuUtilizationTracker:
    """Samples NVML (utilisation, memory, SM clock, power, throttle reasons) from a background thread.
    Read-only: no setting of the device is touched. Without NVML every sample is empty."""

    def __init__(self, device_index: int = 0, interval_s: float = 0.2):
        self.idx, self.interval = device_index, interval_s
        self.samples: List[Dict[str, float]] = []
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(device_index)
        except Exception:
            self._nv = self._h = None

    def sample(self) -> Dict[str, float]:
        if self._nv is None:
            return {}
        nv, h = self._nv, self._h
        out: Dict[str, float] = {"time": time.time()}
        try:
            u = nv.nvmlDeviceGetUtilizationRates(h)
            m = nv.nvmlDeviceGetMemoryInfo(h)
            out.update(gpu_util=u.gpu, mem_util=u.memory, mem_used=m.used, mem_total=m.total,
                       sm_mhz=nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), sm_max_mhz=nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM),
                       power_w=nv.nvmlDeviceGetPowerUsage(h) / 1000.0, throttle_reasons=nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                       if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
        except Exception:
            pass
        return out

    def start(self):
        def loop():
            while not self._stop.wait(self.interval):
                s = self.sample()
                if s:
                    self.samples.append(s)
        self._t = threading.Thread(target=loop, daemon=True, name="mlf-gpu-util")
        self._t.start()

    def stop(self) -> Dict[str, float]:
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2.0)
        if not self.samples:
            return {}
        ks = [k for k in self.samples[0] if k not in ("time", "throttle_reasons")]
        return {k: sum(s.get(k, 0) for s in self.samples) / len(self.samples) for k in ks}


# ------------------------------------------------------------------ NVTX ranges and timeline export
_NVTX_ENABLED = False


def enable_nvtx(on: bool = True):
    """NVTX ranges cost a push / pop each even with no tool attached; they are off until enabled (``MLF_NVTX=1`` in
    the environment enables them at import)."""
    global _NVTX_ENABLED
    _NVTX_ENABLED = bool(on) and torch.cuda.is_available()


def nvtx_enabled() -> bool:
    return _NVTX_ENABLED


@contextlib.contextmanager
def nvtx_range(name: str):
    """Named range on the calling thread, visible in Nsight Systems / Nsight Compute timelines and in
    ``torch.profiler`` traces (as user annotations). The engine and the parallel wrappers mark forward, backward,
    optimizer and each collective with it."""
    if not _NVTX_ENABLED:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_mark(name: str):
    if _NVTX_ENABLED:
        torch.cuda.nvtx.mark(name)


class TimelineProfiler:
    """Kernel-level timeline of a few steps through ``torch.profiler`` (CUPTI under the hood), exported as a Chrome
    trace; ranges opened with :func:`nvtx_range` / ``record_function`` appear as annotations. For analysis only:
    numbers measured while it runs are not benchmark results.

        with TimelineProfiler("trace.json", steps=3) as tp:
            for _ in range(3):
                engine.step(ids, tgt); tp.step()
        print(tp.top_kernels(10))
    """

    def __init__(self, path: Optional[str] = None, steps: int = 3, with_stack: bool = False, record_shapes: bool = False):
        self.path, self.steps = path, steps
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, with_stack=with_stack, record_shapes=record_shapes)
        self._n = 0

    def __enter__(self):
        self._prof.__enter__()
        return self

    def step(self):
        self._n += 1

    def __exit__(self, *a):
        self._prof.__exit__(*a)
        if self.path:
            self._prof.export_chrome_trace(self.path)

    def top_kernels(self, n: int = 10) -> List[Tuple[str, float, int]]:
        """(name, total device microseconds, calls) of the kernels that took the most device time."""
        rows = []
        for e in self._prof.key_averages():
            dev = getattr(e, "device_time_total", None)
            if dev is None:
                dev = getattr(e, "cuda_time_total", 0.0)
            if dev and dev > 0:
                rows.append((e.key, float(dev), int(e.count)))
        rows.sort(key=lambda r: -r[1])
        return rows[:n]


class annotate(contextlib.ContextDecorator):
    """``with annotate("forward"):`` = an NVTX range (when enabled) and a ``torch.profiler.record_function`` scope."""

    def __init__(self, name: str):
        self.name = name
        self._rf = None

    def __enter__(self):
        if _NVTX_ENABLED:
            torch.cuda.nvtx.range_push(self.name)
        self._rf = torch.profiler.record_function(self.name)
        self._rf.__enter__()
        return self

    def __exit__(self, *a):
        self._rf.__exit__(*a)
        if _NVTX_ENABLED:
            torch.cuda.nvtx.range_pop()
        return False


import os as _os  # noqa: E402

if _os.environ.get("MLF_NVTX") == "1":
    enable_nvtx(True)


class PercentileCalculator:
    """Percentiles of a sample set with linear interpolation between order statistics
    (src/MLFramework.Visualization/Profiling/Statistics/PercentileCalculator.cs)."""

    def __init__(self, values: Sequence[float] = ()):
        self._v = sorted(float(x) for x in values)

    def add(self, x: float):
        import bisect
        bisect.insort(self._v, float(x))

    def __len__(self):
        return len(self._v)

    def percentile(self, q: float) -> float:
        if not (0.0 <= q <= 100.0):
            raise ValueError("percentile lies in [0, 100]")
        return percentile(self._v, q)

    def percentiles(self, qs: Sequence[float]) -> Dict[float, float]:
        return {q: self.percentile(q) for q in qs}

    def summary(self) -> Dict[str, float]:
        if not self._v:
            return {"count": 0}
        return {"count": len(self._v), "min": self._v[0], "max": self._v[-1], "mean": sum(self._v) / len(self._v),
                "p50": self.percentile(50), "p90": self.percentile(90), "p95": self.percentile(95), "p99": self.percentile(99)}


class DurationTracker:
    """Durations by name in nanoseconds: totals, counts, extremes and percentiles; ``track(name)`` times a block
    (src/MLFramework.Visualization/Profiling/Statistics/DurationTracker.cs)."""

    def __init__(self, max_samples_per_name: int = 10_000):
        self.max_samples = max_samples_per_name
        self._d: Dict[str, List[int]] = {}
        self._total: Dict[str, int] = {}
        self._count: Dict[str, int] = {}
        self._lock = threading.Lock()

    def record(self, name: str, duration_ns: int):
        if duration_ns < 0:
            raise ValueError("a duration cannot be negative")
        with self._lock:
            lst = self._d.setdefault(name, [])
            lst.append(int(duration_ns))
            if len(lst) > self.max_samples:
                del lst[:len(lst) - self.max_samples]
            self._total[name] = self._total.get(name, 0) + int(duration_ns)
            self._count[name] = self._count.get(name, 0) + 1

    @contextlib.contextmanager
    def track(self, name: str):
        t0 = time.perf_counter_ns()
        try:
            yield
        finally:
            self.record(name, time.perf_counter_ns() - t0)

    def names(self) -> List[str]:
        with self._lock:
            return sorted(self._d)

    def statistics(self, name: str) -> Dict[str, float]:
        with self._lock:
            v = list(self._d.get(name, ()))
            total, count = self._total.get(name, 0), self._count.get(name, 0)
        if not v:
            return {"count": 0}
        pc = PercentileCalculator(v)
        return {"count": count, "total_ns": total, "mean_ns": total / count, "min_ns": min(v), "max_ns": max(v),
                "p50_ns": pc.percentile(50), "p95_ns": pc.percentile(95), "p99_ns": pc.percentile(99)}

    def reset(self, name: Optional[str] = None):
        with self._lock:
            if name is None:
                self._d.clear(); self._total.clear(); self._count.clear()
            else:
                self._d.pop(name, None); self._total.pop(name, None); self._count.pop(name, None)
