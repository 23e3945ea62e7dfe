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
from dataclasses import dataclass, field
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
