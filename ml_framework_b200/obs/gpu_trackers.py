"""Per-vendor GPU trackers behind one utilisation tracker.

Reference: src/MLFramework.Visualization/GPU/{GPUUtilizationTracker.cs:28-315, IGPUTracker.cs, GPUDeviceInfo.cs,
GPUStatistics.cs, GPUUtilizationSample.cs}, GPU/Vendor/{CudaGpuTracker.cs (NVML enum names, values simulated),
RocmGpuTracker.cs, GenericGpuTracker.cs}. The CUDA tracker here reads NVML for real through ``pynvml`` - utilisation,
memory, temperature, power, SM clock and the clock-event reasons - and only reads: no call that changes a clock, a
power limit or any other device setting is made. The NVML module is injectable so tests run against a fake.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

# NVML clock-event reason bits (public NVML header values)
REASON_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}


def decode_reasons(mask: int) -> List[str]:
    return [name for bit, name in REASON_BITS.items() if mask & bit]


@dataclass
class GPUDeviceInfo:
    device_id: int
    name: str
    vendor: str
    total_memory_bytes: int
    compute_capability: str = ""
    sm_count: int = 0
    driver_version: str = ""


@dataclass
class GPUUtilizationSample:
    device_id: int
    timestamp: float
    utilization_percent: float = 0.0
    memory_used_bytes: int = 0
    memory_total_bytes: int = 0
    temperature_c: float = 0.0
    power_w: float = 0.0
    sm_clock_mhz: float = 0.0
    sm_clock_max_mhz: float = 0.0
    reasons: List[str] = field(default_factory=list)

    @property
    def memory_percent(self) -> float:
        return 100.0 * self.memory_used_bytes / self.memory_total_bytes if self.memory_total_bytes else 0.0


@dataclass
class GPUStatistics:
    device_id: int
    sample_count: int = 0
    average_utilization: float = 0.0
    peak_utilization: float = 0.0
    average_memory_bytes: float = 0.0
    peak_memory_bytes: int = 0
    average_power_w: float = 0.0
    peak_power_w: float = 0.0
    peak_temperature_c: float = 0.0
    median_sm_clock_mhz: float = 0.0
    sm_clock_max_mhz: float = 0.0
    reasons_seen: List[str] = field(default_factory=list)
    duration_s: float = 0.0

    @staticmethod
    def from_samples(device_id: int, samples: List[GPUUtilizationSample]) -> "GPUStatistics":
        if not samples:
            return GPUStatistics(device_id)
        n = len(samples)
        clocks = sorted(s.sm_clock_mhz for s in samples)
        seen: List[str] = []
        for s in samples:
            for r in s.reasons:
                if r not in seen:
                    seen.append(r)
        return GPUStatistics(device_id, n, sum(s.utilization_percent for s in samples) / n, max(s.utilization_percent for s in samples),
                             sum(s.memory_used_bytes for s in samples) / n, max(s.memory_used_bytes for s in samples),
                             sum(s.power_w for s in samples) / n, max(s.power_w for s in samples), max(s.temperature_c for s in samples),
                             clocks[n // 2], max(s.sm_clock_max_mhz for s in samples), seen, samples[-1].timestamp - samples[0].timestamp)

    def throttled(self) -> bool:
        """True when a thermal or hardware slowdown was seen (a power cap under a dense GEMM is normal and not counted)."""
        return any(r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "hw_power_brake_slowdown") for r in self.reasons_seen)


class GpuTracker:
    vendor = "generic"

    def is_available(self) -> bool:
        raise NotImplementedError

    def device_count(self) -> int:
        raise NotImplementedError

    def device_info(self, device_id: int) -> GPUDeviceInfo:
        raise NotImplementedError

    def sample(self, device_id: int) -> GPUUtilizationSample:
        raise NotImplementedError


class CudaGpuTracker(GpuTracker):
    vendor = "nvidia"

    def __init__(self, nvml=None):
        self._nv = nvml
        self._ok = nvml is not None
        if nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nv, self._ok = pynvml, True
            except Exception:       # noqa: BLE001 - no NVML here: the tracker reports itself unavailable
                self._ok = False
        self._handles: Dict[int, object] = {}

    def is_available(self) -> bool:
        return self._ok

    def _h(self, i: int):
        if i not in self._handles:
            self._handles[i] = self._nv.nvmlDeviceGetHandleByIndex(i)
        return self._handles[i]

    def device_count(self) -> int:
        return int(self._nv.nvmlDeviceGetCount()) if self._ok else 0

    def device_info(self, device_id: int) -> GPUDeviceInfo:
        nv, h = self._nv, self._h(device_id)
        name = nv.nvmlDeviceGetName(h)
        name = name.decode() if isinstance(name, bytes) else str(name)
        cc = ""
        if hasattr(nv, "nvmlDeviceGetCudaComputeCapability"):
            try:
                major, minor = nv.nvmlDeviceGetCudaComputeCapability(h)
                cc = f"{major}.{minor}"
            except Exception:       # noqa: BLE001
                pass
        drv = ""
        if hasattr(nv, "nvmlSystemGetDriverVersion"):
            try:
                d = nv.nvmlSystemGetDriverVersion()
                drv = d.decode() if isinstance(d, bytes) else str(d)
            except Exception:       # noqa: BLE001
                pass
        return GPUDeviceInfo(device_id, name, self.vendor, int(nv.nvmlDeviceGetMemoryInfo(h).total), cc, 0, drv)

    def sample(self, device_id: int) -> GPUUtilizationSample:
        nv, h = self._nv, self._h(device_id)
        s = GPUUtilizationSample(device_id, time.time())

        def get(fn, default=0):
            try:
                return fn()
            except Exception:       # noqa: BLE001 - a counter this device does not expose stays at its default
                return default
        s.utilization_percent = float(get(lambda: nv.nvmlDeviceGetUtilizationRates(h).gpu))
        m = get(lambda: nv.nvmlDeviceGetMemoryInfo(h), None)
        if m is not None:
            s.memory_used_bytes, s.memory_total_bytes = int(m.used), int(m.total)
        s.temperature_c = float(get(lambda: nv.nvmlDeviceGetTemperature(h, getattr(nv, "NVML_TEMPERATURE_GPU", 0))))
        s.power_w = get(lambda: nv.nvmlDeviceGetPowerUsage(h)) / 1000.0
        s.sm_clock_mhz = float(get(lambda: nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
        s.sm_clock_max_mhz = float(get(lambda: nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
        fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        s.reasons = decode_reasons(int(get(lambda: fn(h)))) if fn is not None else []
        return s


class RocmGpuTracker(GpuTracker):
    """AMD devices are outside this framework's target; the tracker exists so that vendor selection has the same
    shape as the reference's and always reports itself unavailable."""
    vendor = "amd"

    def is_available(self) -> bool:
        return False

    def device_count(self) -> int:
        return 0

    def device_info(self, device_id):
        raise RuntimeError("ROCm devices are not supported")

    def sample(self, device_id):
        raise RuntimeError("ROCm devices are not supported")


class GenericGpuTracker(GpuTracker):
    """What the CUDA runtime alone can tell (through torch): names, memory in use; no utilisation, power or clocks."""
    vendor = "generic"

    def is_available(self) -> bool:
        return torch.cuda.is_available()

    def device_count(self) -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    def device_info(self, device_id: int) -> GPUDeviceInfo:
        p = torch.cuda.get_device_properties(device_id)
        return GPUDeviceInfo(device_id, p.name, self.vendor, p.total_memory, f"{p.major}.{p.minor}", p.multi_processor_count)

    def sample(self, device_id: int) -> GPUUtilizationSample:
        free, total = torch.cuda.mem_get_info(device_id)
        return GPUUtilizationSample(device_id, time.time(), memory_used_bytes=total - free, memory_total_bytes=total)


class GPUUtilizationTracker:
    """Picks the first available tracker (NVML, then the runtime-only one) and samples the tracked devices on a
    background thread. ``start_tracking(-1)`` tracks every device."""

    def __init__(self, trackers: Optional[List[GpuTracker]] = None, sampling_interval_s: float = 1.0, max_samples_per_device: int = 100_000):
        cands = trackers if trackers is not None else [CudaGpuTracker(), RocmGpuTracker(), GenericGpuTracker()]
        self.tracker: Optional[GpuTracker] = next((t for t in cands if t.is_available()), None)
        self.sampling_interval_s, self.max_samples = sampling_interval_s, max_samples_per_device
        self.enabled = True
        self._samples: Dict[int, List[GPUUtilizationSample]] = {}
        self._tracked: List[int] = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None

    @property
    def is_available(self) -> bool:
        return self.tracker is not None

    def available_devices(self) -> List[GPUDeviceInfo]:
        if self.tracker is None:
            return []
        return [self.tracker.device_info(i) for i in range(self.tracker.device_count())]

    def device_info(self, device_id: int) -> GPUDeviceInfo:
        if self.tracker is None:
            raise RuntimeError("no GPU tracker available")
        if not (0 <= device_id < self.tracker.device_count()):
            raise IndexError(f"device {device_id} out of range")
        return self.tracker.device_info(device_id)

    def set_sampling_interval(self, seconds: float):
        if seconds <= 0:
            raise ValueError("interval must be positive")
        self.sampling_interval_s = seconds

    def enable(self):
        self.enabled = True

    def disable(self):
        self.enabled = False

    def sample_utilization(self):
        if self.tracker is None or not self.enabled:
            return
        for d in self._tracked:
            s = self.tracker.sample(d)
            with self._lock:
                lst = self._samples.setdefault(d, [])
                lst.append(s)
                if len(lst) > self.max_samples:
                    del lst[:len(lst) - self.max_samples]

    def start_tracking(self, device_id: int = -1):
        if self.tracker is None:
            return
        self._tracked = list(range(self.tracker.device_count())) if device_id < 0 else [device_id]
        if self._t is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.wait(self.sampling_interval_s):
                self.sample_utilization()
        self._t = threading.Thread(target=loop, daemon=True, name="mlf-gpu-tracker")
        self._t.start()

    def stop_tracking(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2.0)
            self._t = None

    def samples(self, device_id: int, start: float = 0.0, end: float = float("inf")) -> List[GPUUtilizationSample]:
        with self._lock:
            return [s for s in self._samples.get(device_id, ()) if start <= s.timestamp <= end]

    def statistics(self, device_id: int) -> GPUStatistics:
        return GPUStatistics.from_samples(device_id, self.samples(device_id))

    def all_statistics(self) -> Dict[int, GPUStatistics]:
        with self._lock:
            ids = list(self._samples)
        return {d: self.statistics(d) for d in ids}

    def clear(self):
        with self._lock:
            self._samples.clear()
