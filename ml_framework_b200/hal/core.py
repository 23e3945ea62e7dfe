"""Hardware abstraction: devices, streams, events, backends, allocators, dynamic-shape memory.

The reference abstracts back-ends behind ``IBackend / IDevice / IStream / IEvent / IMemoryAllocator``
(src/MLFramework/HAL/IBackend.cs:8-41, IDevice.cs:6-41, IStream.cs:6-31, IMemoryAllocator.cs:6-42)
with an ``Operation`` enum (HAL/Operation.cs:6-39), a CPU back-end (CpuBackend.cs:14-35), a CUDA
back-end that supports only element-wise / reduction ops (HAL/CUDA/CudaBackend.cs:33-82) and caching
/ simple allocators (CachingAllocator.cs:46-95, SimpleAllocator.cs). Here there is one accelerator
back-end, the B200, whose ops are this package's own kernels (bf16) or PyTorch (other dtypes); the CPU
back-end exists for tests and host-side tensors. Streams and events are CUDA streams / events.

Dynamic-shape memory (src/MLFramework/Memory/PredictiveAllocator.cs, AdaptivePaddingStrategy.cs,
MemoryPressureHandler.cs, ShapeBounds.cs): allocate for the shape you expect to see next, pad to
avoid re-allocation, and shed cached blocks under pressure.
"""
from __future__ import annotations

import enum
import math
import threading
import time
from collections import defaultdict, deque
from dataclasses import dataclass
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch


class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"


class Operation(enum.Enum):
    ADD = "add"; SUBTRACT = "subtract"; MULTIPLY = "multiply"; DIVIDE = "divide"; MATMUL = "matmul"
    TRANSPOSE = "transpose"; SUM = "sum"; MEAN = "mean"; MAX = "max"; MIN = "min"; COPY = "copy"; FILL = "fill"
    RELU = "relu"; SIGMOID = "sigmoid"; TANH = "tanh"; CONV2D = "conv2d"; MAXPOOL2D = "maxpool2d"; CAST = "cast"
    RESHAPE = "reshape"


@dataclass(frozen=True)
class DeviceId:
    type: DeviceType
    index: int = 0

    def torch(self) -> torch.device:
        return torch.device(self.type.value, self.index) if self.type == DeviceType.CUDA else torch.device("cpu")

    def __str__(self):
        return f"{self.type.value}:{self.index}"


class Event:
    """CUDA event on an accelerator device; an immediately complete marker on the CPU."""

    def __init__(self, device: "Device", timing: bool = True):
        self.device = device
        self._ev = torch.cuda.Event(enable_timing=timing) if device.is_cuda else None
        self._recorded = False

    def record(self, stream: Optional["Stream"] = None):
        if self._ev is not None:
            self._ev.record(stream._s if stream is not None else torch.cuda.current_stream(self.device.torch))
        self._recorded = True

    def query(self) -> bool:
        return self._ev.query() if self._ev is not None else self._recorded

    def synchronize(self):
        if self._ev is not None:
            self._ev.synchronize()

    def elapsed_ms(self, later: "Event") -> float:
        return self._ev.elapsed_time(later._ev) if self._ev is not None else 0.0


class Stream:
    def __init__(self, device: "Device", priority: int = 0):
        self.device = device
        self._s = torch.cuda.Stream(device.torch, priority=priority) if device.is_cuda else None
        self._queue: List[Callable[[], None]] = []

    def enqueue(self, fn: Callable[[], None]):
        """Run ``fn`` with this stream current (CPU streams execute in order, immediately)."""
        if self._s is None:
            fn()
        else:
            with torch.cuda.stream(self._s):
                fn()

    def record_event(self) -> Event:
        e = Event(self.device)
        e.record(self)
        return e

    def wait_event(self, ev: Event):
        if self._s is not None and ev._ev is not None:
            self._s.wait_event(ev._ev)

    def synchronize(self):
        if self._s is not None:
            self._s.synchronize()

    @property
    def handle(self) -> int:
        return self._s.cuda_stream if self._s is not None else 0


# ------------------------------------------------------------------ allocators
@dataclass
class MemoryBuffer:
    tensor: torch.Tensor
    size: int
    allocator: "MemoryAllocator"
    freed: bool = False

    @property
    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def free(self):
        if not self.freed:
            self.allocator.free(self)


class MemoryAllocator:
    def __init__(self, device: "Device"):
        self.device = device
        self.allocated_bytes = 0
        self.peak_bytes = 0
        self.n_allocs = 0
        self._lock = threading.Lock()

    def _raw(self, size: int) -> torch.Tensor:
        return torch.empty(size, dtype=torch.uint8, device=self.device.torch)

    def allocate(self, size: int) -> MemoryBuffer:
        raise NotImplementedError

    def free(self, buf: MemoryBuffer):
        raise NotImplementedError

    def empty_cache(self):
        pass

    def _account(self, delta: int):
        self.allocated_bytes += delta
        self.peak_bytes = max(self.peak_bytes, self.allocated_bytes)


class SimpleAllocator(MemoryAllocator):
    """Every allocate is a fresh device allocation; every free releases it."""

    def allocate(self, size: int) -> MemoryBuffer:
        if size <= 0:
            raise ValueError("allocation size must be positive")
        with self._lock:
            self.n_allocs += 1
            self._account(size)
        return MemoryBuffer(self._raw(size), size, self)

    def free(self, buf: MemoryBuffer):
        with self._lock:
            if buf.freed:
                raise RuntimeError("double free")
            buf.freed = True
            self._account(-buf.size)
        buf.tensor = None


class CachingAllocator(MemoryAllocator):
    """Size-class free lists: sizes round up to 512 B below 1 MiB, to 2 MiB above (the granularity
    of the device's large pages), so that variable-shape workloads re-use blocks."""

    SMALL, LARGE = 512, 2 << 20

    def __init__(self, device: "Device", max_cached_bytes: int = 8 << 30):
        super().__init__(device)
        self._free: Dict[int, List[torch.Tensor]] = defaultdict(list)
        self.cached_bytes = 0
        self.max_cached_bytes = max_cached_bytes
        self.hits = self.misses = 0

    @classmethod
    def round_size(cls, size: int) -> int:
        g = cls.SMALL if size < (1 << 20) else cls.LARGE
        return (size + g - 1) // g * g

    def allocate(self, size: int) -> MemoryBuffer:
        if size <= 0:
            raise ValueError("allocation size must be positive")
        r = self.round_size(size)
        with self._lock:
            lst = self._free.get(r)
            if lst:
                t = lst.pop()
                self.cached_bytes -= r
                self.hits += 1
            else:
                t = None
                self.misses += 1
            self.n_allocs += 1
            self._account(r)
        if t is None:
            t = self._raw(r)
        return MemoryBuffer(t, r, self)

    def free(self, buf: MemoryBuffer):
        with self._lock:
            if buf.freed:
                raise RuntimeError("double free")
            buf.freed = True
            self._account(-buf.size)
            if self.cached_bytes + buf.size <= self.max_cached_bytes:
                self._free[buf.size].append(buf.tensor)
                self.cached_bytes += buf.size
        buf.tensor = None

    def empty_cache(self):
        with self._lock:
            self._free.clear()
            self.cached_bytes = 0


# ------------------------------------------------------------------ devices / backends
class Device:
    def __init__(self, dev_id: DeviceId, backend: "Backend"):
        self.id, self.backend = dev_id, backend
        self.torch = dev_id.torch()
        self.is_cuda = dev_id.type == DeviceType.CUDA
        self.allocator: MemoryAllocator = CachingAllocator(self)
        self._default_stream: Optional[Stream] = None

    def create_stream(self, priority: int = 0) -> Stream:
        return Stream(self, priority)

    def create_event(self) -> Event:
        return Event(self)

    def synchronize(self):
        if self.is_cuda:
            torch.cuda.synchronize(self.torch)

    def properties(self) -> Dict[str, object]:
        if not self.is_cuda:
            import os
            return {"name": "cpu", "cores": os.cpu_count()}
        p = torch.cuda.get_device_properties(self.torch)
        return {"name": p.name, "sms": p.multi_processor_count, "memory_bytes": p.total_memory, "capability": (p.major, p.minor)}

    def allocate(self, size: int) -> MemoryBuffer:
        return self.allocator.allocate(size)


class Backend:
    name = "base"
    device_type = DeviceType.CPU

    def device_count(self) -> int:
        return 1

    def is_available(self) -> bool:
        return True

    def supports(self, op: Operation) -> bool:
        return True

    def execute(self, op: Operation, inputs: Sequence[torch.Tensor], **kw) -> torch.Tensor:
        return _torch_execute(op, inputs, **kw)

    def device(self, index: int = 0) -> Device:
        return Device(DeviceId(self.device_type, index), self)


def _torch_execute(op: Operation, x: Sequence[torch.Tensor], **kw) -> torch.Tensor:
    import torch.nn.functional as F
    a = x[0]
    b = x[1] if len(x) > 1 else None
    if op == Operation.ADD: return a + b
    if op == Operation.SUBTRACT: return a - b
    if op == Operation.MULTIPLY: return a * b
    if op == Operation.DIVIDE: return a / b
    if op == Operation.MATMUL: return a @ b
    if op == Operation.TRANSPOSE: return a.transpose(kw.get("dim0", -2), kw.get("dim1", -1))
    if op == Operation.SUM: return a.sum(kw["dim"]) if "dim" in kw else a.sum()
    if op == Operation.MEAN: return a.mean(kw["dim"]) if "dim" in kw else a.mean()
    if op == Operation.MAX: return a.amax(kw["dim"]) if "dim" in kw else a.max()
    if op == Operation.MIN: return a.amin(kw["dim"]) if "dim" in kw else a.min()
    if op == Operation.COPY: return a.clone()
    if op == Operation.FILL: return torch.full_like(a, kw["value"])
    if op == Operation.RELU: return torch.relu(a)
    if op == Operation.SIGMOID: return torch.sigmoid(a)
    if op == Operation.TANH: return torch.tanh(a)
    if op == Operation.CONV2D: return F.conv2d(a, b, x[2] if len(x) > 2 else None, kw.get("stride", 1), kw.get("padding", 0))
    if op == Operation.MAXPOOL2D: return F.max_pool2d(a, kw.get("kernel", 2), kw.get("stride", None))
    if op == Operation.CAST: return a.to(kw["dtype"])
    if op == Operation.RESHAPE: return a.reshape(kw["shape"])
    raise NotImplementedError(op)


class CpuBackend(Backend):
    name = "cpu"
    device_type = DeviceType.CPU


class B200Backend(Backend):
    """bf16 2-D matmul and element-wise ops go to this package's kernels; everything else to PyTorch
    on the same device (the reference's CUDA back-end has no matmul / conv at all)."""
    name = "b200"
    device_type = DeviceType.CUDA

    def device_count(self) -> int:
        return torch.cuda.device_count()

    def is_available(self) -> bool:
        return torch.cuda.is_available()

    def execute(self, op: Operation, inputs: Sequence[torch.Tensor], **kw) -> torch.Tensor:
        a = inputs[0]
        if a.is_cuda and a.dtype == torch.bfloat16:
            from ..ops import native
            from ..ops.gemm import gemm
            b = inputs[1] if len(inputs) > 1 else None
            if op == Operation.MATMUL and a.dim() == 2 and b.dim() == 2 and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
                return gemm(a, b, b_mn=True)            # b is [K, N]: the kernel reads it MN-major
            ew = {Operation.ADD: "add", Operation.SUBTRACT: "sub", Operation.MULTIPLY: "mul", Operation.DIVIDE: "div"}
            if op in ew and b is not None and b.shape == a.shape and a.is_contiguous() and b.is_contiguous() and hasattr(native, "ew_binary"):
                return native.ew_binary(a, b, ew[op])
        return _torch_execute(op, inputs, **kw)


class BackendRegistry:
    _backends: Dict[str, Backend] = {}

    @classmethod
    def register(cls, b: Backend):
        cls._backends[b.name] = b

    @classmethod
    def get(cls, name: str) -> Backend:
        if name not in cls._backends:
            raise KeyError(f"backend {name!r} is not registered; known: {sorted(cls._backends)}")
        return cls._backends[name]

    @classmethod
    def available(cls) -> List[str]:
        return [n for n, b in cls._backends.items() if b.is_available()]

    @classmethod
    def best(cls) -> Backend:
        return cls._backends["b200"] if cls._backends["b200"].is_available() else cls._backends["cpu"]


BackendRegistry.register(CpuBackend())
BackendRegistry.register(B200Backend())


# ------------------------------------------------------------------ dynamic-shape memory
@dataclass
class ShapeBounds:
    min_shape: Tuple[int, ...]
    max_shape: Tuple[int, ...]
    expected_shape: Optional[Tuple[int, ...]] = None

    def __post_init__(self):
        if len(self.min_shape) != len(self.max_shape) or any(a > b for a, b in zip(self.min_shape, self.max_shape)):
            raise ValueError("min_shape must be element-wise <= max_shape with equal rank")

    def contains(self, shape: Sequence[int]) -> bool:
        return len(shape) == len(self.min_shape) and all(a <= s <= b for a, s, b in zip(self.min_shape, shape, self.max_shape))

    def max_elements(self) -> int:
        return math.prod(self.max_shape)


class AdaptivePaddingStrategy:
    """Pad requested sizes by a factor that grows when re-allocations are frequent and shrinks when
    the padding goes unused (AdaptivePaddingStrategy.cs)."""

    def __init__(self, initial: float = 1.2, lo: float = 1.0, hi: float = 2.0):
        self.factor, self.lo, self.hi = initial, lo, hi
        self._resizes = self._uses = 0

    def padded(self, n: int) -> int:
        return int(math.ceil(n * self.factor))

    def observe(self, resized: bool):
        self._uses += 1
        self._resizes += int(resized)
        if self._uses >= 16:
            rate = self._resizes / self._uses
            if rate > 0.25:
                self.factor = min(self.hi, self.factor * 1.1)
            elif rate < 0.05:
                self.factor = max(self.lo, self.factor * 0.97)
            self._resizes = self._uses = 0


class MemoryHandle:
    def __init__(self, buf: MemoryBuffer, shape: Tuple[int, ...], dtype: torch.dtype):
        self.buffer, self.shape, self.dtype = buf, shape, dtype

    @property
    def capacity_elements(self) -> int:
        return self.buffer.size // torch.empty((), dtype=self.dtype).element_size()

    def view(self, shape: Sequence[int]) -> torch.Tensor:
        n = math.prod(shape)
        if n > self.capacity_elements:
            raise ValueError("shape exceeds the handle's capacity")
        return self.buffer.tensor.view(self.dtype)[:n].view(*shape)


class PredictiveAllocator:
    """Keeps a history of requested shapes per tensor name and allocates for the predicted next shape
    (max of the recent window, padded), so that a growing sequence length re-allocates rarely."""

    def __init__(self, allocator: MemoryAllocator, window: int = 32, padding: Optional[AdaptivePaddingStrategy] = None):
        self.alloc, self.window = allocator, window
        self.padding = padding or AdaptivePaddingStrategy()
        self._hist: Dict[str, Deque[int]] = defaultdict(lambda: deque(maxlen=window))
        self._handles: Dict[str, MemoryHandle] = {}
        self.reallocations = 0
        self._allocations = 0
        self._bytes_allocated = 0
        self._bytes_wasted = 0
        self._util_sum, self._util_n = 0.0, 0

    def stats(self) -> "AllocationStats":
        """Allocation counts, bytes handed out, bytes that padding left unused, mean utilisation of a request."""
        return AllocationStats(self._allocations, self.reallocations, self._bytes_allocated, self._bytes_wasted,
                               self._util_sum / self._util_n if self._util_n else 0.0)

    def predict_elements(self, name: str) -> int:
        h = self._hist[name]
        return max(h) if h else 0

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype, bounds: Optional[ShapeBounds] = None) -> torch.Tensor:
        if bounds is not None and not bounds.contains(shape):
            raise ValueError(f"shape {tuple(shape)} outside bounds {bounds.min_shape}..{bounds.max_shape}")
        n = math.prod(shape)
        self._hist[name].append(n)
        h = self._handles.get(name)
        resized = h is None or h.dtype != dtype or h.capacity_elements < n
        if resized:
            want = self.padding.padded(max(n, self.predict_elements(name)))
            if bounds is not None:
                want = min(want, bounds.max_elements())
            want = max(want, n)
            if h is not None:
                h.buffer.free()
                self.reallocations += 1
            esz = torch.empty((), dtype=dtype).element_size()
            h = MemoryHandle(self.alloc.allocate(want * esz), tuple(shape), dtype)
            self._handles[name] = h
            self._allocations += 1
            self._bytes_allocated += want * esz
            self._bytes_wasted += (want - n) * esz
        self._util_sum += n / max(1, h.capacity_elements)
        self._util_n += 1
        self.padding.observe(resized)
        return h.view(shape)

    def release(self, name: str):
        h = self._handles.pop(name, None)
        if h is not None:
            h.buffer.free()


class MemoryPressureHandler:
    """Calls registered release callbacks (lowest priority first) until usage drops below the low
    watermark (MemoryPressureHandler.cs)."""

    def __init__(self, capacity_bytes: int, high: float = 0.9, low: float = 0.75, usage_fn: Optional[Callable[[], int]] = None):
        self.capacity, self.high, self.low = capacity_bytes, high, low
        self._usage_fn = usage_fn or (lambda: torch.cuda.memory_allocated() if torch.cuda.is_available() else 0)
        self._callbacks: List[Tuple[int, Callable[[], int]]] = []
        self.events = 0

    def register(self, release: Callable[[], int], priority: int = 0):
        self._callbacks.append((priority, release))
        self._callbacks.sort(key=lambda t: t[0])

    def pressure(self) -> float:
        return self._usage_fn() / max(1, self.capacity)

    def check(self) -> int:
        if self.pressure() < self.high:
            return 0
        self.events += 1
        freed = 0
        for _, cb in self._callbacks:
            freed += cb()
            if self.pressure() < self.low:
                break
        return freed


# ------------------------------------------------------------------ allocation statistics, model-level memory pressure
@dataclass
class AllocationStats:
    """Reference: src/MLFramework/Memory/AllocationStats.cs."""
    total_allocations: int = 0
    total_resizes: int = 0
    total_bytes_allocated: int = 0
    total_bytes_wasted: int = 0
    average_utilization: float = 0.0

    def to_report(self) -> str:
        waste = 100.0 * self.total_bytes_wasted / self.total_bytes_allocated if self.total_bytes_allocated else 0.0
        return (f"allocations: {self.total_allocations} ({self.total_resizes} resizes), {self.total_bytes_allocated} bytes, "
                f"{self.total_bytes_wasted} bytes of padding ({waste:.1f} %), mean utilisation {self.average_utilization * 100:.1f} %")


class ModelMemoryInfo:
    """One loaded model version as the eviction policy sees it (src/MLFramework/Memory/ModelMemoryInfo.cs): the weight
    falls with the time since the last use and rises with the number of uses, a day per use."""

    SECONDS_PER_USE = 86400.0

    def __init__(self, model_name: str, version: str, memory_bytes: int, clock: Callable[[], float] = time.time):
        if memory_bytes < 0:
            raise ValueError("memory_bytes cannot be negative")
        self.model_name, self.version, self.memory_bytes = model_name, version, int(memory_bytes)
        self._clock = clock
        self.last_access_time = clock()
        self.access_count = 0
        self.is_pinned = False

    @property
    def weight(self) -> float:
        """Lower = a better candidate for eviction."""
        return self.last_access_time + self.access_count * self.SECONDS_PER_USE

    def record_access(self) -> None:
        self.last_access_time = self._clock()
        self.access_count += 1


@dataclass
class EvictionResult:
    evicted_versions: List[str]
    bytes_freed: int
    sufficient: bool

    def __str__(self):
        return f"evicted {len(self.evicted_versions)} model(s), freed {self.bytes_freed} bytes, {'enough' if self.sufficient else 'NOT enough'}"


class ModelMemoryPressureHandler:
    """Keeps the loaded model versions under a byte threshold: ``evict_if_needed(required)`` unloads unpinned versions,
    lowest weight first, skipping those the ``can_evict`` callback protects (requests in flight), until usage plus the
    requirement fits (src/MLFramework/Memory/MemoryPressureHandler.cs:9-180)."""

    def __init__(self, memory_threshold_bytes: int, unload_model: Callable[[str, str], None],
                 can_evict: Optional[Callable[[str, str], bool]] = None, clock: Callable[[], float] = time.time):
        if memory_threshold_bytes <= 0:
            raise ValueError("the memory threshold must be positive")
        self._threshold, self._unload, self._can_evict, self._clock = int(memory_threshold_bytes), unload_model, can_evict, clock
        self._models: Dict[str, ModelMemoryInfo] = {}
        self._lock = threading.RLock()
        self.evictions = 0

    @staticmethod
    def _key(name: str, version: str) -> str:
        return f"{name}:{version}"

    def track_model_load(self, model_name: str, version: str, memory_bytes: int) -> None:
        with self._lock:
            self._models[self._key(model_name, version)] = ModelMemoryInfo(model_name, version, memory_bytes, self._clock)

    def track_model_access(self, model_name: str, version: str) -> None:
        with self._lock:
            m = self._models.get(self._key(model_name, version))
            if m is not None:
                m.record_access()

    def _pin(self, model_name: str, version: str, value: bool) -> None:
        with self._lock:
            k = self._key(model_name, version)
            if k not in self._models:
                raise KeyError(f"model {k} is not tracked")
            self._models[k].is_pinned = value

    def pin_model(self, model_name: str, version: str) -> None:
        self._pin(model_name, version, True)

    def unpin_model(self, model_name: str, version: str) -> None:
        self._pin(model_name, version, False)

    def untrack_model(self, model_name: str, version: str) -> bool:
        with self._lock:
            return self._models.pop(self._key(model_name, version), None) is not None

    def get_total_memory_usage(self) -> int:
        with self._lock:
            return sum(m.memory_bytes for m in self._models.values())

    def set_memory_threshold(self, threshold_bytes: int) -> None:
        if threshold_bytes <= 0:
            raise ValueError("the memory threshold must be positive")
        self._threshold = int(threshold_bytes)

    def get_loaded_models_info(self) -> List[ModelMemoryInfo]:
        with self._lock:
            return list(self._models.values())

    def evict_if_needed(self, required_bytes: int = 0) -> EvictionResult:
        """Makes room for ``required_bytes`` more under the threshold."""
        with self._lock:
            usage = self.get_total_memory_usage()
            target = self._threshold - max(0, int(required_bytes))
            if usage <= target:
                return EvictionResult([], 0, True)
            gone, freed = [], 0
            for m in sorted((m for m in self._models.values() if not m.is_pinned), key=lambda m: m.weight):
                if usage - freed <= target:
                    break
                if self._can_evict is not None and not self._can_evict(m.model_name, m.version):
                    continue
                k = self._key(m.model_name, m.version)
                self._models.pop(k)
                self._unload(m.model_name, m.version)
                gone.append(k)
                freed += m.memory_bytes
                self.evictions += 1
            return EvictionResult(gone, freed, usage - freed <= target)
