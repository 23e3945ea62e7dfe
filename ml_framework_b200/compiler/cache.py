"""Shape-keyed kernel caches, lazy specialisation, autotuning and shape profiling.

Reference: src/MLFramework/Cache/ShapeSignature.cs, Cache/LRUKernelCache.cs, Compilation/
LazyCompilationManager.cs, ShapeVariantGenerator.cs, Autotuning/Autotuner.cs (+ search space, benchmark
runner, tuning cache), Profiling/GlobalShapeProfiler.cs, ShapeHistogram.cs.

Used here for the choices the hand-written kernels leave open per shape: GEMM column tile
(64 / 128 / 256 / CTA pair), number of copy CTAs of a fused gather, decode split size. The autotuner
times candidates with CUDA events (warm-up, then median of repeats) and remembers the winner per shape
signature; the persistent tuning cache is a JSON file.
"""
from __future__ import annotations

import json
import os
import threading
import time
from collections import Counter, OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generic, Iterable, List, Optional, Sequence, Tuple, TypeVar

import torch

V = TypeVar("V")


@dataclass(frozen=True)
class ShapeSignature:
    op: str
    shapes: Tuple[Tuple[int, ...], ...]
    dtype: str = "bf16"
    extra: Tuple = ()

    @staticmethod
    def of(op: str, *tensors: torch.Tensor, extra: Tuple = ()) -> "ShapeSignature":
        return ShapeSignature(op, tuple(tuple(t.shape) for t in tensors), str(tensors[0].dtype) if tensors else "", extra)

    def key(self) -> str:
        return f"{self.op}|{self.shapes}|{self.dtype}|{self.extra}"


class LRUKernelCache(Generic[V]):
    def __init__(self, capacity: int = 256):
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.capacity = capacity
        self._d: "OrderedDict[str, V]" = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = self.evictions = 0

    def get(self, sig: ShapeSignature) -> Optional[V]:
        with self._lock:
            k = sig.key()
            if k in self._d:
                self._d.move_to_end(k)
                self.hits += 1
                return self._d[k]
            self.misses += 1
            return None

    def put(self, sig: ShapeSignature, value: V):
        with self._lock:
            k = sig.key()
            self._d[k] = value
            self._d.move_to_end(k)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)
                self.evictions += 1

    def get_or_create(self, sig: ShapeSignature, factory: Callable[[], V]) -> V:
        v = self.get(sig)
        if v is None:
            v = factory()
            self.put(sig, v)
        return v

    def __len__(self):
        return len(self._d)

    def stats(self) -> Dict[str, float]:
        tot = self.hits + self.misses
        return {"size": len(self._d), "hits": self.hits, "misses": self.misses, "evictions": self.evictions,
                "hit_rate": self.hits / tot if tot else 0.0}


class ShapeVariantGenerator:
    """Buckets for dynamic dimensions: powers of two between bounds, so a lazily specialised kernel
    covers a range of shapes."""

    @staticmethod
    def buckets(lo: int, hi: int) -> List[int]:
        out, v = [], 1
        while v < lo:
            v *= 2
        while v < hi:
            out.append(v)
            v *= 2
        out.append(hi)
        return out

    @staticmethod
    def bucket_for(n: int, buckets: Sequence[int]) -> int:
        for b in buckets:
            if n <= b:
                return b
        raise ValueError(f"{n} exceeds the largest bucket {buckets[-1]}")


class LazyCompilationManager:
    """Builds a specialisation the first time a signature is seen; ``precompile`` fills it ahead of time."""

    def __init__(self, builder: Callable[[ShapeSignature], Any], cache: Optional[LRUKernelCache] = None):
        self.builder, self.cache = builder, cache or LRUKernelCache(256)
        self.compilations = 0
        self.compile_seconds = 0.0

    def get(self, sig: ShapeSignature):
        def make():
            t0 = time.perf_counter()
            v = self.builder(sig)
            self.compile_seconds += time.perf_counter() - t0
            self.compilations += 1
            return v
        return self.cache.get_or_create(sig, make)

    def precompile(self, sigs: Iterable[ShapeSignature]):
        for s in sigs:
            self.get(s)


# ------------------------------------------------------------------ autotuner
def cuda_event_timer(fn: Callable[[], None], warmup: int = 3, repeats: int = 10) -> float:
    """Median milliseconds of ``fn`` on the current stream (wall clock on CPU)."""
    if not torch.cuda.is_available():
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
        return sorted(ts)[len(ts) // 2]
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


class TuningCache:
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self._d: Dict[str, Dict[str, Any]] = {}
        if path and os.path.exists(path):
            with open(path) as f:
                self._d = json.load(f)

    def get(self, sig: ShapeSignature):
        return self._d.get(sig.key())

    def put(self, sig: ShapeSignature, config: Dict[str, Any], ms: float):
        self._d[sig.key()] = {"config": config, "ms": ms}
        if self.path:
            tmp = self.path + ".tmp"
            with open(tmp, "w") as f:
                json.dump(self._d, f, indent=1)
            os.replace(tmp, self.path)


class Autotuner:
    def __init__(self, cache: Optional[TuningCache] = None, timer: Callable = cuda_event_timer):
        self.cache, self.timer = cache or TuningCache(), timer
        self.trials = 0

    def tune(self, sig: ShapeSignature, candidates: Sequence[Dict[str, Any]], run: Callable[[Dict[str, Any]], None]) -> Dict[str, Any]:
        hit = self.cache.get(sig)
        if hit is not None:
            return hit["config"]
        best, best_ms = None, float("inf")
        for cfg in candidates:
            try:
                ms = self.timer(lambda: run(cfg))
            except Exception:
                continue
            self.trials += 1
            if ms < best_ms:
                best, best_ms = cfg, ms
        if best is None:
            raise RuntimeError(f"no candidate ran for {sig.key()}")
        self.cache.put(sig, best, best_ms)
        return best


def gemm_search_space(M: int, N: int, K: int) -> List[Dict[str, Any]]:
    """Column tiles worth trying for a plain GEMM (512 = CTA pair)."""
    out = [{"tile_n": t} for t in (64, 128, 256) if N >= t]
    if M >= 256 and N >= 256:
        out.append({"tile_n": 512})
    return out


# ------------------------------------------------------------------ shape profiler
class ShapeHistogram:
    def __init__(self):
        self.counts: Counter = Counter()

    def record(self, shape: Tuple[int, ...]):
        self.counts[tuple(shape)] += 1

    def top(self, k: int = 5) -> List[Tuple[Tuple[int, ...], int]]:
        return self.counts.most_common(k)

    def coverage(self, k: int) -> float:
        tot = sum(self.counts.values())
        return sum(c for _, c in self.top(k)) / tot if tot else 0.0


class GlobalShapeProfiler:
    _inst: Optional["GlobalShapeProfiler"] = None

    def __init__(self):
        self.hist: Dict[str, ShapeHistogram] = {}
        self.enabled = True

    @classmethod
    def instance(cls) -> "GlobalShapeProfiler":
        if cls._inst is None:
            cls._inst = GlobalShapeProfiler()
        return cls._inst

    def record(self, op: str, shape: Sequence[int]):
        if self.enabled:
            self.hist.setdefault(op, ShapeHistogram()).record(tuple(shape))

    def specialisations(self, op: str, coverage: float = 0.9, max_k: int = 8) -> List[Tuple[int, ...]]:
        """Smallest set of most frequent shapes covering ``coverage`` of calls."""
        h = self.hist.get(op)
        if h is None:
            return []
        for k in range(1, max_k + 1):
            if h.coverage(k) >= coverage:
                return [s for s, _ in h.top(k)]
        return [s for s, _ in h.top(max_k)]


@dataclass
class ShapeStatistics:
    """Summary of the shapes one operation was called with (src/MLFramework/Profiling/ShapeStatistics.cs)."""
    op: str
    calls: int
    distinct_shapes: int
    most_common: Tuple[int, ...]
    most_common_share: float
    min_dims: Tuple[int, ...]
    max_dims: Tuple[int, ...]
    mean_elements: float
    dynamic_dims: Tuple[int, ...]            # positions that varied between calls

    @staticmethod
    def from_histogram(op: str, h: ShapeHistogram) -> Optional["ShapeStatistics"]:
        if not h.counts:
            return None
        calls = sum(h.counts.values())
        (top, n), = h.top(1)
        rank = len(top)
        same = [s for s in h.counts if len(s) == rank]
        mins = tuple(min(s[i] for s in same) for i in range(rank))
        maxs = tuple(max(s[i] for s in same) for i in range(rank))

        def numel(s):
            k = 1
            for d in s:
                k *= d
            return k
        mean = sum(numel(s) * c for s, c in h.counts.items()) / calls
        return ShapeStatistics(op, calls, len(h.counts), top, n / calls, mins, maxs, mean, tuple(i for i in range(rank) if mins[i] != maxs[i]))


@dataclass
class ShapeSpecializationPlan:
    op: str
    specialize: List[Tuple[int, ...]]         # compile a variant for each of these exact shapes
    bucket_dims: Dict[int, List[int]]          # dynamic positions -> bucket upper bounds for the generic variants
    expected_hit_rate: float


class ShapeProfileOptimizer:
    """Turns recorded shapes into a compilation plan: exact variants for the few shapes that make up most calls,
    power-of-two buckets (capped at the largest seen) along the dimensions that vary for everything else
    (src/MLFramework/Profiling/ShapeProfileOptimizer.cs)."""

    def __init__(self, profiler: Optional[GlobalShapeProfiler] = None, coverage: float = 0.9, max_variants: int = 8, min_calls: int = 10):
        self.prof = profiler or GlobalShapeProfiler.instance()
        self.coverage, self.max_variants, self.min_calls = coverage, max_variants, min_calls

    def statistics(self, op: str) -> Optional[ShapeStatistics]:
        h = self.prof.hist.get(op)
        return ShapeStatistics.from_histogram(op, h) if h is not None else None

    def plan(self, op: str) -> Optional[ShapeSpecializationPlan]:
        st = self.statistics(op)
        if st is None or st.calls < self.min_calls:
            return None
        spec = self.prof.specialisations(op, self.coverage, self.max_variants)
        h = self.prof.hist[op]
        hit = sum(h.counts[s] for s in spec) / st.calls
        buckets: Dict[int, List[int]] = {}
        for i in st.dynamic_dims:
            b, out = 1, []
            while b < st.max_dims[i]:
                if b >= st.min_dims[i]:
                    out.append(b)
                b *= 2
            out.append(st.max_dims[i])
            buckets[i] = out
        return ShapeSpecializationPlan(op, spec, buckets, hit)

    def plan_all(self) -> Dict[str, ShapeSpecializationPlan]:
        out = {}
        for op in self.prof.hist:
            p = self.plan(op)
            if p is not None:
                out[op] = p
        return out

    def apply(self, manager, op: str, compile_fn: Callable[[Tuple[int, ...]], object]) -> int:
        """Pre-compiles the planned exact variants through ``compile_fn(shape)``; returns how many were built."""
        p = self.plan(op)
        if p is None:
            return 0
        n = 0
        for shape in p.specialize:
            compile_fn(shape)
            n += 1
        return n
