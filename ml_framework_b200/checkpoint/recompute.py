"""Recomputation machinery around activation checkpointing: who recomputes what, in which order, what it costs.

:mod:`ml_framework_b200.checkpoint.activation` holds the autograd function that drops and recomputes a block's
intermediates. This module is the bookkeeping the reference keeps beside it:

* ``DependencyGraph`` - which layer's recomputation needs which other layers first
  (src/MLFramework/Checkpointing/DependencyGraph.cs:24-200);
* ``RecomputationCache`` - a byte-bounded LRU of recomputed activations (RecomputationCache.cs:28-154);
* ``RecomputationEngine`` / ``AsyncRecomputationEngine`` - registered recompute closures run in dependency order,
  per-layer counts and times (RecomputationEngine.cs:39-264, AsyncRecomputationEngine.cs:17-111). The asynchronous
  engine runs closures on worker threads; on a CUDA device each worker uses a side stream of its own and the caller's
  stream waits on an event, so a recomputation overlaps the backward kernels already queued;
* ``MemoryTracker`` - allocation / release accounting per layer with a limit and callbacks (MemoryTracking.cs:30-451);
* ``BackwardHookManager`` - hooks by layer id, invoked when the gradient of a tensor attached to that layer arrives
  (BackwardHookManager.cs:35-208);
* ``CheckpointedGradientAccumulator`` - named gradients averaged over N micro-steps
  (CheckpointedGradientAccumulator.cs:22-209);
* the five strategy objects with a factory (Strategies/*.cs);
* ``CheckpointProfiler`` / ``CheckpointMonitor`` / ``OptimizationRecommender`` (Profiling/*.cs);
* ``DistributedCheckpointManager``, ``ModelParallelCheckpointStrategy``, ``PipelineParallelCheckpointManager``
  (Distributed/*.cs) over this package's process-group facade.
"""
from __future__ import annotations

import enum
import json
import threading
import time
from collections import OrderedDict, defaultdict
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from .activation import CheckpointConfig, CheckpointStrategyKind


class RecomputationError(RuntimeError):
    pass


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


# ------------------------------------------------------------------ dependency order
class DependencyGraph:
    def __init__(self):
        self._deps: Dict[str, List[str]] = {}

    def add_dependency(self, layer_id: str, depends_on: Iterable[str] = ()):
        cur = self._deps.setdefault(layer_id, [])
        for d in depends_on:
            if d == layer_id:
                raise ValueError(f"layer {layer_id!r} cannot depend on itself")
            if d not in cur:
                cur.append(d)
            self._deps.setdefault(d, [])

    def dependencies(self, layer_id: str) -> List[str]:
        return list(self._deps.get(layer_id, ()))

    def topological_order(self, layer_ids: Iterable[str]) -> List[str]:
        """The requested layers and everything they need, dependencies first. Raises on a cycle."""
        order: List[str] = []
        state: Dict[str, int] = {}            # 1 = on the stack, 2 = done
        for root in layer_ids:
            stack = [(root, iter(self._deps.get(root, ())))]
            if state.get(root) == 2:
                continue
            state[root] = 1
            while stack:
                node, it = stack[-1]
                for d in it:
                    s = state.get(d)
                    if s == 1:
                        raise RecomputationError(f"dependency cycle through {d!r}")
                    if s is None:
                        state[d] = 1
                        stack.append((d, iter(self._deps.get(d, ()))))
                        break
                else:
                    state[node] = 2
                    order.append(node)
                    stack.pop()
        return order

    def has_cycle(self) -> bool:
        try:
            self.topological_order(list(self._deps))
            return False
        except RecomputationError:
            return True

    def clear(self):
        self._deps.clear()


# ------------------------------------------------------------------ cache
@dataclass
class CacheStats:
    entries: int = 0
    size_bytes: int = 0
    max_size_bytes: int = 0
    hits: int = 0
    misses: int = 0
    evictions: int = 0

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0


class RecomputationCache:
    """Least-recently-used activations up to ``max_size_bytes``; an activation larger than the whole cache is not kept."""

    def __init__(self, max_size_bytes: int):
        if max_size_bytes <= 0:
            raise ValueError("max_size_bytes must be positive")
        self.max_size_bytes = int(max_size_bytes)
        self._items: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self._bytes = 0
        self._lock = threading.Lock()
        self._hits = self._misses = self._evictions = 0

    def get(self, layer_id: str) -> Optional[torch.Tensor]:
        with self._lock:
            t = self._items.get(layer_id)
            if t is None:
                self._misses += 1
                return None
            self._items.move_to_end(layer_id)
            self._hits += 1
            return t

    def add(self, layer_id: str, activation: torch.Tensor) -> bool:
        n = _nbytes(activation)
        with self._lock:
            if layer_id in self._items:
                self._bytes -= _nbytes(self._items.pop(layer_id))
            if n > self.max_size_bytes:
                return False
            while self._bytes + n > self.max_size_bytes and self._items:
                _, old = self._items.popitem(last=False)
                self._bytes -= _nbytes(old)
                self._evictions += 1
            self._items[layer_id] = activation
            self._bytes += n
            return True

    def contains(self, layer_id: str) -> bool:
        with self._lock:
            return layer_id in self._items

    def clear(self):
        with self._lock:
            self._items.clear()
            self._bytes = 0

    def stats(self) -> CacheStats:
        with self._lock:
            return CacheStats(len(self._items), self._bytes, self.max_size_bytes, self._hits, self._misses, self._evictions)


# ------------------------------------------------------------------ engines
@dataclass
class LayerRecomputationStats:
    layer_id: str
    call_count: int = 0
    total_ms: float = 0.0
    last_ms: float = 0.0

    @property
    def average_ms(self) -> float:
        return self.total_ms / self.call_count if self.call_count else 0.0


@dataclass
class RecomputationStats:
    total_recomputations: int = 0
    total_ms: float = 0.0
    registered_layers: int = 0
    cache: Optional[CacheStats] = None
    layers: Dict[str, LayerRecomputationStats] = field(default_factory=dict)


class RecomputationEngine:
    def __init__(self, cache: Optional[RecomputationCache] = None):
        self._fns: Dict[str, Callable[[], torch.Tensor]] = {}
        self.graph = DependencyGraph()
        self.cache = cache
        self._stats: Dict[str, LayerRecomputationStats] = {}
        self._lock = threading.Lock()

    def register_recompute_function(self, layer_id: str, fn: Callable[[], torch.Tensor], dependencies: Sequence[str] = ()):
        if not layer_id:
            raise ValueError("layer id must not be empty")
        if not callable(fn):
            raise TypeError("recompute function must be callable")
        with self._lock:
            self._fns[layer_id] = fn
            self.graph.add_dependency(layer_id, dependencies)
            self._stats.setdefault(layer_id, LayerRecomputationStats(layer_id))

    def has_recompute_function(self, layer_id: str) -> bool:
        return layer_id in self._fns

    def _run_one(self, layer_id: str) -> torch.Tensor:
        if self.cache is not None:
            hit = self.cache.get(layer_id)
            if hit is not None:
                return hit
        fn = self._fns.get(layer_id)
        if fn is None:
            raise RecomputationError(f"no recompute function registered for layer {layer_id!r}")
        t0 = time.perf_counter()
        try:
            out = fn()
        except Exception as e:
            raise RecomputationError(f"recomputation of layer {layer_id!r} failed: {e}") from e
        ms = (time.perf_counter() - t0) * 1e3
        with self._lock:
            s = self._stats[layer_id]
            s.call_count += 1
            s.total_ms += ms
            s.last_ms = ms
        if self.cache is not None and isinstance(out, torch.Tensor):
            self.cache.add(layer_id, out)
        return out

    def recompute(self, layer_id: str) -> torch.Tensor:
        """Recomputes ``layer_id`` after the layers it depends on (those that have closures registered)."""
        out = None
        for lid in self.graph.topological_order([layer_id]):
            if lid == layer_id or lid in self._fns:
                r = self._run_one(lid)
                if lid == layer_id:
                    out = r
        return out

    def recompute_multiple(self, layer_ids: Iterable[str]) -> Dict[str, torch.Tensor]:
        wanted = list(layer_ids)
        res: Dict[str, torch.Tensor] = {}
        for lid in self.graph.topological_order(wanted):
            if lid in self._fns:
                r = self._run_one(lid)
                if lid in wanted:
                    res[lid] = r
            elif lid in wanted:
                raise RecomputationError(f"no recompute function registered for layer {lid!r}")
        return res

    def layer_stats(self, layer_id: str) -> Optional[LayerRecomputationStats]:
        return self._stats.get(layer_id)

    def stats(self) -> RecomputationStats:
        with self._lock:
            ls = {k: LayerRecomputationStats(**asdict(v)) for k, v in self._stats.items()}
        return RecomputationStats(sum(s.call_count for s in ls.values()), sum(s.total_ms for s in ls.values()), len(self._fns),
                                  self.cache.stats() if self.cache is not None else None, ls)

    def clear(self):
        with self._lock:
            self._fns.clear()
            self._stats.clear()
            self.graph.clear()
        if self.cache is not None:
            self.cache.clear()


class AsyncRecomputationEngine:
    """Recompute closures on worker threads. With ``device`` a CUDA device, every closure runs under a side stream
    (one per worker thread) that first waits for the work queued on the submitting stream; ``result()`` of the
    returned future makes the consumer's current stream wait on the closure's completion event instead of the host."""

    def __init__(self, max_workers: int = 2, device: Optional[torch.device] = None):
        if max_workers <= 0:
            max_workers = 2
        self._pool = ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="mlf-recompute")
        self._fns: Dict[str, Callable[[], torch.Tensor]] = {}
        self.device = torch.device(device) if device is not None else None
        self._tls = threading.local()
        self._closed = False

    def register_recompute_function(self, layer_id: str, fn: Callable[[], torch.Tensor]):
        if not layer_id:
            raise ValueError("layer id must not be empty")
        self._fns[layer_id] = fn

    def _stream(self):
        s = getattr(self._tls, "stream", None)
        if s is None:
            s = self._tls.stream = torch.cuda.Stream(device=self.device)
        return s

    def recompute_async(self, layer_id: str) -> Future:
        if self._closed:
            raise RecomputationError("engine is closed")
        fn = self._fns.get(layer_id)
        if fn is None:
            raise RecomputationError(f"no recompute function registered for layer {layer_id!r}")
        on_cuda = self.device is not None and self.device.type == "cuda"
        ready = torch.cuda.current_stream(self.device).record_event() if on_cuda else None

        def run():
            if not on_cuda:
                return fn()
            s = self._stream()
            s.wait_event(ready)
            with torch.cuda.stream(s):
                out = fn()
                done = s.record_event()
            if isinstance(out, torch.Tensor):
                out.record_stream(s)
            return _StreamResult(out, done, self.device)

        fut = self._pool.submit(run)
        return _UnwrappingFuture(fut) if on_cuda else fut

    def recompute_multiple_async(self, layer_ids: Iterable[str]) -> Dict[str, Future]:
        return {lid: self.recompute_async(lid) for lid in layer_ids}

    def wait_all(self, futures: Dict[str, Future], timeout: Optional[float] = None) -> Dict[str, torch.Tensor]:
        return {k: f.result(timeout) for k, f in futures.items()}

    def close(self):
        self._closed = True
        self._pool.shutdown(wait=True)


@dataclass
class _StreamResult:
    value: object
    done: object
    device: torch.device


class _UnwrappingFuture:
    def __init__(self, inner: Future):
        self._inner = inner

    def done(self) -> bool:
        return self._inner.done()

    def result(self, timeout: Optional[float] = None):
        r = self._inner.result(timeout)
        torch.cuda.current_stream(r.device).wait_event(r.done)
        return r.value


# ------------------------------------------------------------------ memory accounting
@dataclass
class LayerMemoryStats:
    layer_id: str
    current_bytes: int = 0
    peak_bytes: int = 0
    allocations: int = 0
    deallocations: int = 0


@dataclass
class TrackedMemoryStats:
    current_bytes: int = 0
    peak_bytes: int = 0
    total_allocated_bytes: int = 0
    total_freed_bytes: int = 0
    allocation_count: int = 0
    deallocation_count: int = 0
    limit_bytes: Optional[int] = None
    layers: int = 0


class MemoryTracker:
    """Counts the bytes each layer holds. ``on_limit_exceeded(layer_id, current, limit)`` fires once per crossing."""

    def __init__(self, limit_bytes: Optional[int] = None):
        self._layers: Dict[str, LayerMemoryStats] = {}
        self._sizes: Dict[str, List[int]] = defaultdict(list)
        self._s = TrackedMemoryStats(limit_bytes=limit_bytes)
        self._lock = threading.Lock()
        self._over = False
        self.on_allocated: List[Callable[[str, int], None]] = []
        self.on_deallocated: List[Callable[[str, int], None]] = []
        self.on_limit_exceeded: List[Callable[[str, int, int], None]] = []

    def record_allocation(self, layer_id: str, size_bytes: int):
        if size_bytes < 0:
            raise ValueError("size must be non-negative")
        fire = False
        with self._lock:
            l = self._layers.setdefault(layer_id, LayerMemoryStats(layer_id))
            l.current_bytes += size_bytes
            l.peak_bytes = max(l.peak_bytes, l.current_bytes)
            l.allocations += 1
            self._sizes[layer_id].append(size_bytes)
            s = self._s
            s.current_bytes += size_bytes
            s.peak_bytes = max(s.peak_bytes, s.current_bytes)
            s.total_allocated_bytes += size_bytes
            s.allocation_count += 1
            if s.limit_bytes is not None and s.current_bytes > s.limit_bytes and not self._over:
                self._over = fire = True
            cur, lim = s.current_bytes, s.limit_bytes
        for cb in self.on_allocated:
            cb(layer_id, size_bytes)
        if fire:
            for cb in self.on_limit_exceeded:
                cb(layer_id, cur, lim)

    def record_tensor(self, layer_id: str, t: torch.Tensor):
        self.record_allocation(layer_id, _nbytes(t))

    def record_deallocation(self, layer_id: str) -> int:
        """Releases the layer's most recent allocation; returns its size (0 when nothing was held)."""
        with self._lock:
            sizes = self._sizes.get(layer_id)
            if not sizes:
                return 0
            n = sizes.pop()
            l = self._layers[layer_id]
            l.current_bytes -= n
            l.deallocations += 1
            s = self._s
            s.current_bytes -= n
            s.total_freed_bytes += n
            s.deallocation_count += 1
            if s.limit_bytes is None or s.current_bytes <= s.limit_bytes:
                self._over = False
        for cb in self.on_deallocated:
            cb(layer_id, n)
        return n

    def set_memory_limit(self, limit_bytes: Optional[int]):
        if limit_bytes is not None and limit_bytes <= 0:
            raise ValueError("limit must be positive")
        with self._lock:
            self._s.limit_bytes = limit_bytes
            self._over = False

    def stats(self) -> TrackedMemoryStats:
        with self._lock:
            s = TrackedMemoryStats(**asdict(self._s))
            s.layers = len(self._layers)
            return s

    def layer_stats(self, layer_id: str) -> Optional[LayerMemoryStats]:
        with self._lock:
            l = self._layers.get(layer_id)
            return LayerMemoryStats(**asdict(l)) if l is not None else None

    def reset_stats(self):
        with self._lock:
            lim = self._s.limit_bytes
            self._s = TrackedMemoryStats(limit_bytes=lim)
            self._layers.clear()
            self._sizes.clear()
            self._over = False


# ------------------------------------------------------------------ backward hooks by layer id
class BackwardHookManager:
    def __init__(self):
        self._hooks: Dict[int, tuple] = {}            # handle -> (layer id, fn)
        self._by_layer: Dict[str, List[int]] = defaultdict(list)
        self._next = 1
        self._lock = threading.Lock()
        self._attached: List[object] = []

    def register_hook(self, layer_id: str, hook: Callable[[torch.Tensor], Optional[torch.Tensor]]) -> int:
        if not layer_id:
            raise ValueError("layer id must not be empty")
        with self._lock:
            h = self._next
            self._next += 1
            self._hooks[h] = (layer_id, hook)
            self._by_layer[layer_id].append(h)
            return h

    def remove_hook(self, handle: int) -> bool:
        with self._lock:
            e = self._hooks.pop(handle, None)
            if e is None:
                return False
            self._by_layer[e[0]].remove(handle)
            return True

    def remove_hooks_for_layer(self, layer_id: str) -> int:
        with self._lock:
            hs = self._by_layer.pop(layer_id, [])
            for h in hs:
                self._hooks.pop(h, None)
            return len(hs)

    def clear_all_hooks(self):
        with self._lock:
            self._hooks.clear()
            self._by_layer.clear()
        for h in self._attached:
            h.remove()
        self._attached.clear()

    def invoke_hooks(self, layer_id: str, gradient: torch.Tensor) -> torch.Tensor:
        """Calls the layer's hooks in registration order; a hook that returns a tensor replaces the gradient.
        A hook that raises does not stop the others; the first error is raised after all ran."""
        with self._lock:
            fns = [self._hooks[h][1] for h in self._by_layer.get(layer_id, ())]
        err = None
        for fn in fns:
            try:
                r = fn(gradient)
                if isinstance(r, torch.Tensor):
                    gradient = r
            except Exception as e:       # noqa: BLE001 - collected and re-raised below
                err = err or e
        if err is not None:
            raise err
        return gradient

    def attach(self, tensor: torch.Tensor, layer_id: str):
        """The layer's hooks run when autograd delivers ``tensor``'s gradient."""
        if not tensor.requires_grad:
            raise ValueError("tensor does not require grad")
        h = tensor.register_hook(lambda g, lid=layer_id: self.invoke_hooks(lid, g))
        self._attached.append(h)
        return h

    def hook_count_for_layer(self, layer_id: str) -> int:
        with self._lock:
            return len(self._by_layer.get(layer_id, ()))

    def has_hook(self, handle: int) -> bool:
        with self._lock:
            return handle in self._hooks


# ------------------------------------------------------------------ gradient accumulation over micro-steps
class CheckpointedGradientAccumulator:
    def __init__(self, accumulation_steps: int):
        if accumulation_steps <= 0:
            raise ValueError("accumulation_steps must be positive")
        self.accumulation_steps = accumulation_steps
        self._sum: Dict[str, torch.Tensor] = {}
        self.current_step = 0

    def accumulate(self, gradients: Dict[str, torch.Tensor]):
        for k, g in gradients.items():
            acc = self._sum.get(k)
            if acc is None:
                self._sum[k] = g.detach().clone()
            else:
                if acc.shape != g.shape:
                    raise ValueError(f"gradient {k!r} changed shape {tuple(acc.shape)} -> {tuple(g.shape)}")
                acc.add_(g.detach())
        self.current_step += 1

    def should_apply_gradients(self) -> bool:
        return self.current_step >= self.accumulation_steps

    def peek_gradients(self) -> Dict[str, torch.Tensor]:
        n = max(self.current_step, 1)
        return {k: v / n for k, v in self._sum.items()}

    def get_accumulated_gradients(self) -> Dict[str, torch.Tensor]:
        """Averaged gradients; the accumulator starts over."""
        out = self.peek_gradients()
        self.reset()
        return out

    def get_gradient(self, name: str) -> Optional[torch.Tensor]:
        v = self._sum.get(name)
        return None if v is None else v / max(self.current_step, 1)

    def remove_gradient(self, name: str) -> bool:
        return self._sum.pop(name, None) is not None

    def reset(self):
        self._sum.clear()
        self.current_step = 0


# ------------------------------------------------------------------ strategies
class CheckpointStrategy:
    name = "base"

    def should_checkpoint(self, layer_id: str, activation: Optional[torch.Tensor], layer_index: int) -> bool:
        raise NotImplementedError

    def reset(self):
        pass


class IntervalCheckpointStrategy(CheckpointStrategy):
    name = "interval"

    def __init__(self, interval: int = 2):
        if interval <= 0:
            raise ValueError("interval must be positive")
        self.interval = interval

    def should_checkpoint(self, layer_id, activation, layer_index):
        return layer_index % self.interval == 0


class SelectiveCheckpointStrategy(CheckpointStrategy):
    name = "selective"

    def __init__(self, checkpoint_layers: Iterable[str] = (), exclude_layers: Iterable[str] = ()):
        self.include, self.exclude = set(checkpoint_layers), set(exclude_layers)
        both = self.include & self.exclude
        if both:
            raise ValueError(f"layers both selected and excluded: {sorted(both)}")

    def should_checkpoint(self, layer_id, activation, layer_index):
        if layer_id in self.exclude:
            return False
        return layer_id in self.include if self.include else True


class SizeBasedCheckpointStrategy(CheckpointStrategy):
    name = "size_based"

    def __init__(self, min_activation_size_bytes: int = 1 << 20, exclude_layers: Iterable[str] = ()):
        if min_activation_size_bytes < 0:
            raise ValueError("size threshold must be non-negative")
        self.min_bytes, self.exclude = min_activation_size_bytes, set(exclude_layers)

    def should_checkpoint(self, layer_id, activation, layer_index):
        if layer_id in self.exclude or activation is None:
            return False
        return _nbytes(activation) >= self.min_bytes


class MemoryAwareCheckpointStrategy(CheckpointStrategy):
    """Keeps activations while they fit in the budget; once the running total would cross it, the layer is recomputed."""
    name = "memory_aware"

    def __init__(self, max_memory_percentage: float = 0.8, total_memory_bytes: int = 180 << 30, tracker: Optional[MemoryTracker] = None):
        if not (0.0 < max_memory_percentage <= 1.0):
            raise ValueError("max_memory_percentage must be in (0, 1]")
        self.budget = int(max_memory_percentage * total_memory_bytes)
        self.tracker = tracker
        self._kept = 0

    def should_checkpoint(self, layer_id, activation, layer_index):
        n = _nbytes(activation) if activation is not None else 0
        held = self.tracker.stats().current_bytes if self.tracker is not None else self._kept
        if held + n > self.budget:
            return True
        self._kept += n
        return False

    def reset(self):
        self._kept = 0


class SmartCheckpointStrategy(CheckpointStrategy):
    """Learns per-layer activation sizes and recompute costs and recomputes the layers with the most bytes saved per
    millisecond of recomputation until the kept set fits the budget. Before anything is known it behaves like the
    interval rule."""
    name = "smart"

    def __init__(self, max_memory_percentage: float = 0.8, total_memory_bytes: int = 180 << 30, fallback_interval: int = 2):
        self.budget = int(max_memory_percentage * total_memory_bytes)
        self.fallback = IntervalCheckpointStrategy(fallback_interval)
        self.sizes: Dict[str, int] = {}
        self.cost_ms: Dict[str, float] = {}
        self._chosen: Optional[set] = None

    def observe(self, layer_id: str, activation_bytes: int, recompute_ms: Optional[float] = None):
        self.sizes[layer_id] = activation_bytes
        if recompute_ms is not None:
            self.cost_ms[layer_id] = recompute_ms
        self._chosen = None

    def plan(self) -> List[str]:
        total, chosen = sum(self.sizes.values()), []
        rank = sorted(self.sizes, key=lambda k: -(self.sizes[k] / max(self.cost_ms.get(k, 1.0), 1e-3)))
        for k in rank:
            if total <= self.budget:
                break
            chosen.append(k)
            total -= self.sizes[k]
        self._chosen = set(chosen)
        return chosen

    def should_checkpoint(self, layer_id, activation, layer_index):
        if layer_id not in self.sizes:
            if activation is not None:
                self.observe(layer_id, _nbytes(activation))
            return self.fallback.should_checkpoint(layer_id, activation, layer_index)
        if self._chosen is None:
            self.plan()
        return layer_id in self._chosen


def make_strategy(cfg: CheckpointConfig, tracker: Optional[MemoryTracker] = None) -> CheckpointStrategy:
    cfg.validate()
    k = cfg.strategy
    if k == CheckpointStrategyKind.INTERVAL:
        return IntervalCheckpointStrategy(cfg.interval)
    if k == CheckpointStrategyKind.SELECTIVE:
        return SelectiveCheckpointStrategy(cfg.checkpoint_layers, cfg.exclude_layers)
    if k == CheckpointStrategyKind.SIZE_BASED:
        return SizeBasedCheckpointStrategy(cfg.min_activation_size_bytes, cfg.exclude_layers)
    if k == CheckpointStrategyKind.MEMORY_AWARE:
        return MemoryAwareCheckpointStrategy(cfg.max_memory_percentage, cfg.device_memory_bytes, tracker)
    return SmartCheckpointStrategy(cfg.max_memory_percentage, cfg.device_memory_bytes, cfg.interval)


# ------------------------------------------------------------------ profiling
class CheckpointEventType(enum.Enum):
    CHECKPOINT = "checkpoint"
    RECOMPUTE = "recompute"
    CACHE_HIT = "cache_hit"
    CACHE_MISS = "cache_miss"
    RETRIEVE = "retrieve"
    DEALLOCATE = "deallocate"


@dataclass
class CheckpointEvent:
    type: CheckpointEventType
    layer_id: str
    duration_ms: float = 0.0
    memory_bytes: int = 0
    timestamp: float = field(default_factory=time.time)


@dataclass
class LayerProfile:
    layer_id: str
    checkpoint_count: int = 0
    recompute_count: int = 0
    cache_hits: int = 0
    cache_misses: int = 0
    total_checkpoint_ms: float = 0.0
    total_recompute_ms: float = 0.0
    total_memory_saved: int = 0

    @property
    def cache_hit_rate(self) -> float:
        n = self.cache_hits + self.cache_misses
        return self.cache_hits / n if n else 0.0

    @property
    def average_recompute_ms(self) -> float:
        return self.total_recompute_ms / self.recompute_count if self.recompute_count else 0.0


@dataclass
class ProfilingSummary:
    duration_ms: float
    total_checkpoint_ms: float
    total_recompute_ms: float
    total_memory_saved: int
    total_events: int
    cache_hit_rate: float
    layer_profiles: List[LayerProfile]


class CheckpointProfiler:
    def __init__(self, max_events: int = 100_000):
        self.max_events = max_events
        self._events: List[CheckpointEvent] = []
        self._layers: Dict[str, LayerProfile] = {}
        self._t0: Optional[float] = None
        self._t1: Optional[float] = None
        self._lock = threading.Lock()

    @property
    def is_profiling(self) -> bool:
        return self._t0 is not None and self._t1 is None

    def start_profiling(self):
        with self._lock:
            self._events.clear()
            self._layers.clear()
            self._t0, self._t1 = time.perf_counter(), None

    def stop_profiling(self):
        with self._lock:
            if self._t0 is not None and self._t1 is None:
                self._t1 = time.perf_counter()

    def record_event(self, type: CheckpointEventType, layer_id: str, duration_ms: float = 0.0, memory_bytes: int = 0):
        if not self.is_profiling:
            return
        with self._lock:
            if len(self._events) < self.max_events:
                self._events.append(CheckpointEvent(type, layer_id, duration_ms, memory_bytes))
            p = self._layers.setdefault(layer_id, LayerProfile(layer_id))
            if type == CheckpointEventType.CHECKPOINT:
                p.checkpoint_count += 1
                p.total_checkpoint_ms += duration_ms
                p.total_memory_saved += memory_bytes
            elif type == CheckpointEventType.RECOMPUTE:
                p.recompute_count += 1
                p.total_recompute_ms += duration_ms
            elif type == CheckpointEventType.CACHE_HIT:
                p.cache_hits += 1
            elif type == CheckpointEventType.CACHE_MISS:
                p.cache_misses += 1

    def layer_profile(self, layer_id: str) -> Optional[LayerProfile]:
        return self._layers.get(layer_id)

    def all_layer_profiles(self) -> Dict[str, LayerProfile]:
        return dict(self._layers)

    def summary(self) -> ProfilingSummary:
        with self._lock:
            ps = list(self._layers.values())
            end = self._t1 if self._t1 is not None else time.perf_counter()
            dur = (end - self._t0) * 1e3 if self._t0 is not None else 0.0
            hits, misses = sum(p.cache_hits for p in ps), sum(p.cache_misses for p in ps)
            return ProfilingSummary(dur, sum(p.total_checkpoint_ms for p in ps), sum(p.total_recompute_ms for p in ps),
                                    sum(p.total_memory_saved for p in ps), len(self._events),
                                    hits / (hits + misses) if hits + misses else 0.0, ps)

    def generate_report(self) -> str:
        s = self.summary()
        lines = [f"activation checkpointing: {s.total_events} events in {s.duration_ms:.1f} ms",
                 f"  checkpoint time {s.total_checkpoint_ms:.2f} ms, recompute time {s.total_recompute_ms:.2f} ms, "
                 f"memory saved {s.total_memory_saved / 2**20:.1f} MiB, cache hit rate {s.cache_hit_rate:.0%}"]
        for p in sorted(s.layer_profiles, key=lambda p: -p.total_recompute_ms):
            lines.append(f"  {p.layer_id}: {p.checkpoint_count} checkpoints, {p.recompute_count} recomputes "
                         f"({p.average_recompute_ms:.3f} ms each), {p.total_memory_saved / 2**20:.1f} MiB saved")
        return "\n".join(lines)

    def export_json(self) -> str:
        s = self.summary()
        d = asdict(s)
        for p, src in zip(d["layer_profiles"], s.layer_profiles):
            p["cache_hit_rate"] = src.cache_hit_rate
        return json.dumps(d)


class CheckpointMonitor:
    """Polls a profiler and calls back when the memory saved or the time spent recomputing crosses a threshold."""

    def __init__(self, profiler: CheckpointProfiler, memory_threshold_bytes: int = 1 << 30, recompute_threshold_ms: float = 1000.0,
                 interval_s: float = 1.0):
        self.profiler = profiler
        self.memory_threshold_bytes, self.recompute_threshold_ms = memory_threshold_bytes, recompute_threshold_ms
        self.on_memory_threshold: List[Callable[[int, int], None]] = []
        self.on_recompute_threshold: List[Callable[[float, float], None]] = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._loop, args=(interval_s,), daemon=True, name="mlf-ckpt-monitor")
        self._t.start()

    def check_now(self):
        s = self.profiler.summary()
        if s.total_memory_saved > self.memory_threshold_bytes:
            for cb in self.on_memory_threshold:
                cb(s.total_memory_saved, self.memory_threshold_bytes)
        if s.total_recompute_ms > self.recompute_threshold_ms:
            for cb in self.on_recompute_threshold:
                cb(s.total_recompute_ms, self.recompute_threshold_ms)

    def _loop(self, interval_s):
        while not self._stop.wait(interval_s):
            self.check_now()

    def close(self):
        self._stop.set()
        self._t.join(timeout=2.0)


class RecommendationType(enum.Enum):
    REDUCE_RECOMPUTATION = "reduce_recomputation"
    IMPROVE_CACHE_HIT_RATE = "improve_cache_hit_rate"
    IMPROVE_EFFICIENCY = "improve_efficiency"
    ADJUST_CHECKPOINT_STRATEGY = "adjust_checkpoint_strategy"
    ENABLE_ASYNC_RECOMPUTATION = "enable_async_recomputation"
    INCREASE_CHECKPOINT_FREQUENCY = "increase_checkpoint_frequency"


class RecommendationPriority(enum.Enum):
    HIGH = 0
    MEDIUM = 1
    LOW = 2


@dataclass
class OptimizationRecommendation:
    type: RecommendationType
    priority: RecommendationPriority
    title: str
    description: str
    affected_layer_id: Optional[str] = None
    expected_impact: str = ""


def _fmt_ms(ms: float) -> str:
    return f"{ms:.0f}ms" if ms < 1e3 else (f"{ms / 1e3:.1f}s" if ms < 6e4 else f"{ms / 6e4:.1f}m")


class OptimizationRecommender:
    """Rules over a profiling summary (at most three layers per rule, worst first): recomputed more than twice per
    checkpoint -> keep it; cache hit rate under one half after ten checkpoints -> enlarge the cache; checkpointing
    costs over three times the recomputation -> stop checkpointing it; recomputation over 30 % of the profiled time
    -> recompute asynchronously."""

    def generate(self, s: ProfilingSummary) -> List[OptimizationRecommendation]:
        out: List[OptimizationRecommendation] = []
        ps = s.layer_profiles
        for p in sorted((p for p in ps if p.recompute_count > 2 * p.checkpoint_count), key=lambda p: -p.total_recompute_ms)[:3]:
            out.append(OptimizationRecommendation(
                RecommendationType.REDUCE_RECOMPUTATION, RecommendationPriority.HIGH, f"Reduce recomputation for layer '{p.layer_id}'",
                f"recomputed {p.recompute_count} times for {p.checkpoint_count} checkpoints; keep its activation or checkpoint more often",
                p.layer_id, f"could save {_fmt_ms(p.total_recompute_ms)} of recomputation"))
        for p in sorted((p for p in ps if p.checkpoint_count > 10 and p.cache_hit_rate < 0.5), key=lambda p: p.cache_hit_rate)[:3]:
            out.append(OptimizationRecommendation(
                RecommendationType.IMPROVE_CACHE_HIT_RATE, RecommendationPriority.MEDIUM, f"Improve cache hit rate for layer '{p.layer_id}'",
                f"cache hit rate {p.cache_hit_rate:.0%}; enlarge the recomputation cache or change the strategy",
                p.layer_id, f"hit rate could reach ~{min(1.0, p.cache_hit_rate + 0.3):.0%}"))
        for p in sorted((p for p in ps if p.total_memory_saved > 0 and p.total_checkpoint_ms > 3 * p.total_recompute_ms),
                        key=lambda p: -p.total_checkpoint_ms)[:3]:
            gain = (p.total_checkpoint_ms - p.total_recompute_ms) * 100 / p.total_checkpoint_ms
            out.append(OptimizationRecommendation(
                RecommendationType.IMPROVE_EFFICIENCY, RecommendationPriority.LOW, f"Improve checkpointing efficiency for layer '{p.layer_id}'",
                "checkpoint overhead is high compared to its recomputation; skip checkpointing this layer",
                p.layer_id, f"could reduce overhead by ~{gain:.0f}%"))
        if s.duration_ms > 0 and s.total_recompute_ms > 0.3 * s.duration_ms:
            out.append(OptimizationRecommendation(
                RecommendationType.ENABLE_ASYNC_RECOMPUTATION, RecommendationPriority.MEDIUM, "Recompute on a side stream",
                f"recomputation takes {s.total_recompute_ms / s.duration_ms:.0%} of the profiled time",
                None, "overlaps recomputation with the backward kernels already queued"))
        out.sort(key=lambda r: r.priority.value)
        return out


# ------------------------------------------------------------------ distributed variants
@dataclass
class DistributedMemoryStats:
    per_rank_bytes: List[int]

    @property
    def total_bytes(self) -> int:
        return sum(self.per_rank_bytes)

    @property
    def max_bytes(self) -> int:
        return max(self.per_rank_bytes) if self.per_rank_bytes else 0

    @property
    def min_bytes(self) -> int:
        return min(self.per_rank_bytes) if self.per_rank_bytes else 0

    @property
    def average_bytes(self) -> float:
        return self.total_bytes / len(self.per_rank_bytes) if self.per_rank_bytes else 0.0

    @property
    def imbalance(self) -> float:
        """max / mean - 1: zero when every rank holds the same amount."""
        return self.max_bytes / self.average_bytes - 1.0 if self.average_bytes else 0.0


class DistributedCheckpointManager:
    """Activation checkpoints of a group of ranks. A checkpoint lives on the rank that registered it; other ranks fetch
    it with a broadcast from its owner (``retrieve_or_fetch`` is collective when ``source_rank`` is given)."""

    def __init__(self, pg, tracker: Optional[MemoryTracker] = None):
        self.pg = pg
        self.rank, self.world_size = pg.rank, pg.world_size
        self._store: Dict[str, torch.Tensor] = {}
        self.tracker = tracker or MemoryTracker()

    def register_checkpoint(self, layer_id: str, activation: torch.Tensor):
        self._store[layer_id] = activation
        self.tracker.record_tensor(layer_id, activation)

    def register_checkpoint_broadcast(self, layer_id: str, activation: torch.Tensor, source_rank: int = 0):
        """Every rank ends up holding the source rank's activation (collective)."""
        t = activation if self.rank == source_rank else torch.empty_like(activation)
        self.pg.broadcast(t, src=source_rank)
        self.register_checkpoint(layer_id, t)

    def synchronize_checkpoints(self):
        self.pg.barrier()

    def has_checkpoint(self, layer_id: str) -> bool:
        return layer_id in self._store

    def retrieve_or_fetch(self, layer_id: str, source_rank: Optional[int] = None) -> torch.Tensor:
        if source_rank is None:
            if layer_id not in self._store:
                raise KeyError(f"rank {self.rank} holds no checkpoint for layer {layer_id!r}")
            return self._store[layer_id]
        meta = None
        if self.rank == source_rank:
            if layer_id not in self._store:
                raise KeyError(f"source rank {source_rank} holds no checkpoint for layer {layer_id!r}")
            src = self._store[layer_id]
            meta = (tuple(src.shape), str(src.dtype).replace("torch.", ""))
        meta = self.pg.broadcast_object(meta, src=source_rank)
        if self.rank == source_rank:
            t = self._store[layer_id]
        else:
            ref = next(iter(self._store.values()), None)
            dev = ref.device if ref is not None else torch.device("cpu")
            t = torch.empty(meta[0], dtype=getattr(torch, meta[1]), device=dev)
        self.pg.broadcast(t, src=source_rank)
        return t

    def clear_checkpoints_distributed(self):
        for lid in list(self._store):
            self.tracker.record_deallocation(lid)
        self._store.clear()
        self.pg.barrier()

    def aggregated_memory_stats(self) -> DistributedMemoryStats:
        return DistributedMemoryStats([int(b) for b in self.pg.all_gather_object(self.tracker.stats().current_bytes)])


class ModelParallelCheckpointStrategy:
    """Under tensor parallelism a replicated activation is kept by the first rank of each tensor-parallel group only;
    layers can be pinned to a rank explicitly."""

    def __init__(self, rank: int, tensor_parallel_size: int):
        if tensor_parallel_size <= 0:
            raise ValueError("tensor_parallel_size must be positive")
        self.rank, self.tp = rank, tensor_parallel_size
        self._layer_rank: Dict[str, int] = {}

    def should_checkpoint(self, layer_id: str, activation: Optional[torch.Tensor] = None, is_tensor_parallel: bool = False) -> bool:
        if layer_id in self._layer_rank:
            return self._layer_rank[layer_id] == self.rank
        if is_tensor_parallel:
            return self.rank % self.tp == 0
        return True

    def checkpoint_rank(self, layer_id: str) -> int:
        return self._layer_rank.get(layer_id, 0)

    def register_layer_rank(self, layer_id: str, rank: int):
        self._layer_rank[layer_id] = rank


class PipelineParallelCheckpointManager:
    """Per-stage activation checkpoints of a pipeline; ``next_stage_boundaries`` are the tensors the following stage
    consumes (this stage's boundary outputs)."""

    def __init__(self, stage: int, num_stages: int):
        if not (0 <= stage < num_stages):
            raise ValueError("stage out of range")
        self.stage, self.num_stages = stage, num_stages
        self._by_stage: Dict[int, List[tuple]] = defaultdict(list)

    def register_stage_checkpoint(self, stage: int, layer_id: str, activation: torch.Tensor, is_boundary: bool = False):
        if not (0 <= stage < self.num_stages):
            raise ValueError("stage out of range")
        self._by_stage[stage].append((layer_id, activation, is_boundary))

    def stage_checkpoints(self, stage: int) -> List[torch.Tensor]:
        return [t for _, t, _ in self._by_stage.get(stage, ())]

    def next_stage_boundaries(self) -> List[torch.Tensor]:
        if self.stage + 1 >= self.num_stages:
            return []
        return [t for _, t, b in self._by_stage.get(self.stage, ()) if b]

    def clear_stage_checkpoints(self, stage: Optional[int] = None):
        if stage is None:
            self._by_stage.clear()
        else:
            self._by_stage.pop(stage, None)
