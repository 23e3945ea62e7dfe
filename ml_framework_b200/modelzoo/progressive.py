"""Progressive model loading: layers arrive when they are needed, and can leave again.

Reference: src/ModelZoo/Progressive — ProgressiveModelLoader.cs:10-346, LazyParameter.cs:10-234,
ProgressiveLoadContext.cs:9-187, ProgressiveLoadOptions.cs:8-55, LayerLoadOrder.cs:6-150,
LayerLoadingStrategy.cs:6-27, UnloadStrategy.cs:6-22, MemoryManager.cs:8-225,
ModelZooProgressiveExtensions.cs:9-112.

The model is built with its parameters on the ``meta`` device (shapes, no storage). Each
layer (a leaf of the container tree) owns the state-dict keys under its name; a forward
pre-hook makes the layer resident before it runs, reading just its tensors from the weight
file (``torch.save`` files through a memory map, the zoo's own format through its index).
Background strategies load ahead of the forward pass; the unload strategies send layers back
to ``meta`` under a byte budget or a layer-count cap, least recently used first. Unloading
is for inference: autograd keeps no claim on a layer that has left.
"""
from __future__ import annotations

import enum
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from .transfer import layers as _module_layers

__all__ = [
    "LayerLoadingStrategy", "UnloadStrategy", "ModelArchitectureType", "LayerLoadOrder",
    "ProgressiveLoadOptions", "LayerMemoryInfo", "MemoryManager", "WeightSource", "DictSource",
    "TorchFileSource", "ZooFileSource", "open_weight_source", "LazyLayer", "ProgressiveLoadContext",
    "ProgressiveModelLoader", "load_progressive",
]


class LayerLoadingStrategy(enum.Enum):
    ON_DEMAND = "on_demand"      # a layer loads when the forward pass reaches it
    SEQUENTIAL = "sequential"    # one background worker walks the load order
    PARALLEL = "parallel"        # up to max_concurrent_loads workers
    PREFETCH = "prefetch"        # on demand, plus the next prefetch_count layers in the background


class UnloadStrategy(enum.Enum):
    NEVER = "never"
    MEMORY_PRESSURE = "memory_pressure"   # over memory_pressure_threshold bytes: oldest use leaves first
    LRU = "lru"                           # at most max_loaded_layers resident


class ModelArchitectureType(enum.Enum):
    CNN = "cnn"
    TRANSFORMER = "transformer"
    RNN = "rnn"
    MLP = "mlp"
    CUSTOM = "custom"


class LayerLoadOrder:
    """Layers in the order they will be wanted, with optional "needs" edges: a layer's
    dependencies come out before it (LayerLoadOrder.cs:87-122)."""

    def __init__(self, architecture_type: ModelArchitectureType = ModelArchitectureType.CUSTOM):
        self.architecture_type = architecture_type
        self.ordered_layers: List[str] = []
        self.dependencies: Dict[str, List[str]] = {}

    @classmethod
    def for_cnn(cls):
        return cls(ModelArchitectureType.CNN)

    @classmethod
    def for_transformer(cls):
        return cls(ModelArchitectureType.TRANSFORMER)

    @classmethod
    def for_rnn(cls):
        return cls(ModelArchitectureType.RNN)

    @classmethod
    def for_architecture(cls, architecture: str):
        a = architecture.lower()
        if "cnn" in a or "conv" in a or "resnet" in a:
            return cls.for_cnn()
        if any(k in a for k in ("transformer", "attention", "gpt", "llama", "bert")):
            return cls.for_transformer()
        if any(k in a for k in ("rnn", "lstm", "gru")):
            return cls.for_rnn()
        return cls(ModelArchitectureType.MLP if "mlp" in a else ModelArchitectureType.CUSTOM)

    @classmethod
    def from_model(cls, model: nn.Module, architecture: str = "custom"):
        o = cls.for_architecture(architecture)
        for name, m in _module_layers(model):
            if next(m.parameters(), None) is not None or next(m.buffers(), None) is not None:
                o.add_layer(name)
        return o

    def add_layer(self, layer_name: str):
        if layer_name is None:
            raise ValueError("the layer name is required")
        if layer_name not in self.ordered_layers:
            self.ordered_layers.append(layer_name)

    def add_dependency(self, layer_name: str, dependency_name: str):
        self.dependencies.setdefault(layer_name, [])
        if dependency_name not in self.dependencies[layer_name]:
            self.dependencies[layer_name].append(dependency_name)

    def get_load_order(self) -> List[str]:
        out: List[str] = []
        seen: set = set()

        def visit(layer: str):
            if layer in seen:
                return
            seen.add(layer)
            for d in self.dependencies.get(layer, ()):
                visit(d)
            out.append(layer)
        for layer in self.ordered_layers:
            visit(layer)
        return out


@dataclass
class ProgressiveLoadOptions:
    strategy: LayerLoadingStrategy = LayerLoadingStrategy.ON_DEMAND
    max_concurrent_loads: int = 3
    prefetch_count: int = 1
    unload_strategy: UnloadStrategy = UnloadStrategy.NEVER
    max_loaded_layers: int = -1
    memory_pressure_threshold: int = 100 * 1024 * 1024


@dataclass
class LayerMemoryInfo:
    layer_name: str
    size_in_bytes: int
    load_time: float
    last_access_time: float


class MemoryManager:
    """Who is resident, how large, and used when (MemoryManager.cs:8-225)."""

    def __init__(self, options: ProgressiveLoadOptions, clock: Callable[[], float] = time.monotonic):
        self._o, self._clock = options, clock
        self._loaded: Dict[str, LayerMemoryInfo] = {}
        self._lru: List[str] = []                     # most recent first
        self._lock = threading.Lock()
        self.total_loaded_bytes = 0

    @property
    def loaded_layer_count(self) -> int:
        return len(self._loaded)

    def register_layer(self, layer_name: str, size_in_bytes: int) -> None:
        with self._lock:
            if layer_name in self._loaded:
                self.total_loaded_bytes -= self._loaded[layer_name].size_in_bytes
                self._lru.remove(layer_name)
            now = self._clock()
            self._loaded[layer_name] = LayerMemoryInfo(layer_name, size_in_bytes, now, now)
            self._lru.insert(0, layer_name)
            self.total_loaded_bytes += size_in_bytes

    def record_access(self, layer_name: str) -> None:
        with self._lock:
            info = self._loaded.get(layer_name)
            if info is None:
                return
            info.last_access_time = self._clock()
            self._lru.remove(layer_name)
            self._lru.insert(0, layer_name)

    def unregister_layer(self, layer_name: str) -> int:
        with self._lock:
            info = self._loaded.pop(layer_name, None)
            if info is None:
                return 0
            self._lru.remove(layer_name)
            self.total_loaded_bytes -= info.size_in_bytes
            return info.size_in_bytes

    def has_memory_pressure(self) -> bool:
        u = self._o.unload_strategy
        if u is UnloadStrategy.MEMORY_PRESSURE:
            return self.total_loaded_bytes > self._o.memory_pressure_threshold
        if u is UnloadStrategy.LRU:
            return self._o.max_loaded_layers > 0 and len(self._loaded) > self._o.max_loaded_layers
        return False

    def get_layers_to_unload(self, count: Optional[int] = None, keep: Iterable[str] = ()) -> List[str]:
        """Least recently used first; enough of them to end the pressure (at most ``count``),
        never one of ``keep``."""
        u, keep = self._o.unload_strategy, set(keep)
        if u is UnloadStrategy.NEVER:
            return []
        out: List[str] = []
        with self._lock:
            cand = [n for n in reversed(self._lru) if n not in keep]
            if u is UnloadStrategy.LRU:
                excess = len(self._loaded) - self._o.max_loaded_layers if self._o.max_loaded_layers > 0 else 0
                out = cand[:max(0, excess)]
            else:
                to_free, freed = self.total_loaded_bytes - self._o.memory_pressure_threshold, 0
                for n in cand:
                    if freed >= to_free:
                        break
                    out.append(n)
                    freed += self._loaded[n].size_in_bytes
        return out if count is None else out[:count]

    def get_memory_info(self) -> Dict[str, LayerMemoryInfo]:
        with self._lock:
            return dict(self._loaded)

    def clear(self) -> None:
        with self._lock:
            self._loaded.clear()
            self._lru.clear()
            self.total_loaded_bytes = 0


# ------------------------------------------------------------------ weight sources
class WeightSource:
    """Random access to named tensors of a weight file."""

    def keys(self) -> List[str]:
        raise NotImplementedError

    def read(self, names: Sequence[str]) -> Dict[str, torch.Tensor]:
        raise NotImplementedError


class DictSource(WeightSource):
    def __init__(self, state: Dict[str, torch.Tensor]):
        self._s = state
        self.reads: List[List[str]] = []

    def keys(self):
        return list(self._s)

    def read(self, names):
        self.reads.append(list(names))
        return {n: self._s[n] for n in names}


class TorchFileSource(WeightSource):
    """A ``torch.save`` state dict, memory-mapped: a tensor's pages are read when it is copied."""

    def __init__(self, path: str):
        self._s = torch.load(path, map_location="cpu", mmap=True, weights_only=True)

    def keys(self):
        return list(self._s)

    def read(self, names):
        return {n: self._s[n] for n in names}


class ZooFileSource(WeightSource):
    """The zoo's self-describing format: the header's index gives each tensor's offset."""

    def __init__(self, path: str, verify_checksums: bool = True):
        from .serialization import ModelDeserializer
        self._path, self._d = path, ModelDeserializer(verify_checksums)
        with open(path, "rb") as f:
            self._names = [e["name"] for e in self._d.read_header(f)["tensors"]]

    def keys(self):
        return list(self._names)

    def read(self, names):
        return self._d.deserialize_file(self._path, names)


def open_weight_source(path: str) -> WeightSource:
    from .serialization import MAGIC
    with open(path, "rb") as f:
        magic = f.read(len(MAGIC))
    return ZooFileSource(path) if magic == MAGIC else TorchFileSource(path)


# ------------------------------------------------------------------ one lazily resident layer
#: Name of the layer that holds tensors owned by containers themselves.
ROOT_LAYER = "(root)"


def _owner(root: nn.Module, dotted: str):
    *path, leaf = dotted.split(".")
    m = root
    for p in path:
        m = getattr(m, p)
    return m, leaf


class LazyLayer:
    """The tensors of one layer: resident or on ``meta`` (the counterpart of LazyParameter.cs)."""

    def __init__(self, layer_name: str, module: nn.Module, keys: Dict[str, str], source: WeightSource,
                 device: torch.device, dtype: Optional[torch.dtype] = None):
        self.layer_name, self.module = layer_name, module
        self._keys = keys                                   # name inside the module -> state-dict key
        self._source, self._device, self._dtype = source, device, dtype
        self._lock = threading.Lock()
        self.is_loaded = False
        self.on_layer_loaded: List[Callable[["LazyLayer"], None]] = []
        self.on_layer_unloaded: List[Callable[["LazyLayer"], None]] = []
        self.size_in_bytes = sum(t.numel() * (torch.empty((), dtype=dtype or t.dtype).element_size())
                                 for t in self._tensors().values())

    def _tensors(self) -> Dict[str, torch.Tensor]:
        out = dict(self.module.named_parameters())
        out.update(dict(self.module.named_buffers()))
        return {k: v for k, v in out.items() if k in self._keys}

    def ensure_loaded(self) -> bool:
        """Makes the layer resident; ``True`` if this call did the loading."""
        with self._lock:
            if self.is_loaded:
                return False
            got = self._source.read(list(self._keys.values()))
            params = dict(self.module.named_parameters())
            for local, key in self._keys.items():
                src = got[key]
                owner, leaf = _owner(self.module, local)
                cur = getattr(owner, leaf)
                if tuple(cur.shape) != tuple(src.shape):
                    raise ValueError(f"{self.layer_name}.{local}: file has shape {tuple(src.shape)}, model {tuple(cur.shape)}")
                dt = self._dtype if (self._dtype is not None and src.is_floating_point()) else cur.dtype
                val = src.to(device=self._device, dtype=dt, copy=True)
                if local in params:
                    owner._parameters[leaf] = nn.Parameter(val, requires_grad=cur.requires_grad)
                else:
                    owner._buffers[leaf] = val
            self.is_loaded = True
        for cb in self.on_layer_loaded:
            cb(self)
        return True

    def unload(self) -> bool:
        with self._lock:
            if not self.is_loaded:
                return False
            params = dict(self.module.named_parameters())
            for local in self._keys:
                owner, leaf = _owner(self.module, local)
                cur = getattr(owner, leaf)
                ghost = torch.empty(cur.shape, dtype=cur.dtype, device="meta")
                if local in params:
                    owner._parameters[leaf] = nn.Parameter(ghost, requires_grad=cur.requires_grad)
                else:
                    owner._buffers[leaf] = ghost
            self.is_loaded = False
        for cb in self.on_layer_unloaded:
            cb(self)
        return True


# ------------------------------------------------------------------ context and loader
class ProgressiveLoadContext:
    """Shared state of one progressive load (ProgressiveLoadContext.cs:9-187)."""

    def __init__(self, metadata, device, options: ProgressiveLoadOptions, layer_load_order: LayerLoadOrder,
                 clock: Callable[[], float] = time.monotonic):
        self.metadata, self.device, self.options = metadata, torch.device(device), options
        self.layer_load_order = layer_load_order
        self.loaded_layers: set = set()
        self.total_layers = len(layer_load_order.get_load_order())
        self.memory_manager = MemoryManager(options, clock)
        self.ever_loaded: set = set()
        self._lock = threading.Lock()

    @property
    def loading_strategy(self) -> LayerLoadingStrategy:
        return self.options.strategy

    @property
    def loading_progress(self) -> float:
        """Share of layers that have been resident at least once."""
        return len(self.ever_loaded) / self.total_layers if self.total_layers else 1.0

    def is_layer_loaded(self, layer_name: str) -> bool:
        return layer_name in self.loaded_layers

    def mark_layer_loaded(self, layer_name: str, size_in_bytes: int = 0):
        with self._lock:
            self.loaded_layers.add(layer_name)
            self.ever_loaded.add(layer_name)
        self.memory_manager.register_layer(layer_name, size_in_bytes)

    def mark_layer_unloaded(self, layer_name: str):
        with self._lock:
            self.loaded_layers.discard(layer_name)
        self.memory_manager.unregister_layer(layer_name)

    def is_fully_loaded(self) -> bool:
        return len(self.ever_loaded) >= self.total_layers

    def get_next_layers_to_load(self, current_layer: Optional[str] = None) -> List[str]:
        order, s = self.layer_load_order.get_load_order(), self.options.strategy
        if s is LayerLoadingStrategy.ON_DEMAND:
            return []
        if s is LayerLoadingStrategy.PARALLEL:
            return [n for n in order if n not in self.loaded_layers][:self.options.max_concurrent_loads]
        start = order.index(current_layer) + 1 if current_layer in order else 0
        return [n for n in order[start:] if n not in self.loaded_layers][:self.options.prefetch_count]


class ProgressiveModelLoader:
    """Attaches lazy layers to ``model`` (built on ``meta``, or anywhere: resident tensors are then
    overwritten on first use) and runs the chosen strategy (ProgressiveModelLoader.cs:10-346)."""

    def __init__(self, model: nn.Module, source: WeightSource, options: Optional[ProgressiveLoadOptions] = None,
                 device="cpu", dtype: Optional[torch.dtype] = None, metadata=None,
                 layer_load_order: Optional[LayerLoadOrder] = None, strict: bool = True,
                 clock: Callable[[], float] = time.monotonic):
        self.model, self.source = model, source
        self.options = options or ProgressiveLoadOptions()
        arch = getattr(metadata, "architecture", "custom") if metadata is not None else "custom"
        order = layer_load_order or LayerLoadOrder.from_model(model, arch)
        self.context = ProgressiveLoadContext(metadata, device, self.options, order, clock)
        self.on_layer_loaded: List[Callable[[str], None]] = []
        self.on_progress_changed: List[Callable[[float], None]] = []
        self.on_fully_loaded: List[Callable[[], None]] = []
        self._lazy: Dict[str, LazyLayer] = {}
        self._hooks = []
        self._pool: Optional[ThreadPoolExecutor] = None
        self._done = threading.Event()
        self._fired_full = False
        self._evt_lock = threading.Lock()
        have = set(source.keys())
        by_name = dict(_module_layers(model))
        # tensors that sit on a container itself (a root-level parameter, say) belong to no layer: they
        # form one more, loaded first and never unloaded, since no hook can tell when they are used
        claimed = {f"{n}.{k}" if n else k for n, m in by_name.items() if n in order.get_load_order()
                   for k in [*dict(m.named_parameters()), *dict(m.named_buffers())]}
        loose = [k for k in [*dict(model.named_parameters()), *dict(model.named_buffers())] if k not in claimed]
        if loose and ROOT_LAYER not in order.ordered_layers:
            order.ordered_layers.insert(0, ROOT_LAYER)
            self.context.total_layers += 1
        missing: List[str] = []
        for name in order.get_load_order():
            if name == ROOT_LAYER:
                keys = {k: k for k in loose if k in have}
                missing += [k for k in loose if k not in have]
                self.register_layer(name, model, keys, dtype)
                continue
            if name not in by_name:
                raise KeyError(f"the load order names layer {name!r}, which the model does not have")
            m = by_name[name]
            local = [k for k, _ in m.named_parameters()] + [k for k, _ in m.named_buffers()]
            keys = {k: (f"{name}.{k}" if name else k) for k in local}
            missing += [v for v in keys.values() if v not in have]
            keys = {k: v for k, v in keys.items() if v in have}
            self.register_layer(name, m, keys, dtype)
        if strict and missing:
            raise KeyError(f"the weight file lacks {len(missing)} tensors, e.g. {missing[:4]}")
        self.missing_keys = missing
        if self.context.total_layers == 0:
            self._done.set()
        if self.options.strategy in (LayerLoadingStrategy.SEQUENTIAL, LayerLoadingStrategy.PARALLEL):
            self._start_background_walk()

    # ---- registration
    @property
    def lazy_layers(self) -> Dict[str, LazyLayer]:
        return dict(self._lazy)

    def register_layer(self, name: str, module: nn.Module, keys: Dict[str, str], dtype=None) -> LazyLayer:
        lazy = LazyLayer(name, module, keys, self.source, self.context.device, dtype)
        lazy.on_layer_loaded.append(self._loaded)
        lazy.on_layer_unloaded.append(lambda l: self.context.mark_layer_unloaded(l.layer_name))
        self._lazy[name] = lazy
        self._hooks.append(module.register_forward_pre_hook(lambda mod, args, n=name: self._before_forward(n)))
        return lazy

    def get_layer(self, layer_name: str) -> Optional[LazyLayer]:
        return self._lazy.get(layer_name)

    # ---- events
    def _loaded(self, lazy: LazyLayer):
        self.context.mark_layer_loaded(lazy.layer_name, lazy.size_in_bytes)
        for cb in self.on_layer_loaded:
            cb(lazy.layer_name)
        p = self.context.loading_progress
        for cb in self.on_progress_changed:
            cb(p)
        fire = False
        with self._evt_lock:
            if self.context.is_fully_loaded() and not self._fired_full:
                self._fired_full = fire = True
        if fire:
            self._done.set()
            for cb in self.on_fully_loaded:
                cb()

    # ---- the forward path
    def _before_forward(self, name: str):
        lazy = self._lazy[name]
        lazy.ensure_loaded()
        self.context.memory_manager.record_access(name)
        if self.options.strategy is LayerLoadingStrategy.PREFETCH:
            self.prefetch_next_layers(name)
        self.manage_memory(keep=(name, ROOT_LAYER))

    # ---- loading ahead
    def _executor(self) -> ThreadPoolExecutor:
        if self._pool is None:
            workers = 1 if self.options.strategy is LayerLoadingStrategy.SEQUENTIAL else max(1, self.options.max_concurrent_loads)
            self._pool = ThreadPoolExecutor(workers, thread_name_prefix="mlf-progressive")
        return self._pool

    def _start_background_walk(self):
        for name in self.context.layer_load_order.get_load_order():
            self._executor().submit(self._lazy[name].ensure_loaded)

    def prefetch_layer(self, layer_name: str):
        """Starts loading in the background; returns the future."""
        if layer_name not in self._lazy:
            raise KeyError(layer_name)
        return self._executor().submit(self._lazy[layer_name].ensure_loaded)

    def prefetch_layers(self, layer_names: Sequence[str]):
        return [self.prefetch_layer(n) for n in layer_names]

    def prefetch_next_layers(self, current_layer: Optional[str] = None):
        return self.prefetch_layers(self.context.get_next_layers_to_load(current_layer))

    def load_all(self) -> None:
        """Loads what is not resident, in load order, on the calling thread."""
        for name in self.context.layer_load_order.get_load_order():
            self._lazy[name].ensure_loaded()

    # ---- memory
    def manage_memory(self, keep: Iterable[str] = ()) -> List[str]:
        mm = self.context.memory_manager
        if not mm.has_memory_pressure():
            return []
        gone = mm.get_layers_to_unload(keep={*keep, ROOT_LAYER})
        for n in gone:
            self._lazy[n].unload()
        return gone

    # ---- progress
    def get_loading_progress(self) -> float:
        return self.context.loading_progress

    def is_fully_loaded(self) -> bool:
        return self.context.is_fully_loaded()

    def wait_for_fully_loaded(self, timeout_ms: int = 60000) -> bool:
        return self._done.wait(timeout_ms / 1000.0)

    def close(self):
        """Removes the hooks and stops the workers; resident layers stay as they are."""
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None


def load_progressive(model_factory: Callable[[], nn.Module], weights_path: str,
                     options: Optional[ProgressiveLoadOptions] = None, device="cpu",
                     dtype: Optional[torch.dtype] = None, metadata=None, strict: bool = True):
    """Builds the model on ``meta`` and attaches a loader over ``weights_path``; returns
    (model, loader). The first forward pass pulls the layers in."""
    with torch.device("meta"):
        model = model_factory()
    loader = ProgressiveModelLoader(model, open_weight_source(weights_path), options, device, dtype, metadata, strict=strict)
    return model, loader
