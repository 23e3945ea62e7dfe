"""Activation checkpointing (recompute in backward instead of storing).

``checkpoint(fn, *args)`` runs ``fn`` without keeping its intermediate activations and recomputes
them when the gradient arrives; RNG state is restored for the recomputation so dropout matches.
``CheckpointManager`` decides *which* layers to checkpoint with the reference's strategies
(src/MLFramework/Checkpointing/CheckpointConfig.cs:40-90: Interval (every 2nd layer by default),
Selective (layer lists), SizeBased (min activation size 1 MB), MemoryAware (budget 80 % of device
memory), Smart (largest activations first until under budget)), registers / retrieves-or-recomputes
activations by layer id (CheckpointManager.cs:40-87, RecomputationEngine.cs:39-96) and tracks the
memory saved (MemoryTracking.cs).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as nn


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensor, *args):
        ctx.fn = fn
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
        ctx.inputs = args
        with torch.no_grad():
            out = fn(*args)
        return out

    @staticmethod
    def backward(ctx, *grads):
        cpu_now = torch.get_rng_state()
        torch.set_rng_state(ctx.cpu_rng)
        cuda_now = None
        if ctx.cuda_rng is not None:
            cuda_now = torch.cuda.get_rng_state()
            torch.cuda.set_rng_state(ctx.cuda_rng)
        detached = [a.detach().requires_grad_(a.requires_grad) if isinstance(a, torch.Tensor) else a for a in ctx.inputs]
        with torch.enable_grad():
            out = ctx.fn(*detached)
        torch.set_rng_state(cpu_now)
        if cuda_now is not None:
            torch.cuda.set_rng_state(cuda_now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if isinstance(a, torch.Tensor) and a.requires_grad else None for a in detached)


def checkpoint(fn: Callable, *args):
    """Run ``fn(*args)`` keeping only its inputs; intermediates are recomputed during backward.
    Gradients of parameters used inside ``fn`` flow as usual (to ``.grad`` or ``main_grad``)."""
    if not torch.is_grad_enabled():
        return fn(*args)
    return _CheckpointFn.apply(fn, len(args), *args)


class CheckpointStrategyKind(enum.Enum):
    INTERVAL = "interval"
    SELECTIVE = "selective"
    SIZE_BASED = "size_based"
    MEMORY_AWARE = "memory_aware"
    SMART = "smart"


@dataclass
class CheckpointConfig:
    strategy: CheckpointStrategyKind = CheckpointStrategyKind.INTERVAL
    interval: int = 2
    checkpoint_layers: Sequence[str] = ()
    exclude_layers: Sequence[str] = ()
    min_activation_size_bytes: int = 1 << 20
    max_memory_percentage: float = 0.8
    recompute_cache_bytes: int = 100 << 20
    device_memory_bytes: int = 180 << 30

    def validate(self):
        if self.interval <= 0:
            raise ValueError("interval must be positive")
        if not (0.0 < self.max_memory_percentage <= 1.0):
            raise ValueError("max_memory_percentage must be in (0, 1]")


class CheckpointConfigBuilder:
    def __init__(self):
        self._c = CheckpointConfig()

    def with_strategy(self, s): self._c.strategy = s; return self
    def with_interval(self, n): self._c.interval = n; return self
    def with_layers(self, names): self._c.checkpoint_layers = tuple(names); return self
    def excluding(self, names): self._c.exclude_layers = tuple(names); return self
    def with_memory_budget(self, pct): self._c.max_memory_percentage = pct; return self

    def build(self):
        self._c.validate()
        return self._c


@dataclass
class MemoryStats:
    stored_bytes: int = 0
    saved_bytes: int = 0
    recomputations: int = 0
    peak_stored_bytes: int = 0


class CheckpointManager:
    def __init__(self, config: Optional[CheckpointConfig] = None):
        self.cfg = config or CheckpointConfig()
        self.cfg.validate()
        self._store: Dict[str, torch.Tensor] = {}
        self._recompute: Dict[str, Callable[[], torch.Tensor]] = {}
        self.stats = MemoryStats()

    # ---- policy
    def should_checkpoint(self, layer_name: str, layer_index: int, activation_bytes: int = 0) -> bool:
        c = self.cfg
        if layer_name in c.exclude_layers:
            return False
        k = c.strategy
        if k == CheckpointStrategyKind.INTERVAL:
            return layer_index % c.interval == 0
        if k == CheckpointStrategyKind.SELECTIVE:
            return layer_name in c.checkpoint_layers
        if k == CheckpointStrategyKind.SIZE_BASED:
            return activation_bytes >= c.min_activation_size_bytes
        budget = c.max_memory_percentage * c.device_memory_bytes
        if k == CheckpointStrategyKind.MEMORY_AWARE:
            return self.stats.stored_bytes + activation_bytes > budget
        return activation_bytes >= c.min_activation_size_bytes and self.stats.stored_bytes + activation_bytes > 0.5 * budget

    def plan(self, layer_sizes: Dict[str, int]) -> List[str]:
        """Smart strategy as a planner: checkpoint the largest activations first until the rest fits."""
        budget = self.cfg.max_memory_percentage * self.cfg.device_memory_bytes
        total, chosen = sum(layer_sizes.values()), []
        for name, size in sorted(layer_sizes.items(), key=lambda kv: -kv[1]):
            if total <= budget:
                break
            chosen.append(name)
            total -= size
        return chosen

    # ---- store / recompute
    def register_checkpoint(self, layer_id: str, activation: torch.Tensor, recompute_fn: Optional[Callable[[], torch.Tensor]] = None):
        n = activation.numel() * activation.element_size()
        if recompute_fn is not None:
            self._recompute[layer_id] = recompute_fn
            self.stats.saved_bytes += n
        else:
            self._store[layer_id] = activation
            self.stats.stored_bytes += n
            self.stats.peak_stored_bytes = max(self.stats.peak_stored_bytes, self.stats.stored_bytes)

    def retrieve_or_recompute(self, layer_id: str) -> torch.Tensor:
        if layer_id in self._store:
            return self._store[layer_id]
        if layer_id in self._recompute:
            self.stats.recomputations += 1
            return self._recompute[layer_id]()
        raise KeyError(f"no checkpoint registered for layer {layer_id!r}")

    def clear(self):
        self._store.clear()
        self._recompute.clear()
        self.stats.stored_bytes = 0


class CheckpointedModuleWrapper(nn.Module):
    """Wraps a module so its forward is checkpointed (Extensions/CheckpointedModuleWrapper.cs)."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module

    def forward(self, *args):
        return checkpoint(self.module, *args)


def apply_activation_checkpointing(layers: nn.ModuleList, manager: Optional[CheckpointManager] = None) -> int:
    """Wrap the layers the manager's policy selects; returns how many were wrapped."""
    mgr = manager or CheckpointManager()
    n = 0
    for i, layer in enumerate(list(layers)):
        if not isinstance(layer, CheckpointedModuleWrapper) and mgr.should_checkpoint(f"layer{i}", i):
            layers[i] = CheckpointedModuleWrapper(layer)
            n += 1
    return n


# ------------------------------------------------------------------ scopes and selective wrapping
import contextlib as _contextlib
import threading as _threading

_scope = _threading.local()


@_contextlib.contextmanager
def checkpoint_scope(enabled: bool = True):
    """Inside the block ``maybe_checkpoint`` recomputes; outside it runs the function normally. Scopes nest; the
    innermost decides (src/MLFramework/Autograd/CheckpointScope.cs:40)."""
    prev = getattr(_scope, "on", False)
    _scope.on = bool(enabled)
    try:
        yield
    finally:
        _scope.on = prev


def in_checkpoint_scope() -> bool:
    return getattr(_scope, "on", False)


def maybe_checkpoint(fn: Callable, *args):
    return checkpoint(fn, *args) if in_checkpoint_scope() else fn(*args)


def checkpoint_sequential(functions: Sequence[Callable], segments: int, x):
    """Runs ``functions`` one after the other in ``segments`` groups, keeping only the activations between groups."""
    fs = list(functions)
    if segments <= 0:
        raise ValueError("segments must be positive")
    per = max(1, -(-len(fs) // segments))

    def run(group):
        def f(t):
            for fn in group:
                t = fn(t)
            return t
        return f
    for i in range(0, len(fs), per):
        x = checkpoint(run(fs[i:i + per]), x)
    return x


def selective_checkpointing(model: nn.Module, predicate: Callable[[str, nn.Module], bool]) -> List[str]:
    """Wraps every sub-module for which ``predicate(path, module)`` holds (outermost match wins); returns their paths
    (src/MLFramework/Autograd/CheckpointManager.cs:158)."""
    wrapped: List[str] = []

    def walk(parent: nn.Module, prefix: str):
        for name, child in list(parent.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            if isinstance(child, CheckpointedModuleWrapper):
                continue
            if predicate(path, child):
                setattr(parent, name, CheckpointedModuleWrapper(child))
                wrapped.append(path)
            else:
                walk(child, path)
    walk(model, "")
    return wrapped


def tensor_checkpoint_bytes(*tensors: torch.Tensor) -> int:
    """Bytes a set of saved activations holds (what recomputing them would free)."""
    seen, n = set(), 0
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            n += t.numel() * t.element_size()
    return n
