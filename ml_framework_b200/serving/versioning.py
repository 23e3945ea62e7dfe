"""Model version lifecycle, routing policies and monitoring.

Reference: src/MLFramework/ModelVersioning/{ModelRegistry,ModelVersionManager,ModelHotSwapper,VersionRouter,
VersionMonitor}.cs + model / enum files: lifecycle states (Registered -> Staging -> Production -> Deprecated ->
Archived), routing modes (latest, pinned, percentage, shadow), monitor with alert thresholds and metric
comparison between versions. Built on ``deployment.py``'s registry and swapper.
"""
from __future__ import annotations

import enum
import time
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

from .deployment import ModelHotSwapper, ModelMetadata, ModelRegistry, SemanticVersion, TrafficSplitter


class VersionState(enum.Enum):
    REGISTERED = "registered"
    STAGING = "staging"
    PRODUCTION = "production"
    DEPRECATED = "deprecated"
    ARCHIVED = "archived"


_ALLOWED = {
    VersionState.REGISTERED: {VersionState.STAGING, VersionState.ARCHIVED},
    VersionState.STAGING: {VersionState.PRODUCTION, VersionState.REGISTERED, VersionState.ARCHIVED},
    VersionState.PRODUCTION: {VersionState.DEPRECATED, VersionState.STAGING},
    VersionState.DEPRECATED: {VersionState.ARCHIVED, VersionState.PRODUCTION},
    VersionState.ARCHIVED: set(),
}


class ModelVersionManager:
    def __init__(self, registry: Optional[ModelRegistry] = None, swapper: Optional[ModelHotSwapper] = None):
        self.reg = registry or ModelRegistry()
        self.sw = swapper or ModelHotSwapper(self.reg)
        self.state: Dict[Tuple[str, str], VersionState] = {}
        self.log: List[Tuple[float, str, str, str, str]] = []

    def register(self, name: str, version: str, model: Any, **tags):
        SemanticVersion.parse(version)
        self.reg.register(model, ModelMetadata(name, version, tags=dict(tags)))
        self.state[(name, version)] = VersionState.REGISTERED

    def transition(self, name: str, version: str, to: VersionState):
        cur = self.state[(name, version)]
        if to not in _ALLOWED[cur]:
            raise ValueError(f"{name}:{version}: illegal transition {cur.value} -> {to.value}")
        if to == VersionState.PRODUCTION:
            for (n, v), s in list(self.state.items()):          # one production version per model
                if n == name and s == VersionState.PRODUCTION and v != version:
                    self.state[(n, v)] = VersionState.DEPRECATED
            self.sw.swap(name, version) if name in self.sw.active else self.sw.activate(name, version)
        self.state[(name, version)] = to
        self.log.append((time.time(), name, version, cur.value, to.value))

    def promote(self, name: str, version: str):
        if self.state[(name, version)] == VersionState.REGISTERED:
            self.transition(name, version, VersionState.STAGING)
        self.transition(name, version, VersionState.PRODUCTION)

    def production(self, name: str) -> Optional[str]:
        return next((v for (n, v), s in self.state.items() if n == name and s == VersionState.PRODUCTION), None)

    def in_state(self, name: str, s: VersionState) -> List[str]:
        return [v for (n, v), st in self.state.items() if n == name and st == s]


class RoutingMode(enum.Enum):
    LATEST = "latest"
    PINNED = "pinned"
    PERCENTAGE = "percentage"
    SHADOW = "shadow"           # primary answers; the shadow version also runs and its result is discarded


@dataclass
class RoutingPolicy:
    mode: RoutingMode = RoutingMode.LATEST
    pinned: Optional[str] = None
    weights: Dict[str, float] = field(default_factory=dict)
    shadow: Optional[str] = None


class PolicyRouter:
    def __init__(self, manager: ModelVersionManager):
        self.m = manager
        self.policies: Dict[str, RoutingPolicy] = {}
        self._split: Dict[str, TrafficSplitter] = {}

    def set_policy(self, name: str, p: RoutingPolicy):
        if p.mode == RoutingMode.PINNED and not p.pinned:
            raise ValueError("pinned mode needs a version")
        if p.mode == RoutingMode.PERCENTAGE:
            self._split[name] = TrafficSplitter(p.weights)
        self.policies[name] = p

    def route(self, name: str, sticky_key: Optional[str] = None) -> Tuple[str, Optional[str]]:
        """Returns (version that answers, shadow version or None)."""
        p = self.policies.get(name, RoutingPolicy())
        if p.mode == RoutingMode.PINNED:
            return p.pinned, None
        if p.mode == RoutingMode.PERCENTAGE:
            return self._split[name].choose(sticky_key), None
        primary = self.m.production(name) or self.m.reg.latest(name)
        return primary, (p.shadow if p.mode == RoutingMode.SHADOW else None)

    def infer(self, name: str, fn: Callable[[Any], Any], sticky_key: Optional[str] = None):
        v, shadow = self.route(name, sticky_key)
        out = self.m.sw.serve(name, fn, v)
        if shadow is not None:
            try:
                self.m.sw.serve(name, fn, shadow)
            except Exception:
                pass
        return out


@dataclass
class Alert:
    name: str
    version: str
    metric: str
    value: float
    threshold: float
    time: float = field(default_factory=time.time)


class VersionMonitor:
    def __init__(self, thresholds: Optional[Dict[str, float]] = None):
        self.thresholds = thresholds or {"error_rate": 0.05, "latency_p99_s": 1.0}
        self._lat: Dict[Tuple[str, str], List[float]] = defaultdict(list)
        self._err: Dict[Tuple[str, str], int] = defaultdict(int)
        self._n: Dict[Tuple[str, str], int] = defaultdict(int)
        self.alerts: List[Alert] = []

    def record(self, name: str, version: str, latency_s: float, ok: bool = True):
        k = (name, version)
        self._lat[k].append(latency_s)
        self._n[k] += 1
        self._err[k] += int(not ok)

    def metrics(self, name: str, version: str) -> Dict[str, float]:
        k = (name, version)
        lat = sorted(self._lat[k])
        n = self._n[k]
        return {"requests": n, "error_rate": self._err[k] / n if n else 0.0, "latency_mean_s": sum(lat) / n if n else 0.0,
                "latency_p99_s": lat[min(n - 1, int(0.99 * n))] if n else 0.0}

    def check(self, name: str, version: str) -> List[Alert]:
        m = self.metrics(name, version)
        new = [Alert(name, version, k, m[k], t) for k, t in self.thresholds.items() if m.get(k, 0.0) > t]
        self.alerts += new
        return new

    def compare(self, name: str, a: str, b: str) -> Dict[str, float]:
        ma, mb = self.metrics(name, a), self.metrics(name, b)
        return {k: mb[k] - ma[k] for k in ma}
