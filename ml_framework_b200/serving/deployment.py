"""Model deployment: loading, registry, hot swap with draining, rollback, routing, traffic splitting,
experiments.

Reference (src/MLFramework/Serving/): Deployment/{ModelLoader,ModelRegistry,ModelHotswapper,RollbackManager,
MetadataSerializer}.cs; Routing/{VersionRouter,HeaderRouter,SemanticVersion,RoutingRule}.cs; Traffic/
TrafficSplitter.cs (weighted A/B and canary); ExperimentTracker.cs; ReferenceTracker.cs (reference counts
per model version so a swap waits for in-flight requests); InferenceTracker.cs, RequestTracker.cs.
"""
from __future__ import annotations

import contextlib
import enum
import fnmatch
import functools
import hashlib
import json
import math
import random
import re
import threading
import time
from collections import defaultdict, deque
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple


@functools.total_ordering
class SemanticVersion:
    _re = re.compile(r"^v?(\d+)\.(\d+)\.(\d+)(?:-([0-9A-Za-z.-]+))?(?:\+([0-9A-Za-z.-]+))?$")

    def __init__(self, major: int, minor: int = 0, patch: int = 0, prerelease: str = "", build: str = ""):
        self.major, self.minor, self.patch, self.prerelease, self.build = major, minor, patch, prerelease, build

    @classmethod
    def parse(cls, s: str) -> "SemanticVersion":
        m = cls._re.match(s.strip())
        if not m:
            raise ValueError(f"not a semantic version: {s!r}")
        return cls(int(m[1]), int(m[2]), int(m[3]), m[4] or "", m[5] or "")

    def _key(self):
        pre = tuple((0, int(p)) if p.isdigit() else (1, p) for p in self.prerelease.split(".")) if self.prerelease else ()
        return (self.major, self.minor, self.patch, 0 if self.prerelease else 1, pre)

    def __eq__(self, o):
        return isinstance(o, SemanticVersion) and self._key() == o._key()

    def __lt__(self, o):
        return self._key() < o._key()

    def __hash__(self):
        return hash(self._key())

    def compatible_with(self, o: "SemanticVersion") -> bool:
        return self.major == o.major and self >= o

    def __str__(self):
        s = f"{self.major}.{self.minor}.{self.patch}"
        return s + (f"-{self.prerelease}" if self.prerelease else "") + (f"+{self.build}" if self.build else "")

    __repr__ = __str__


@dataclass
class ModelMetadata:
    name: str
    version: str
    framework: str = "ml_framework_b200"
    created: float = field(default_factory=time.time)
    checksum: str = ""
    tags: Dict[str, str] = field(default_factory=dict)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_json(s: str) -> "ModelMetadata":
        return ModelMetadata(**json.loads(s))


class ReferenceTracker:
    """In-flight request counts per key; ``wait_idle`` blocks until a key has none (draining)."""

    def __init__(self):
        self._n: Dict[str, int] = defaultdict(int)
        self._cv = threading.Condition()

    @contextlib.contextmanager
    def acquire(self, key: str):
        with self._cv:
            self._n[key] += 1
        try:
            yield
        finally:
            with self._cv:
                self._n[key] -= 1
                self._cv.notify_all()

    def count(self, key: str) -> int:
        return self._n[key]

    def wait_idle(self, key: str, timeout: float = 30.0) -> bool:
        end = time.monotonic() + timeout
        with self._cv:
            while self._n[key] > 0:
                left = end - time.monotonic()
                if left <= 0:
                    return False
                self._cv.wait(left)
        return True


class ModelRegistry:
    def __init__(self):
        self._m: Dict[Tuple[str, str], Tuple[Any, ModelMetadata]] = {}
        self._lock = threading.RLock()

    def register(self, model: Any, meta: ModelMetadata):
        with self._lock:
            key = (meta.name, meta.version)
            if key in self._m:
                raise ValueError(f"{meta.name}:{meta.version} already registered")
            self._m[key] = (model, meta)

    def unregister(self, name: str, version: str):
        with self._lock:
            self._m.pop((name, version), None)

    def get(self, name: str, version: str):
        with self._lock:
            if (name, version) not in self._m:
                raise KeyError(f"model {name}:{version} not found")
            return self._m[(name, version)][0]

    def versions(self, name: str) -> List[str]:
        with self._lock:
            return sorted((v for n, v in self._m if n == name), key=SemanticVersion.parse)

    def latest(self, name: str) -> str:
        v = self.versions(name)
        if not v:
            raise KeyError(f"no versions of {name}")
        return v[-1]


class ModelLoader:
    """``factory(path) -> model``; verifies the SHA-256 recorded in the side-car metadata (``<path>.meta.json``)."""

    def __init__(self, factory: Callable[[str], Any]):
        self.factory = factory

    @staticmethod
    def checksum(path: str) -> str:
        h = hashlib.sha256()
        with open(path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
        return h.hexdigest()

    def load(self, path: str, meta: Optional[ModelMetadata] = None):
        if meta is not None and meta.checksum and self.checksum(path) != meta.checksum:
            raise IOError(f"checksum mismatch for {path}")
        return self.factory(path)


class ModelHotSwapper:
    """The active version of each model name; ``swap`` makes the new version active at once, then waits
    for requests on the old one to drain before releasing it. ``serve`` runs a call under a reference."""

    def __init__(self, registry: ModelRegistry, refs: Optional[ReferenceTracker] = None):
        self.reg, self.refs = registry, refs or ReferenceTracker()
        self.active: Dict[str, str] = {}
        self.history: Dict[str, List[str]] = defaultdict(list)
        self._lock = threading.Lock()

    def activate(self, name: str, version: str):
        self.reg.get(name, version)
        with self._lock:
            self.active[name] = version
            self.history[name].append(version)

    def swap(self, name: str, new_version: str, drain_timeout: float = 30.0, unload_old: bool = False) -> bool:
        self.reg.get(name, new_version)
        with self._lock:
            old = self.active.get(name)
            self.active[name] = new_version
            self.history[name].append(new_version)
        if old is None or old == new_version:
            return True
        drained = self.refs.wait_idle(f"{name}:{old}", drain_timeout)
        if drained and unload_old:
            self.reg.unregister(name, old)
        return drained

    def serve(self, name: str, fn: Callable[[Any], Any], version: Optional[str] = None):
        with self._lock:
            v = version or self.active[name]
        with self.refs.acquire(f"{name}:{v}"):
            return fn(self.reg.get(name, v))


class RollbackManager:
    """Sliding-window error-rate monitor per model; when the rate exceeds the threshold (with enough
    samples) the previous version is swapped back in."""

    def __init__(self, swapper: ModelHotSwapper, error_threshold: float = 0.1, window: int = 100, min_samples: int = 20):
        self.sw, self.thr, self.window, self.min = swapper, error_threshold, window, min_samples
        self._res: Dict[str, Deque[bool]] = defaultdict(lambda: deque(maxlen=window))
        self.rollbacks: List[Tuple[str, str, str]] = []

    def record(self, name: str, ok: bool) -> bool:
        r = self._res[name]
        r.append(ok)
        if len(r) >= self.min and (1 - sum(r) / len(r)) > self.thr:
            return self.rollback(name)
        return False

    def error_rate(self, name: str) -> float:
        r = self._res[name]
        return 1 - sum(r) / len(r) if r else 0.0

    def rollback(self, name: str) -> bool:
        h = self.sw.history[name]
        cur = self.sw.active.get(name)
        prev = next((v for v in reversed(h[:-1]) if v != cur), None)
        if prev is None:
            return False
        self.sw.swap(name, prev)
        self.rollbacks.append((name, cur, prev))
        self._res[name].clear()
        return True


# ------------------------------------------------------------------ routing / traffic
@dataclass
class RoutingRule:
    header: str
    pattern: str            # glob
    version: str
    priority: int = 0


class HeaderRouter:
    def __init__(self, rules: Optional[List[RoutingRule]] = None, default: Optional[str] = None):
        self.rules, self.default = sorted(rules or [], key=lambda r: -r.priority), default

    def add(self, rule: RoutingRule):
        self.rules.append(rule)
        self.rules.sort(key=lambda r: -r.priority)

    def route(self, headers: Dict[str, str]) -> Optional[str]:
        low = {k.lower(): v for k, v in headers.items()}
        for r in self.rules:
            v = low.get(r.header.lower())
            if v is not None and fnmatch.fnmatch(v, r.pattern):
                return r.version
        return self.default


class VersionRouter:
    """Resolves a requested version constraint ("1.2.3", "^1.2.0" = compatible, "latest") to a registered one."""

    def __init__(self, registry: ModelRegistry):
        self.reg = registry

    def resolve(self, name: str, constraint: str = "latest") -> str:
        vs = self.reg.versions(name)
        if not vs:
            raise KeyError(f"no versions of {name}")
        if constraint == "latest":
            return vs[-1]
        if constraint.startswith("^"):
            base = SemanticVersion.parse(constraint[1:])
            ok = [v for v in vs if SemanticVersion.parse(v).compatible_with(base)]
            if not ok:
                raise KeyError(f"no version of {name} compatible with {base}")
            return ok[-1]
        if constraint in vs:
            return constraint
        raise KeyError(f"{name}:{constraint} not registered")


class TrafficSplitter:
    """Weighted split across versions. With ``sticky_key`` the choice is a hash of the key, so one
    user keeps one arm; otherwise it is random."""

    def __init__(self, weights: Dict[str, float], seed: int = 0):
        self.set_weights(weights)
        self._rng = random.Random(seed)
        self.counts: Dict[str, int] = defaultdict(int)

    def set_weights(self, weights: Dict[str, float]):
        tot = sum(weights.values())
        if tot <= 0 or any(w < 0 for w in weights.values()):
            raise ValueError("weights must be non-negative with a positive sum")
        self.weights = {k: w / tot for k, w in weights.items()}

    @classmethod
    def canary(cls, stable: str, canary: str, fraction: float, seed: int = 0):
        return cls({stable: 1 - fraction, canary: fraction}, seed)

    def choose(self, sticky_key: Optional[str] = None) -> str:
        u = int(hashlib.sha256(sticky_key.encode()).hexdigest()[:12], 16) / float(1 << 48) if sticky_key is not None else self._rng.random()
        acc = 0.0
        for k, w in self.weights.items():
            acc += w
            if u < acc:
                self.counts[k] += 1
                return k
        k = next(reversed(self.weights))
        self.counts[k] += 1
        return k


class ExperimentTracker:
    """Per-arm metric samples with mean / variance and a Welch t statistic between two arms."""

    def __init__(self):
        self.samples: Dict[str, Dict[str, List[float]]] = defaultdict(lambda: defaultdict(list))

    def record(self, arm: str, metric: str, value: float):
        self.samples[arm][metric].append(value)

    def summary(self, arm: str, metric: str) -> Dict[str, float]:
        v = self.samples[arm][metric]
        n = len(v)
        mean = sum(v) / n if n else 0.0
        var = sum((x - mean) ** 2 for x in v) / (n - 1) if n > 1 else 0.0
        return {"n": n, "mean": mean, "var": var}

    def compare(self, a: str, b: str, metric: str) -> Dict[str, float]:
        sa, sb = self.summary(a, metric), self.summary(b, metric)
        se = (sa["var"] / max(1, sa["n"]) + sb["var"] / max(1, sb["n"])) ** 0.5
        return {"diff": sb["mean"] - sa["mean"], "t": (sb["mean"] - sa["mean"]) / se if se > 0 else 0.0, "n_a": sa["n"], "n_b": sb["n"]}


class InferenceTracker:
    def __init__(self):
        self.latencies: Dict[str, List[float]] = defaultdict(list)
        self.errors: Dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def track(self, key: str):
        t0 = time.perf_counter()
        try:
            yield
        except BaseException:
            self.errors[key] += 1
            raise
        finally:
            self.latencies[key].append(time.perf_counter() - t0)

    def p(self, key: str, q: float) -> float:
        v = sorted(self.latencies[key])
        return v[min(len(v) - 1, int(q / 100 * len(v)))] if v else 0.0


# ------------------------------------------------------------------ request routing end to end, records
class MatchType(enum.Enum):
    """How a routing rule compares a header value (Serving/Routing/MatchType.cs)."""
    EXACT = "exact"
    PREFIX = "prefix"
    REGEX = "regex"
    GLOB = "glob"


class RoutingError(LookupError):
    def __init__(self, message: str, model_name: str = "", context: Optional["RoutingContext"] = None):
        super().__init__(message)
        self.model_name, self.context = model_name, context


class ReferenceLeakError(RuntimeError):
    """A version was released while requests still held it (Serving/ReferenceLeakException.cs)."""

    def __init__(self, key: str, count: int):
        super().__init__(f"{key} still has {count} request(s) in flight")
        self.key, self.count = key, count


@dataclass
class TypedRoutingRule:
    header: str
    pattern: str
    version: str
    match_type: MatchType = MatchType.EXACT
    priority: int = 0

    def matches(self, value: str) -> bool:
        if self.match_type is MatchType.EXACT:
            return value == self.pattern
        if self.match_type is MatchType.PREFIX:
            return value.startswith(self.pattern)
        if self.match_type is MatchType.REGEX:
            return re.search(self.pattern, value) is not None
        return fnmatch.fnmatch(value, self.pattern)


@dataclass
class RoutingContext:
    """What a routing decision may look at (Serving/Routing/RoutingContext.cs)."""
    headers: Dict[str, str] = field(default_factory=dict)
    user_id: Optional[str] = None
    experiment_id: Optional[str] = None
    requested_version: Optional[str] = None          # "1.2.3", "^1.2.0" or "latest"
    metadata: Dict[str, Any] = field(default_factory=dict)


@dataclass
class TrafficSplitConfig:
    """Percentages per version, summing to 100 (Serving/Traffic/TrafficSplitConfig.cs)."""
    model_name: str
    version_percentages: Dict[str, float]
    sticky: bool = True

    def validate(self) -> None:
        if not self.version_percentages:
            raise ValueError("a traffic split needs at least one version")
        if any(p < 0 for p in self.version_percentages.values()):
            raise ValueError("percentages cannot be negative")
        total = sum(self.version_percentages.values())
        if abs(total - 100.0) > 1e-6:
            raise ValueError(f"percentages sum to {total:g}, not 100")

    def to_splitter(self, seed: int = 0) -> "TrafficSplitter":
        self.validate()
        return TrafficSplitter({k: v for k, v in self.version_percentages.items() if v > 0}, seed)


class RequestRouter:
    """One decision per request, in this order: an explicit version constraint, the first matching header
    rule, the model's traffic split (sticky per user when the split says so), the active version."""

    def __init__(self, registry: ModelRegistry, swapper: Optional[ModelHotSwapper] = None):
        self.registry, self.swapper = registry, swapper
        self.versions = VersionRouter(registry)
        self._rules: Dict[str, List[TypedRoutingRule]] = defaultdict(list)
        self._splits: Dict[str, Tuple[TrafficSplitConfig, TrafficSplitter]] = {}
        self.decisions: Dict[str, int] = defaultdict(int)

    def add_rule(self, model_name: str, rule: TypedRoutingRule) -> None:
        self._rules[model_name].append(rule)
        self._rules[model_name].sort(key=lambda r: -r.priority)

    def set_traffic_split(self, config: TrafficSplitConfig, seed: int = 0) -> None:
        for v in config.version_percentages:
            self.registry.get(config.model_name, v)
        self._splits[config.model_name] = (config, config.to_splitter(seed))

    def clear_traffic_split(self, model_name: str) -> bool:
        return self._splits.pop(model_name, None) is not None

    def route(self, model_name: str, context: Optional[RoutingContext] = None) -> str:
        ctx = context or RoutingContext()
        try:
            if ctx.requested_version:
                self.decisions["explicit"] += 1
                return self.versions.resolve(model_name, ctx.requested_version)
            low = {k.lower(): v for k, v in ctx.headers.items()}
            for r in self._rules.get(model_name, ()):
                v = low.get(r.header.lower())
                if v is not None and r.matches(v):
                    self.registry.get(model_name, r.version)
                    self.decisions["rule"] += 1
                    return r.version
            if model_name in self._splits:
                cfg, splitter = self._splits[model_name]
                self.decisions["split"] += 1
                return splitter.choose(ctx.user_id if cfg.sticky else None)
            self.decisions["default"] += 1
            if self.swapper is not None and model_name in self.swapper.active:
                return self.swapper.active[model_name]
            return self.registry.latest(model_name)
        except KeyError as e:
            raise RoutingError(f"cannot route {model_name}: {e.args[0]}", model_name, ctx) from e


@dataclass
class ExperimentMetrics:
    """One arm of an experiment, summarised (Serving/ExperimentMetrics.cs)."""
    experiment_id: str
    version: str
    request_count: int = 0
    success_count: int = 0
    mean_latency_ms: float = 0.0
    p95_latency_ms: float = 0.0
    custom: Dict[str, float] = field(default_factory=dict)

    @property
    def success_rate(self) -> float:
        return self.success_count / self.request_count if self.request_count else 0.0

    @property
    def error_rate(self) -> float:
        return 1.0 - self.success_rate if self.request_count else 0.0

    @classmethod
    def from_samples(cls, experiment_id: str, version: str, latencies_ms: Sequence[float], successes: Sequence[bool],
                     custom: Optional[Dict[str, float]] = None) -> "ExperimentMetrics":
        if len(latencies_ms) != len(successes):
            raise ValueError("one success flag per latency sample")
        lat = sorted(latencies_ms)
        p95 = lat[min(len(lat) - 1, int(math.ceil(0.95 * len(lat))) - 1)] if lat else 0.0
        return cls(experiment_id, version, len(lat), sum(bool(s) for s in successes), sum(lat) / len(lat) if lat else 0.0, p95,
                   dict(custom or {}))


class DeploymentStatus(enum.Enum):
    PENDING = "pending"
    ACTIVE = "active"
    DRAINING = "draining"
    RETIRED = "retired"
    FAILED = "failed"
    ROLLED_BACK = "rolled_back"


@dataclass
class DeploymentRecord:
    model_name: str
    version: str
    status: DeploymentStatus
    deployed_at: float
    retired_at: Optional[float] = None
    previous_version: Optional[str] = None
    note: str = ""


class DeploymentLog:
    """What was deployed when, on top of a hot swapper: ``deploy`` swaps and records, ``rollback`` goes back
    to the previous record; releasing a version that still serves requests raises ``ReferenceLeakError``."""

    def __init__(self, swapper: ModelHotSwapper, clock: Callable[[], float] = time.time):
        self.swapper, self._clock = swapper, clock
        self.records: List[DeploymentRecord] = []

    def current(self, model_name: str) -> Optional[DeploymentRecord]:
        return next((r for r in reversed(self.records) if r.model_name == model_name and r.status is DeploymentStatus.ACTIVE), None)

    def history(self, model_name: str) -> List[DeploymentRecord]:
        return [r for r in self.records if r.model_name == model_name]

    def deploy(self, model_name: str, version: str, drain_timeout: float = 30.0, note: str = "") -> DeploymentRecord:
        prev = self.current(model_name)
        rec = DeploymentRecord(model_name, version, DeploymentStatus.PENDING, self._clock(), None, prev.version if prev else None, note)
        self.records.append(rec)
        try:
            if prev is None:
                self.swapper.activate(model_name, version)
                drained = True
            else:
                prev.status = DeploymentStatus.DRAINING
                drained = self.swapper.swap(model_name, version, drain_timeout)
        except KeyError:
            rec.status = DeploymentStatus.FAILED
            if prev is not None:
                prev.status = DeploymentStatus.ACTIVE
            raise
        rec.status = DeploymentStatus.ACTIVE
        if prev is not None and drained:
            prev.status, prev.retired_at = DeploymentStatus.RETIRED, self._clock()
        return rec

    def rollback(self, model_name: str, drain_timeout: float = 30.0) -> Optional[DeploymentRecord]:
        cur = self.current(model_name)
        if cur is None or cur.previous_version is None:
            return None
        target = cur.previous_version
        self.swapper.swap(model_name, target, drain_timeout)
        cur.status, cur.retired_at = DeploymentStatus.ROLLED_BACK, self._clock()
        rec = DeploymentRecord(model_name, target, DeploymentStatus.ACTIVE, self._clock(), None, cur.version, f"rollback from {cur.version}")
        self.records.append(rec)
        return rec

    def release(self, model_name: str, version: str) -> None:
        """Unregisters a version that is no longer active; refuses while requests still hold it."""
        if self.swapper.active.get(model_name) == version:
            raise ValueError(f"{model_name}:{version} is the active version")
        key = f"{model_name}:{version}"
        n = self.swapper.refs.count(key)
        if n > 0:
            raise ReferenceLeakError(key, n)
        self.swapper.reg.unregister(model_name, version)
