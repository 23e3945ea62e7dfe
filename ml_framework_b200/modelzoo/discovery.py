"""Model discovery: search with filters and sorting, latency / memory estimators, constraint-based recommendation.

Reference: src/ModelZoo/Discovery/{ModelSearchQuery.cs, ModelSearchQueryBuilder.cs, ModelSearchService.cs:28-139,
SearchSortBy.cs, ModelConstraints.cs, DeploymentEnv.cs, DeviceType.cs, LatencyEstimator.cs:29-70, MemoryEstimator.cs:33-82,
ModelRecommendationEngine.cs:34-197, RecommendationStrategy.cs, ModelRecommendation.cs}. The estimators here are a
roofline over the target's measured numbers (tensor throughput and memory bandwidth of a B200, or a host CPU),
computed from the architecture's parameter and KV-cache sizes, not a per-parameter constant.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from .zoo import ModelInfo, ZooRegistry


class SearchSortBy(enum.Enum):
    NAME = "name"
    PARAMETERS = "parameters"
    ACCURACY = "accuracy"
    FILE_SIZE = "file_size"
    RELEVANCE = "relevance"


class DeviceType(enum.Enum):
    B200 = "b200"
    CPU = "cpu"


class DeploymentEnv(enum.Enum):
    CLOUD = "cloud"          # throughput matters most
    EDGE = "edge"            # memory and file size matter most
    REALTIME = "realtime"    # latency matters most


@dataclass
class DeviceProfile:
    tflops: float            # dense bf16 matrix throughput actually reachable
    mem_gbs: float           # memory bandwidth actually reachable
    memory_bytes: int
    launch_us_per_layer: float

PROFILES = {DeviceType.B200: DeviceProfile(1400.0, 6600.0, 180 << 30, 12.0),
            DeviceType.CPU: DeviceProfile(2.0, 100.0, 256 << 30, 40.0)}


def _accuracy(i: ModelInfo) -> Optional[float]:
    return (i.metrics or {}).get("accuracy")


def _size(i: ModelInfo, dtype_bytes: int = 2) -> int:
    return i.file_size if i.file_size is not None else i.num_params() * dtype_bytes


@dataclass
class ModelSearchQuery:
    text: str = ""
    task: Optional[str] = None
    architecture: Optional[str] = None
    min_accuracy: Optional[float] = None
    max_accuracy: Optional[float] = None
    min_file_size: Optional[int] = None
    max_file_size: Optional[int] = None
    min_parameters: Optional[int] = None
    max_parameters: Optional[int] = None
    license: Optional[str] = None
    tags: Tuple[str, ...] = ()
    pretrained_dataset: Optional[str] = None
    framework_version: Optional[str] = None
    custom_filters: Dict[str, Callable[[ModelInfo], bool]] = field(default_factory=dict)
    sort_by: SearchSortBy = SearchSortBy.NAME
    sort_descending: bool = False
    limit: int = 100

    def validate(self):
        for lo, hi, what in ((self.min_accuracy, self.max_accuracy, "accuracy"), (self.min_file_size, self.max_file_size, "file size"),
                             (self.min_parameters, self.max_parameters, "parameters")):
            if lo is not None and hi is not None and lo > hi:
                raise ValueError(f"minimum {what} exceeds the maximum")
        if self.limit <= 0:
            raise ValueError("limit must be positive")


class ModelSearchQueryBuilder:
    def __init__(self):
        self._q = ModelSearchQuery()

    def with_text(self, t): self._q.text = t; return self
    def with_task(self, t): self._q.task = t; return self
    def with_architecture(self, a): self._q.architecture = a; return self
    def with_accuracy(self, lo=None, hi=None): self._q.min_accuracy, self._q.max_accuracy = lo, hi; return self
    def with_file_size(self, lo=None, hi=None): self._q.min_file_size, self._q.max_file_size = lo, hi; return self
    def with_parameters(self, lo=None, hi=None): self._q.min_parameters, self._q.max_parameters = lo, hi; return self
    def with_license(self, l): self._q.license = l; return self
    def with_tags(self, *tags): self._q.tags = tuple(tags); return self
    def with_filter(self, name, fn): self._q.custom_filters[name] = fn; return self
    def sort_by(self, key: SearchSortBy, descending: bool = False): self._q.sort_by, self._q.sort_descending = key, descending; return self
    def limit(self, n): self._q.limit = n; return self

    def build(self) -> ModelSearchQuery:
        self._q.validate()
        return self._q


@dataclass
class ModelSearchResult:
    model: ModelInfo
    score: float                      # relevance in [0, 1]
    matched: List[str]                # which criteria contributed


class ModelSearchService:
    def __init__(self, registry: ZooRegistry):
        self.registry = registry

    def _match(self, i: ModelInfo, q: ModelSearchQuery) -> Optional[ModelSearchResult]:
        matched, score, crit = [], 0.0, 0
        if q.text:
            crit += 1
            words = q.text.lower().split()
            hay = f"{i.name} {i.description} {' '.join(i.tags)} {i.architecture}".lower()
            hit = sum(w in hay for w in words)
            if hit == 0:
                return None
            score += hit / len(words) * (1.0 if q.text.lower() in i.name.lower() else 0.8)
            matched.append("text")
        def need(cond, name):
            nonlocal crit, score
            crit += 1
            if not cond:
                return False
            score += 1.0
            matched.append(name)
            return True
        if q.task is not None and not need(i.task == q.task, "task"): return None
        if q.architecture is not None and not need(i.architecture.lower() == q.architecture.lower(), "architecture"): return None
        if q.license is not None and not need(i.license.lower() == q.license.lower(), "license"): return None
        if q.pretrained_dataset is not None and not need(i.pretrained_dataset.lower() == q.pretrained_dataset.lower(), "dataset"): return None
        if q.framework_version is not None and not need(i.framework_version == q.framework_version, "framework_version"): return None
        if q.tags and not need(all(t in i.tags for t in q.tags), "tags"): return None
        acc = _accuracy(i)
        if q.min_accuracy is not None or q.max_accuracy is not None:
            ok = acc is not None and (q.min_accuracy is None or acc >= q.min_accuracy) and (q.max_accuracy is None or acc <= q.max_accuracy)
            if not need(ok, "accuracy"): return None
        if q.min_file_size is not None or q.max_file_size is not None:
            sz = _size(i)
            if not need((q.min_file_size is None or sz >= q.min_file_size) and (q.max_file_size is None or sz <= q.max_file_size), "file_size"): return None
        if q.min_parameters is not None or q.max_parameters is not None:
            n = i.num_params()
            if not need((q.min_parameters is None or n >= q.min_parameters) and (q.max_parameters is None or n <= q.max_parameters), "parameters"): return None
        for name, fn in q.custom_filters.items():
            if not need(bool(fn(i)), name): return None
        return ModelSearchResult(i, score / crit if crit else 1.0, matched)

    def search(self, q: ModelSearchQuery) -> List[ModelSearchResult]:
        q.validate()
        res = [r for r in (self._match(i, q) for i in self.registry.list()) if r is not None]
        key = {SearchSortBy.NAME: lambda r: r.model.name, SearchSortBy.PARAMETERS: lambda r: r.model.num_params(),
               SearchSortBy.ACCURACY: lambda r: _accuracy(r.model) if _accuracy(r.model) is not None else -1.0,
               SearchSortBy.FILE_SIZE: lambda r: _size(r.model), SearchSortBy.RELEVANCE: lambda r: r.score}[q.sort_by]
        res.sort(key=key, reverse=q.sort_descending)
        return res[:q.limit]

    def search_by_task(self, task: str, limit: int = 10):
        return self.search(ModelSearchQuery(task=task, limit=limit))

    def search_by_accuracy(self, min_accuracy: float, task: Optional[str] = None, limit: int = 10):
        return self.search(ModelSearchQuery(task=task, min_accuracy=min_accuracy, sort_by=SearchSortBy.ACCURACY, sort_descending=True, limit=limit))

    def search_by_architecture(self, architecture: str, limit: int = 10):
        return self.search(ModelSearchQuery(architecture=architecture, limit=limit))

    def search_by_size(self, max_size: int, task: Optional[str] = None, limit: int = 10):
        return self.search(ModelSearchQuery(task=task, max_file_size=max_size, sort_by=SearchSortBy.FILE_SIZE, limit=limit))

    def advanced_search(self, build: Callable[[ModelSearchQueryBuilder], object]):
        b = ModelSearchQueryBuilder()
        build(b)
        return self.search(b.build())


# ------------------------------------------------------------------ estimators
def _arch(i: ModelInfo) -> Tuple[int, int, int, int]:
    """(layers, model width, KV heads x head dim, vocabulary) from the architecture config; zeros when unknown."""
    c = i.config
    d = c.get("d_model", 0)
    hd = c.get("head_dim", d // max(c.get("n_heads", 1), 1) if d else 0)
    return c.get("n_layers", 0), d, c.get("n_kv_heads", c.get("n_heads", 0)) * hd, c.get("vocab_size", 0)


class MemoryEstimator:
    """Bytes needed to run a model: weights + KV cache for the context held + activations of one layer (+ gradients,
    fp32 master copy and Adam moments when training)."""

    def estimate(self, i: ModelInfo, batch_size: int = 1, seq_len: int = 1, dtype_bytes: int = 2, training: bool = False) -> int:
        p = i.num_params()
        L, d, kv, _ = _arch(i)
        weights = p * dtype_bytes
        tokens = batch_size * seq_len
        if training:
            return weights + p * dtype_bytes + p * 12 + tokens * d * L * 34
        kv_cache = 2 * L * kv * tokens * dtype_bytes
        act = tokens * max(d, 1) * 8 * dtype_bytes
        return weights + kv_cache + act

    def fits(self, i: ModelInfo, device: DeviceType, **kw) -> bool:
        return self.estimate(i, **kw) <= PROFILES[device].memory_bytes * 0.9


class LatencyEstimator:
    """Milliseconds for one forward pass over ``batch x seq`` new tokens against ``context`` cached ones: the slower
    of the matrix work at the device's tensor throughput and the bytes that must stream (weights once, KV cache once)
    at its memory bandwidth, plus a launch cost per layer."""

    def estimate(self, i: ModelInfo, device: DeviceType = DeviceType.B200, batch_size: int = 1, seq_len: int = 1, context: int = 0,
                 dtype_bytes: int = 2) -> float:
        prof = PROFILES[device]
        p = i.num_params()
        L, d, kv, _ = _arch(i)
        tokens = batch_size * seq_len
        flops = 2.0 * p * tokens + 4.0 * L * d * tokens * (context + seq_len / 2)
        bytes_ = p * dtype_bytes + 2 * L * kv * batch_size * (context + seq_len) * dtype_bytes
        t = max(flops / (prof.tflops * 1e12), bytes_ / (prof.mem_gbs * 1e9)) + L * prof.launch_us_per_layer * 1e-6
        return t * 1e3

    def tokens_per_second(self, i: ModelInfo, device: DeviceType = DeviceType.B200, batch_size: int = 1, context: int = 0) -> float:
        return batch_size / (self.estimate(i, device, batch_size, 1, context) * 1e-3)


# ------------------------------------------------------------------ recommendation
class RecommendationStrategy(enum.Enum):
    ACCURACY_FIRST = "accuracy_first"
    PERFORMANCE_FIRST = "performance_first"
    MEMORY_CONSTRAINED = "memory_constrained"
    BALANCED = "balanced"


@dataclass
class ModelConstraints:
    task: Optional[str] = None
    max_latency_ms: Optional[float] = None
    max_memory_bytes: Optional[int] = None
    min_accuracy: Optional[float] = None
    max_file_size: Optional[int] = None
    device: DeviceType = DeviceType.B200
    batch_size: int = 1
    seq_len: int = 1
    context: int = 0
    environment: Optional[DeploymentEnv] = None

    def with_task(self, t): self.task = t; return self
    def with_device(self, d): self.device = d; return self
    def with_batch(self, b, seq_len=1, context=0): self.batch_size, self.seq_len, self.context = b, seq_len, context; return self
    def with_environment(self, e): self.environment = e; return self

    def with_max_latency(self, ms):
        if ms <= 0:
            raise ValueError("max latency must be positive")
        self.max_latency_ms = ms
        return self

    def with_max_memory(self, n):
        if n <= 0:
            raise ValueError("max memory must be positive")
        self.max_memory_bytes = n
        return self

    def with_min_accuracy(self, a):
        if not (0.0 <= a <= 1.0):
            raise ValueError("accuracy lies in [0, 1]")
        self.min_accuracy = a
        return self


@dataclass
class ModelRecommendation:
    model: ModelInfo
    score: float
    estimated_latency_ms: float
    estimated_memory_bytes: int
    reasons: List[str]


class ModelRecommendationEngine:
    def __init__(self, registry: ZooRegistry, latency: Optional[LatencyEstimator] = None, memory: Optional[MemoryEstimator] = None):
        self.registry, self.lat, self.mem = registry, latency or LatencyEstimator(), memory or MemoryEstimator()

    @staticmethod
    def strategy_for(env: Optional[DeploymentEnv]) -> RecommendationStrategy:
        return {DeploymentEnv.CLOUD: RecommendationStrategy.ACCURACY_FIRST, DeploymentEnv.EDGE: RecommendationStrategy.MEMORY_CONSTRAINED,
                DeploymentEnv.REALTIME: RecommendationStrategy.PERFORMANCE_FIRST}.get(env, RecommendationStrategy.BALANCED)

    def _candidates(self, c: ModelConstraints) -> List[ModelRecommendation]:
        out = []
        for i in self.registry.list():
            if c.task is not None and i.task != c.task:
                continue
            lat = self.lat.estimate(i, c.device, c.batch_size, c.seq_len, c.context)
            mem = self.mem.estimate(i, c.batch_size, c.seq_len + c.context)
            acc = _accuracy(i)
            if c.max_latency_ms is not None and lat > c.max_latency_ms: continue
            if c.max_memory_bytes is not None and mem > c.max_memory_bytes: continue
            if c.min_accuracy is not None and (acc is None or acc < c.min_accuracy): continue
            if c.max_file_size is not None and _size(i) > c.max_file_size: continue
            if mem > PROFILES[c.device].memory_bytes: continue
            out.append(ModelRecommendation(i, 0.0, lat, mem, []))
        return out

    def recommend_with_strategy(self, c: ModelConstraints, strategy: RecommendationStrategy, top_n: int = 3) -> List[ModelRecommendation]:
        cands = self._candidates(c)
        if not cands:
            return []
        max_lat = max(r.estimated_latency_ms for r in cands)
        max_mem = max(r.estimated_memory_bytes for r in cands)
        max_par = max(r.model.num_params() for r in cands) or 1
        w = {RecommendationStrategy.ACCURACY_FIRST: (0.7, 0.15, 0.15), RecommendationStrategy.PERFORMANCE_FIRST: (0.15, 0.7, 0.15),
             RecommendationStrategy.MEMORY_CONSTRAINED: (0.15, 0.15, 0.7), RecommendationStrategy.BALANCED: (0.34, 0.33, 0.33)}[strategy]
        for r in cands:
            acc = _accuracy(r.model)
            # without a measured accuracy, capacity (parameter count) stands in for quality
            q = acc if acc is not None else r.model.num_params() / max_par
            fast = 1.0 - r.estimated_latency_ms / max_lat if max_lat > 0 else 1.0
            small = 1.0 - r.estimated_memory_bytes / max_mem if max_mem > 0 else 1.0
            r.score = w[0] * q + w[1] * fast + w[2] * small
            r.reasons = [f"quality {q:.2f}" + ("" if acc is not None else " (by capacity)"), f"latency {r.estimated_latency_ms:.2f} ms",
                         f"memory {r.estimated_memory_bytes / 2**30:.1f} GiB", f"strategy {strategy.value}"]
        cands.sort(key=lambda r: -r.score)
        return cands[:top_n]

    def recommend_for_constraints(self, c: ModelConstraints, top_n: int = 3) -> List[ModelRecommendation]:
        return self.recommend_with_strategy(c, self.strategy_for(c.environment), top_n)

    def recommend_for(self, task: str, device: DeviceType = DeviceType.B200, **kw) -> Optional[ModelRecommendation]:
        r = self.recommend_for_constraints(ModelConstraints(task=task, device=device, **kw), 1)
        return r[0] if r else None

    def alternatives(self, name: str, count: int = 3) -> List[ModelInfo]:
        """Other models of the same task, nearest in parameter count (same architecture first)."""
        base = self.registry.get(name)
        n0 = base.num_params()
        others = [i for i in self.registry.list() if i.name != base.name and i.task == base.task]
        others.sort(key=lambda i: (i.architecture != base.architecture, abs(i.num_params() - n0)))
        return others[:count]
