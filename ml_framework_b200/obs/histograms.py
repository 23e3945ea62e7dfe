"""Histogram and distribution logging with moments, quantiles and outlier detection.

Reference: src/MLFramework.Visualization/Histograms/{HistogramLogger.cs:40-290, HistogramData.cs, TensorDistribution.cs},
Histograms/Statistics/{MomentsCalculator.cs:16-125, QuantileCalculator.cs:14-47, OutlierDetector.cs:15-172 (z-score and
inter-quartile rules, dead-neuron count)}. Statistics are computed with tensor ops on whatever device holds the values
(one pass over a weight tensor on the GPU instead of a host copy of it); only the summary goes to the host.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch


def _flat(values) -> torch.Tensor:
    t = values if isinstance(values, torch.Tensor) else torch.as_tensor(values)
    return t.detach().reshape(-1).float()


class MomentsCalculator:
    @staticmethod
    def mean_std(values) -> Tuple[float, float]:
        v = _flat(values)
        if v.numel() == 0:
            return 0.0, 0.0
        return float(v.mean()), float(v.std(unbiased=False))

    @staticmethod
    def skewness(values, mean: Optional[float] = None, std: Optional[float] = None) -> float:
        v = _flat(values)
        if v.numel() < 2:
            return 0.0
        m = float(v.mean()) if mean is None else mean
        s = float(v.std(unbiased=False)) if std is None else std
        return float((((v - m) / s) ** 3).mean()) if s > 0 else 0.0

    @staticmethod
    def kurtosis(values, mean: Optional[float] = None, std: Optional[float] = None) -> float:
        """Excess kurtosis (a normal distribution gives 0)."""
        v = _flat(values)
        if v.numel() < 2:
            return 0.0
        m = float(v.mean()) if mean is None else mean
        s = float(v.std(unbiased=False)) if std is None else std
        return float((((v - m) / s) ** 4).mean()) - 3.0 if s > 0 else 0.0

    @classmethod
    def both(cls, values) -> Tuple[float, float]:
        m, s = cls.mean_std(values)
        return cls.skewness(values, m, s), cls.kurtosis(values, m, s)


class QuantileCalculator:
    """Linear interpolation between order statistics (position ``q * (n - 1)``)."""

    @staticmethod
    def calculate(values, q: float) -> float:
        return QuantileCalculator.calculate_multiple(values, [q])[0]

    @staticmethod
    def calculate_multiple(values, qs: Sequence[float]) -> List[float]:
        if any(not (0.0 <= q <= 1.0) for q in qs):
            raise ValueError("quantiles must lie in [0, 1]")
        v = _flat(values)
        if v.numel() == 0:
            raise ValueError("no data")
        s, _ = torch.sort(v)
        n = s.numel()
        out = []
        for q in qs:
            pos = q * (n - 1)
            lo, hi = int(math.floor(pos)), int(math.ceil(pos))
            out.append(float(s[lo] + (s[hi] - s[lo]) * (pos - lo)))
        return out


class OutlierDetector:
    @staticmethod
    def bounds_by_std(values, threshold: float = 3.0) -> Tuple[float, float]:
        m, s = MomentsCalculator.mean_std(values)
        return m - threshold * s, m + threshold * s

    @staticmethod
    def by_std(values, threshold: float = 3.0) -> Tuple[int, List[int]]:
        v = _flat(values)
        if v.numel() == 0:
            return 0, []
        lo, hi = OutlierDetector.bounds_by_std(v, threshold)
        idx = torch.nonzero((v < lo) | (v > hi)).reshape(-1)
        return int(idx.numel()), idx.tolist()

    @staticmethod
    def by_iqr(values, multiplier: float = 1.5) -> Tuple[int, List[int]]:
        v = _flat(values)
        if v.numel() == 0:
            return 0, []
        q1, q3 = QuantileCalculator.calculate_multiple(v, [0.25, 0.75])
        lo, hi = q1 - multiplier * (q3 - q1), q3 + multiplier * (q3 - q1)
        idx = torch.nonzero((v < lo) | (v > hi)).reshape(-1)
        return int(idx.numel()), idx.tolist()

    @staticmethod
    def outlier_values(values, threshold: float = 3.0) -> List[float]:
        v = _flat(values)
        _, idx = OutlierDetector.by_std(v, threshold)
        return v[idx].tolist() if idx else []

    @staticmethod
    def count_dead_neurons(values, near_zero: float = 0.0) -> int:
        """Activations whose magnitude is at most ``near_zero`` (exactly zero by default: a ReLU unit that never fires)."""
        return int((_flat(values).abs() <= near_zero).sum())


@dataclass
class HistogramBinConfig:
    bin_count: int = 30
    min_value: Optional[float] = None      # None: the data's minimum
    max_value: Optional[float] = None
    log_scale: bool = False                # bins uniform in log10(|x|); zeros go to the first bin

    def validate(self):
        if self.bin_count <= 0:
            raise ValueError("bin_count must be positive")
        if self.min_value is not None and self.max_value is not None and self.min_value >= self.max_value:
            raise ValueError("min_value must be below max_value")


@dataclass
class HistogramData:
    name: str
    step: int
    bin_edges: List[float]
    bin_counts: List[int]
    min: float
    max: float
    mean: float
    std: float
    count: int
    underflow: int = 0                     # values below / above a fixed range
    overflow: int = 0

    def normalized(self) -> List[float]:
        n = sum(self.bin_counts)
        return [c / n for c in self.bin_counts] if n else [0.0] * len(self.bin_counts)

    def mode_bin(self) -> Tuple[float, float]:
        i = max(range(len(self.bin_counts)), key=self.bin_counts.__getitem__)
        return self.bin_edges[i], self.bin_edges[i + 1]


@dataclass
class TensorDistribution:
    name: str
    step: int
    count: int
    min: float
    max: float
    mean: float
    std: float
    skewness: float
    kurtosis: float
    quantiles: Dict[str, float]
    outliers_std: int
    outliers_iqr: int
    dead: int
    nan: int
    inf: int

    @property
    def dead_fraction(self) -> float:
        return self.dead / self.count if self.count else 0.0

    def warnings(self) -> List[str]:
        w = []
        if self.nan or self.inf:
            w.append(f"{self.nan} NaN and {self.inf} Inf values")
        if self.dead_fraction > 0.5:
            w.append(f"{self.dead_fraction:.0%} of the values are dead (zero)")
        if self.std == 0 and self.count > 1:
            w.append("constant tensor")
        if abs(self.kurtosis) > 10:
            w.append(f"heavy tails (excess kurtosis {self.kurtosis:.1f})")
        return w


def build_histogram(name: str, values, config: Optional[HistogramBinConfig] = None, step: int = 0) -> HistogramData:
    cfg = config or HistogramBinConfig()
    cfg.validate()
    v = _flat(values)
    v = v[torch.isfinite(v)]
    if v.numel() == 0:
        return HistogramData(name, step, [0.0, 1.0], [0], 0.0, 0.0, 0.0, 0.0, 0)
    x = torch.log10(v.abs().clamp_min(1e-38)) if cfg.log_scale else v
    lo = float(x.min()) if cfg.min_value is None else cfg.min_value
    hi = float(x.max()) if cfg.max_value is None else cfg.max_value
    if hi <= lo:
        hi = lo + 1.0
    counts = torch.histc(x.float(), bins=cfg.bin_count, min=lo, max=hi)
    w = (hi - lo) / cfg.bin_count
    m, s = MomentsCalculator.mean_std(v)
    return HistogramData(name, step, [lo + i * w for i in range(cfg.bin_count + 1)], [int(c) for c in counts.tolist()],
                         float(v.min()), float(v.max()), m, s, int(v.numel()), int((x < lo).sum()), int((x > hi).sum()))


def build_distribution(name: str, values, step: int = 0) -> TensorDistribution:
    raw = _flat(values)
    nan, inf = int(torch.isnan(raw).sum()), int(torch.isinf(raw).sum())
    v = raw[torch.isfinite(raw)]
    if v.numel() == 0:
        return TensorDistribution(name, step, 0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, {}, 0, 0, 0, nan, inf)
    m, s = MomentsCalculator.mean_std(v)
    qs = QuantileCalculator.calculate_multiple(v, [0.01, 0.05, 0.25, 0.5, 0.75, 0.95, 0.99])
    return TensorDistribution(name, step, int(v.numel()), float(v.min()), float(v.max()), m, s, MomentsCalculator.skewness(v, m, s),
                              MomentsCalculator.kurtosis(v, m, s), dict(zip(("p1", "p5", "p25", "p50", "p75", "p95", "p99"), qs)),
                              OutlierDetector.by_std(v)[0], OutlierDetector.by_iqr(v)[0], OutlierDetector.count_dead_neurons(v), nan, inf)


class HistogramLogger:
    """Histograms and distributions by name and step; ``step = -1`` numbers a series automatically. ``events`` (an
    ``EventSystem``) receives a histogram event per log call when given."""

    def __init__(self, events=None, default_bins: Optional[HistogramBinConfig] = None, max_steps_per_name: int = 1000):
        self.events, self.default_bin_config = events, default_bins or HistogramBinConfig()
        self.max_steps_per_name = max_steps_per_name
        self._h: Dict[str, Dict[int, HistogramData]] = {}
        self._d: Dict[str, Dict[int, TensorDistribution]] = {}

    @staticmethod
    def _step(series: Dict[int, object], step: int) -> int:
        return step if step >= 0 else (max(series) + 1 if series else 0)

    def _trim(self, series: Dict[int, object]):
        while len(series) > self.max_steps_per_name:
            del series[min(series)]

    def log_histogram(self, name: str, values, step: int = -1, config: Optional[HistogramBinConfig] = None) -> HistogramData:
        if not name:
            raise ValueError("name must not be empty")
        ser = self._h.setdefault(name, {})
        h = build_histogram(name, values, config or self.default_bin_config, self._step(ser, step))
        ser[h.step] = h
        self._trim(ser)
        if self.events is not None:
            from .events import Event, EventType
            self.events.publish(Event(EventType.HISTOGRAM, name, h.step, {"edges": h.bin_edges, "counts": h.bin_counts, "mean": h.mean, "std": h.std}))
        return h

    def log_distribution(self, name: str, values, step: int = -1) -> TensorDistribution:
        if not name:
            raise ValueError("name must not be empty")
        ser = self._d.setdefault(name, {})
        d = build_distribution(name, values, self._step(ser, step))
        ser[d.step] = d
        self._trim(ser)
        return d

    def log_module(self, model: torch.nn.Module, step: int = -1, gradients: bool = True) -> List[str]:
        """One distribution per parameter (``<name>``) and per gradient (``<name>.grad``); returns the warnings found."""
        out = []
        for n, p in model.named_parameters():
            out += [f"{n}: {w}" for w in self.log_distribution(n, p, step).warnings()]
            if gradients and p.grad is not None:
                out += [f"{n}.grad: {w}" for w in self.log_distribution(n + ".grad", p.grad, step).warnings()]
        return out

    def get_histogram(self, name: str, step: int) -> Optional[HistogramData]:
        return self._h.get(name, {}).get(step)

    def get_distribution(self, name: str, step: int) -> Optional[TensorDistribution]:
        return self._d.get(name, {}).get(step)

    def histograms_over_time(self, name: str) -> List[HistogramData]:
        return [self._h[name][k] for k in sorted(self._h.get(name, {}))]

    def distributions_over_time(self, name: str) -> List[TensorDistribution]:
        return [self._d[name][k] for k in sorted(self._d.get(name, {}))]

    def histogram_names(self) -> List[str]:
        return sorted(self._h)

    def distribution_names(self) -> List[str]:
        return sorted(self._d)

    def clear(self, name: Optional[str] = None):
        if name is None:
            self._h.clear()
            self._d.clear()
        else:
            self._h.pop(name, None)
            self._d.pop(name, None)
