"""TensorBoard-style façade over the event system (reference: src/MLFramework.Visualization/
TensorBoardVisualizer.cs:14-540, VisualizerBuilder.cs, Histograms/*, Graphs/*, Configuration/
ConfigurationLoader.cs:36-213 with ``MLFRAMEWORK_VISUALIZATION_*`` environment overrides)."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from .events import (AsyncEventCollector, Event, EventCollector, EventCollectorConfig, EventSystem, EventType, FileStorageBackend, MemoryStorageBackend, ScalarLogger, StorageBackend)
from .profiler import Profiler


@dataclass
class VisualizationConfiguration:
    log_dir: str = "./runs"
    enabled: bool = True
    async_collection: bool = True
    flush_interval_s: float = 1.0
    buffer_capacity: int = 1000
    histogram_bins: int = 30
    storage: str = "file"

    def validate(self):
        if self.buffer_capacity <= 0 or self.histogram_bins <= 0 or self.flush_interval_s <= 0:
            raise ValueError("buffer_capacity, histogram_bins and flush_interval_s must be positive")
        if self.storage not in ("file", "memory", "binary"):
            raise ValueError(f"unknown storage {self.storage!r}")


class ConfigurationLoader:
    PREFIX = "MLFRAMEWORK_VISUALIZATION_"

    @staticmethod
    def from_json(text: str) -> VisualizationConfiguration:
        c = VisualizationConfiguration(**json.loads(text))
        c.validate()
        return c

    @classmethod
    def from_file(cls, path: str) -> VisualizationConfiguration:
        with open(path) as f:
            return cls.from_json(f.read())

    @classmethod
    def from_environment(cls, base: Optional[VisualizationConfiguration] = None, env=os.environ) -> VisualizationConfiguration:
        c = base or VisualizationConfiguration()
        for name, typ in (("log_dir", str), ("enabled", bool), ("async_collection", bool), ("flush_interval_s", float),
                          ("buffer_capacity", int), ("histogram_bins", int), ("storage", str)):
            v = env.get(cls.PREFIX + name.upper())
            if v is not None:
                setattr(c, name, v.lower() in ("1", "true", "yes") if typ is bool else typ(v))
        c.validate()
        return c


def histogram_summary(values: torch.Tensor, bins: int = 30) -> Dict[str, Any]:
    v = values.detach().float().flatten().cpu()
    if v.numel() == 0:
        return {"count": 0}
    mean, std = v.mean().item(), v.std(unbiased=False).item()
    lo, hi = v.min().item(), v.max().item()
    counts = torch.histc(v, bins=bins, min=lo, max=hi if hi > lo else lo + 1).tolist()
    q = torch.quantile(v, torch.tensor([0.01, 0.25, 0.5, 0.75, 0.99])).tolist()
    z = (v - mean) / (std if std > 0 else 1.0)
    return {"count": v.numel(), "min": lo, "max": hi, "mean": mean, "std": std, "skew": (z ** 3).mean().item(),
            "kurtosis": (z ** 4).mean().item() - 3.0, "quantiles": dict(zip(("p1", "p25", "p50", "p75", "p99"), q)),
            "outliers": int((z.abs() > 3).sum()), "bins": counts, "nan": int(torch.isnan(v).sum()), "inf": int(torch.isinf(v).sum())}


def module_graph(model: torch.nn.Module) -> Dict[str, Any]:
    nodes = [{"name": n or "<root>", "type": type(m).__name__, "params": sum(p.numel() for p in m.parameters(recurse=False))}
             for n, m in model.named_modules()]
    edges = [{"from": n.rsplit(".", 1)[0] if "." in n else "<root>", "to": n} for n, _ in model.named_modules() if n]
    return {"nodes": nodes, "edges": edges}


class Visualizer:
    def __init__(self, config: Optional[VisualizationConfiguration] = None, backend: Optional[StorageBackend] = None):
        self.cfg = config or VisualizationConfiguration()
        self.cfg.validate()
        self.events = EventSystem()
        if backend is None:
            if self.cfg.storage == "binary":
                from .event_file import BinaryFileStorageBackend
                backend = BinaryFileStorageBackend(self.cfg.log_dir)
            else:
                backend = FileStorageBackend(self.cfg.log_dir) if self.cfg.storage == "file" else MemoryStorageBackend()
        self.backend = backend
        ccfg = EventCollectorConfig(buffer_capacity=self.cfg.buffer_capacity, flush_interval_s=self.cfg.flush_interval_s)
        self.collector = (AsyncEventCollector if self.cfg.async_collection else EventCollector)(backend, ccfg)
        self.events.subscribe(self.collector.collect)
        self.scalars = ScalarLogger(self.events)
        self.profiler = Profiler()
        from .graphs import GraphLogger
        from .histograms import HistogramBinConfig, HistogramLogger
        self.histograms = HistogramLogger(default_bins=HistogramBinConfig(self.cfg.histogram_bins))
        self.graphs = GraphLogger()

    def log_distribution(self, name: str, values: torch.Tensor, step: int = -1):
        """Moments, quantiles, outlier and dead-value counts of a tensor, kept by name and step (``self.histograms``)."""
        if self.cfg.enabled:
            return self.histograms.log_distribution(name, values, step)

    def log_autograd_graph(self, output: torch.Tensor, model: Optional[torch.nn.Module] = None, name: str = "step"):
        """The operation graph autograd recorded behind ``output`` (the loss), as a graph event plus an analysis."""
        if not self.cfg.enabled:
            return None
        from .graphs import GraphSerializer, graph_from_autograd
        g = graph_from_autograd(output, dict(model.named_parameters()) if model is not None else None, name)
        self.graphs.log_graph(g)
        self.events.publish(Event(EventType.GRAPH, name, 0, GraphSerializer.to_dict(g)))
        return self.graphs.analyze_graph(name)

    def log_scalar(self, name: str, value: float, step: int = 0):
        if self.cfg.enabled:
            self.scalars.log(name, value, step)

    def log_histogram(self, name: str, values: torch.Tensor, step: int = 0):
        if self.cfg.enabled:
            self.events.publish(Event(EventType.HISTOGRAM, name, step, histogram_summary(values, self.cfg.histogram_bins)))

    def log_graph(self, model: torch.nn.Module, name: str = "model"):
        if self.cfg.enabled:
            self.events.publish(Event(EventType.GRAPH, name, 0, module_graph(model)))

    def log_hyperparameters(self, hparams: Dict[str, Any], metrics: Optional[Dict[str, float]] = None):
        if self.cfg.enabled:
            self.events.publish(Event(EventType.HYPERPARAMETERS, "hparams", 0, {"hparams": hparams, "metrics": metrics or {}}))

    def log_text(self, name: str, text: str, step: int = 0):
        if self.cfg.enabled:
            self.events.publish(Event(EventType.TEXT, name, step, text))

    def log_image(self, name: str, image: torch.Tensor, step: int = 0):
        """Stores shape + per-channel statistics and an 8-bit thumbnail (<= 64 x 64) of a CHW image."""
        if not self.cfg.enabled:
            return
        img = image.detach().float().cpu()
        st = max(1, math.ceil(max(img.shape[-2:]) / 64))
        thumb = (img[..., ::st, ::st].clamp(0, 1) * 255).to(torch.uint8)
        self.events.publish(Event(EventType.IMAGE, name, step, {"shape": list(img.shape), "thumb": thumb.tolist()}))

    def start_profile(self, name: str):
        return self.profiler.scope(name)

    def record_instant(self, name: str):
        self.profiler.record_instant(name)

    def flush(self):
        self.collector.flush()

    def export(self, path: str):
        self.flush()
        data = {"scalars": {k: {"steps": s.steps, "values": s.values} for k, s in self.scalars.series.items()},
                "profile": {k: vars(r) for k, r in self.profiler.results().items()}}
        with open(path, "w") as f:
            json.dump(data, f, indent=1)

    def close(self):
        self.collector.close()


class VisualizerBuilder:
    def __init__(self):
        self._c = VisualizationConfiguration()
        self._backend: Optional[StorageBackend] = None

    def with_log_dir(self, d): self._c.log_dir = d; return self
    def with_async(self, b=True): self._c.async_collection = b; return self
    def with_storage(self, kind): self._c.storage = kind; return self
    def with_backend(self, b): self._backend = b; return self
    def with_histogram_bins(self, n): self._c.histogram_bins = n; return self
    def enabled(self, b=True): self._c.enabled = b; return self

    def build(self) -> Visualizer:
        return Visualizer(self._c, self._backend)
