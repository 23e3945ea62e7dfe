"""Sectioned configuration of the visualisation stack with validation, a fluent builder and loaders.

Reference: src/MLFramework.Visualization/Configuration/{VisualizationConfiguration.cs,
StorageConfiguration.cs, LoggingConfiguration.cs, ProfilingConfiguration.cs,
MemoryProfilingConfiguration.cs, GPUTrackingConfiguration.cs, EventCollectionConfiguration.cs,
ConfigurationValidator.cs:8-247, ValidationResult.cs, VisualizationConfigurationBuilder.cs:6-258,
ConfigurationLoader.cs:8-235}.

``FullVisualizationConfiguration.to_flat()`` gives the flat settings that ``obs.visualizer.Visualizer``
consumes; ``make_visualizer`` builds one and applies the logging switches (scalars, histograms,
graphs, hyper-parameters, prefix) that the flat form has no field for.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

__all__ = [
    "StorageConfiguration", "LoggingConfiguration", "ProfilingConfiguration", "MemoryProfilingConfiguration",
    "GPUTrackingConfiguration", "EventCollectionConfiguration", "FullVisualizationConfiguration",
    "ConfigValidationResult", "ConfigurationValidator", "VisualizationConfigurationBuilder",
    "SectionedConfigurationLoader", "make_visualizer",
]


@dataclass
class StorageConfiguration:
    backend_type: str = "file"                 # file | memory | binary
    log_directory: str = "./logs"
    connection_string: Optional[str] = None
    write_buffer_size: int = 100
    flush_interval_s: float = 1.0
    enable_async_writes: bool = True


@dataclass
class LoggingConfiguration:
    log_scalars: bool = True
    log_histograms: bool = True
    log_graphs: bool = True
    log_hyperparameters: bool = True
    scalar_log_prefix: str = ""
    histogram_bin_count: int = 30
    auto_smooth_scalars: bool = True
    default_smoothing_window: int = 10


@dataclass
class ProfilingConfiguration:
    enable_profiling: bool = True
    profile_forward_pass: bool = True
    profile_backward_pass: bool = True
    profile_optimizer_step: bool = False
    profile_cpu: bool = True
    profile_gpu: bool = True
    max_stored_operations: int = 10000


@dataclass
class MemoryProfilingConfiguration:
    enable_memory_profiling: bool = False
    capture_stack_traces: bool = False
    max_stack_trace_depth: int = 10
    snapshot_interval_ms: int = 1000
    auto_snapshot: bool = True


@dataclass
class GPUTrackingConfiguration:
    enable_gpu_tracking: bool = False
    sampling_interval_ms: int = 1000
    track_temperature: bool = True
    track_power: bool = True


@dataclass
class EventCollectionConfiguration:
    enable_async: bool = True
    buffer_capacity: int = 1000
    batch_size: int = 100
    enable_backpressure: bool = True
    max_queue_length: int = 10000


@dataclass
class FullVisualizationConfiguration:
    storage: StorageConfiguration = field(default_factory=StorageConfiguration)
    logging: LoggingConfiguration = field(default_factory=LoggingConfiguration)
    profiling: ProfilingConfiguration = field(default_factory=ProfilingConfiguration)
    memory_profiling: MemoryProfilingConfiguration = field(default_factory=MemoryProfilingConfiguration)
    gpu_tracking: GPUTrackingConfiguration = field(default_factory=GPUTrackingConfiguration)
    event_collection: EventCollectionConfiguration = field(default_factory=EventCollectionConfiguration)
    is_enabled: bool = True
    verbose_logging: bool = False

    def to_flat(self):
        from .visualizer import VisualizationConfiguration
        return VisualizationConfiguration(
            log_dir=self.storage.log_directory, enabled=self.is_enabled,
            async_collection=self.event_collection.enable_async and self.storage.enable_async_writes,
            flush_interval_s=self.storage.flush_interval_s, buffer_capacity=self.event_collection.buffer_capacity,
            histogram_bins=self.logging.histogram_bin_count, storage=self.storage.backend_type)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


class ConfigValidationResult:
    def __init__(self, errors: Optional[List[str]] = None, warnings: Optional[List[str]] = None):
        self.errors: List[str] = list(errors or [])
        self.warnings: List[str] = list(warnings or [])

    @property
    def is_valid(self) -> bool:
        return not self.errors

    def add_error(self, e: str) -> None:
        self.errors.append(e)

    def add_warning(self, w: str) -> None:
        self.warnings.append(w)

    def summary(self) -> str:
        head = "configuration is valid" if self.is_valid else f"configuration is invalid: {len(self.errors)} error(s)"
        lines = [head] + [f"  error: {e}" for e in self.errors] + [f"  warning: {w}" for w in self.warnings]
        return "\n".join(lines)


class ConfigurationValidator:
    """Errors stop a build; warnings point at settings that work but cost (ConfigurationValidator.cs)."""

    BACKENDS = ("file", "memory", "binary")

    def validate(self, c: Optional[FullVisualizationConfiguration]) -> ConfigValidationResult:
        r = ConfigValidationResult()
        if c is None:
            r.add_error("configuration cannot be None")
            return r
        for name in ("storage", "logging", "profiling", "memory_profiling", "gpu_tracking", "event_collection"):
            if getattr(c, name) is None:
                r.add_error(f"{name} configuration cannot be None")
        if not r.is_valid:
            return r
        s, lg, p, m, g, e = c.storage, c.logging, c.profiling, c.memory_profiling, c.gpu_tracking, c.event_collection
        if not s.log_directory or not s.log_directory.strip():
            r.add_error("storage.log_directory cannot be empty")
        if s.write_buffer_size <= 0:
            r.add_error("storage.write_buffer_size must be positive")
        elif s.write_buffer_size > 100000:
            r.add_warning("storage.write_buffer_size is very large, may consume significant memory")
        if s.flush_interval_s <= 0:
            r.add_error("storage.flush_interval_s must be positive")
        elif s.flush_interval_s > 300:
            r.add_warning("storage.flush_interval_s is very long, data may be lost if the process crashes")
        if not s.backend_type or not s.backend_type.strip():
            r.add_error("storage.backend_type cannot be empty")
        elif s.backend_type not in self.BACKENDS:
            r.add_error(f"storage.backend_type must be one of {', '.join(self.BACKENDS)}")
        if lg.histogram_bin_count <= 0:
            r.add_error("logging.histogram_bin_count must be positive")
        elif lg.histogram_bin_count > 1000:
            r.add_warning("logging.histogram_bin_count is very large, may impact performance")
        if lg.default_smoothing_window <= 0:
            r.add_error("logging.default_smoothing_window must be positive")
        elif lg.default_smoothing_window > 1000:
            r.add_warning("logging.default_smoothing_window is very large, smoothing will be very aggressive")
        if p.max_stored_operations <= 0:
            r.add_error("profiling.max_stored_operations must be positive")
        elif p.max_stored_operations > 100000:
            r.add_warning("profiling.max_stored_operations is very large, may consume significant memory")
        if p.enable_profiling and not p.profile_cpu and not p.profile_gpu:
            r.add_warning("profiling is enabled but neither CPU nor GPU profiling is selected")
        if m.max_stack_trace_depth <= 0:
            r.add_error("memory_profiling.max_stack_trace_depth must be positive")
        elif m.max_stack_trace_depth > 50:
            r.add_warning("memory_profiling.max_stack_trace_depth is very large, may impact performance")
        if m.snapshot_interval_ms <= 0:
            r.add_error("memory_profiling.snapshot_interval_ms must be positive")
        elif m.snapshot_interval_ms < 100 and m.auto_snapshot:
            r.add_warning("memory_profiling.snapshot_interval_ms is very small, may impact performance")
        if m.capture_stack_traces and not m.enable_memory_profiling:
            r.add_warning("memory_profiling.capture_stack_traces is enabled but memory profiling is disabled")
        if g.sampling_interval_ms <= 0:
            r.add_error("gpu_tracking.sampling_interval_ms must be positive")
        elif g.sampling_interval_ms < 100 and g.enable_gpu_tracking:
            r.add_warning("gpu_tracking.sampling_interval_ms is very small, may impact performance")
        if g.enable_gpu_tracking and not g.track_temperature and not g.track_power:
            r.add_warning("gpu tracking is enabled but neither temperature nor power tracking is selected")
        if e.buffer_capacity <= 0:
            r.add_error("event_collection.buffer_capacity must be positive")
        elif e.buffer_capacity > 100000:
            r.add_warning("event_collection.buffer_capacity is very large, may consume significant memory")
        if e.batch_size <= 0:
            r.add_error("event_collection.batch_size must be positive")
        elif e.buffer_capacity > 0 and e.batch_size > e.buffer_capacity:
            r.add_error("event_collection.batch_size cannot be larger than buffer_capacity")
        if e.max_queue_length <= 0:
            r.add_error("event_collection.max_queue_length must be positive")
        elif e.batch_size > e.max_queue_length:
            r.add_error("event_collection.batch_size cannot be larger than max_queue_length")
        return r

    def validate_or_raise(self, c: FullVisualizationConfiguration) -> None:
        r = self.validate(c)
        if not r.is_valid:
            raise ValueError(r.summary())


class VisualizationConfigurationBuilder:
    """Fluent construction; ``build`` validates (VisualizationConfigurationBuilder.cs:6-258)."""

    def __init__(self):
        self._c = FullVisualizationConfiguration()

    def _set(self, section: str, name: str, value):
        setattr(getattr(self._c, section), name, value)
        return self

    def with_storage(self, storage: StorageConfiguration):
        self._c.storage = storage
        return self

    def with_storage_directory(self, d: str): return self._set("storage", "log_directory", d)
    def with_storage_backend(self, kind: str): return self._set("storage", "backend_type", kind)

    def with_logging(self, logging: LoggingConfiguration):
        self._c.logging = logging
        return self

    def with_log_prefix(self, p: str): return self._set("logging", "scalar_log_prefix", p)
    def with_scalar_logging(self, on: bool): return self._set("logging", "log_scalars", on)
    def with_histogram_bin_count(self, n: int): return self._set("logging", "histogram_bin_count", n)

    def with_profiling(self, profiling: ProfilingConfiguration):
        self._c.profiling = profiling
        return self

    def enable_profiling(self, on: bool = True): return self._set("profiling", "enable_profiling", on)
    def enable_cpu_profiling(self, on: bool = True): return self._set("profiling", "profile_cpu", on)
    def enable_gpu_profiling(self, on: bool = True): return self._set("profiling", "profile_gpu", on)
    def with_max_stored_operations(self, n: int): return self._set("profiling", "max_stored_operations", n)

    def with_memory_profiling(self, mp: MemoryProfilingConfiguration):
        self._c.memory_profiling = mp
        return self

    def enable_memory_profiling(self, on: bool = True): return self._set("memory_profiling", "enable_memory_profiling", on)
    def with_memory_snapshot_interval_ms(self, ms: int): return self._set("memory_profiling", "snapshot_interval_ms", ms)

    def with_gpu_tracking(self, g: GPUTrackingConfiguration):
        self._c.gpu_tracking = g
        return self

    def enable_gpu_tracking(self, on: bool = True): return self._set("gpu_tracking", "enable_gpu_tracking", on)
    def with_gpu_sampling_interval_ms(self, ms: int): return self._set("gpu_tracking", "sampling_interval_ms", ms)

    def with_event_collection(self, e: EventCollectionConfiguration):
        self._c.event_collection = e
        return self

    def enable_async_event_collection(self, on: bool = True): return self._set("event_collection", "enable_async", on)
    def with_event_buffer_capacity(self, n: int): return self._set("event_collection", "buffer_capacity", n)
    def with_event_batch_size(self, n: int): return self._set("event_collection", "batch_size", n)

    def enable(self, on: bool = True):
        self._c.is_enabled = on
        return self

    def with_verbose_logging(self, on: bool = True):
        self._c.verbose_logging = on
        return self

    def build(self) -> FullVisualizationConfiguration:
        ConfigurationValidator().validate_or_raise(self._c)
        return self._c

    def build_without_validation(self) -> FullVisualizationConfiguration:
        return self._c

    def build_with_validation(self) -> Tuple[FullVisualizationConfiguration, ConfigValidationResult]:
        return self._c, ConfigurationValidator().validate(self._c)


_SECTIONS = {"storage": StorageConfiguration, "logging": LoggingConfiguration, "profiling": ProfilingConfiguration,
             "memory_profiling": MemoryProfilingConfiguration, "gpu_tracking": GPUTrackingConfiguration,
             "event_collection": EventCollectionConfiguration}


def _coerce(cur, raw: str):
    if isinstance(cur, bool):
        if raw.strip().lower() in ("1", "true", "yes", "on"):
            return True
        if raw.strip().lower() in ("0", "false", "no", "off"):
            return False
        raise ValueError(f"not a boolean: {raw!r}")
    if isinstance(cur, int):
        return int(raw)
    if isinstance(cur, float):
        return float(raw)
    return raw


class SectionedConfigurationLoader:
    """JSON (nested by section; unknown keys are errors), environment variables
    ``<PREFIX><SECTION>__<FIELD>`` / ``<PREFIX><FIELD>`` over any base, defaults."""

    PREFIX = "MLFRAMEWORK_VISUALIZATION_"

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> FullVisualizationConfiguration:
        c = FullVisualizationConfiguration()
        for k, v in d.items():
            if k in _SECTIONS:
                known = {f.name for f in dataclasses.fields(_SECTIONS[k])}
                bad = set(v) - known
                if bad:
                    raise KeyError(f"unknown {k} settings: {sorted(bad)}")
                setattr(c, k, _SECTIONS[k](**v))
            elif k in ("is_enabled", "verbose_logging"):
                setattr(c, k, bool(v))
            else:
                raise KeyError(f"unknown configuration section {k!r}")
        return c

    @classmethod
    def from_json(cls, text: str) -> FullVisualizationConfiguration:
        return cls.from_dict(json.loads(text))

    @classmethod
    def from_file(cls, path: str) -> FullVisualizationConfiguration:
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        with open(path) as f:
            return cls.from_json(f.read())

    @classmethod
    def from_environment(cls, base: Optional[FullVisualizationConfiguration] = None, env=None) -> FullVisualizationConfiguration:
        env = os.environ if env is None else env
        c = base or FullVisualizationConfiguration()
        for key, raw in env.items():
            if not key.startswith(cls.PREFIX):
                continue
            rest = key[len(cls.PREFIX):].lower()
            if "__" in rest:
                section, name = rest.split("__", 1)
                if section not in _SECTIONS or not hasattr(getattr(c, section), name):
                    raise KeyError(f"environment variable {key} names no setting")
                setattr(getattr(c, section), name, _coerce(getattr(getattr(c, section), name), raw))
            elif rest in ("is_enabled", "verbose_logging"):
                setattr(c, rest, _coerce(True, raw))
            else:
                raise KeyError(f"environment variable {key} names no setting")
        return c

    @classmethod
    def load(cls, path: Optional[str] = None, env=None, validate: bool = True) -> FullVisualizationConfiguration:
        """File (when given), then environment overrides, then validation."""
        c = cls.from_environment(cls.from_file(path) if path else None, env)
        if validate:
            ConfigurationValidator().validate_or_raise(c)
        return c

    @staticmethod
    def save(c: FullVisualizationConfiguration, path: str) -> None:
        with open(path, "w") as f:
            json.dump(c.to_dict(), f, indent=1)


def make_visualizer(config: FullVisualizationConfiguration, backend=None):
    """A ``Visualizer`` that honours the sectioned settings: disabled kinds of records are dropped, scalar
    names get the prefix, the profiler keeps at most ``max_stored_operations`` records per name."""
    from .visualizer import Visualizer
    ConfigurationValidator().validate_or_raise(config)
    v = Visualizer(config.to_flat(), backend)
    lg = config.logging
    if not lg.log_scalars:
        v.log_scalar = lambda *a, **k: None
    elif lg.scalar_log_prefix:
        inner = v.log_scalar
        v.log_scalar = lambda name, value, step=0: inner(lg.scalar_log_prefix + name, value, step)
    if not lg.log_histograms:
        v.log_histogram = lambda *a, **k: None
        v.log_distribution = lambda *a, **k: None
    if not lg.log_graphs:
        v.log_graph = lambda *a, **k: None
        v.log_autograd_graph = lambda *a, **k: None
    if not lg.log_hyperparameters:
        v.log_hyperparameters = lambda *a, **k: None
    if not config.profiling.enable_profiling:
        import contextlib
        v.start_profile = lambda name: contextlib.nullcontext()
        v.record_instant = lambda name: None
    v.full_config = config
    return v
