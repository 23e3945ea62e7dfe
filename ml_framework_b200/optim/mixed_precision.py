"""Mixed-precision optimizer wrapper: reduced-precision training weights, fp32 master weights, dynamic loss
scaling with skip-on-overflow, gradient clipping, automatic fall-back to fp32 after a run of overflows, and a
step-time monitor.

Behaviour follows the reference (src/MLFramework/Optimizers/MixedPrecision/MixedPrecisionOptimizer.cs:107-138,
:295-310: process gradients -> skip on overflow -> base step; after ``max_consecutive_overflows`` skipped steps in
a row with ``enable_auto_fallback`` the optimizer switches to fp32 for good; MixedPrecisionOptions.cs:9-125 for
the defaults: fp16, scale 65536, x2 / x0.5, interval 2000, fp32 layer patterns BatchNorm / LayerNorm /
InstanceNorm / GroupNorm, clip at norm 1.0, fall-back after 10; PrecisionManager.cs:75-215 for the conversion
rules and exclusions; PerformanceMonitor.cs:89-160 for the step timer). The reference leaves the conversions as
pass-through ("when tensor infrastructure is ready"); here they are real: training weights are bf16 / fp16 copies
of fp32 masters, excluded layers stay fp32, and ``sync_training_weights`` rounds the masters back after each step.
"""
from __future__ import annotations

import dataclasses
import enum
import fnmatch
import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig

_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


@dataclass
class MixedPrecisionOptions:
    precision: str = "bf16"                  # fp32 | fp16 | bf16 (the reference defaults to fp16; B200 trains in bf16)
    auto_detect_precision: bool = True
    initial_loss_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    max_loss_scale: float = 1e9
    min_loss_scale: float = 1.0
    growth_interval: int = 2000
    enable_dynamic_loss_scaling: bool = True
    auto_exclude_sensitive_layers: bool = True
    fp32_layer_patterns: List[str] = field(default_factory=lambda: ["*BatchNorm*", "*LayerNorm*", "*InstanceNorm*", "*GroupNorm*",
                                                                     "*norm*", "*ln_*", "*ln1*", "*ln2*"])
    max_grad_norm: float = 1.0
    enable_gradient_clipping: bool = True
    max_consecutive_overflows: int = 10
    enable_auto_fallback: bool = True
    enable_performance_monitoring: bool = True
    log_fallback_events: bool = False

    def validate(self):
        if self.precision not in _DTYPES:
            raise ValueError(f"precision must be one of {sorted(_DTYPES)}")
        if self.initial_loss_scale <= 0 or self.min_loss_scale <= 0 or self.max_loss_scale < self.min_loss_scale:
            raise ValueError("loss-scale bounds must be positive and ordered")
        if self.growth_factor <= 1.0 or not (0.0 < self.backoff_factor < 1.0):
            raise ValueError("growth_factor must be > 1 and backoff_factor in (0, 1)")
        if self.growth_interval <= 0 or self.max_consecutive_overflows <= 0:
            raise ValueError("growth_interval and max_consecutive_overflows must be positive")
        if self.max_grad_norm <= 0:
            raise ValueError("max_grad_norm must be positive")


def detect_precision() -> str:
    """bf16 where the device has bf16 tensor cores (every sm_80+ part), fp16 on older GPUs, fp32 on the CPU
    (the reference's HardwareDetector.cs:20-65)."""
    if not torch.cuda.is_available():
        return "fp32"
    major, _ = torch.cuda.get_device_capability()
    return "bf16" if major >= 8 else "fp16"


@dataclass
class PrecisionConversionStats:
    total_conversions: int = 0
    training_precision_conversions: int = 0
    fp32_conversions: int = 0
    skipped_conversions: int = 0
    excluded_layers: int = 0


class PrecisionManager:
    """Which tensors train in reduced precision and the conversions between training and master copies."""

    def __init__(self, options: Optional[MixedPrecisionOptions] = None):
        self.options = options or MixedPrecisionOptions()
        self.target = _DTYPES[self.options.precision]
        self._patterns: List[str] = list(self.options.fp32_layer_patterns) if self.options.auto_exclude_sensitive_layers else []
        self.stats = PrecisionConversionStats()

    @property
    def is_reduced_precision(self) -> bool:
        return self.target != torch.float32

    def should_exclude_layer(self, name: Optional[str]) -> bool:
        return bool(name) and any(fnmatch.fnmatchcase(name, p) or fnmatch.fnmatchcase(name.lower(), p.lower()) for p in self._patterns)

    def exclude_layers_matching(self, pattern: str):
        if pattern not in self._patterns:
            self._patterns.append(pattern)

    def remove_exclusion(self, pattern: str) -> bool:
        if pattern in self._patterns:
            self._patterns.remove(pattern)
            return True
        return False

    def clear_exclusions(self):
        self._patterns.clear()

    def exclusion_patterns(self) -> List[str]:
        return list(self._patterns)

    def convert_to_training_precision(self, t: torch.Tensor, layer_name: Optional[str] = None) -> torch.Tensor:
        self.stats.total_conversions += 1
        if self.should_exclude_layer(layer_name):
            self.stats.excluded_layers += 1
            return t if t.dtype == torch.float32 else t.float()
        if t.dtype == self.target:
            self.stats.skipped_conversions += 1
            return t
        self.stats.training_precision_conversions += 1
        return t.to(self.target)

    def convert_to_fp32(self, t: torch.Tensor) -> torch.Tensor:
        self.stats.total_conversions += 1
        if t.dtype == torch.float32:
            self.stats.skipped_conversions += 1
            return t
        self.stats.fp32_conversions += 1
        return t.float()

    def convert_weights(self, weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: self.convert_to_training_precision(v, k) for k, v in weights.items()}

    def create_master_weights(self, training: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: self.convert_to_fp32(v).detach().clone() for k, v in training.items()}

    def sync_training_weights(self, masters: Dict[str, torch.Tensor], training: Dict[str, torch.Tensor]):
        """Rounds the fp32 masters into the training copies in place."""
        with torch.no_grad():
            for k, m in masters.items():
                training[k].copy_(m)


@dataclass
class PerformanceStats:
    average_step_time_ms: float = 0.0
    last_step_time_ms: float = 0.0
    min_step_time_ms: float = 0.0
    max_step_time_ms: float = 0.0
    std_dev_step_time_ms: float = 0.0
    total_time_seconds: float = 0.0
    step_count: int = 0
    steps_per_second: float = 0.0


class PerformanceMonitor:
    def __init__(self, clock=time.perf_counter):
        self.clock = clock
        self.reset()

    def reset(self):
        self._t0 = None
        self._n = 0
        self._sum = self._sumsq = 0.0
        self._min, self._max, self._last = math.inf, -math.inf, 0.0

    def start_step(self):
        self._t0 = self.clock()

    def end_step(self):
        if self._t0 is None:
            return
        ms = (self.clock() - self._t0) * 1e3
        self._t0 = None
        self._n += 1
        self._sum += ms
        self._sumsq += ms * ms
        self._min, self._max, self._last = min(self._min, ms), max(self._max, ms), ms

    def get_stats(self) -> PerformanceStats:
        if self._n == 0:
            return PerformanceStats()
        avg = self._sum / self._n
        var = max(0.0, self._sumsq / self._n - avg * avg)
        return PerformanceStats(avg, self._last, self._min, self._max, math.sqrt(var), self._sum / 1e3, self._n,
                                1000.0 / avg if avg > 0 else 0.0)

    def get_summary(self) -> str:
        s = self.get_stats()
        return (f"steps {s.step_count}, {s.average_step_time_ms:.3f} ms/step (min {s.min_step_time_ms:.3f}, max "
                f"{s.max_step_time_ms:.3f}, sd {s.std_dev_step_time_ms:.3f}), {s.steps_per_second:.1f} steps/s")


@dataclass
class MixedPrecisionOptimizerStats:
    step_count: int
    skipped_steps: int
    has_fallback: bool
    target_precision: str
    loss_scale: float
    consecutive_overflows: int
    performance: Optional[PerformanceStats] = None

    @property
    def skip_rate(self) -> float:
        return self.skipped_steps / self.step_count if self.step_count else 0.0


class MixedPrecisionOptimizer:
    """Wraps a model and a base optimizer factory.

    The model's parameters become reduced-precision training weights (excluded layers stay fp32); fp32 master copies are
    what ``base_optimizer_factory(master_params)`` optimizes. ``step()`` takes the gradients of the training weights:
    unscales them into the masters' ``.grad``, skips the step on overflow (backing the scale off), clips by global
    norm, steps the base optimizer, rounds the masters back into the training weights and updates the scale. After
    ``max_consecutive_overflows`` skipped steps in a row the training weights are switched to fp32 for the rest of the
    run (``has_fallback``) and loss scaling is turned off.
    """

    def __init__(self, model: nn.Module, base_optimizer_factory, options: Optional[MixedPrecisionOptions] = None):
        self.options = options or MixedPrecisionOptions()
        self.options.validate()
        if self.options.auto_detect_precision and self.options.precision != "fp32":
            det = detect_precision()
            dev = next(model.parameters()).device.type
            if det == "fp32" and dev == "cpu" and self.options.precision == "fp16":
                self.options.precision = "bf16"        # fp16 arithmetic is not usable on the CPU
        self.model = model
        self.precision = PrecisionManager(self.options)
        self.monitor = PerformanceMonitor() if self.options.enable_performance_monitoring else None
        self.named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        device = self.named[0][1].device
        # exclusion patterns see the parameter's path with the class of the module that owns it, so that
        # "*LayerNorm*" finds a norm layer whatever its attribute is called
        owner = {id(p): type(m).__name__ for m in model.modules() for p in m.parameters(recurse=False)}
        self.masters: Dict[str, torch.Tensor] = {}
        with torch.no_grad():
            for n, p in self.named:
                self.masters[n] = nn.Parameter(p.detach().float().clone())
                p.data = self.precision.convert_to_training_precision(p.data, f"{n}:{owner.get(id(p), '')}")
        self.base = base_optimizer_factory(list(self.masters.values()))
        o = self.options
        self.scaler = DynamicLossScaler(DynamicScalerConfig(initial_scale=o.initial_loss_scale, growth_factor=o.growth_factor,
                                                            backoff_factor=o.backoff_factor, growth_interval=o.growth_interval,
                                                            min_scale=o.min_loss_scale, max_scale=o.max_loss_scale,
                                                            enabled=o.enable_dynamic_loss_scaling and self.precision.is_reduced_precision),
                                        device=device)
        self.step_count = 0
        self.skipped_steps = 0
        self.consecutive_overflows = 0
        self.has_fallback = False
        self.last_grad_norm: Optional[float] = None

    # ---- loss scaling
    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return self.scaler.scale_loss(loss)

    def zero_grad(self):
        for _, p in self.named:
            p.grad = None
        for m in self.masters.values():
            m.grad = None

    # ---- the step
    def step(self) -> bool:
        """Returns True when the update was applied, False when it was skipped because of an overflow."""
        if self.monitor is not None:
            self.monitor.start_step()
        self.step_count += 1
        inv = 1.0 / self.scaler.scale if self.scaler.enabled else 1.0
        overflow = False
        sumsq = 0.0
        for n, p in self.named:
            m = self.masters[n]
            if p.grad is None:
                m.grad = None
                continue
            g = p.grad.detach().float() * inv
            if not bool(torch.isfinite(g).all()):
                overflow = True
                break
            m.grad = g
            sumsq += float(g.pow(2).sum())
        if overflow:
            self.skipped_steps += 1
            self.consecutive_overflows += 1
            self.scaler.found_inf.fill_(1)
            self.scaler.update()
            if self.options.enable_auto_fallback and self.consecutive_overflows >= self.options.max_consecutive_overflows:
                self.fallback_to_fp32()
            if self.monitor is not None:
                self.monitor.end_step()
            return False
        self.consecutive_overflows = 0
        norm = math.sqrt(sumsq)
        self.last_grad_norm = norm
        if self.options.enable_gradient_clipping and norm > self.options.max_grad_norm:
            c = self.options.max_grad_norm / (norm + 1e-6)
            for m in self.masters.values():
                if m.grad is not None:
                    m.grad.mul_(c)
        self.base.step()
        self.precision.sync_training_weights({n: self.masters[n].data for n, _ in self.named}, {n: p.data for n, p in self.named})
        self.scaler.update()
        if self.monitor is not None:
            self.monitor.end_step()
        return True

    def fallback_to_fp32(self):
        """Training weights become fp32 copies of the masters; loss scaling stops. Irreversible."""
        if self.has_fallback:
            return
        self.has_fallback = True
        with torch.no_grad():
            for n, p in self.named:
                p.data = self.masters[n].data.clone()
        self.precision.target = torch.float32
        self.scaler.enabled = False
        if self.options.log_fallback_events:
            print(f"[MixedPrecisionOptimizer] falling back to fp32 after {self.consecutive_overflows} consecutive overflows")

    def get_stats(self) -> MixedPrecisionOptimizerStats:
        return MixedPrecisionOptimizerStats(self.step_count, self.skipped_steps, self.has_fallback,
                                            "fp32" if self.has_fallback else self.options.precision, self.scaler.scale,
                                            self.consecutive_overflows, self.monitor.get_stats() if self.monitor else None)

    def state_dict(self) -> Dict:
        return {"masters": {k: v.detach().cpu().clone() for k, v in self.masters.items()}, "scaler": self.scaler.state_dict(),
                "step_count": self.step_count, "skipped_steps": self.skipped_steps, "has_fallback": self.has_fallback,
                "base": self.base.state_dict() if hasattr(self.base, "state_dict") else None}

    def load_state_dict(self, sd: Dict):
        with torch.no_grad():
            for k, v in sd["masters"].items():
                self.masters[k].copy_(v)
        self.scaler.load_state_dict(sd["scaler"])
        self.step_count, self.skipped_steps = sd["step_count"], sd["skipped_steps"]
        if sd.get("has_fallback"):
            self.fallback_to_fp32()
        else:
            self.precision.sync_training_weights({n: self.masters[n].data for n, _ in self.named}, {n: p.data for n, p in self.named})
        if sd.get("base") is not None and hasattr(self.base, "load_state_dict"):
            self.base.load_state_dict(sd["base"])


# ------------------------------------------------------------------ precision helpers, gradient layer, checkpoints
class Precision(enum.Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"

    @property
    def dtype(self) -> torch.dtype:
        return _DTYPES[self.value]


@dataclass(frozen=True)
class PrecisionCapability:
    supports_fp16: bool
    supports_bf16: bool
    supports_fp32: bool = True

    @property
    def is_fp16_available(self) -> bool:
        return self.supports_fp16

    @property
    def is_bf16_available(self) -> bool:
        return self.supports_bf16


class HardwareDetector:
    """What the current device computes in natively, asked once (HardwareDetector.cs:5-60)."""

    _cached: Optional[PrecisionCapability] = None

    @classmethod
    def detect_capabilities(cls) -> PrecisionCapability:
        if cls._cached is None:
            if torch.cuda.is_available():
                major, _ = torch.cuda.get_device_capability()
                cls._cached = PrecisionCapability(supports_fp16=major >= 6, supports_bf16=major >= 8)
            else:
                cls._cached = PrecisionCapability(supports_fp16=False, supports_bf16=True)     # CPU kernels exist for bf16 only
        return cls._cached

    @classmethod
    def get_recommended_precision(cls) -> Precision:
        return Precision(detect_precision())

    @classmethod
    def reset_cache(cls) -> None:
        cls._cached = None


class PrecisionConverter:
    """Conversions between the three training precisions (PrecisionConverter.cs)."""

    @staticmethod
    def convert(t: torch.Tensor, target: Precision) -> torch.Tensor:
        if not t.is_floating_point():
            raise TypeError(f"cannot change the precision of a {t.dtype} tensor")
        return t if t.dtype == target.dtype else t.to(target.dtype)

    @staticmethod
    def detect_precision(t: torch.Tensor) -> Precision:
        for p in Precision:
            if t.dtype == p.dtype:
                return p
        raise TypeError(f"{t.dtype} is not a training precision")

    @staticmethod
    def is_conversion_safe(source: Precision, target: Precision, t: Optional[torch.Tensor] = None) -> bool:
        """Widening is always safe. Narrowing to bf16 keeps the range; narrowing to fp16 is safe only while
        the values fit its range, which needs the tensor to decide (without one: not safe)."""
        if source == target or target is Precision.FP32:
            return True
        if target is Precision.BF16 and source is Precision.FP32:
            return True
        if t is None or not t.numel():
            return t is not None
        lim = torch.finfo(target.dtype).max
        return bool(torch.isfinite(t).all() and t.abs().max() <= lim)


@dataclass
class LossScalerStats:
    current_scale: float
    steps_since_last_overflow: int
    total_steps: int
    total_overflows: int


@dataclass
class GradientProcessingStats:
    loss_scale: float
    clip_count: int
    last_gradient_norm: float
    clipping_enabled: bool
    max_grad_norm: float
    loss_scaler_stats: LossScalerStats

    def __str__(self):
        clip = f"clip at {self.max_grad_norm:g} ({self.clip_count} times)" if self.clipping_enabled else "no clipping"
        return f"loss scale {self.loss_scale:g}, last gradient norm {self.last_gradient_norm:.4g}, {clip}"


class GradientConversionLayer:
    """Between backward and the optimizer: unscale, detect overflow, clip by global norm, as one call on a
    dictionary of gradients (GradientConversionLayer.cs:10-230)."""

    def __init__(self, options: Optional[MixedPrecisionOptions] = None, loss_scaler: Optional[DynamicLossScaler] = None, device="cpu"):
        self.options = options or MixedPrecisionOptions()
        self.options.validate()
        o = self.options
        self.scaler = loss_scaler or DynamicLossScaler(DynamicScalerConfig(
            initial_scale=o.initial_loss_scale, growth_factor=o.growth_factor, backoff_factor=o.backoff_factor,
            growth_interval=o.growth_interval, min_scale=o.min_loss_scale, max_scale=o.max_loss_scale,
            enabled=o.enable_dynamic_loss_scaling), device=device)
        self.clip_count = 0
        self.last_gradient_norm = 0.0

    @property
    def loss_scale(self) -> float:
        return self.scaler.scale

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return self.scaler.scale_loss(loss)

    def clip_gradients(self, gradients: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Scales every gradient by ``max_grad_norm / norm`` when the global norm exceeds the bound (in place)."""
        if not gradients:
            return gradients
        norm = float(torch.sqrt(sum((g.float() ** 2).sum() for g in gradients.values())))
        self.last_gradient_norm = norm
        if self.options.enable_gradient_clipping and norm > self.options.max_grad_norm:
            k = self.options.max_grad_norm / (norm + 1e-6)
            for g in gradients.values():
                g.mul_(k)
            self.clip_count += 1
        return gradients

    def process_gradients(self, gradients: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], bool]:
        """(fp32 gradients ready for the optimizer, whether to skip the step). Updates the loss scale."""
        inv = 1.0 / self.scaler.scale if self.scaler.enabled else 1.0
        out = {k: g.float() * inv for k, g in gradients.items()}
        overflow = any(not bool(torch.isfinite(g).all()) for g in out.values())
        if overflow:
            self.scaler.found_inf.fill_(1)
        self.scaler.update()
        if overflow:
            return {}, True
        return self.clip_gradients(out), False

    def get_stats(self) -> GradientProcessingStats:
        s = self.scaler.get_stats()
        ls = LossScalerStats(s.scale, s.growth_tracker, s.total_steps, s.skipped_steps)
        return GradientProcessingStats(self.loss_scale, self.clip_count, self.last_gradient_norm, self.options.enable_gradient_clipping,
                                       self.options.max_grad_norm, ls)

    def reset(self) -> None:
        self.clip_count, self.last_gradient_norm = 0, 0.0
        self.scaler.load_state_dict({"scale": self.options.initial_loss_scale, "tracker": 0, "total_steps": 0, "skipped": 0})


@dataclass
class MixedPrecisionCheckpoint:
    """Everything needed to continue a mixed-precision run exactly (Checkpointing.cs:11-82)."""
    version: int = 1
    timestamp: float = field(default_factory=time.time)
    master_weights: Dict[str, torch.Tensor] = field(default_factory=dict)
    training_weights: Dict[str, torch.Tensor] = field(default_factory=dict)
    current_loss_scale: float = 1.0
    steps_since_last_overflow: int = 0
    consecutive_overflows: int = 0
    total_overflows: int = 0
    step_count: int = 0
    has_fallback: bool = False
    skipped_steps: int = 0
    options: Optional[Dict] = None
    scaler_state: Optional[Dict] = None
    base_optimizer_state: Optional[Dict] = None
    metadata: Dict[str, str] = field(default_factory=dict)


class MixedPrecisionCheckpointManager:
    VERSION = 1

    @classmethod
    def create_checkpoint(cls, optimizer: "MixedPrecisionOptimizer", metadata: Optional[Dict[str, str]] = None) -> MixedPrecisionCheckpoint:
        sd = optimizer.state_dict()
        sc = sd["scaler"]
        return MixedPrecisionCheckpoint(
            cls.VERSION, time.time(), sd["masters"], {n: p.detach().cpu().clone() for n, p in optimizer.named},
            sc["scale"], sc["tracker"], optimizer.consecutive_overflows, sc["skipped"], sd["step_count"], sd["has_fallback"],
            sd["skipped_steps"], dataclasses.asdict(optimizer.options), sc, sd["base"], dict(metadata or {}))

    @staticmethod
    def save_checkpoint(checkpoint: MixedPrecisionCheckpoint, path: str) -> None:
        tmp = path + ".tmp"
        torch.save(dataclasses.asdict(checkpoint), tmp)
        os.replace(tmp, path)

    @staticmethod
    def load_checkpoint(path: str) -> MixedPrecisionCheckpoint:
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        d = torch.load(path, map_location="cpu", weights_only=False)
        known = {f.name for f in dataclasses.fields(MixedPrecisionCheckpoint)}
        return MixedPrecisionCheckpoint(**{k: v for k, v in d.items() if k in known})

    @classmethod
    def validate_checkpoint(cls, c: MixedPrecisionCheckpoint) -> bool:
        if c is None or c.version != cls.VERSION or not c.master_weights:
            return False
        if set(c.master_weights) != set(c.training_weights):
            return False
        if any(c.master_weights[k].shape != c.training_weights[k].shape for k in c.master_weights):
            return False
        if not (c.current_loss_scale > 0 and math.isfinite(c.current_loss_scale)) or c.step_count < 0 or c.skipped_steps < 0:
            return False
        return all(bool(torch.isfinite(w).all()) for w in c.master_weights.values())

    @classmethod
    def restore_checkpoint(cls, optimizer: "MixedPrecisionOptimizer", c: MixedPrecisionCheckpoint) -> None:
        if not cls.validate_checkpoint(c):
            raise ValueError("the mixed-precision checkpoint is not valid")
        missing = set(optimizer.masters) ^ set(c.master_weights)
        if missing:
            raise KeyError(f"checkpoint and optimizer disagree on parameters: {sorted(missing)[:4]}")
        optimizer.load_state_dict({"masters": c.master_weights, "scaler": c.scaler_state or
                                   {"scale": c.current_loss_scale, "tracker": c.steps_since_last_overflow,
                                    "total_steps": c.step_count, "skipped": c.total_overflows},
                                   "step_count": c.step_count, "skipped_steps": c.skipped_steps, "has_fallback": c.has_fallback,
                                   "base": c.base_optimizer_state})
        optimizer.consecutive_overflows = c.consecutive_overflows

    @classmethod
    def load_and_restore(cls, optimizer: "MixedPrecisionOptimizer", path: str) -> MixedPrecisionCheckpoint:
        c = cls.load_checkpoint(path)
        cls.restore_checkpoint(optimizer, c)
        return c
