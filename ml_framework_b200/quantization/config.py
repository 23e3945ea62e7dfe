"""Configuration-driven quantisation: settings, per-layer overrides, model traversal, static and
dynamic post-training quantisation with an accuracy guard, QAT wrappers and conversion reports,
accuracy metrics and reports, CPU feature detection.

Reference: src/MLFramework/Quantization — DataStructures/{QuantizationConfig.cs:6-162,
QuantizationType.cs, CalibrationMethod.cs}, Calibration/CalibratorFactory.cs, PTQ/{ModelTraversal.cs,
DynamicQuantization.cs:14-204, StaticQuantization.cs:15-225}, QAT/{LayerwiseConfig.cs:9-301,
QATModuleWrapper.cs:11-259, MovingAverageStatistics.cs, ModelConversion.cs:10-438},
Evaluation/{AccuracyReport.cs, AccuracyComparison.cs, AccuracyReporter.cs:9-276,
SensitivityAnalysisResult.cs, Metrics/*.cs}, Backends/{ARMBackend,x86Backend}/*FeatureDetection.cs.
"""
from __future__ import annotations

import copy
import enum
import json
import math
import platform
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .core import (Calibrator, EntropyCalibrator, FakeQuantize, MinMaxCalibrator, MovingAverageCalibrator, PercentileCalibrator,
                   PTQQuantizer, QATLinear, QuantizationMode, QuantizationParameters, QuantizedLinear, _FakeQuantSTE, compute_qparams)

__all__ = [
    "QuantizationType", "CalibrationMethod", "QuantizationConfig", "CalibratorFactory", "LayerConfigEntry", "LayerwiseConfig",
    "ModelTraversal", "StaticQuantization", "DynamicQuantization", "MovingAverageStatistics", "ObserverStatistics",
    "QATModuleWrapper", "ModelConversionReport", "ModelConversionResult", "ModelVerificationResult", "ModelConversion",
    "AccuracyMetric", "TopKAccuracy", "CrossEntropyLoss", "MAE", "RMSE", "SensitivityAnalysisResult", "AccuracyReport",
    "AccuracyComparison", "ReportFormat", "AccuracyReporter", "X86FeatureDetection", "ARMFeatureDetection",
]


class QuantizationType(enum.Enum):
    INT8 = "int8"
    UINT8 = "uint8"

    def range(self) -> Tuple[int, int]:
        return (-128, 127) if self is QuantizationType.INT8 else (0, 255)


class CalibrationMethod(enum.Enum):
    MIN_MAX = "min_max"
    ENTROPY = "entropy"
    PERCENTILE = "percentile"
    MOVING_AVERAGE = "moving_average"


@dataclass
class QuantizationConfig:
    weight_quantization: QuantizationMode = QuantizationMode.SYMMETRIC
    activation_quantization: QuantizationMode = QuantizationMode.SYMMETRIC
    calibration_method: CalibrationMethod = CalibrationMethod.MIN_MAX
    calibration_batch_size: int = 32
    quantization_type: QuantizationType = QuantizationType.INT8
    fallback_to_fp32: bool = True            # a layer whose quantisation costs more than the threshold stays fp32
    accuracy_threshold: float = 0.01
    enable_per_channel_quantization: bool = True
    enable_mixed_precision: bool = False

    def validate(self) -> bool:
        if self.calibration_batch_size <= 0:
            raise ValueError("calibration_batch_size must be positive")
        if not 0.0 <= self.accuracy_threshold <= 1.0:
            raise ValueError("accuracy_threshold must lie in [0, 1]")
        if self.quantization_type is QuantizationType.UINT8 and self.activation_quantization is QuantizationMode.SYMMETRIC:
            raise ValueError("unsigned 8-bit activations need the asymmetric mode")
        return True

    @classmethod
    def create_default(cls):
        return cls()

    @classmethod
    def create_aggressive(cls):
        """Everything quantised, tolerance 5 %, entropy calibration."""
        return cls(calibration_method=CalibrationMethod.ENTROPY, fallback_to_fp32=False, accuracy_threshold=0.05,
                   enable_mixed_precision=False)

    @classmethod
    def create_conservative(cls):
        """Percentile ranges, asymmetric activations, tolerance 0.5 %, sensitive layers kept in fp32."""
        return cls(activation_quantization=QuantizationMode.ASYMMETRIC, calibration_method=CalibrationMethod.PERCENTILE,
                   calibration_batch_size=64, fallback_to_fp32=True, accuracy_threshold=0.005, enable_mixed_precision=True)

    def __str__(self):
        return (f"QuantizationConfig(w={self.weight_quantization.value}, a={self.activation_quantization.value}, "
                f"cal={self.calibration_method.value}, type={self.quantization_type.value}, threshold={self.accuracy_threshold})")


class CalibratorFactory:
    def create(self, method: CalibrationMethod, **kw) -> Calibrator:
        if method is CalibrationMethod.MIN_MAX:
            return MinMaxCalibrator()
        if method is CalibrationMethod.ENTROPY:
            return EntropyCalibrator(**kw)
        if method is CalibrationMethod.PERCENTILE:
            return PercentileCalibrator(kw.get("percentile", 99.9))
        if method is CalibrationMethod.MOVING_AVERAGE:
            return MovingAverageCalibrator(kw.get("momentum", 0.9))
        raise ValueError(f"unknown calibration method {method!r}")

    def create_percentile(self, percentile: float) -> Calibrator:
        if not 50.0 < percentile <= 100.0:
            raise ValueError("the percentile must lie in (50, 100]")
        return PercentileCalibrator(percentile)

    def create_moving_average(self, momentum: float = 0.9) -> Calibrator:
        return MovingAverageCalibrator(momentum)


# ------------------------------------------------------------------ per-layer configuration
@dataclass
class LayerConfigEntry:
    layer_name: str
    config: QuantizationConfig
    enabled: bool = True

    def __str__(self):
        return f"{self.layer_name}: {'on' if self.enabled else 'off'}, {self.config}"


class LayerwiseConfig:
    """A global configuration with per-layer overrides and switches (LayerwiseConfig.cs:9-301)."""

    def __init__(self, global_config: Optional[QuantizationConfig] = None):
        self.global_config = global_config or QuantizationConfig.create_default()
        self.layer_configs: Dict[str, LayerConfigEntry] = {}

    @property
    def configured_layers(self) -> List[str]:
        return list(self.layer_configs)

    def set_layer_config(self, layer_name: str, config: QuantizationConfig, enabled: bool = True):
        if not layer_name:
            raise ValueError("the layer name is required")
        if config is None:
            raise ValueError("the configuration is required")
        self.layer_configs[layer_name] = LayerConfigEntry(layer_name, config, enabled)

    def get_layer_config(self, layer_name: str) -> Optional[LayerConfigEntry]:
        return self.layer_configs.get(layer_name)

    def get_effective_config(self, layer_name: str) -> QuantizationConfig:
        e = self.layer_configs.get(layer_name)
        return e.config if e is not None else self.global_config

    def is_layer_enabled(self, layer_name: str) -> bool:
        e = self.layer_configs.get(layer_name)
        return True if e is None else e.enabled

    def _entry(self, layer_name: str) -> LayerConfigEntry:
        if layer_name not in self.layer_configs:
            self.layer_configs[layer_name] = LayerConfigEntry(layer_name, copy.deepcopy(self.global_config), True)
        return self.layer_configs[layer_name]

    def disable_layer(self, layer_name: str):
        self._entry(layer_name).enabled = False

    def enable_layer(self, layer_name: str):
        self._entry(layer_name).enabled = True

    def set_layer_mode(self, layer_name: str, weight_mode: QuantizationMode, activation_mode: QuantizationMode):
        e = self._entry(layer_name)
        e.config.weight_quantization, e.config.activation_quantization = weight_mode, activation_mode

    def remove_layer_config(self, layer_name: str) -> bool:
        return self.layer_configs.pop(layer_name, None) is not None

    def clear_all_layer_configs(self):
        self.layer_configs.clear()

    def get_layer_configuration_dictionary(self) -> Dict[str, QuantizationConfig]:
        return {k: e.config for k, e in self.layer_configs.items() if e.enabled}

    def get_disabled_layers(self) -> List[str]:
        return [k for k, e in self.layer_configs.items() if not e.enabled]

    def get_enabled_layers(self) -> List[str]:
        return [k for k, e in self.layer_configs.items() if e.enabled]

    def validate(self) -> bool:
        self.global_config.validate()
        for e in self.layer_configs.values():
            e.config.validate()
        return True

    def clone(self) -> "LayerwiseConfig":
        return copy.deepcopy(self)


# ------------------------------------------------------------------ model traversal
class ModelTraversal:
    """Which layers of a model can be quantised, and how (ModelTraversal.cs)."""

    QUANTIZABLE = (nn.Linear, nn.Conv1d, nn.Conv2d)
    PER_CHANNEL = (nn.Linear, nn.Conv1d, nn.Conv2d)
    IMPLEMENTED = (nn.Linear,)              # kinds this package has an integer kernel path for

    def get_all_layers(self, model: nn.Module) -> List[Tuple[str, nn.Module]]:
        return [(n, m) for n, m in model.named_modules() if n and not list(m.children())]

    def get_quantizable_layers(self, model: nn.Module, implemented_only: bool = True) -> List[Tuple[str, nn.Module]]:
        kinds = self.IMPLEMENTED if implemented_only else self.QUANTIZABLE
        return [(n, m) for n, m in self.get_all_layers(model) if isinstance(m, kinds)]

    @staticmethod
    def get_layer_name(model: nn.Module, layer: nn.Module) -> str:
        for n, m in model.named_modules():
            if m is layer:
                return n
        raise KeyError("the layer is not part of the model")

    def is_quantizable(self, layer: nn.Module) -> bool:
        return isinstance(layer, self.QUANTIZABLE)

    def supports_per_channel_quantization(self, layer: nn.Module) -> bool:
        return isinstance(layer, self.PER_CHANNEL)


def _forward(model, batch, forward):
    return forward(model, batch) if forward else model(batch)


class _ConfiguredPTQ:
    def __init__(self, traversal: Optional[ModelTraversal] = None, calibrator_factory: Optional[CalibratorFactory] = None):
        self.traversal, self.factory = traversal or ModelTraversal(), calibrator_factory or CalibratorFactory()
        self.skipped_layers: List[str] = []
        self.fallback_layers: List[str] = []
        self.quantized_layers: List[str] = []

    def _targets(self, model, config: QuantizationConfig, layers: Optional[LayerwiseConfig]):
        self.skipped_layers, self.fallback_layers, self.quantized_layers = [], [], []
        out = []
        for n, m in self.traversal.get_quantizable_layers(model):
            if layers is not None and not layers.is_layer_enabled(n):
                self.skipped_layers.append(n)
                continue
            out.append((n, m, layers.get_effective_config(n) if layers is not None else config))
        return out

    def _guard(self, model, name, original, quantized, cfg: QuantizationConfig, metric, baseline):
        """Swaps ``quantized`` in; swaps back when the metric drops by more than the layer's threshold."""
        PTQQuantizer._swap(model, name, quantized)
        if metric is None or not cfg.fallback_to_fp32:
            self.quantized_layers.append(name)
            return
        if baseline - metric(model) > cfg.accuracy_threshold:
            PTQQuantizer._swap(model, name, original)
            self.fallback_layers.append(name)
        else:
            self.quantized_layers.append(name)


class StaticQuantization(_ConfiguredPTQ):
    """Calibrates activation ranges on data, then swaps each enabled layer for its integer form; with a
    ``metric`` (higher is better) a layer that costs more than its threshold goes back to fp32."""

    def quantize(self, model: nn.Module, calibration_batches: Iterable, config: Optional[QuantizationConfig] = None,
                 layerwise: Optional[LayerwiseConfig] = None, forward: Optional[Callable] = None,
                 metric: Optional[Callable[[nn.Module], float]] = None) -> nn.Module:
        config = config or (layerwise.global_config if layerwise else QuantizationConfig.create_default())
        (layerwise.validate() if layerwise else config.validate())
        targets = self._targets(model, config, layerwise)
        cals: Dict[str, Calibrator] = {}
        hooks = []
        for n, m, cfg in targets:
            cals[n] = self.factory.create(cfg.calibration_method)
            hooks.append(m.register_forward_pre_hook(lambda mod, inp, n=n: cals[n].observe(inp[0])))
        model.eval()
        seen = 0
        with torch.no_grad():
            for b in calibration_batches:
                _forward(model, b, forward)
                seen += 1
        for h in hooks:
            h.remove()
        if targets and seen == 0:
            raise ValueError("static quantisation needs at least one calibration batch")
        baseline = metric(model) if metric is not None else None
        for n, m, cfg in targets:
            lo, hi = cfg.quantization_type.range()
            qp = cals[n].qparams(cfg.activation_quantization, lo, hi)
            self._guard(model, n, m, QuantizedLinear(m, qp), cfg, metric, baseline)
        return model


class DynamicQuantization(_ConfiguredPTQ):
    """Integer weights now, activation ranges measured per call: no calibration data."""

    def quantize(self, model: nn.Module, config: Optional[QuantizationConfig] = None, layerwise: Optional[LayerwiseConfig] = None,
                 metric: Optional[Callable[[nn.Module], float]] = None) -> nn.Module:
        config = config or (layerwise.global_config if layerwise else QuantizationConfig.create_default())
        (layerwise.validate() if layerwise else config.validate())
        model.eval()
        baseline = metric(model) if metric is not None else None
        for n, m, cfg in self._targets(model, config, layerwise):
            self._guard(model, n, m, QuantizedLinear(m, None), cfg, metric, baseline)
        return model


# ------------------------------------------------------------------ QAT wrapper and conversion
class MovingAverageStatistics:
    """Exponential moving mean with exact extremes and variance (MovingAverageStatistics.cs)."""

    def __init__(self, momentum: float = 0.9):
        if not 0.0 <= momentum < 1.0:
            raise ValueError("momentum must lie in [0, 1)")
        self.momentum = momentum
        self.reset()

    def reset(self):
        self.mean, self.min, self.max = 0.0, math.inf, -math.inf
        self._sum = self._sum_sq = 0.0
        self.count = 0

    def update(self, value: float):
        v = float(value)
        self.mean = v if self.count == 0 else self.momentum * self.mean + (1 - self.momentum) * v
        self.min, self.max = min(self.min, v), max(self.max, v)
        self._sum += v
        self._sum_sq += v * v
        self.count += 1

    def update_batch(self, values: Iterable[float]):
        for v in values:
            self.update(v)

    def update_tensor(self, t: torch.Tensor):
        """One step per tensor: its mean feeds the moving mean, its elements the extremes and the variance."""
        x = t.detach().float()
        if not x.numel():
            return
        m = float(x.mean())
        self.mean = m if self.count == 0 else self.momentum * self.mean + (1 - self.momentum) * m
        self.min, self.max = min(self.min, float(x.min())), max(self.max, float(x.max()))
        self._sum += float(x.sum())
        self._sum_sq += float((x * x).sum())
        self.count += x.numel()

    @property
    def variance(self) -> float:
        if not self.count:
            return 0.0
        mu = self._sum / self.count
        return max(0.0, self._sum_sq / self.count - mu * mu)

    def get_statistics(self) -> Dict[str, float]:
        return {"mean": self.mean, "min": self.min, "max": self.max, "variance": self.variance, "count": self.count}


@dataclass
class ObserverStatistics:
    min: float
    max: float
    mean: float
    variance: float
    count: int


class QATModuleWrapper(nn.Module):
    """Any layer with a weight, trained through fake quantisation of its weight and of its input; keeps
    observer statistics of both (QATModuleWrapper.cs:11-259)."""

    def __init__(self, module: nn.Module, config: Optional[QuantizationConfig] = None, momentum: float = 0.9):
        super().__init__()
        if not hasattr(module, "weight") or module.weight is None:
            raise ValueError(f"{type(module).__name__} has no weight to quantise")
        self.wrapped_module = module
        self.config = config or QuantizationConfig.create_default()
        lo, hi = self.config.quantization_type.range()
        self.act_fq = FakeQuantize(self.config.activation_quantization, momentum, lo, hi)
        self._w_stats, self._a_stats = MovingAverageStatistics(momentum), MovingAverageStatistics(momentum)
        self.weight_quantization_parameters: Optional[QuantizationParameters] = None

    @property
    def activation_quantization_parameters(self) -> Optional[QuantizationParameters]:
        c = self.act_fq.cal
        return c.qparams(self.act_fq.mode, self.act_fq.qmin, self.act_fq.qmax) if c.lo is not None else None

    def _weight_qparams(self, w: torch.Tensor) -> QuantizationParameters:
        flat = w.detach().float().reshape(w.shape[0], -1)
        if self.config.enable_per_channel_quantization:
            return compute_qparams(flat.amin(1), flat.amax(1), self.config.weight_quantization, axis=0)
        return compute_qparams(flat.min(), flat.max(), self.config.weight_quantization)

    def forward(self, x):
        if self.training:
            self._a_stats.update_tensor(x)
            self._w_stats.update_tensor(self.wrapped_module.weight)
        x = self.act_fq(x)
        w = self.wrapped_module.weight
        qp = self._weight_qparams(w)
        self.weight_quantization_parameters = qp
        wq = _FakeQuantSTE.apply(w.reshape(w.shape[0], -1), qp).view_as(w)
        m = self.wrapped_module
        if isinstance(m, nn.Linear):
            return F.linear(x, wq, m.bias)
        if isinstance(m, nn.Conv2d):
            return F.conv2d(x, wq, m.bias, m.stride, m.padding, m.dilation, m.groups)
        if isinstance(m, nn.Conv1d):
            return F.conv1d(x, wq, m.bias, m.stride, m.padding, m.dilation, m.groups)
        raise TypeError(f"no fake-quantised forward for {type(m).__name__}")

    def quantize_weights(self) -> Tuple[torch.Tensor, QuantizationParameters]:
        """The integer weight and its parameters as conversion will use them."""
        from .core import quantize
        w = self.wrapped_module.weight.detach()
        qp = self._weight_qparams(w)
        self.weight_quantization_parameters = qp
        return quantize(w.reshape(w.shape[0], -1).contiguous(), qp).view_as(w), qp

    @staticmethod
    def _stats(s: MovingAverageStatistics) -> Optional[ObserverStatistics]:
        return ObserverStatistics(s.min, s.max, s.mean, s.variance, s.count) if s.count else None

    def get_activation_observer_statistics(self) -> Optional[ObserverStatistics]:
        return self._stats(self._a_stats)

    def get_weight_observer_statistics(self) -> Optional[ObserverStatistics]:
        return self._stats(self._w_stats)

    def reset_observers(self):
        self._a_stats.reset(); self._w_stats.reset()
        self.act_fq.cal = MovingAverageCalibrator(self.act_fq.cal.momentum if hasattr(self.act_fq.cal, "momentum") else 0.9)

    def has_fake_quantization_nodes(self) -> bool:
        return True

    def get_fake_quantization_node_count(self) -> int:
        return 2                                          # weight and input


@dataclass
class ModelConversionReport:
    start_time: float = 0.0
    end_time: float = 0.0
    source_layer_count: int = 0
    source_fake_quant_nodes: int = 0
    quantized_layers: int = 0
    weight_scale_range: Tuple[float, float] = (0.0, 0.0)
    activation_scale_range: Tuple[float, float] = (0.0, 0.0)
    success: bool = False
    error_message: Optional[str] = None

    @property
    def duration_s(self) -> float:
        return self.end_time - self.start_time


@dataclass
class ModelConversionResult:
    quantized_model: Optional[nn.Module]
    report: ModelConversionReport


@dataclass
class ModelVerificationResult:
    start_time: float = 0.0
    end_time: float = 0.0
    passed_checks: List[str] = field(default_factory=list)
    failed_checks: List[str] = field(default_factory=list)
    success: bool = False
    error_message: Optional[str] = None

    @property
    def duration_s(self) -> float:
        return self.end_time - self.start_time


class ModelConversion:
    """From a trained QAT model to the integer model, with a report, and checks of the result
    (ModelConversion.cs:10-438)."""

    @staticmethod
    def _qat_layers(model: nn.Module):
        return [(n, m) for n, m in model.named_modules() if isinstance(m, (QATLinear, QATModuleWrapper))]

    @classmethod
    def extract_trained_parameters(cls, qat_model: nn.Module) -> Dict[str, Optional[QuantizationParameters]]:
        """The learned activation parameters per QAT layer (``None`` where the observer saw no data)."""
        out: Dict[str, Optional[QuantizationParameters]] = {}
        for n, m in cls._qat_layers(qat_model):
            fq = m.act_fq
            out[n] = fq.cal.qparams(fq.mode, fq.qmin, fq.qmax) if fq.cal.lo is not None else None
        return out

    @classmethod
    def convert_to_quantized(cls, qat_model: nn.Module) -> nn.Module:
        res = cls.convert_with_report(qat_model)
        if not res.report.success:
            raise RuntimeError(f"conversion failed: {res.report.error_message}")
        return res.quantized_model

    @classmethod
    def convert_with_report(cls, qat_model: nn.Module) -> ModelConversionResult:
        rep = ModelConversionReport(start_time=time.time())
        try:
            layers = cls._qat_layers(qat_model)
            rep.source_layer_count = sum(1 for n, m in qat_model.named_modules() if n and not list(m.children()))
            rep.source_fake_quant_nodes = sum(2 for _ in layers)
            if not layers:
                raise ValueError("the model has no QAT layers: prepare it for QAT first")
            params = cls.extract_trained_parameters(qat_model)
            model = copy.deepcopy(qat_model)
            w_scales, a_scales = [], []
            for n, m in cls._qat_layers(model):
                inner = m.linear if isinstance(m, QATLinear) else m.wrapped_module
                if not isinstance(inner, nn.Linear):
                    continue                              # stays a fake-quantised float layer: no integer kernel for it
                q = QuantizedLinear(inner, params[n])
                PTQQuantizer._swap(model, n, q)
                rep.quantized_layers += 1
                w_scales += [float(q.w_scale.min()), float(q.w_scale.max())]
                if params[n] is not None:
                    a_scales.append(float(params[n].scale.reshape(-1)[0]))
            if w_scales:
                rep.weight_scale_range = (min(w_scales), max(w_scales))
            if a_scales:
                rep.activation_scale_range = (min(a_scales), max(a_scales))
            rep.success = rep.quantized_layers > 0
            if not rep.success:
                rep.error_message = "no QAT layer had an integer form"
            rep.end_time = time.time()
            return ModelConversionResult(model.eval() if rep.success else None, rep)
        except Exception as e:                           # noqa: BLE001 - the report carries the failure
            rep.success, rep.error_message, rep.end_time = False, str(e), time.time()
            return ModelConversionResult(None, rep)

    @staticmethod
    def verify_quantized_model(quantized: nn.Module, reference: Optional[nn.Module] = None, sample: Optional[torch.Tensor] = None,
                               min_sqnr_db: float = 15.0) -> ModelVerificationResult:
        r = ModelVerificationResult(start_time=time.time())

        def check(name: str, ok: bool):
            (r.passed_checks if ok else r.failed_checks).append(name)
        try:
            qs = [m for m in quantized.modules() if isinstance(m, QuantizedLinear)]
            check("has quantized layers", bool(qs))
            check("no fake-quantisation nodes left in converted layers", not any(isinstance(m, QATLinear) for m in quantized.modules()))
            check("weights are int8", all(m.w_q.dtype == torch.int8 for m in qs))
            check("weight scales are positive and finite", all(bool((m.w_scale > 0).all() and torch.isfinite(m.w_scale).all()) for m in qs))
            check("activation parameters are finite", all(m.act_qparams is None or bool(torch.isfinite(m.act_qparams.scale).all()) for m in qs))
            if sample is not None:
                with torch.no_grad():
                    y = quantized(sample)
                check("output is finite", bool(torch.isfinite(y.float()).all()))
                if reference is not None:
                    from .core import sqnr_db
                    with torch.no_grad():
                        ref = reference(sample)
                    check(f"output within {min_sqnr_db:g} dB of the reference", sqnr_db(ref.float(), y.float()) >= min_sqnr_db)
            r.success = not r.failed_checks
        except Exception as e:                           # noqa: BLE001
            r.success, r.error_message = False, str(e)
        r.end_time = time.time()
        return r


# ------------------------------------------------------------------ metrics and accuracy reports
class AccuracyMetric:
    """Accumulates over batches: ``update(prediction, target)``, ``compute()``, ``reset()``."""

    name = "metric"
    higher_is_better = True

    def __init__(self):
        self.reset()

    def reset(self):
        self._num, self._den = 0.0, 0

    def compute(self) -> float:
        return self._num / self._den if self._den else 0.0

    def update(self, prediction: torch.Tensor, target: torch.Tensor) -> None:
        raise NotImplementedError


class TopKAccuracy(AccuracyMetric):
    def __init__(self, k: int = 1):
        if k <= 0:
            raise ValueError("k must be positive")
        self.k, self.name = k, f"top{k}_accuracy"
        super().__init__()

    def update(self, prediction, target):
        top = prediction.reshape(-1, prediction.shape[-1]).topk(min(self.k, prediction.shape[-1]), dim=-1).indices
        self._num += float((top == target.reshape(-1, 1)).any(-1).sum())
        self._den += target.numel()


class CrossEntropyLoss(AccuracyMetric):
    name, higher_is_better = "cross_entropy", False

    def update(self, prediction, target):
        self._num += float(F.cross_entropy(prediction.reshape(-1, prediction.shape[-1]).float(), target.reshape(-1), reduction="sum"))
        self._den += target.numel()


class MAE(AccuracyMetric):
    name, higher_is_better = "mae", False

    def update(self, prediction, target):
        self._num += float((prediction.float() - target.float()).abs().sum())
        self._den += target.numel()


class RMSE(AccuracyMetric):
    name, higher_is_better = "rmse", False

    def update(self, prediction, target):
        self._num += float(((prediction.float() - target.float()) ** 2).sum())
        self._den += target.numel()

    def compute(self):
        return math.sqrt(self._num / self._den) if self._den else 0.0


@dataclass
class SensitivityAnalysisResult:
    layer_name: str
    accuracy_impact: float                 # drop of the metric when only this layer is quantised
    is_sensitive: bool
    recommended_action: str = ""


@dataclass
class AccuracyReport:
    fp32_accuracy: float = 0.0
    quantized_accuracy: float = 0.0
    is_acceptable: bool = True
    acceptable_threshold: float = 0.01
    per_layer_results: List[SensitivityAnalysisResult] = field(default_factory=list)
    timestamp: float = field(default_factory=time.time)
    metadata: Dict[str, Any] = field(default_factory=dict)

    @property
    def accuracy_drop(self) -> float:
        return self.fp32_accuracy - self.quantized_accuracy

    def get_sensitive_layers(self) -> List[SensitivityAnalysisResult]:
        return [r for r in self.per_layer_results if r.is_sensitive]

    def get_recommended_fp32_layers(self) -> List[str]:
        return [r.layer_name for r in self.per_layer_results if r.is_sensitive]

    def get_quantizable_layers(self) -> List[str]:
        return [r.layer_name for r in self.per_layer_results if not r.is_sensitive]


class AccuracyComparison:
    """Evaluates the float and the quantised model on the same data with one metric, and optionally each
    layer's share by quantising one layer at a time (AccuracyComparison.cs)."""

    def __init__(self, metric: Optional[AccuracyMetric] = None, forward: Optional[Callable] = None):
        self.metric, self.forward = metric or TopKAccuracy(1), forward

    def evaluate(self, model: nn.Module, data: Iterable[Tuple[Any, torch.Tensor]]) -> float:
        self.metric.reset()
        model.eval()
        with torch.no_grad():
            for x, y in data:
                self.metric.update(_forward(model, x, self.forward), y)
        return self.metric.compute()

    def _drop(self, base: float, value: float) -> float:
        return base - value if self.metric.higher_is_better else value - base

    def compare_models(self, fp32_model: nn.Module, quantized_model: nn.Module, data: Sequence[Tuple[Any, torch.Tensor]],
                       threshold: float = 0.01, per_layer: bool = False) -> AccuracyReport:
        a, b = self.evaluate(fp32_model, data), self.evaluate(quantized_model, data)
        drop = self._drop(a, b)
        rep = AccuracyReport(a, b, drop <= threshold, threshold, metadata={"metric": self.metric.name, "batches": len(data),
                                                                             "higher_is_better": self.metric.higher_is_better})
        if not self.metric.higher_is_better:             # keep "drop = fp32 - quantised" meaningful: store negated losses
            rep.metadata["note"] = "lower is better: accuracy fields hold the metric itself, the drop is its increase"
        if per_layer:
            for n, m in ModelTraversal().get_quantizable_layers(fp32_model):
                PTQQuantizer._swap(fp32_model, n, QuantizedLinear(m, None))
                try:
                    impact = self._drop(a, self.evaluate(fp32_model, data))
                finally:
                    PTQQuantizer._swap(fp32_model, n, m)
                sens = impact > threshold
                rep.per_layer_results.append(SensitivityAnalysisResult(
                    n, impact, sens, "keep in fp32" if sens else "quantise to int8"))
            rep.per_layer_results.sort(key=lambda r: -r.accuracy_impact)
        return rep

    def get_accuracy_delta(self, report: AccuracyReport) -> float:
        return self._drop(report.fp32_accuracy, report.quantized_accuracy)

    @staticmethod
    def get_per_layer_metrics(report: AccuracyReport) -> List[SensitivityAnalysisResult]:
        return list(report.per_layer_results)


class ReportFormat(enum.Enum):
    TEXT = "text"
    JSON = "json"
    MARKDOWN = "markdown"


class AccuracyReporter:
    def generate_text_report(self, r: AccuracyReport) -> str:
        bar = "=" * 60
        drop = r.metadata.get("drop", r.accuracy_drop if r.metadata.get("higher_is_better", True) else -r.accuracy_drop)
        out = [bar, "Quantisation accuracy report", bar,
               time.strftime("Generated: %Y-%m-%d %H:%M:%S UTC", time.gmtime(r.timestamp)), "",
               f"FP32:       {r.fp32_accuracy:.4f}", f"Quantised:  {r.quantized_accuracy:.4f}",
               f"Drop:       {drop:.4f} (threshold {r.acceptable_threshold:.4f})",
               f"Result:     {'ACCEPTABLE' if r.is_acceptable else 'NOT ACCEPTABLE'}", ""]
        if r.per_layer_results:
            out.append("Per-layer sensitivity (largest first):")
            width = max(len(x.layer_name) for x in r.per_layer_results)
            for x in r.per_layer_results:
                out.append(f"  {x.layer_name:<{width}}  {x.accuracy_impact:+.4f}  {'SENSITIVE' if x.is_sensitive else 'ok':<9}  {x.recommended_action}")
            out += ["", f"Keep in fp32: {', '.join(r.get_recommended_fp32_layers()) or 'none'}",
                    f"Quantise:     {', '.join(r.get_quantizable_layers()) or 'none'}", ""]
        if r.metadata:
            out.append("Metadata:")
            out += [f"  {k}: {v}" for k, v in r.metadata.items()]
        return "\n".join(out + [bar]) + "\n"

    def generate_json_report(self, r: AccuracyReport) -> str:
        return json.dumps({
            "timestamp": r.timestamp, "fp32_accuracy": r.fp32_accuracy, "quantized_accuracy": r.quantized_accuracy,
            "accuracy_drop": r.accuracy_drop, "acceptable_threshold": r.acceptable_threshold, "is_acceptable": r.is_acceptable,
            "per_layer_results": [{"layer_name": x.layer_name, "accuracy_impact": x.accuracy_impact, "is_sensitive": x.is_sensitive,
                                   "recommended_action": x.recommended_action} for x in r.per_layer_results],
            "metadata": r.metadata, "recommended_fp32_layers": r.get_recommended_fp32_layers(),
            "quantizable_layers": r.get_quantizable_layers()}, indent=1, default=str)

    def generate_markdown_report(self, r: AccuracyReport) -> str:
        out = ["# Quantisation accuracy report", "", "| | value |", "|---|---|", f"| FP32 | {r.fp32_accuracy:.4f} |",
               f"| quantised | {r.quantized_accuracy:.4f} |", f"| drop | {r.accuracy_drop:.4f} |",
               f"| threshold | {r.acceptable_threshold:.4f} |", f"| result | {'acceptable' if r.is_acceptable else '**not acceptable**'} |", ""]
        if r.per_layer_results:
            out += ["| layer | impact | sensitive | action |", "|---|---|---|---|"]
            out += [f"| `{x.layer_name}` | {x.accuracy_impact:+.4f} | {'yes' if x.is_sensitive else 'no'} | {x.recommended_action} |"
                    for x in r.per_layer_results]
        return "\n".join(out) + "\n"

    def save_report(self, r: AccuracyReport, path: str, format: ReportFormat = ReportFormat.TEXT) -> None:
        text = {ReportFormat.TEXT: self.generate_text_report, ReportFormat.JSON: self.generate_json_report,
                ReportFormat.MARKDOWN: self.generate_markdown_report}[format](r)
        with open(path, "w") as f:
            f.write(text)


# ------------------------------------------------------------------ CPU feature detection
def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith(("flags", "features")):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


class X86FeatureDetection:
    """Instruction-set extensions that matter for 8-bit arithmetic on x86 hosts."""

    FEATURES = ("sse4_1", "avx", "avx2", "avx512f", "avx512bw", "avx512_vnni", "avx_vnni", "amx_int8")

    @staticmethod
    def is_available() -> bool:
        return platform.machine().lower() in ("x86_64", "amd64", "i386", "i686")

    @classmethod
    def get_detected_features(cls, flags: Optional[set] = None) -> List[str]:
        flags = _cpu_flags() if flags is None else flags
        return [f for f in cls.FEATURES if f in flags]

    @classmethod
    def has_int8_dot_product(cls, flags: Optional[set] = None) -> bool:
        f = set(cls.get_detected_features(flags))
        return bool(f & {"avx512_vnni", "avx_vnni", "amx_int8"})


class ARMFeatureDetection:
    FEATURES = ("asimd", "neon", "asimddp", "i8mm", "sve", "sve2")

    @staticmethod
    def is_available() -> bool:
        return platform.machine().lower() in ("aarch64", "arm64", "armv7l", "armv8l")

    @classmethod
    def get_detected_features(cls, flags: Optional[set] = None) -> List[str]:
        flags = _cpu_flags() if flags is None else flags
        return [f for f in cls.FEATURES if f in flags]

    @classmethod
    def has_int8_dot_product(cls, flags: Optional[set] = None) -> bool:
        f = set(cls.get_detected_features(flags))
        return bool(f & {"asimddp", "i8mm"})
