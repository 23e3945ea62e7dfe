"""Quantisation workflows around the core operators: calibration process, evaluation and reports, QAT training
integration and checkpointing, per-layer sensitivity with a mixed-precision plan.

Reference (src/MLFramework/Quantization/): PTQ/CalibrationProcess.cs, PTQ/SensitivityAnalysis.cs,
QAT/{QATPreparer, ModelPreparation, ModelConversion, QATCheckpointing, TrainingIntegration}.cs,
Evaluation/* (top-k / MAE / RMSE / cross-entropy metrics, per-layer sensitivity, regression detector, reports),
Operations/PerChannelOperations.cs.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .core import (Calibrator, FakeQuantize, MinMaxCalibrator, PTQQuantizer, QuantizationMode, QuantizationParameters, QuantizedLinear, compute_qparams, dequantize, mae, quantize, rmse, sqnr_db, top_k_accuracy)


# ------------------------------------------------------------------ per-channel helpers
class PerChannelOperations:
    """Per-channel parameters and round trips for weight tensors of any rank (channel axis 0 by default)."""

    @staticmethod
    def qparams(w: torch.Tensor, axis: int = 0, mode: QuantizationMode = QuantizationMode.SYMMETRIC, qmin: int = -128, qmax: int = 127) -> QuantizationParameters:
        w2 = w.detach().float().movedim(axis, 0).reshape(w.shape[axis], -1)
        return compute_qparams(w2.amin(1), w2.amax(1), mode, qmin, qmax, axis=0)

    @staticmethod
    def quantize(w: torch.Tensor, qp: QuantizationParameters, axis: int = 0) -> torch.Tensor:
        w2 = w.detach().movedim(axis, 0)
        q = quantize(w2.reshape(w2.shape[0], -1).contiguous(), qp)
        return q.reshape(w2.shape).movedim(0, axis).contiguous()

    @staticmethod
    def dequantize(q: torch.Tensor, qp: QuantizationParameters, axis: int = 0, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        q2 = q.movedim(axis, 0)
        x = dequantize(q2.reshape(q2.shape[0], -1).contiguous(), qp, dtype)
        return x.reshape(q2.shape).movedim(0, axis).contiguous()

    @staticmethod
    def error(w: torch.Tensor, axis: int = 0) -> Dict[str, float]:
        """Round-trip error of per-channel against per-tensor quantisation of the same tensor."""
        w = w.detach()
        qp_c = PerChannelOperations.qparams(w, axis)
        rc = PerChannelOperations.dequantize(PerChannelOperations.quantize(w, qp_c, axis), qp_c, axis)
        lo, hi = w.detach().float().min(), w.detach().float().max()
        qp_t = compute_qparams(lo, hi)
        rt = dequantize(quantize(w.detach().reshape(1, -1).contiguous(), qp_t), qp_t).reshape(w.shape)
        return {"per_channel_sqnr_db": sqnr_db(w, rc), "per_tensor_sqnr_db": sqnr_db(w, rt), "per_channel_rmse": rmse(w, rc), "per_tensor_rmse": rmse(w, rt)}


# ------------------------------------------------------------------ calibration process
@dataclass
class CalibrationResult:
    batches: int
    samples: int
    ranges: Dict[str, Tuple[float, float]]
    converged: bool


class CalibrationProcess:
    """Feeds calibration batches through a model with observers on every Linear input, stops when ``max_batches`` is
    reached or the observed ranges moved by less than ``tolerance`` (relative) over ``patience`` batches."""

    def __init__(self, calibrator_factory: Callable[[], Calibrator] = MinMaxCalibrator, max_batches: int = 100, tolerance: float = 0.0,
                 patience: int = 3, skip: Sequence[str] = ()):
        self.quantizer = PTQQuantizer(calibrator_factory, skip)
        self.max_batches, self.tolerance, self.patience = max_batches, tolerance, patience

    def run(self, model: nn.Module, batches: Iterable, forward: Optional[Callable] = None) -> Tuple[Dict[str, Calibrator], CalibrationResult]:
        targets = self.quantizer._targets(model)
        cals = {n: self.quantizer.factory() for n, _ in targets}
        hooks = [m.register_forward_pre_hook(lambda mod, inp, c=cals[n]: c.observe(inp[0].detach())) for n, m in targets]
        fwd = forward or (lambda mdl, b: mdl(b[0] if isinstance(b, (tuple, list)) else b))
        nb = ns = still = 0
        prev: Dict[str, Tuple[float, float]] = {}
        converged = False
        was_training = model.training
        model.eval()
        try:
            with torch.no_grad():
                for b in batches:
                    if nb >= self.max_batches:
                        break
                    fwd(model, b)
                    nb += 1
                    x = b[0] if isinstance(b, (tuple, list)) else b
                    ns += int(x.shape[0]) if isinstance(x, torch.Tensor) and x.dim() else 1
                    cur = {n: tuple(float(v.reshape(-1).abs().max()) for v in c.range()) for n, c in cals.items()}
                    if self.tolerance > 0 and prev:
                        moved = max(abs(cur[n][i] - prev[n][i]) / max(abs(prev[n][i]), 1e-12) for n in cur for i in (0, 1))
                        still = still + 1 if moved < self.tolerance else 0
                        if still >= self.patience:
                            converged = True
                            break
                    prev = cur
        finally:
            for h in hooks:
                h.remove()
            model.train(was_training)
        ranges = {n: tuple(float(v.reshape(-1)[0]) for v in c.range()) for n, c in cals.items()} if nb else {}
        return cals, CalibrationResult(nb, ns, ranges, converged)

    def quantize(self, model: nn.Module, batches: Iterable, forward: Optional[Callable] = None) -> Tuple[nn.Module, CalibrationResult]:
        cals, res = self.run(model, batches, forward)
        for n, m in self.quantizer._targets(model):
            PTQQuantizer._swap(model, n, QuantizedLinear(m, cals[n].qparams()))
        return model, res


# ------------------------------------------------------------------ evaluation
@dataclass
class EvaluationMetrics:
    top1: Optional[float] = None
    top5: Optional[float] = None
    cross_entropy: Optional[float] = None
    mae_vs_reference: Optional[float] = None
    rmse_vs_reference: Optional[float] = None
    sqnr_db: Optional[float] = None
    samples: int = 0


class ModelEvaluator:
    """Runs a model over ``(inputs, targets)`` batches; with a reference model also measures output drift."""

    def evaluate(self, model: nn.Module, batches: Iterable, reference: Optional[nn.Module] = None) -> EvaluationMetrics:
        n = 0
        c1 = c5 = ce = 0.0
        outs, refs = [], []
        have_targets = True
        model.eval()
        with torch.no_grad():
            for b in batches:
                x, y = (b[0], b[1]) if isinstance(b, (tuple, list)) and len(b) > 1 else (b[0] if isinstance(b, (tuple, list)) else b, None)
                out = model(x).float()
                if reference is not None:
                    outs.append(out)
                    refs.append(reference(x).float())
                bs = out.shape[0]
                if y is not None and out.dim() == 2:
                    c1 += top_k_accuracy(out, y, 1) * bs
                    c5 += top_k_accuracy(out, y, min(5, out.shape[-1])) * bs
                    ce += float(F.cross_entropy(out, y, reduction="sum"))
                else:
                    have_targets = False
                n += bs
        m = EvaluationMetrics(samples=n)
        if have_targets and n:
            m.top1, m.top5, m.cross_entropy = c1 / n, c5 / n, ce / n
        if outs:
            o, r = torch.cat(outs), torch.cat(refs)
            m.mae_vs_reference, m.rmse_vs_reference, m.sqnr_db = mae(o, r), rmse(o, r), sqnr_db(r, o)
        return m


@dataclass
class RegressionThresholds:
    max_top1_drop: float = 0.01
    max_ce_increase: float = 0.05
    min_sqnr_db: float = 20.0


@dataclass
class RegressionFinding:
    metric: str
    baseline: Optional[float]          # None for metrics that have no baseline value (drift of the quantised output)
    quantized: float
    limit: float


class RegressionDetector:
    def __init__(self, thresholds: Optional[RegressionThresholds] = None):
        self.t = thresholds or RegressionThresholds()

    def check(self, baseline: EvaluationMetrics, quantized: EvaluationMetrics) -> List[RegressionFinding]:
        out = []
        if baseline.top1 is not None and quantized.top1 is not None and baseline.top1 - quantized.top1 > self.t.max_top1_drop:
            out.append(RegressionFinding("top1", baseline.top1, quantized.top1, self.t.max_top1_drop))
        if baseline.cross_entropy is not None and quantized.cross_entropy is not None and quantized.cross_entropy - baseline.cross_entropy > self.t.max_ce_increase:
            out.append(RegressionFinding("cross_entropy", baseline.cross_entropy, quantized.cross_entropy, self.t.max_ce_increase))
        if quantized.sqnr_db is not None and quantized.sqnr_db < self.t.min_sqnr_db:
            out.append(RegressionFinding("sqnr_db", None, quantized.sqnr_db, self.t.min_sqnr_db))
        return out


def model_bytes(model: nn.Module) -> int:
    seen, n = set(), 0
    for t in list(model.parameters()) + list(model.buffers()):
        if id(t) not in seen:
            seen.add(id(t))
            n += t.numel() * t.element_size()
    return n


@dataclass
class LayerSensitivity:
    layer: str
    metric_drop: float
    weight_sqnr_db: float
    parameters: int


@dataclass
class MixedPrecisionPlan:
    quantize: List[str]
    keep_full_precision: List[str]
    estimated_drop: float


class PerLayerSensitivityAnalyzer:
    """Quantises one Linear at a time, measures what the metric loses, and plans which layers to leave in full
    precision so that the summed loss stays within a budget (largest layers are quantised first: most bytes saved per
    unit of metric lost)."""

    def analyze(self, model: nn.Module, metric: Callable[[nn.Module], float]) -> List[LayerSensitivity]:
        base = metric(model)
        out = []
        for n, m in [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear)]:
            PTQQuantizer._swap(model, n, QuantizedLinear(m, None))
            drop = base - metric(model)
            PTQQuantizer._swap(model, n, m)
            out.append(LayerSensitivity(n, drop, PerChannelOperations.error(m.weight)["per_channel_sqnr_db"], m.weight.numel()))
        return sorted(out, key=lambda s: -s.metric_drop)

    @staticmethod
    def plan(sens: Sequence[LayerSensitivity], max_total_drop: float) -> MixedPrecisionPlan:
        order = sorted(sens, key=lambda s: (max(s.metric_drop, 0.0) / max(s.parameters, 1), -s.parameters))
        total, q, keep = 0.0, [], []
        for s in order:
            d = max(s.metric_drop, 0.0)
            if total + d <= max_total_drop:
                q.append(s.layer)
                total += d
            else:
                keep.append(s.layer)
        return MixedPrecisionPlan(q, keep, total)


@dataclass
class QuantizationReport:
    model_name: str
    baseline: EvaluationMetrics
    quantized: EvaluationMetrics
    baseline_bytes: int
    quantized_bytes: int
    regressions: List[RegressionFinding] = field(default_factory=list)
    sensitivity: List[LayerSensitivity] = field(default_factory=list)

    @property
    def compression_ratio(self) -> float:
        return self.baseline_bytes / self.quantized_bytes if self.quantized_bytes else 0.0

    def to_json(self) -> str:
        d = asdict(self)
        d["compression_ratio"] = self.compression_ratio
        return json.dumps(d, indent=1)

    def to_markdown(self) -> str:
        f = lambda v: "-" if v is None else f"{v:.4f}"      # noqa: E731
        lines = [f"# Quantisation report: {self.model_name}", "",
                 f"size {self.baseline_bytes / 2**20:.2f} MiB -> {self.quantized_bytes / 2**20:.2f} MiB ({self.compression_ratio:.2f}x)", "",
                 "| metric | baseline | quantised |", "|---|---|---|",
                 f"| top-1 | {f(self.baseline.top1)} | {f(self.quantized.top1)} |", f"| top-5 | {f(self.baseline.top5)} | {f(self.quantized.top5)} |",
                 f"| cross-entropy | {f(self.baseline.cross_entropy)} | {f(self.quantized.cross_entropy)} |",
                 f"| output SQNR (dB) | - | {f(self.quantized.sqnr_db)} |", ""]
        lines.append("regressions: " + (", ".join(f"{r.metric} ({f(r.baseline)} -> {r.quantized:.4f}, limit {r.limit})" for r in self.regressions) or "none"))
        if self.sensitivity:
            lines += ["", "| layer | metric drop | weight SQNR (dB) | parameters |", "|---|---|---|---|"]
            lines += [f"| {s.layer} | {s.metric_drop:.4f} | {s.weight_sqnr_db:.1f} | {s.parameters} |" for s in self.sensitivity]
        return "\n".join(lines) + "\n"


def build_report(name: str, fp_model: nn.Module, q_model: nn.Module, batches: Sequence, thresholds: Optional[RegressionThresholds] = None,
                 sensitivity: Sequence[LayerSensitivity] = ()) -> QuantizationReport:
    ev = ModelEvaluator()
    base = ev.evaluate(fp_model, batches)
    quant = ev.evaluate(q_model, batches, reference=fp_model)
    return QuantizationReport(name, base, quant, model_bytes(fp_model), model_bytes(q_model), RegressionDetector(thresholds).check(base, quant), list(sensitivity))


# ------------------------------------------------------------------ QAT integration
@dataclass
class QATSchedule:
    observer_warmup_steps: int = 0        # fake-quant off, observers collecting
    freeze_observers_after: Optional[int] = None      # ranges fixed from this step on
    freeze_batchnorm_after: Optional[int] = None


class QATTrainingIntegration:
    """Step-driven control of a QAT-prepared model: observers warm up first, fake quantisation switches on after the
    warm-up, observers (and batch-norm statistics) freeze late in training so that the ranges the converted model
    will use are the ones the last steps trained against."""

    def __init__(self, model: nn.Module, schedule: Optional[QATSchedule] = None):
        self.model, self.s = model, schedule or QATSchedule()
        self.step_count = 0
        self._apply()

    def fake_quant_modules(self) -> List[FakeQuantize]:
        return [m for m in self.model.modules() if isinstance(m, FakeQuantize)]

    def _apply(self):
        s, k = self.s, self.step_count
        fq_on = k >= s.observer_warmup_steps
        obs_on = s.freeze_observers_after is None or k < s.freeze_observers_after
        for m in self.fake_quant_modules():
            m.fake_quant_enabled, m.observer_enabled = fq_on, obs_on
        if s.freeze_batchnorm_after is not None and k >= s.freeze_batchnorm_after:
            for m in self.model.modules():
                if isinstance(m, nn.modules.batchnorm._BatchNorm):
                    m.eval()

    def on_step_end(self):
        self.step_count += 1
        self._apply()

    def state(self) -> Dict[str, Any]:
        fq = self.fake_quant_modules()
        return {"step": self.step_count, "fake_quant_enabled": bool(fq and fq[0].fake_quant_enabled), "observers_enabled": bool(fq and fq[0].observer_enabled)}


class QATCheckpointing:
    """Saves / restores a QAT-prepared model with what ``state_dict`` does not carry: the observers' running ranges and
    the enable flags, plus the integration's step counter."""

    @staticmethod
    def _observers(model: nn.Module) -> Dict[str, FakeQuantize]:
        return {n: m for n, m in model.named_modules() if isinstance(m, FakeQuantize)}

    @classmethod
    def state(cls, model: nn.Module, integration: Optional[QATTrainingIntegration] = None) -> Dict[str, Any]:
        obs = {}
        for n, m in cls._observers(model).items():
            obs[n] = {"lo": None if m.cal.lo is None else m.cal.lo.detach().cpu(), "hi": None if m.cal.hi is None else m.cal.hi.detach().cpu(),
                      "observer_enabled": m.observer_enabled, "fake_quant_enabled": m.fake_quant_enabled}
        return {"model": model.state_dict(), "observers": obs, "step": integration.step_count if integration is not None else 0}

    @classmethod
    def save(cls, path: str, model: nn.Module, integration: Optional[QATTrainingIntegration] = None, optimizer=None):
        st = cls.state(model, integration)
        if optimizer is not None:
            st["optimizer"] = optimizer.state_dict()
        tmp = path + ".tmp"
        torch.save(st, tmp)
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str, model: nn.Module, integration: Optional[QATTrainingIntegration] = None, optimizer=None) -> int:
        st = torch.load(path, map_location="cpu", weights_only=False)
        own = cls._observers(model)
        missing = set(st["observers"]) ^ set(own)
        if missing:
            raise KeyError(f"observer sets differ: {sorted(missing)}")
        model.load_state_dict(st["model"])
        for n, o in st["observers"].items():
            m = own[n]
            m.cal.lo, m.cal.hi = o["lo"], o["hi"]
            m.observer_enabled, m.fake_quant_enabled = o["observer_enabled"], o["fake_quant_enabled"]
        if integration is not None:
            integration.step_count = st["step"]
            integration._apply()
        if optimizer is not None and "optimizer" in st:
            optimizer.load_state_dict(st["optimizer"])
        return st["step"]
