"""Quantisation: int8 operations, calibrators, post-training quantisation, quantisation-aware training,
evaluation.

Reference (src/MLFramework/Quantization/): Operations/{Quantization,Dequantization,PerChannel}Operations.cs
and QuantizationUtils.cs; Calibration/{MinMax,Entropy,MovingAverage,Percentile}Calibrator.cs; PTQ/{PTQQuantizer,
StaticQuantization,DynamicQuantization,CalibrationProcess,SensitivityAnalysis}.cs; QAT/{FakeQuantize,
FakeQuantizeLayer,StraightThroughEstimator,ActivationObserver,QATPreparer,ModelConversion}.cs; Evaluation/*
(Top-K, MAE, RMSE, per-layer sensitivity, regression detector); Backends/GPUBackend (int8 path is a TODO
there). On a CUDA tensor the element-wise work runs in this package's kernels (``csrc/ops/quant.cu``).
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class QuantizationMode(enum.Enum):
    SYMMETRIC = "symmetric"
    ASYMMETRIC = "asymmetric"


@dataclass
class QuantizationParameters:
    scale: torch.Tensor                 # [] or [channels], fp32
    zero_point: torch.Tensor            # int32, same shape
    qmin: int = -128
    qmax: int = 127
    axis: Optional[int] = None          # None = per tensor; 0 / 1 = per row / column of the 2-D view

    @property
    def per_channel(self) -> bool:
        return self.axis is not None


def compute_qparams(lo: torch.Tensor, hi: torch.Tensor, mode: QuantizationMode = QuantizationMode.SYMMETRIC, qmin: int = -128,
                    qmax: int = 127, axis: Optional[int] = None, eps: float = 1e-8) -> QuantizationParameters:
    lo, hi = torch.minimum(lo.float(), torch.zeros_like(lo, dtype=torch.float32)), torch.maximum(hi.float(), torch.zeros_like(hi, dtype=torch.float32))
    if mode == QuantizationMode.SYMMETRIC:
        amax = torch.maximum(lo.abs(), hi.abs())
        scale = (amax / max(abs(qmin), qmax)).clamp_min(eps)
        zp = torch.zeros_like(scale, dtype=torch.int32)
    else:
        scale = ((hi - lo) / (qmax - qmin)).clamp_min(eps)
        zp = (qmin - torch.round(lo / scale)).clamp(qmin, qmax).to(torch.int32)
    return QuantizationParameters(scale, zp, qmin, qmax, axis)


def _as2d(x: torch.Tensor, axis: Optional[int]) -> Tuple[torch.Tensor, Optional[int]]:
    """2-D view with the channel axis as rows (axis 0) or columns (last axis); other axes are not supported per channel."""
    if axis is None:
        return x.reshape(1, -1) if x.dim() < 2 else x.reshape(-1, x.shape[-1]), None
    axis = axis % x.dim()
    if axis == 0:
        return x.reshape(x.shape[0], -1), 0
    if axis == x.dim() - 1:
        return x.reshape(-1, x.shape[-1]), 1
    raise ValueError("per-channel axis must be the first or the last dimension")


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous()


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def quantize(x: torch.Tensor, qp: QuantizationParameters) -> torch.Tensor:
    x2, ax = _as2d(x, qp.axis)
    if _native(x):
        from .. import _lib
        out = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
        s, z = qp.scale.to(x.device, torch.float32).reshape(-1).contiguous(), qp.zero_point.to(x.device, torch.int32).reshape(-1).contiguous()
        rc = _lib.get().mlf_quantize_i8(_ptr(out), _ptr(x2), 0 if x.dtype == torch.float32 else 1, C.c_longlong(x2.shape[0]), x2.shape[1],
                                        _ptr(s), _ptr(z), -1 if ax is None else ax, qp.qmin, qp.qmax, C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_quantize_i8")
        return out.view(x.shape)
    s, z = _bcast(qp, x2, ax)
    return (torch.round(x2.float() / s) + z).clamp(qp.qmin, qp.qmax).to(torch.int8).view(x.shape)


def _bcast(qp, x2, ax):
    s, z = qp.scale.to(x2.device).float().reshape(-1), qp.zero_point.to(x2.device).float().reshape(-1)
    if ax == 0:
        return s[:, None], z[:, None]
    if ax == 1:
        return s[None, :], z[None, :]
    return s[0], z[0]


def dequantize(q: torch.Tensor, qp: QuantizationParameters, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    q2, ax = _as2d(q, qp.axis)
    if q.is_cuda and q.is_contiguous() and dtype in (torch.float32, torch.bfloat16):
        from .. import _lib
        out = torch.empty(q2.shape, dtype=dtype, device=q.device)
        s, z = qp.scale.to(q.device, torch.float32).reshape(-1).contiguous(), qp.zero_point.to(q.device, torch.int32).reshape(-1).contiguous()
        rc = _lib.get().mlf_dequantize_i8(_ptr(out), _ptr(q2), 0 if dtype == torch.float32 else 1, C.c_longlong(q2.shape[0]), q2.shape[1],
                                          _ptr(s), _ptr(z), -1 if ax is None else ax, C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_dequantize_i8")
        return out.view(q.shape)
    s, z = _bcast(qp, q2, ax)
    return ((q2.float() - z) * s).to(dtype).view(q.shape)


def fake_quantize(x: torch.Tensor, qp: QuantizationParameters, want_mask: bool = False):
    """quantise + dequantise in one pass; ``mask`` marks elements that were not clamped (the straight-through
    estimator passes gradients only there)."""
    x2, ax = _as2d(x, qp.axis)
    if _native(x):
        from .. import _lib
        out = torch.empty_like(x2)
        mask = torch.empty(x2.shape, dtype=torch.uint8, device=x.device) if want_mask else None
        s, z = qp.scale.to(x.device, torch.float32).reshape(-1).contiguous(), qp.zero_point.to(x.device, torch.int32).reshape(-1).contiguous()
        rc = _lib.get().mlf_fake_quant(_ptr(out), _ptr(mask), _ptr(x2), 0 if x.dtype == torch.float32 else 1, C.c_longlong(x2.shape[0]),
                                       x2.shape[1], _ptr(s), _ptr(z), -1 if ax is None else ax, qp.qmin, qp.qmax, C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_fake_quant")
        return (out.view(x.shape), mask.view(x.shape).bool()) if want_mask else out.view(x.shape)
    s, z = _bcast(qp, x2, ax)
    qf = torch.round(x2.float() / s) + z
    out = ((qf.clamp(qp.qmin, qp.qmax) - z) * s).to(x.dtype).view(x.shape)
    if want_mask:
        return out, ((qf >= qp.qmin) & (qf <= qp.qmax)).view(x.shape)
    return out


def tensor_minmax(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if _native(x):
        from .. import _lib
        out = torch.empty(2, dtype=torch.float32, device=x.device)
        sc = torch.empty(2, dtype=torch.int32, device=x.device)
        rc = _lib.get().mlf_minmax(_ptr(out), _ptr(x), 0 if x.dtype == torch.float32 else 1, C.c_longlong(x.numel()), _ptr(sc),
                                   C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_minmax")
        return out[0], out[1]
    return x.min().float(), x.max().float()


# ------------------------------------------------------------------ calibrators
class Calibrator:
    def observe(self, x: torch.Tensor):
        raise NotImplementedError

    def range(self) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def qparams(self, mode=QuantizationMode.SYMMETRIC, qmin=-128, qmax=127) -> QuantizationParameters:
        lo, hi = self.range()
        return compute_qparams(lo, hi, mode, qmin, qmax)


class MinMaxCalibrator(Calibrator):
    def __init__(self):
        self.lo = self.hi = None

    def observe(self, x):
        lo, hi = tensor_minmax(x.detach())
        self.lo = lo if self.lo is None else torch.minimum(self.lo, lo)
        self.hi = hi if self.hi is None else torch.maximum(self.hi, hi)

    def range(self):
        if self.lo is None:
            raise RuntimeError("calibrator saw no data")
        return self.lo, self.hi


class MovingAverageCalibrator(Calibrator):
    def __init__(self, momentum: float = 0.9):
        self.m, self.lo, self.hi = momentum, None, None

    def observe(self, x):
        lo, hi = tensor_minmax(x.detach())
        self.lo = lo if self.lo is None else self.m * self.lo + (1 - self.m) * lo
        self.hi = hi if self.hi is None else self.m * self.hi + (1 - self.m) * hi

    def range(self):
        if self.lo is None:
            raise RuntimeError("calibrator saw no data")
        return self.lo, self.hi


class PercentileCalibrator(Calibrator):
    def __init__(self, percentile: float = 99.99, max_samples: int = 1 << 20):
        self.p, self.max_samples, self.samples = percentile, max_samples, []

    def observe(self, x):
        v = x.detach().float().flatten()
        if v.numel() > self.max_samples:
            v = v[torch.randperm(v.numel(), device=v.device)[:self.max_samples]]
        self.samples.append(v.cpu())

    def range(self):
        v = torch.cat(self.samples)
        if v.numel() > (1 << 24):
            v = v[torch.randperm(v.numel())[:1 << 24]]
        q = torch.tensor([1 - self.p / 100.0, self.p / 100.0])
        lo, hi = torch.quantile(v, q).unbind()
        return lo, hi


class EntropyCalibrator(Calibrator):
    """KL-divergence calibration: choose the clipping threshold whose quantised histogram is closest to
    the observed one (2048-bin histogram of |x|, 128 quantisation levels)."""

    def __init__(self, bins: int = 2048, levels: int = 128):
        self.bins, self.levels, self.hist, self.amax = bins, levels, None, 0.0

    def observe(self, x):
        v = x.detach().float().abs().flatten().cpu()
        amax = float(v.max())
        if self.hist is None or amax > self.amax:
            if self.hist is not None:                          # re-bin the old histogram into the wider range
                old_centers = (torch.arange(self.bins) + 0.5) * (self.amax / self.bins)
                new = torch.zeros(self.bins)
                idx = (old_centers / amax * self.bins).long().clamp(max=self.bins - 1)
                new.index_add_(0, idx, self.hist)
                self.hist = new
            else:
                self.hist = torch.zeros(self.bins)
            self.amax = max(amax, 1e-12)
        self.hist += torch.histc(v, self.bins, 0, self.amax)

    def range(self):
        h = self.hist
        best_kl, best_i = float("inf"), self.bins
        for i in range(self.levels, self.bins + 1, 16):
            p = h[:i].clone()
            p[i - 1] += h[i:].sum()
            chunks = torch.tensor_split(h[:i], self.levels)
            q = torch.cat([torch.where(c > 0, c.sum() / max(1, int((c > 0).sum())), torch.zeros_like(c)) for c in chunks])
            ps, qs = p / p.sum(), q / max(float(q.sum()), 1e-12)
            m = ps > 0
            kl = float((ps[m] * (ps[m] / qs[m].clamp_min(1e-12)).log()).sum())
            if kl < best_kl:
                best_kl, best_i = kl, i
        t = torch.tensor(best_i * self.amax / self.bins)
        return -t, t


# ------------------------------------------------------------------ quantised layers, PTQ
class QuantizedLinear(nn.Module):
    """int8 weights (per output channel, symmetric) and int8 activations (per tensor: static parameters from
    calibration or dynamic per call). The integer product runs on the tensor cores through
    ``torch._int_mm`` when shapes allow, else in fp32 on the dequantised operands."""

    def __init__(self, linear: nn.Linear, act_qparams: Optional[QuantizationParameters] = None):
        super().__init__()
        w = linear.weight.detach()
        self.w_qp = compute_qparams(w.float().amin(1), w.float().amax(1), QuantizationMode.SYMMETRIC, axis=0)
        self.register_buffer("w_q", quantize(w.contiguous(), self.w_qp))
        self.register_buffer("w_scale", self.w_qp.scale.to(w.device))
        self.bias = linear.bias
        self.act_qparams = act_qparams
        self.out_dtype = linear.weight.dtype

    def forward(self, x):
        xq_p = self.act_qparams
        if xq_p is None:
            lo, hi = tensor_minmax(x.detach().contiguous())
            xq_p = compute_qparams(lo, hi, QuantizationMode.SYMMETRIC)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        xq = quantize(x2, xq_p)
        M, K = xq.shape
        N = self.w_q.shape[0]
        if xq.is_cuda and M > 16 and K % 8 == 0 and N % 8 == 0 and int(xq_p.zero_point.reshape(-1)[0]) == 0:
            acc = torch._int_mm(xq, self.w_q.t()).float()
        else:
            acc = (xq.float() - xq_p.zero_point.to(x.device).float().reshape(-1)[0]) @ self.w_q.float().t()
        y = acc * (xq_p.scale.to(x.device).float().reshape(-1)[0] * self.w_scale.to(x.device)[None, :])
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(self.out_dtype).view(*x.shape[:-1], N)


class ActivationObserver(nn.Module):
    def __init__(self, calibrator: Optional[Calibrator] = None):
        super().__init__()
        self.cal = calibrator or MinMaxCalibrator()
        self.enabled = True

    def forward(self, x):
        if self.enabled:
            self.cal.observe(x)
        return x


class PTQQuantizer:
    """Static: observe activations at every Linear input over calibration batches, then swap in
    ``QuantizedLinear`` with fixed activation parameters. Dynamic: swap without calibration."""

    def __init__(self, calibrator_factory: Callable[[], Calibrator] = MinMaxCalibrator, skip: Sequence[str] = ()):
        self.factory, self.skip = calibrator_factory, tuple(skip)

    def _targets(self, model: nn.Module):
        return [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and not any(s in n for s in self.skip)]

    def calibrate(self, model: nn.Module, batches: Iterable, forward: Optional[Callable] = None) -> Dict[str, Calibrator]:
        cals: Dict[str, Calibrator] = {}
        hooks = []
        for n, m in self._targets(model):
            cals[n] = self.factory()
            hooks.append(m.register_forward_pre_hook(lambda mod, inp, n=n: cals[n].observe(inp[0])))
        model.eval()
        with torch.no_grad():
            for b in batches:
                forward(model, b) if forward else model(b)
        for h in hooks:
            h.remove()
        return cals

    @staticmethod
    def _swap(model: nn.Module, name: str, new: nn.Module):
        parent = model
        parts = name.split(".")
        for p in parts[:-1]:
            parent = getattr(parent, p)
        setattr(parent, parts[-1], new)

    def quantize_static(self, model: nn.Module, batches: Iterable, forward: Optional[Callable] = None) -> nn.Module:
        cals = self.calibrate(model, batches, forward)
        for n, m in self._targets(model):
            self._swap(model, n, QuantizedLinear(m, cals[n].qparams()))
        return model

    def quantize_dynamic(self, model: nn.Module) -> nn.Module:
        for n, m in self._targets(model):
            self._swap(model, n, QuantizedLinear(m, None))
        return model


def sensitivity_analysis(model: nn.Module, batches: Sequence, metric: Callable[[nn.Module], float]) -> List[Tuple[str, float]]:
    """Quantise one Linear at a time (dynamic), measure the metric drop, restore; sorted most sensitive first."""
    base = metric(model)
    out = []
    for n, m in [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear)]:
        PTQQuantizer._swap(model, n, QuantizedLinear(m, None))
        out.append((n, base - metric(model)))
        PTQQuantizer._swap(model, n, m)
    return sorted(out, key=lambda t: -t[1])


# ------------------------------------------------------------------ QAT
class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, qp):
        out, mask = fake_quantize(x.contiguous(), qp, want_mask=True)
        ctx.save_for_backward(mask)
        return out

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return g * mask.to(g.dtype), None


class FakeQuantize(nn.Module):
    """Observes the running range (moving average) while training and applies fake quantisation with a
    straight-through gradient."""

    def __init__(self, mode=QuantizationMode.SYMMETRIC, momentum: float = 0.9, qmin=-128, qmax=127):
        super().__init__()
        self.mode, self.qmin, self.qmax = mode, qmin, qmax
        self.cal = MovingAverageCalibrator(momentum)
        self.observer_enabled = self.fake_quant_enabled = True

    def forward(self, x):
        if self.training and self.observer_enabled:
            self.cal.observe(x)
        if not self.fake_quant_enabled or self.cal.lo is None:
            return x
        return _FakeQuantSTE.apply(x, self.cal.qparams(self.mode, self.qmin, self.qmax))


class QATLinear(nn.Module):
    def __init__(self, linear: nn.Linear):
        super().__init__()
        self.linear = linear
        self.act_fq = FakeQuantize()

    def forward(self, x):
        w = self.linear.weight
        qp = compute_qparams(w.detach().float().amin(1), w.detach().float().amax(1), QuantizationMode.SYMMETRIC, axis=0)
        return F.linear(self.act_fq(x), _FakeQuantSTE.apply(w, qp), self.linear.bias)


def prepare_qat(model: nn.Module, skip: Sequence[str] = ()) -> nn.Module:
    for n, m in [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and not any(s in n for s in skip)]:
        PTQQuantizer._swap(model, n, QATLinear(m))
    return model


def convert_qat(model: nn.Module) -> nn.Module:
    for n, m in [(n, m) for n, m in model.named_modules() if isinstance(m, QATLinear)]:
        qp = m.act_fq.cal.qparams(m.act_fq.mode) if m.act_fq.cal.lo is not None else None
        PTQQuantizer._swap(model, n, QuantizedLinear(m.linear, qp))
    return model


# ------------------------------------------------------------------ evaluation
def top_k_accuracy(logits: torch.Tensor, target: torch.Tensor, k: int = 1) -> float:
    return float((logits.topk(k, -1).indices == target[:, None]).any(-1).float().mean())


def mae(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().mean())


def rmse(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(((a.float() - b.float()) ** 2).mean().sqrt())


def sqnr_db(ref: torch.Tensor, q: torch.Tensor) -> float:
    ref, q = ref.detach(), q.detach()
    n = ((ref.float() - q.float()) ** 2).sum()
    return float(10 * torch.log10((ref.float() ** 2).sum() / n.clamp_min(1e-30)))


@dataclass
class RegressionReport:
    baseline: float
    quantized: float
    drop: float
    regressed: bool


def detect_regression(baseline: float, quantized: float, tolerance: float = 0.01) -> RegressionReport:
    return RegressionReport(baseline, quantized, baseline - quantized, (baseline - quantized) > tolerance)
