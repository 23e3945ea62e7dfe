"""Optimizers: AdamW / Adam (fused, flat), SGD, and the ``Optimizer`` base contract.

``AdamW`` follows the reference's Adam (src/MLFramework/Optimizers/Adam.cs:95-213): defaults
lr 1e-3, betas (0.9, 0.999), eps 1e-8, decoupled weight decay applied before the Adam step,
optional amsgrad; ``state_dict`` / ``load_state_dict`` mirror ``GetState/LoadState``
(Optimizers/Optimizer.cs:141-172). Parameters in bf16 keep an fp32 master copy plus m and v
("mixed-precision optimizer", Optimizers/MixedPrecision/MixedPrecisionOptimizer.cs:107-138).
On CUDA one fused kernel updates each flat buffer; on CPU the same math runs in PyTorch.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.nn as nn

from ..ops import native, reference
from ..parallel.flat import FlatParams


class Optimizer:
    """Base contract: ``step``, ``zero_grad``, learning-rate access, state dict, scheduler hook."""

    def __init__(self, lr: float):
        self.lr = lr
        self.step_count = 0
        self.scheduler = None

    def set_learning_rate(self, lr: float):
        self.lr = lr

    def get_learning_rate(self) -> float:
        return self.lr

    def set_scheduler(self, scheduler):
        self.scheduler = scheduler

    def _step_scheduler(self):
        if self.scheduler is not None:
            self.lr = self.scheduler.step()

    def step(self, **_):
        raise NotImplementedError

    def zero_grad(self, set_to_zero: bool = False):
        raise NotImplementedError


class _Segment:
    """One contiguous run of optimizer work: parameter storage, gradient source, fp32 state."""

    def __init__(self, param_flat: torch.Tensor, grad_getter, needs_master: bool):
        self.param_flat = param_flat
        self.grad_getter = grad_getter
        self.master = param_flat.detach().float().clone() if needs_master else param_flat.detach()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.vmax = None
        self.needs_master = needs_master


def _segments(params_or_flat, state_shard=None) -> List[_Segment]:
    segs = []
    if isinstance(params_or_flat, FlatParams):
        fp = params_or_flat
        segs.append(_Segment(fp.flat, lambda fp=fp: fp.grad, fp.flat.dtype != torch.float32))
        return segs
    for p in params_or_flat:
        if isinstance(p, FlatParams):
            segs.extend(_segments(p))
            continue
        if not p.requires_grad:
            continue

        def getter(p=p):
            mg = getattr(p, "main_grad", None)
            if mg is not None and getattr(p, "_main_grad_started", False):
                return mg.reshape(-1)
            return p.grad.reshape(-1) if p.grad is not None else None
        segs.append(_Segment(p.data.view(-1), getter, p.dtype != torch.float32))
    return segs


class AdamW(Optimizer):
    def __init__(self, params: Union[FlatParams, Iterable[nn.Parameter]], lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, amsgrad: bool = False):
        super().__init__(lr)
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1) or weight_decay < 0:
            raise ValueError("invalid AdamW hyper-parameters")
        self.betas, self.eps, self.weight_decay, self.amsgrad = betas, eps, weight_decay, amsgrad
        self._source = params if isinstance(params, FlatParams) else list(params)
        self.segments = _segments(self._source)
        if amsgrad:
            for s in self.segments:
                s.vmax = torch.zeros_like(s.master)

    def step(self, grad_scale: float = 1.0, inv_scale: Optional[torch.Tensor] = None,
             found_inf: Optional[torch.Tensor] = None) -> None:
        """One update. ``inv_scale`` (device scalar, 1/loss_scale) and ``found_inf`` (device int
        flag; non-zero skips the update) let AMP run without a host synchronisation."""
        self.step_count += 1
        b1, b2 = self.betas
        for s in self.segments:
            g = s.grad_getter()
            if g is None:
                continue
            if s.master.is_cuda:
                native.adamw_(s.master, s.m, s.v, g, s.param_flat if s.needs_master else None, lr=self.lr, beta1=b1,
                              beta2=b2, eps=self.eps, weight_decay=self.weight_decay, step=self.step_count,
                              grad_scale=grad_scale, inv_scale=inv_scale, found_inf=found_inf, vmax=s.vmax)
            else:
                if found_inf is not None and int(found_inf.item()) != 0:
                    continue
                gf = g.float() * grad_scale * (float(inv_scale.item()) if inv_scale is not None else 1.0)
                out = reference.adamw_ref(s.master, s.m, s.v, gf, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                                          weight_decay=self.weight_decay, step=self.step_count, vmax=s.vmax)
                s.master.copy_(out[0]); s.m.copy_(out[1]); s.v.copy_(out[2])
                if s.vmax is not None:
                    s.vmax.copy_(out[3])
                if s.needs_master:
                    s.param_flat.copy_(s.master.to(s.param_flat.dtype))
        self._step_scheduler()

    def zero_grad(self, set_to_zero: bool = False):
        if isinstance(self._source, FlatParams):
            self._source.zero_grad(set_to_zero)
            return
        for p in self._source:
            if isinstance(p, FlatParams):
                p.zero_grad(set_to_zero)
            else:
                p.grad = None
                if getattr(p, "main_grad", None) is not None:
                    p._main_grad_started = False

    def state_dict(self) -> Dict:
        return {"type": type(self).__name__, "lr": self.lr, "betas": list(self.betas), "eps": self.eps,
                "weight_decay": self.weight_decay, "amsgrad": self.amsgrad, "step": self.step_count,
                "segments": [{"master": s.master.detach().cpu().clone(), "m": s.m.cpu().clone(), "v": s.v.cpu().clone(),
                              "vmax": None if s.vmax is None else s.vmax.cpu().clone()} for s in self.segments]}

    def load_state_dict(self, sd: Dict):
        if len(sd["segments"]) != len(self.segments):
            raise ValueError("optimizer state does not match the parameter layout")
        self.lr, self.betas, self.eps = sd["lr"], tuple(sd["betas"]), sd["eps"]
        self.weight_decay, self.step_count = sd["weight_decay"], sd["step"]
        for s, d in zip(self.segments, sd["segments"]):
            s.master.copy_(d["master"]); s.m.copy_(d["m"]); s.v.copy_(d["v"])
            if s.vmax is not None and d.get("vmax") is not None:
                s.vmax.copy_(d["vmax"])
            if s.needs_master:
                s.param_flat.copy_(s.master.to(s.param_flat.dtype))


class Adam(AdamW):
    """Adam with the reference's (decoupled) weight-decay semantics; identical to AdamW here."""


class SGD(Optimizer):
    def __init__(self, params, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0):
        super().__init__(lr)
        self.momentum, self.weight_decay = momentum, weight_decay
        self._source = params if isinstance(params, FlatParams) else list(params)
        self.segments = _segments(self._source)
        for s in self.segments:
            s.v = None
            if momentum == 0.0:
                s.m = None

    def step(self, grad_scale: float = 1.0, inv_scale=None, found_inf=None):
        self.step_count += 1
        for s in self.segments:
            g = s.grad_getter()
            if g is None:
                continue
            if s.master.is_cuda:
                native.sgd_(s.master, s.m, g, s.param_flat if s.needs_master else None, lr=self.lr, momentum=self.momentum,
                            weight_decay=self.weight_decay, grad_scale=grad_scale, inv_scale=inv_scale, found_inf=found_inf)
            else:
                if found_inf is not None and int(found_inf.item()) != 0:
                    continue
                gf = g.float() * grad_scale * (float(inv_scale.item()) if inv_scale is not None else 1.0)
                gf = gf + self.weight_decay * s.master
                if s.m is not None:
                    s.m.mul_(self.momentum).add_(gf)
                    gf = s.m
                s.master.add_(gf, alpha=-self.lr)
                if s.needs_master:
                    s.param_flat.copy_(s.master.to(s.param_flat.dtype))
        self._step_scheduler()

    zero_grad = AdamW.zero_grad

    def state_dict(self):
        return {"type": "SGD", "lr": self.lr, "momentum": self.momentum, "weight_decay": self.weight_decay,
                "step": self.step_count,
                "segments": [{"master": s.master.detach().cpu().clone(), "m": None if s.m is None else s.m.cpu().clone()}
                             for s in self.segments]}

    def load_state_dict(self, sd):
        self.lr, self.momentum, self.weight_decay, self.step_count = sd["lr"], sd["momentum"], sd["weight_decay"], sd["step"]
        for s, d in zip(self.segments, sd["segments"]):
            s.master.copy_(d["master"])
            if s.m is not None and d["m"] is not None:
                s.m.copy_(d["m"])
            if s.needs_master:
                s.param_flat.copy_(s.master.to(s.param_flat.dtype))
