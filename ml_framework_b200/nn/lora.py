"""LoRA: low-rank adapters for Linear and Conv2d, injection, multi-adapter management, I/O.

Conventions follow the reference (its A/B naming is reversed relative to the paper and is kept):
``lora_A`` is ``[out, rank]`` ~ N(0, 0.01) and ``lora_B`` is ``[rank, in]`` zeros, the base layer
is frozen, ``forward = base(x) + dropout(x) @ B^T @ A^T * (alpha / rank)``, ``merge`` adds
``(alpha / rank) * A @ B`` to the base weight and ``unmerge`` subtracts it
(src/MLFramework/LoRA/LoraLinear.cs:34-118, 210-236). Config defaults: rank 8, alpha 16, dropout 0,
target modules q_proj / v_proj, bias none | all | lora_only
(src/RitterFramework.Core/LoRA/LoraConfig.cs:9-123). Injection / removal / enumeration:
src/MLFramework/LoRA/LoraInjector.cs:26-141. Adapter manager: RitterFramework.Core/LoRA/AdapterManager.cs:31-204.
Serialization: src/MLFramework/LoRA/AdapterSerializer.cs:21-99.

On bf16 CUDA tensors the two rank-r products run on the tcgen05 GEMM (K or N = rank, padded to 8).
"""
from __future__ import annotations

import fnmatch
import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fm


@dataclass
class LoraConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: Sequence[str] = ("q_proj", "v_proj")
    bias: str = "none"            # none | all | lora_only
    lora_type: str = "default"    # default | scaled (alpha / sqrt(rank))
    init_std: float = 0.01

    def validate(self):
        if self.rank <= 0:
            raise ValueError("rank must be positive")
        if self.alpha <= 0:
            raise ValueError("alpha must be positive")
        if not (0.0 <= self.dropout < 1.0):
            raise ValueError("dropout must be in [0, 1)")
        if self.bias not in ("none", "all", "lora_only"):
            raise ValueError("bias must be none, all or lora_only")
        if self.lora_type not in ("default", "scaled"):
            raise ValueError("lora_type must be default or scaled")

    @property
    def scaling(self) -> float:
        return self.alpha / (math.sqrt(self.rank) if self.lora_type == "scaled" else self.rank)

    @classmethod
    def for_llama(cls, rank=8):
        return cls(rank=rank, alpha=2 * rank, target_modules=("q_proj", "k_proj", "v_proj", "o_proj", "qkv", "proj"))

    @classmethod
    def for_gpt(cls, rank=8):
        return cls(rank=rank, alpha=2 * rank, target_modules=("c_attn", "c_proj", "qkv", "proj"))

    @classmethod
    def for_bert(cls, rank=8):
        return cls(rank=rank, alpha=2 * rank, target_modules=("query", "value"))


def matches_target(name: str, patterns: Sequence[str]) -> bool:
    """``ModuleTargetPattern``: exact leaf name, dotted suffix, or ``*`` / ``?`` wildcards."""
    leaf = name.rsplit(".", 1)[-1]
    for pat in patterns:
        if any(ch in pat for ch in "*?"):
            if fnmatch.fnmatch(name, pat) or fnmatch.fnmatch(leaf, pat):
                return True
        elif leaf == pat or name == pat or name.endswith("." + pat):
            return True
    return False


class _LoraLinearFn(torch.autograd.Function):
    """``y = x W^T + b (+ residual) + s * (x B^T) A^T`` on the tcgen05 GEMM with the adapter's second product
    accumulated into the base product's output by its own epilogue (``MLF_EPI_ACCUM`` with ``alpha = s``): no
    separate pass adds the two. Backward mirrors it: ``dx = dy W`` then ``+= (s dy A) B`` accumulated the same
    way; ``dA = s dy^T h``, ``dB = (s dy A)^T x``; the frozen base weight gets no gradient."""

    @staticmethod
    def forward(ctx, x, w, bias, lora_a, lora_b, scaling, residual):
        from .. import _lib
        from ..ops.gemm import gemm
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        h = gemm(x2, lora_b)                                                     # [M, r]
        y = gemm(x2, w, bias=bias, aux_in=res2, flags=_lib.EPI_RESIDUAL if residual is not None else 0)
        gemm(h, lora_a, out=y, flags=_lib.EPI_ACCUM, alpha=float(scaling))       # y += s * h A^T, in the epilogue
        ctx.save_for_backward(x2, h, w, lora_a, lora_b)
        ctx.scaling, ctx.x_shape, ctx.has_res = float(scaling), x.shape, residual is not None
        ctx.bias_ref = bias
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .. import _lib
        from ..ops.gemm import gemm
        x2, h, w, lora_a, lora_b = ctx.saved_tensors
        s = ctx.scaling
        dy2 = dy.reshape(-1, w.shape[0])
        if dy2.stride(-1) != 1 or (dy2.stride(0) % 8) != 0:
            dy2 = dy2.contiguous()
        dh = gemm(dy2, lora_a, b_mn=True, alpha=s)                                # [M, r] = s * dy A
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True)
            gemm(dh, lora_b, b_mn=True, out=dx, flags=_lib.EPI_ACCUM)             # dx += dh B
            dx = dx.view(ctx.x_shape)
        da = gemm(dy2, h, a_mn=True, b_mn=True, alpha=s) if ctx.needs_input_grad[3] else None   # [out, r]
        db = gemm(dh, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[4] else None            # [r, in]
        dbias = None
        if ctx.bias_ref is not None and ctx.needs_input_grad[2]:
            dbias = Fm._bgrad(dy2, ctx.bias_ref)
        return dx, None, dbias, da, db, None, (dy if ctx.has_res else None)


class LoRAAdapterBase(nn.Module):
    merged: bool = False
    enabled: bool = True

    def adapter_parameters(self) -> List[nn.Parameter]:
        return [self.lora_A, self.lora_B]

    def adapter_state(self) -> Dict[str, torch.Tensor]:
        return {"lora_A": self.lora_A.detach().clone(), "lora_B": self.lora_B.detach().clone()}

    def load_adapter_state(self, sd: Dict[str, torch.Tensor]):
        with torch.no_grad():
            self.lora_A.copy_(sd["lora_A"])
            self.lora_B.copy_(sd["lora_B"])


class LoraLinear(LoRAAdapterBase):
    def __init__(self, base: nn.Module, config: LoraConfig):
        super().__init__()
        config.validate()
        self.base, self.cfg = base, config
        w = base.weight
        out_f, in_f = w.shape
        for p in base.parameters():
            p.requires_grad_(False)
        if config.bias in ("all", "lora_only") and getattr(base, "bias", None) is not None:
            base.bias.requires_grad_(True)
        g = torch.Generator().manual_seed(42)
        self.lora_A = nn.Parameter((torch.randn(out_f, config.rank, generator=g) * config.init_std).to(w.dtype).to(w.device))
        self.lora_B = nn.Parameter(torch.zeros(config.rank, in_f, dtype=w.dtype, device=w.device))
        self.dropout = nn.Dropout(config.dropout) if config.dropout > 0 else nn.Identity()
        self.scaling = config.scaling

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return getattr(self.base, "bias", None)

    def forward(self, x, residual=None):
        if self.merged or not self.enabled:
            return self.base(x, residual) if residual is not None else self.base(x)
        w, b = self.base.weight, getattr(self.base, "bias", None)
        if (isinstance(self.dropout, nn.Identity) and self.cfg.rank % 8 == 0 and w.dim() == 2
                and Fm._native(x, w, b, self.lora_A, self.lora_B, residual)):
            return _LoraLinearFn.apply(x, w, b, self.lora_A, self.lora_B, self.scaling, residual)
        y = self.base(x, residual) if residual is not None else self.base(x)
        h = Fm.linear(self.dropout(x), self.lora_B)          # [.., rank]
        return y + Fm.linear(h, self.lora_A) * self.scaling

    def delta_weight(self) -> torch.Tensor:
        return (self.lora_A.float() @ self.lora_B.float()) * self.scaling

    @torch.no_grad()
    def merge(self):
        if not self.merged:
            self.base.weight.add_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self):
        if self.merged:
            self.base.weight.sub_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = False


class LoRAConv2d(LoRAAdapterBase):
    """Conv2d adapter: B is a conv with the base kernel size to ``rank`` channels, A a 1x1 conv
    back to ``out_channels`` (src/MLFramework/LoRA/LoRAConv2d.cs)."""

    def __init__(self, base: nn.Conv2d, config: LoraConfig):
        super().__init__()
        config.validate()
        self.base, self.cfg = base, config
        for p in base.parameters():
            p.requires_grad_(False)
        g = torch.Generator().manual_seed(42)
        kh, kw = base.kernel_size
        self.lora_B = nn.Parameter(torch.zeros(config.rank, base.in_channels // base.groups, kh, kw,
                                               dtype=base.weight.dtype, device=base.weight.device))
        self.lora_A = nn.Parameter((torch.randn(base.out_channels, config.rank, 1, 1, generator=g) * config.init_std)
                                   .to(base.weight.dtype).to(base.weight.device))
        self.dropout = nn.Dropout(config.dropout) if config.dropout > 0 else nn.Identity()
        self.scaling = config.scaling

    def forward(self, x):
        y = self.base(x)
        if self.merged or not self.enabled:
            return y
        h = F.conv2d(self.dropout(x), self.lora_B, None, self.base.stride, self.base.padding, self.base.dilation, self.base.groups)
        return y + F.conv2d(h, self.lora_A) * self.scaling

    def delta_weight(self):
        a = self.lora_A.float().flatten(1)                       # [out, r]
        b = self.lora_B.float().flatten(1)                       # [r, in*kh*kw]
        return (a @ b).view_as(self.base.weight) * self.scaling

    @torch.no_grad()
    def merge(self):
        if not self.merged:
            self.base.weight.add_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self):
        if self.merged:
            self.base.weight.sub_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = False


def _is_linear_like(m: nn.Module) -> bool:
    from .layers import Linear
    return isinstance(m, (nn.Linear, Linear))


class LoraInjector:
    @staticmethod
    def inject(model: nn.Module, config: LoraConfig) -> List[str]:
        """Replace every targeted Linear / Conv2d by its adapter wrapper; returns the wrapped names."""
        config.validate()
        wrapped = []
        for name, module in list(model.named_modules()):
            for child_name, child in list(module.named_children()):
                full = f"{name}.{child_name}" if name else child_name
                if isinstance(child, LoRAAdapterBase) or not matches_target(full, config.target_modules):
                    continue
                if _is_linear_like(child):
                    setattr(module, child_name, LoraLinear(child, config))
                    wrapped.append(full)
                elif isinstance(child, nn.Conv2d):
                    setattr(module, child_name, LoRAConv2d(child, config))
                    wrapped.append(full)
        return wrapped

    @staticmethod
    def remove(model: nn.Module, merge: bool = False) -> int:
        n = 0
        for module in list(model.modules()):
            for child_name, child in list(module.named_children()):
                if isinstance(child, LoRAAdapterBase):
                    if merge:
                        child.merge()
                    elif child.merged:
                        child.unmerge()
                    setattr(module, child_name, child.base)
                    n += 1
        return n

    @staticmethod
    def get_lora_layers(model: nn.Module) -> Dict[str, LoRAAdapterBase]:
        return {n: m for n, m in model.named_modules() if isinstance(m, LoRAAdapterBase)}


def apply_lora(model: nn.Module, config: Optional[LoraConfig] = None) -> nn.Module:
    LoraInjector.inject(model, config or LoraConfig())
    freeze_base(model)
    return model


def freeze_base(model: nn.Module):
    adapters = {id(p) for m in model.modules() if isinstance(m, LoRAAdapterBase) for p in m.adapter_parameters()}
    keep_bias = {id(m.base.bias) for m in model.modules() if isinstance(m, LoRAAdapterBase)
                 and m.cfg.bias in ("all", "lora_only") and getattr(m.base, "bias", None) is not None}
    for p in model.parameters():
        p.requires_grad_(id(p) in adapters or id(p) in keep_bias)


def lora_parameters(model: nn.Module) -> List[nn.Parameter]:
    return [p for m in model.modules() if isinstance(m, LoRAAdapterBase) for p in m.adapter_parameters()]


class LoraAdapter:
    """A named set of adapter weights detached from a model."""

    def __init__(self, name: str, config: LoraConfig, weights: Dict[str, Dict[str, torch.Tensor]], metadata: Optional[dict] = None):
        self.name, self.config, self.weights, self.metadata = name, config, weights, metadata or {}

    @classmethod
    def from_model(cls, name: str, model: nn.Module) -> "LoraAdapter":
        layers = LoraInjector.get_lora_layers(model)
        if not layers:
            raise ValueError("model has no LoRA layers")
        cfg = next(iter(layers.values())).cfg
        return cls(name, cfg, {n: m.adapter_state() for n, m in layers.items()})

    def apply_to(self, model: nn.Module):
        layers = LoraInjector.get_lora_layers(model)
        missing = set(self.weights) - set(layers)
        if missing:
            raise KeyError(f"adapter {self.name!r} has weights for unknown layers: {sorted(missing)[:3]}")
        for n, sd in self.weights.items():
            layers[n].load_adapter_state(sd)


class AdapterSerializer:
    @staticmethod
    def save(adapter: LoraAdapter, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        torch.save({"name": adapter.name, "config": asdict(adapter.config), "weights": adapter.weights,
                    "metadata": adapter.metadata, "format": "mlf-lora-1"}, path)

    @staticmethod
    def load(path: str) -> LoraAdapter:
        d = torch.load(path, map_location="cpu", weights_only=False)
        if d.get("format") != "mlf-lora-1":
            raise ValueError("not a LoRA adapter file")
        cfg = LoraConfig(**{**d["config"], "target_modules": tuple(d["config"]["target_modules"])})
        return LoraAdapter(d["name"], cfg, d["weights"], d.get("metadata"))

    @staticmethod
    def save_json(adapter: LoraAdapter, path: str):
        with open(path, "w") as f:
            json.dump({"name": adapter.name, "config": {**asdict(adapter.config), "target_modules": list(adapter.config.target_modules)},
                       "metadata": adapter.metadata,
                       "weights": {n: {k: v.float().tolist() for k, v in sd.items()} for n, sd in adapter.weights.items()}}, f)


class AdapterManager:
    """Several named adapters over one injected model; at most one active at a time."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.adapters: Dict[str, LoraAdapter] = {}
        self.active: Optional[str] = None

    def load_adapter(self, adapter: LoraAdapter, activate: bool = False):
        if adapter.name in self.adapters:
            raise ValueError(f"adapter {adapter.name!r} already loaded")
        self.adapters[adapter.name] = adapter
        if activate:
            self.set_active_adapter(adapter.name)

    def set_active_adapter(self, name: str):
        if name not in self.adapters:
            raise KeyError(name)
        self.deactivate()
        self.adapters[name].apply_to(self.model)
        for m in LoraInjector.get_lora_layers(self.model).values():
            m.enabled = True
        self.active = name

    activate = set_active_adapter

    def deactivate(self):
        for m in LoraInjector.get_lora_layers(self.model).values():
            if m.merged:
                m.unmerge()
            m.enabled = False
        self.active = None

    def unload(self, name: str):
        if self.active == name:
            self.deactivate()
        del self.adapters[name]

    def list_adapters(self) -> List[str]:
        return sorted(self.adapters)
