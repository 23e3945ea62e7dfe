"""Per-operation precision policy (autocast), kernel dtype selection and gradient utilities.

* ``AmpRegistry`` / ``DefaultAmpRules``: which operations run in low precision (whitelist: conv,
  linear, matmul, pooling, batchnorm, dropout, relu/gelu/sigmoid/tanh, element-wise) and which are
  forced to fp32 (blacklist: softmax, log-softmax, log, exp, sqrt, reductions, normalize,
  layernorm, embedding, losses) — src/MLFramework/Amp/DefaultAmpRules.cs:48-110,
  AmpRegistry.cs:32-149.
* ``AutoCast``: context manager that answers ``get_forward_dtype(op)`` / ``get_backward_dtype(op)``
  and casts tensors accordingly (src/MLFramework/Amp/AutoCast.cs:69-159); entering it also enables
  ``torch.autocast`` so ordinary PyTorch modules follow the same policy.
* ``KernelSelector`` / ``KernelRegistry``: which dtype kernel exists for an operation on this
  device (src/MLFramework/Amp/KernelSelector.cs:39-144, KernelCapability.cs:53-79). On B200 every
  GEMM-shaped op has a bf16 tcgen05 kernel; norms, softmax and losses take bf16 I/O with fp32 math.
* ``GradientClipper`` (Amp/GradientClipper.cs:19-153) and ``GradientUtils`` (GradientUtils.cs:17-197).
"""
from __future__ import annotations

import contextlib
import enum
import threading
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional

import torch


class OpPrecision(enum.Enum):
    LOWER = "lower"      # run in the autocast dtype
    FP32 = "fp32"        # always fp32
    KEEP = "keep"        # leave inputs as they are


@dataclass
class AmpConfig:
    """src/MLFramework/Amp/AmpConfig.cs:8-68."""
    enabled: bool = True
    target_dtype: torch.dtype = torch.bfloat16
    backward_dtype: torch.dtype = torch.float32
    loss_scaling: bool = True
    initial_loss_scale: float = 65536.0
    growth_interval: int = 2000

    @classmethod
    def create_fp16(cls):
        return cls(target_dtype=torch.float16)

    @classmethod
    def create_bf16(cls):
        return cls(target_dtype=torch.bfloat16, initial_loss_scale=8.0)


WHITELIST = ["conv1d", "conv2d", "conv3d", "linear", "matmul", "bmm", "maxpool", "avgpool", "batchnorm", "dropout",
             "relu", "gelu", "sigmoid", "tanh", "add", "sub", "mul", "div", "attention", "swiglu"]
BLACKLIST = ["softmax", "log_softmax", "log", "exp", "sqrt", "pow", "sum", "mean", "norm", "normalize", "layernorm",
             "rmsnorm", "embedding", "cross_entropy", "mse_loss", "nll_loss", "bce_loss"]


class AmpRegistry:
    def __init__(self, defaults: bool = True):
        self._rules: Dict[str, OpPrecision] = {}
        self._custom: Dict[str, tuple] = {}
        if defaults:
            for op in WHITELIST:
                self.register_whitelist(op)
            for op in BLACKLIST:
                self.register_blacklist(op)

    def register_whitelist(self, op: str):
        self._rules[op.lower()] = OpPrecision.LOWER

    def register_blacklist(self, op: str):
        self._rules[op.lower()] = OpPrecision.FP32

    def register_custom_op(self, op: str, forward_dtype: torch.dtype, backward_dtype: torch.dtype):
        self._custom[op.lower()] = (forward_dtype, backward_dtype)

    def unregister(self, op: str):
        self._rules.pop(op.lower(), None)
        self._custom.pop(op.lower(), None)

    def rule(self, op: str) -> OpPrecision:
        return self._rules.get(op.lower(), OpPrecision.KEEP)

    def get_forward_dtype(self, op: str, cfg: AmpConfig, input_dtype: torch.dtype = torch.float32) -> torch.dtype:
        op = op.lower()
        if op in self._custom:
            return self._custom[op][0]
        r = self.rule(op)
        if not cfg.enabled or r == OpPrecision.KEEP:
            return input_dtype
        return cfg.target_dtype if r == OpPrecision.LOWER else torch.float32

    def get_backward_dtype(self, op: str, cfg: AmpConfig, input_dtype: torch.dtype = torch.float32) -> torch.dtype:
        op = op.lower()
        if op in self._custom:
            return self._custom[op][1]
        r = self.rule(op)
        if not cfg.enabled or r == OpPrecision.KEEP:
            return input_dtype
        return cfg.target_dtype if r == OpPrecision.LOWER else torch.float32


_tls = threading.local()


class AutoCast(contextlib.AbstractContextManager):
    def __init__(self, config: Optional[AmpConfig] = None, registry: Optional[AmpRegistry] = None, device_type: str = "cuda"):
        self.cfg = config or AmpConfig()
        self.registry = registry or AmpRegistry()
        self.device_type = device_type
        self._torch_ctx = None

    @classmethod
    def fp16(cls, **k):
        return cls(AmpConfig.create_fp16(), **k)

    @classmethod
    def bf16(cls, **k):
        return cls(AmpConfig.create_bf16(), **k)

    def __enter__(self):
        stack = getattr(_tls, "stack", None)
        if stack is None:
            stack = _tls.stack = []
        stack.append(self)
        if self.cfg.enabled and (self.device_type != "cuda" or torch.cuda.is_available()):
            self._torch_ctx = torch.autocast(self.device_type, dtype=self.cfg.target_dtype)
            self._torch_ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._torch_ctx is not None:
            self._torch_ctx.__exit__(*exc)
            self._torch_ctx = None
        _tls.stack.pop()
        return False

    @staticmethod
    def current() -> Optional["AutoCast"]:
        stack = getattr(_tls, "stack", None)
        return stack[-1] if stack else None

    def get_forward_dtype(self, op: str, input_dtype=torch.float32):
        return self.registry.get_forward_dtype(op, self.cfg, input_dtype)

    def get_backward_dtype(self, op: str, input_dtype=torch.float32):
        return self.registry.get_backward_dtype(op, self.cfg, input_dtype)

    def cast(self, t: torch.Tensor, op: str) -> torch.Tensor:
        if not t.is_floating_point():
            return t
        dt = self.get_forward_dtype(op, t.dtype)
        return t if t.dtype == dt else t.to(dt)


# ------------------------------------------------------------------ kernel dtype selection
@dataclass
class KernelCapability:
    dtype: torch.dtype
    tensor_cores: bool = False
    perf_factor: float = 1.0
    available: bool = True


class KernelRegistry:
    """Which dtype variants of each operation this build ships for sm_100a."""

    def __init__(self):
        self._caps: Dict[str, List[KernelCapability]] = {}
        self.register_default_capabilities()

    def register(self, op: str, cap: KernelCapability):
        self._caps.setdefault(op.lower(), []).append(cap)

    def register_default_capabilities(self):
        for op in ("linear", "matmul", "attention", "conv2d"):
            self.register(op, KernelCapability(torch.bfloat16, True, 16.0))
            self.register(op, KernelCapability(torch.float32, False, 1.0))
        for op in ("layernorm", "rmsnorm", "softmax", "cross_entropy", "gelu", "relu", "swiglu", "add", "mul", "embedding"):
            self.register(op, KernelCapability(torch.bfloat16, False, 2.0))
            self.register(op, KernelCapability(torch.float32, False, 1.0))
        self.register("adamw", KernelCapability(torch.float32, False, 1.0))

    def capabilities(self, op: str) -> List[KernelCapability]:
        return self._caps.get(op.lower(), [])


class KernelSelector:
    def __init__(self, registry: Optional[KernelRegistry] = None):
        self.registry = registry or KernelRegistry()

    def get_kernel_dtype(self, op: str, requested: torch.dtype) -> torch.dtype:
        caps = [c for c in self.registry.capabilities(op) if c.available]
        if any(c.dtype == requested for c in caps):
            return requested
        if requested == torch.float16 and any(c.dtype == torch.bfloat16 for c in caps):
            return torch.bfloat16
        return torch.float32

    def select_best_kernel(self, op: str) -> Optional[KernelCapability]:
        caps = [c for c in self.registry.capabilities(op) if c.available]
        return max(caps, key=lambda c: c.perf_factor, default=None)


# ------------------------------------------------------------------ gradient utilities
class GradientUtils:
    @staticmethod
    def unscale(grads: Iterable[torch.Tensor], scale: float) -> List[torch.Tensor]:
        return [None if g is None else g / scale for g in grads]

    @staticmethod
    def unscale_in_place(grads: Iterable[torch.Tensor], scale: float):
        for g in grads:
            if g is not None:
                g.div_(scale)

    @staticmethod
    def check_overflow(grads: Iterable[torch.Tensor]) -> bool:
        return any(g is not None and not bool(torch.isfinite(g).all()) for g in grads)

    @staticmethod
    def find_overflow_gradients(named_grads: Dict[str, torch.Tensor]) -> List[str]:
        return [n for n, g in named_grads.items() if g is not None and not bool(torch.isfinite(g).all())]


class GradientClipper:
    @staticmethod
    def clip_by_value(grads: Iterable[torch.Tensor], clip: float):
        if clip <= 0:
            raise ValueError("clip value must be positive")
        for g in grads:
            if g is not None:
                g.clamp_(-clip, clip)

    @staticmethod
    def global_norm(grads: Iterable[torch.Tensor], process_group=None) -> torch.Tensor:
        grads = [g for g in grads if g is not None]
        if not grads:
            return torch.zeros(())
        if grads[0].is_cuda:
            from ..ops import native
            ss = torch.zeros(1, device=grads[0].device)
            dummy = torch.zeros(1, dtype=torch.int32, device=grads[0].device)
            for g in grads:
                native.amp_unscale_check_(g.contiguous(), dummy, sumsq=ss, write_back=False)
        else:
            ss = torch.stack([g.float().pow(2).sum() for g in grads]).sum().reshape(1)
        if process_group is not None and process_group.world_size > 1:
            process_group.all_reduce(ss)
        return ss.sqrt().squeeze(0)

    @staticmethod
    def clip_by_norm(grads: Iterable[torch.Tensor], max_norm: float, process_group=None, eps: float = 1e-6) -> torch.Tensor:
        """Scale all gradients by min(1, max_norm / global_norm); the norm is reduced over
        ``process_group`` when the gradients are shards (the reference's TP clipper uses the
        local norm only, Layers/TensorParallel/TPGradientManager.cs:102-135)."""
        if max_norm <= 0:
            raise ValueError("max_norm must be positive")
        grads = [g for g in grads if g is not None]
        norm = GradientClipper.global_norm(grads, process_group)
        coef = torch.clamp(max_norm / (norm + eps), max=1.0)
        for g in grads:
            g.mul_(coef.to(g.dtype))
        return norm
