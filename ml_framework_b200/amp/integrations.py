"""AMP integration helpers: optimizer wrapper that reports whether a step was applied, scaler context, overflow
statistics, explicit casts, an autograd function with its own precision policy, dtype helpers.

Reference (src/MLFramework/Amp/): Integrations/AmpOptimizerWrapper.cs:68-119 (``Step`` returns whether the update was
applied), GradScalerContext.cs, OverflowStats.cs, ScaleFactor.cs, AmpCast.cs, Integrations/{AmpAutogradFunction,
AmpAutogradHelper, AmpOptimizerHelper}.cs, AmpTensorExtensions.cs, TensorDtypeExtensions.cs, AutoCastContext.cs
(``Fp16`` / ``Bf16`` constructors), OpPrecisionRule.cs.

The training engine keeps scale, overflow flag and skip decision on the device (no host round trip per step); the
wrapper here is the explicit, host-visible form of the same loop for users who drive their own optimizer: its
``step`` reads the flag back (one small device-to-host copy) because its contract is to RETURN the decision.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .autocast import AmpConfig, AutoCast, OpPrecision
from .grad_scaler import DynamicLossScaler, GradScaler, StaticLossScaler

LOW_PRECISION = (torch.float16, torch.bfloat16)


# ------------------------------------------------------------------ statistics
@dataclass
class OverflowStats:
    total_steps: int = 0
    overflow_steps: int = 0
    consecutive_overflows: int = 0
    max_consecutive_overflows: int = 0
    last_overflow_step: Optional[int] = None
    overflow_parameters: Dict[str, int] = field(default_factory=dict)      # name -> times it held a non-finite gradient

    @property
    def overflow_rate(self) -> float:
        return self.overflow_steps / self.total_steps if self.total_steps else 0.0

    def record(self, overflow: bool, names: Sequence[str] = ()):
        self.total_steps += 1
        if overflow:
            self.overflow_steps += 1
            self.consecutive_overflows += 1
            self.max_consecutive_overflows = max(self.max_consecutive_overflows, self.consecutive_overflows)
            self.last_overflow_step = self.total_steps
            for n in names:
                self.overflow_parameters[n] = self.overflow_parameters.get(n, 0) + 1
        else:
            self.consecutive_overflows = 0


@dataclass(frozen=True)
class ScaleFactor:
    """A loss scale as a value object: positive, finite, with the arithmetic the scaler needs."""
    value: float

    def __post_init__(self):
        if not (self.value > 0 and self.value < float("inf")):
            raise ValueError(f"a scale factor is positive and finite, got {self.value}")

    @property
    def inverse(self) -> float:
        return 1.0 / self.value

    def grow(self, factor: float = 2.0, maximum: float = 2.0 ** 24) -> "ScaleFactor":
        return ScaleFactor(min(self.value * factor, maximum))

    def backoff(self, factor: float = 0.5, minimum: float = 1.0) -> "ScaleFactor":
        return ScaleFactor(max(self.value * factor, minimum))

    def is_power_of_two(self) -> bool:
        m = self.value
        while m > 1:
            m /= 2
        while m < 1:
            m *= 2
        return m == 1.0


# ------------------------------------------------------------------ casts
class AmpCast:
    @staticmethod
    def to(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """Floating-point tensors change type; integer and boolean tensors pass through."""
        return t.to(dtype) if t.is_floating_point() and t.dtype != dtype else t

    @staticmethod
    def to_fp32(t): return AmpCast.to(t, torch.float32)
    @staticmethod
    def to_fp16(t): return AmpCast.to(t, torch.float16)
    @staticmethod
    def to_bf16(t): return AmpCast.to(t, torch.bfloat16)

    @staticmethod
    def cast_all(xs, dtype: torch.dtype):
        if isinstance(xs, torch.Tensor):
            return AmpCast.to(xs, dtype)
        if isinstance(xs, (list, tuple)):
            return type(xs)(AmpCast.cast_all(x, dtype) for x in xs)
        if isinstance(xs, dict):
            return {k: AmpCast.cast_all(v, dtype) for k, v in xs.items()}
        return xs

    @staticmethod
    def promote(*ts: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        """The widest floating-point type among the arguments for all of them (fp32 beats bf16 / fp16; bf16 and fp16
        together give fp32, since neither contains the other)."""
        fl = [t.dtype for t in ts if t.is_floating_point()]
        if not fl:
            return ts
        target = fl[0]
        for d in fl[1:]:
            target = torch.promote_types(target, d)
        return tuple(AmpCast.to(t, target) for t in ts)


def is_low_precision(t: torch.Tensor) -> bool:
    return t.dtype in LOW_PRECISION


def dtype_bytes(dt: torch.dtype) -> int:
    return torch.empty(0, dtype=dt).element_size()


def dtype_range(dt: torch.dtype) -> Tuple[float, float, float]:
    """(largest finite value, smallest normal, machine epsilon)."""
    fi = torch.finfo(dt)
    return float(fi.max), float(fi.tiny), float(fi.eps)


def would_overflow(t: torch.Tensor, dtype: torch.dtype) -> bool:
    """True when casting ``t`` to ``dtype`` would produce an infinity."""
    return bool(t.detach().abs().max() > torch.finfo(dtype).max) if t.numel() else False


def autocast_fp16(**kw) -> AutoCast:
    return AutoCast(AmpConfig.create_fp16(), **kw)


def autocast_bf16(**kw) -> AutoCast:
    return AutoCast(AmpConfig.create_bf16(), **kw)


@dataclass
class OpPrecisionRule:
    """A rule of the precision registry as data: exact name or ``prefix*`` pattern, the precision, and its priority
    (a later, higher-priority rule for the same op wins)."""
    pattern: str
    precision: OpPrecision
    priority: int = 0

    def matches(self, op: str) -> bool:
        return op.startswith(self.pattern[:-1]) if self.pattern.endswith("*") else op == self.pattern

    @staticmethod
    def resolve(rules: Sequence["OpPrecisionRule"], op: str, default: OpPrecision = OpPrecision.KEEP) -> OpPrecision:
        best = None
        for r in rules:
            if r.matches(op) and (best is None or r.priority >= best.priority):
                best = r
        return best.precision if best is not None else default


# ------------------------------------------------------------------ autograd function with a precision policy
class AmpAutogradFunction(torch.autograd.Function):
    """Base for custom functions under mixed precision: subclasses implement ``amp_forward(ctx, *inputs)`` and
    ``amp_backward(ctx, *grads)``; floating-point inputs arrive in ``forward_dtype``, incoming gradients in
    ``backward_dtype``, and the gradients returned are cast back to each input's own dtype."""
    forward_dtype: Optional[torch.dtype] = None      # None: leave inputs as they are
    backward_dtype: Optional[torch.dtype] = torch.float32

    @classmethod
    def forward(cls, ctx, *inputs):
        ctx._in_dtypes = [x.dtype if isinstance(x, torch.Tensor) else None for x in inputs]
        if cls.forward_dtype is not None:
            inputs = tuple(AmpCast.to(x, cls.forward_dtype) if isinstance(x, torch.Tensor) else x for x in inputs)
        return cls.amp_forward(ctx, *inputs)

    @classmethod
    def backward(cls, ctx, *grads):
        if cls.backward_dtype is not None:
            grads = tuple(AmpCast.to(g, cls.backward_dtype) if isinstance(g, torch.Tensor) else g for g in grads)
        out = cls.amp_backward(ctx, *grads)
        out = out if isinstance(out, tuple) else (out,)
        return tuple(g.to(dt) if isinstance(g, torch.Tensor) and dt is not None and dt.is_floating_point else g for g, dt in zip(out, ctx._in_dtypes))

    @staticmethod
    def amp_forward(ctx, *inputs):
        raise NotImplementedError

    @staticmethod
    def amp_backward(ctx, *grads):
        raise NotImplementedError


class AmpAutogradHelper:
    @staticmethod
    def run_in_fp32(fn: Callable[..., torch.Tensor], *inputs: torch.Tensor) -> torch.Tensor:
        """``fn`` on fp32 copies of the inputs, result cast back to the first input's dtype (autograd sees the casts)."""
        out = fn(*[AmpCast.to_fp32(x) for x in inputs])
        return out.to(inputs[0].dtype) if inputs and isinstance(out, torch.Tensor) and inputs[0].is_floating_point() else out

    @staticmethod
    def nonfinite_parameters(named_params: Iterable[Tuple[str, torch.Tensor]]) -> List[str]:
        return [n for n, p in named_params if p.grad is not None and not bool(torch.isfinite(p.grad).all())]


# ------------------------------------------------------------------ optimizer wrapper
class AmpOptimizerWrapper:
    """Wraps any ``torch.optim`` optimizer with loss scaling. ``backward(loss)`` scales and differentiates;
    ``step()`` unscales the gradients, checks them (across the process group when one is given), skips the update on
    overflow, updates the scale, and returns whether the update was applied."""

    def __init__(self, optimizer: torch.optim.Optimizer, scaler=None, process_group=None, max_grad_norm: Optional[float] = None,
                 named_parameters: Optional[Iterable[Tuple[str, torch.Tensor]]] = None):
        self.optimizer = optimizer
        self.scaler = scaler if scaler is not None else DynamicLossScaler()
        self.pg, self.max_grad_norm = process_group, max_grad_norm
        self.stats = OverflowStats()
        self._names = {id(p): n for n, p in (named_parameters or [])}

    def _params(self) -> List[torch.Tensor]:
        return [p for g in self.optimizer.param_groups for p in g["params"]]

    @property
    def scale(self) -> float:
        return float(self.scaler.scale)

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return self.scaler.scale_loss(loss)

    def backward(self, loss: torch.Tensor, **kw):
        self.scale_loss(loss).backward(**kw)

    def zero_grad(self, set_to_none: bool = True):
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def step(self, closure=None) -> bool:
        grads = [p.grad for p in self._params() if p.grad is not None]
        inv = 1.0 / self.scale
        overflow = False
        for g in grads:
            g.mul_(inv)
            if not bool(torch.isfinite(g).all()):
                overflow = True
        if self.pg is not None and self.pg.world_size > 1:
            from ..dist.process_group import ReduceOp
            flag = torch.tensor([1.0 if overflow else 0.0], device=grads[0].device if grads else "cpu")
            self.pg.all_reduce(flag, ReduceOp.MAX)
            overflow = bool(flag.item() > 0)
        bad = [self._names.get(id(p), f"param{i}") for i, p in enumerate(self._params())
               if p.grad is not None and not bool(torch.isfinite(p.grad).all())] if overflow else []
        self.stats.record(overflow, bad)
        self.scaler.found_inf.fill_(1 if overflow else 0)
        if not overflow:
            if self.max_grad_norm is not None:
                torch.nn.utils.clip_grad_norm_(self._params(), self.max_grad_norm)
            self.optimizer.step(closure) if closure is not None else self.optimizer.step()
        self.scaler.update()
        return not overflow

    def state_dict(self) -> Dict[str, Any]:
        return {"optimizer": self.optimizer.state_dict(), "scaler": self.scaler.state_dict(), "stats": dict(self.stats.__dict__)}

    def load_state_dict(self, sd: Dict[str, Any]):
        self.optimizer.load_state_dict(sd["optimizer"])
        self.scaler.load_state_dict(sd["scaler"])
        for k, v in sd.get("stats", {}).items():
            setattr(self.stats, k, v)


class AmpOptimizerHelper:
    @staticmethod
    def wrap(optimizer, config: Optional[AmpConfig] = None, device="cpu", **kw) -> AmpOptimizerWrapper:
        c = config or AmpConfig()
        if not c.loss_scaling:
            return AmpOptimizerWrapper(optimizer, StaticLossScaler(1.0, device), **kw)
        from .grad_scaler import DynamicScalerConfig
        return AmpOptimizerWrapper(optimizer, DynamicLossScaler(DynamicScalerConfig(initial_scale=c.initial_loss_scale, growth_interval=c.growth_interval), device), **kw)

    @staticmethod
    def master_copy(params: Iterable[torch.nn.Parameter]) -> List[torch.Tensor]:
        """fp32 copies of low-precision parameters (what an optimizer updates when the model itself is bf16 / fp16)."""
        return [p.detach().float().clone().requires_grad_(True) for p in params]

    @staticmethod
    def copy_master_to_model(master: Sequence[torch.Tensor], params: Iterable[torch.nn.Parameter]):
        with torch.no_grad():
            for m, p in zip(master, params):
                p.copy_(m.to(p.dtype))

    @staticmethod
    def copy_grads_to_master(params: Iterable[torch.nn.Parameter], master: Sequence[torch.Tensor]):
        for p, m in zip(params, master):
            m.grad = None if p.grad is None else p.grad.detach().float()


@contextlib.contextmanager
def grad_scaler_context(scaler: Optional[GradScaler] = None, device="cpu"):
    """``with grad_scaler_context() as ctx:`` - ``ctx.scale(loss)`` inside the block; on exit the scale is updated
    once (GradScalerContext.cs: scope-bound scaler use)."""
    gs = scaler or GradScaler(device=device)

    class _Ctx:
        scaler = gs
        steps = 0

        def scale(self, loss):
            return gs.scale_loss(loss)

        def step(self, optimizer, **kw):
            self.steps += 1
            return gs.step(optimizer, **kw)
    c = _Ctx()
    try:
        yield c
    finally:
        gs.update()
