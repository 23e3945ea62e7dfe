"""Autograd utilities on top of PyTorch's engine.

* ``CustomFunction`` / ``FunctionContext``: the reference's user-defined forward/backward API
  (src/Autograd/CustomFunction.cs:18-51, FunctionContext.cs:33) as a thin shim over
  ``torch.autograd.Function``.
* ``GradientTape``: record / watch / gradient with nested tapes and retention policy
  (src/MLFramework/Autograd/GradientTape.cs:105-245).
* Higher-order derivatives: ``gradient``, ``jacobian`` (auto / forward / reverse mode), ``hessian``
  (full, diagonal, numerical), ``hvp``, ``jvp``, ``vjp`` (Autograd.cs:25-215, Hessian.cs:233-418,
  Jacobian.cs:211) through ``torch.func``.
* ``GradientChecker`` (finite differences, src/Autograd/GradientChecker.cs:22) and
  ``GradientValidator`` (shape / dtype / NaN / Inf, GradientValidator.cs:24-306) with the reference's
  exception types.
* ``GradientAccumulator`` (micro-batch accumulation, MLFramework/Autograd/GradientAccumulator.cs:55-121)
  and batch-size-aware scaling (GradientScaling.cs:21-112).
* Example functions: ``StableSoftmax``, ``ClampedMSELoss``, ``STEBinary`` (src/Autograd/Functions/*.cs).
"""
from __future__ import annotations

import enum
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch
import torch.func as tf


# ------------------------------------------------------------------ custom functions
class FunctionContext:
    def __init__(self, inner):
        self._ctx = inner
        self.extras: Dict[str, object] = {}

    def save_for_backward(self, *tensors):
        self._ctx.save_for_backward(*tensors)

    @property
    def saved_tensors(self):
        return self._ctx.saved_tensors


class CustomFunction:
    """Subclass and implement ``forward(ctx, *inputs)`` and ``backward(ctx, *grad_outputs)``."""

    def forward(self, ctx: FunctionContext, *inputs):
        raise NotImplementedError

    def backward(self, ctx: FunctionContext, *grad_outputs):
        raise NotImplementedError

    def apply(self, *inputs):
        outer = self

        class _Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *args):
                c = FunctionContext(ctx)
                ctx._mlf = c
                return outer.forward(c, *args)

            @staticmethod
            def backward(ctx, *grads):
                g = outer.backward(ctx._mlf, *grads)
                return g if isinstance(g, tuple) else (g,)
        return _Fn.apply(*inputs)

    def apply_many(self, batches: Sequence[Sequence[torch.Tensor]]):
        return [self.apply(*b) for b in batches]


class AutogradEngine:
    """Registry of named custom functions (src/Autograd/AutogradEngine.cs:36-117)."""

    def __init__(self):
        self._fns: Dict[str, CustomFunction] = {}

    def register_custom_function(self, name: str, fn: CustomFunction):
        if name in self._fns:
            raise ValueError(f"function {name!r} already registered")
        self._fns[name] = fn

    def apply(self, name: str, *inputs):
        return self._fns[name].apply(*inputs)

    @staticmethod
    def backward(loss: torch.Tensor, retain_graph: bool = False):
        loss.backward(retain_graph=retain_graph)


class StableSoftmax(CustomFunction):
    def __init__(self, dim: int = -1):
        self.dim = dim

    def forward(self, ctx, x):
        y = torch.softmax(x - x.amax(self.dim, keepdim=True), self.dim)
        ctx.save_for_backward(y)
        return y

    def backward(self, ctx, g):
        (y,) = ctx.saved_tensors
        return y * (g - (g * y).sum(self.dim, keepdim=True))


class ClampedMSELoss(CustomFunction):
    def __init__(self, clamp: float = 1.0):
        self.clamp = clamp

    def forward(self, ctx, pred, target):
        d = (pred - target).clamp(-self.clamp, self.clamp)
        ctx.save_for_backward(pred, target)
        return (d * d).mean()

    def backward(self, ctx, g):
        pred, target = ctx.saved_tensors
        d = pred - target
        inside = (d.abs() <= self.clamp).to(d.dtype)
        grad = 2.0 * d * inside / d.numel() * g
        return grad, -grad


class STEBinary(CustomFunction):
    """sign(x) forward, straight-through (identity inside [-1, 1]) backward."""

    def forward(self, ctx, x):
        ctx.save_for_backward(x)
        return torch.where(x >= 0, torch.ones_like(x), -torch.ones_like(x))

    def backward(self, ctx, g):
        (x,) = ctx.saved_tensors
        return g * (x.abs() <= 1).to(g.dtype)


# ------------------------------------------------------------------ tape
class GradientRetentionPolicy(enum.Enum):
    KEEP = "keep"
    DISCARD = "discard"


class GradientTape:
    _stack: List["GradientTape"] = []

    def __init__(self, persistent: bool = False, retention: GradientRetentionPolicy = GradientRetentionPolicy.DISCARD):
        self.persistent, self.retention = persistent, retention
        self.watched: List[torch.Tensor] = []
        self._used = False

    def __enter__(self):
        GradientTape._stack.append(self)
        self._grad_ctx = torch.enable_grad()
        self._grad_ctx.__enter__()
        return self

    def __exit__(self, *exc):
        self._grad_ctx.__exit__(*exc)
        GradientTape._stack.pop()
        return False

    def watch(self, t: torch.Tensor) -> torch.Tensor:
        if not t.requires_grad:
            t.requires_grad_(True)
        self.watched.append(t)
        return t

    def gradient(self, target: torch.Tensor, sources, create_graph: bool = False):
        if self._used and not self.persistent:
            raise RuntimeError("a non-persistent tape can compute gradients only once")
        self._used = True
        single = isinstance(sources, torch.Tensor)
        srcs = [sources] if single else list(sources)
        grads = torch.autograd.grad(target, srcs, retain_graph=self.persistent or create_graph, create_graph=create_graph,
                                    allow_unused=True)
        return grads[0] if single else list(grads)


# ------------------------------------------------------------------ higher order
def gradient(f: Callable, x: torch.Tensor) -> torch.Tensor:
    return tf.grad(f)(x)


def jacobian(f: Callable, x: torch.Tensor, mode: str = "auto") -> torch.Tensor:
    if mode == "auto":
        probe = f(x)
        mode = "forward" if x.numel() <= probe.numel() else "reverse"
    return tf.jacfwd(f)(x) if mode == "forward" else tf.jacrev(f)(x)


def hessian(f: Callable, x: torch.Tensor) -> torch.Tensor:
    return tf.hessian(f)(x)


def hessian_diagonal(f: Callable, x: torch.Tensor) -> torch.Tensor:
    flat = x.reshape(-1)
    out = torch.empty_like(flat)
    for i in range(flat.numel()):
        e = torch.zeros_like(flat)
        e[i] = 1.0
        out[i] = hvp(f, x, e.view_as(x)).reshape(-1)[i]
    return out.view_as(x)


def hessian_numerical(f: Callable, x: torch.Tensor, eps: float = 1e-3) -> torch.Tensor:
    n = x.numel()
    H = torch.zeros(n, n, dtype=x.dtype)
    flat = x.reshape(-1).clone()

    def at(v):
        return float(f(v.view_as(x)))
    for i in range(n):
        for j in range(i, n):
            ei, ej = torch.zeros(n, dtype=x.dtype), torch.zeros(n, dtype=x.dtype)
            ei[i], ej[j] = eps, eps
            v = (at(flat + ei + ej) - at(flat + ei - ej) - at(flat - ei + ej) + at(flat - ei - ej)) / (4 * eps * eps)
            H[i, j] = H[j, i] = v
    return H


def hvp(f: Callable, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    return tf.jvp(tf.grad(f), (x,), (v,))[1]


def jvp(f: Callable, x: torch.Tensor, v: torch.Tensor):
    return tf.jvp(f, (x,), (v,))


def vjp(f: Callable, x: torch.Tensor, v: torch.Tensor):
    out, fn = tf.vjp(f, x)
    return out, fn(v)[0]


# ------------------------------------------------------------------ checking / validation
class GradientShapeException(ValueError):
    pass


class GradientTypeException(TypeError):
    pass


class GradientNaNException(ArithmeticError):
    pass


class GradientInfException(ArithmeticError):
    pass


class GradientValidator:
    @staticmethod
    def validate(param: torch.Tensor, grad: torch.Tensor, name: str = ""):
        if grad.shape != param.shape:
            raise GradientShapeException(f"{name}: gradient shape {tuple(grad.shape)} != parameter shape {tuple(param.shape)}")
        if grad.dtype != param.dtype:
            raise GradientTypeException(f"{name}: gradient dtype {grad.dtype} != parameter dtype {param.dtype}")
        if torch.isnan(grad).any():
            raise GradientNaNException(f"{name}: gradient contains NaN")
        if torch.isinf(grad).any():
            raise GradientInfException(f"{name}: gradient contains Inf")
        return True


class GradientChecker:
    @staticmethod
    def check_gradients(f: Callable, inputs: Sequence[torch.Tensor], eps: float = 1e-4, atol: float = 1e-3, rtol: float = 1e-2):
        """Compare analytic gradients of scalar ``f(*inputs)`` with central differences (float64)."""
        xs = [x.detach().double().requires_grad_(True) for x in inputs]
        f(*xs).backward()
        worst = 0.0
        for i, x in enumerate(xs):
            num = torch.zeros_like(x)
            flat, nflat = x.detach().reshape(-1), num.reshape(-1)
            for k in range(flat.numel()):
                orig = flat[k].item()
                flat[k] = orig + eps
                fp = float(f(*[xx.detach() for xx in xs]))
                flat[k] = orig - eps
                fm = float(f(*[xx.detach() for xx in xs]))
                flat[k] = orig
                nflat[k] = (fp - fm) / (2 * eps)
            err = (x.grad - num).abs()
            tol = atol + rtol * num.abs()
            worst = max(worst, float((err - tol).max()))
            if (err > tol).any():
                return False, worst
        return True, worst


# ------------------------------------------------------------------ accumulation
class GradientAccumulator:
    def __init__(self, params: Iterable[torch.nn.Parameter], accumulation_steps: int = 1):
        if accumulation_steps <= 0:
            raise ValueError("accumulation_steps must be positive")
        self.params, self.steps, self.count = list(params), accumulation_steps, 0
        self._acc: List[Optional[torch.Tensor]] = [None] * len(self.params)

    def step(self) -> bool:
        """Fold the current ``.grad`` into the accumulator; True when a full batch is ready."""
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            self._acc[i] = p.grad.detach().clone() if self._acc[i] is None else self._acc[i] + p.grad
            p.grad = None
        self.count += 1
        return self.count >= self.steps

    def apply_gradients(self, average: bool = True):
        for p, g in zip(self.params, self._acc):
            if g is not None:
                p.grad = g / self.steps if average else g
        self._acc, self.count = [None] * len(self.params), 0


def scale_by_batch_size(grads: Sequence[torch.Tensor], batch_size: int, reference_batch_size: int):
    return [g * (reference_batch_size / batch_size) for g in grads]


def weighted_average(grad_sets: Sequence[Sequence[torch.Tensor]], weights: Sequence[float]):
    tot = float(sum(weights))
    return [sum(w * g for w, g in zip(weights, gs)) / tot for gs in zip(*grad_sets)]


# ------------------------------------------------------------------ accumulation with varying batch sizes
class DynamicBatchAccumulator:
    """Accumulates per-batch *mean* gradients of batches of different sizes into the gradient of their union:
    each contribution is weighted by its batch size and the result is divided by the accumulated size
    (src/MLFramework/Autograd/DynamicBatchAccumulator.cs:74-150). ``target_batch_size == 0`` leaves completion to
    the caller (fixed step count)."""

    def __init__(self, target_batch_size: int = 0):
        if target_batch_size < 0:
            raise ValueError("target_batch_size cannot be negative")
        self.target_batch_size = target_batch_size
        self._sum: Optional[torch.Tensor] = None
        self.accumulated_batch_size = 0
        self.current_step = 0
        self.accumulation_count = 0

    def accumulate(self, batch_gradient: torch.Tensor, batch_size: int):
        if batch_size < 1:
            raise ValueError("batch size must be at least 1")
        contrib = batch_gradient.detach() * float(batch_size)
        if self._sum is None:
            self._sum = contrib.clone()
        elif self._sum.shape != contrib.shape:
            raise RuntimeError("gradient shape mismatch in accumulation")
        else:
            self._sum += contrib
        self.accumulated_batch_size += batch_size
        self.current_step += 1
        self.accumulation_count += 1

    def is_complete(self) -> bool:
        return self.target_batch_size > 0 and self.accumulated_batch_size >= self.target_batch_size

    def get_accumulated_gradient(self) -> torch.Tensor:
        if self._sum is None:
            raise RuntimeError("nothing accumulated")
        return self._sum / float(self.accumulated_batch_size)

    @property
    def accumulated_gradient(self) -> Optional[torch.Tensor]:
        return None if self._sum is None else self.get_accumulated_gradient()

    def get_progress(self) -> float:
        if self.target_batch_size <= 0:
            return 0.0
        return min(1.0, self.accumulated_batch_size / self.target_batch_size)

    def set_target_batch_size(self, n: int):
        if n < 0:
            raise ValueError("target_batch_size cannot be negative")
        self.target_batch_size = n

    def reset(self):
        self._sum, self.accumulated_batch_size, self.current_step = None, 0, 0


class GradientAccumulatorDynamic:
    """Named gradient slots whose tensors may have symbolic (dynamic) shapes: a slot accepts a gradient whose
    concrete shape is compatible with the slot's symbolic shape (``None`` / ``-1`` dimensions match anything) and
    sums it into the running total (src/MLFramework/Autograd/GradientAccumulatorDynamic.cs:36-265, whose AddGradients
    is a placeholder returning the first operand; here the sum is real). Gradients of different concrete sizes in a
    dynamic dimension are summed after zero-padding to the largest."""

    def __init__(self):
        self._slots: Dict[str, Dict] = {}
        self._closed = False

    @staticmethod
    def _compatible(shape, sym) -> bool:
        if sym is None:
            return True
        sym = tuple(sym)
        return len(shape) == len(sym) and all(s is None or s == -1 or isinstance(s, str) or int(s) == d for d, s in zip(shape, sym))

    def accumulate(self, identifier: str, grad: torch.Tensor, shape=None):
        if self._closed:
            raise RuntimeError("accumulator is disposed")
        if identifier is None or grad is None:
            raise ValueError("identifier and gradient are required")
        if not self._compatible(tuple(grad.shape), shape):
            raise ValueError(f"gradient of shape {tuple(grad.shape)} does not match the symbolic shape {tuple(shape)}")
        slot = self._slots.get(identifier)
        g = grad.detach()
        if slot is None:
            self._slots[identifier] = {"grad": g.clone(), "shape": None if shape is None else tuple(shape), "count": 1}
            return
        if not self._compatible(tuple(g.shape), slot["shape"]):
            raise ValueError(f"gradient of shape {tuple(g.shape)} does not match slot {identifier!r} of shape {slot['shape']}")
        acc = slot["grad"]
        if acc.shape != g.shape:
            tgt = tuple(max(a, b) for a, b in zip(acc.shape, g.shape))

            def pad(t):
                out = t.new_zeros(tgt)
                out[tuple(slice(0, d) for d in t.shape)] = t
                return out
            acc, g = pad(acc), pad(g)
        slot["grad"] = acc + g
        slot["count"] += 1

    def accumulate_batched(self, identifier: str, grads: Sequence[torch.Tensor], shapes: Sequence):
        if len(grads) != len(shapes):
            raise ValueError(f"gradients and shapes must have the same length, got {len(grads)} and {len(shapes)}")
        for g, s in zip(grads, shapes):
            self.accumulate(identifier, g, s)

    def get_accumulated(self, identifier: str, shape=None) -> Optional[torch.Tensor]:
        slot = self._slots.get(identifier)
        if slot is None:
            return None
        if shape is not None and not self._compatible(tuple(slot["grad"].shape), shape):
            return None
        return slot["grad"]

    def get_accumulation_count(self, identifier: str) -> int:
        slot = self._slots.get(identifier)
        return 0 if slot is None else slot["count"]

    def get_identifiers(self) -> List[str]:
        return list(self._slots)

    def has_gradient(self, identifier: str) -> bool:
        return identifier in self._slots

    def remove(self, identifier: str) -> bool:
        return self._slots.pop(identifier, None) is not None

    def reset(self):
        self._slots.clear()

    @property
    def count(self) -> int:
        return len(self._slots)

    def dispose(self):
        self._slots.clear()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()


class VariableBatchScheduler:
    """A fixed schedule of micro-batch sizes for one accumulation window
    (src/MLFramework/Autograd/VariableBatchScheduler.cs:38-160)."""

    def __init__(self, *batch_sizes):
        sched = list(batch_sizes[0]) if len(batch_sizes) == 1 and isinstance(batch_sizes[0], (list, tuple)) else list(batch_sizes)
        if not sched or any(int(b) < 1 for b in sched):
            raise ValueError("the schedule needs at least one batch size and every size must be at least 1")
        self.batch_schedule = [int(b) for b in sched]
        self.current_step = 0

    @property
    def total_steps(self) -> int:
        return len(self.batch_schedule)

    @property
    def effective_batch_size(self) -> int:
        return sum(self.batch_schedule)

    @property
    def is_complete(self) -> bool:
        return self.current_step >= len(self.batch_schedule)

    def get_current_batch_size(self) -> int:
        if self.is_complete:
            raise RuntimeError("the schedule is complete")
        return self.batch_schedule[self.current_step]

    def get_remaining_steps(self) -> int:
        return max(0, len(self.batch_schedule) - self.current_step)

    def get_effective_batch_size(self, window_size: int) -> int:
        if window_size < 1:
            raise ValueError("window size must be at least 1")
        return sum(self.batch_schedule[self.current_step:self.current_step + window_size])

    def advance(self) -> bool:
        if self.is_complete:
            return False
        self.current_step += 1
        return True

    def get_accumulated_batch_size(self) -> int:
        return sum(self.batch_schedule[:self.current_step])

    def get_progress(self) -> float:
        return self.current_step / len(self.batch_schedule)

    def reset(self):
        self.current_step = 0


class AccumulationContext:
    """Counts micro-steps towards ``target_steps`` and scales registered tensors by ``1 / target_steps`` when ready
    (src/MLFramework/Autograd/AccumulationContext.cs:39-90)."""

    def __init__(self, target_steps: int):
        if target_steps < 1:
            raise ValueError("target_steps must be at least 1")
        self.target_steps, self.accumulation_steps = target_steps, 0
        self._tensors: List[torch.Tensor] = []

    @property
    def is_ready(self) -> bool:
        return self.accumulation_steps >= self.target_steps

    @property
    def scaling_factor(self) -> float:
        return 1.0 / self.target_steps

    def register_tensor(self, t: torch.Tensor):
        self._tensors.append(t)

    def step(self):
        self.accumulation_steps += 1

    def reset(self):
        self.accumulation_steps = 0
        self._tensors.clear()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.reset()
