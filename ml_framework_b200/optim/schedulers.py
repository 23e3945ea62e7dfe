"""Learning-rate schedulers (the reference's sixteen, src/MLFramework/Schedulers/*.cs) behind one
interface: ``get_lr(step) -> float``, ``step() -> float`` (advance and return the new rate),
``state_dict`` / ``load_state_dict`` (Schedulers/StateDict.cs), plus composition
(``ChainedScheduler`` multiplies factors, ``SequentialScheduler`` switches at milestones) and
per-layer rates (``LayerWiseLRDecay``, ``DiscriminativeLR``). ``LRSchedulerCallback`` steps a
scheduler from a training loop (src/MLFramework/Training/LRSchedulerCallback.cs).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence


class LRScheduler:
    def __init__(self, base_lr: float):
        if base_lr < 0:
            raise ValueError("base_lr must be non-negative")
        self.base_lr = base_lr
        self.step_count = 0

    def get_lr(self, step: int) -> float:
        raise NotImplementedError

    def step(self, metric: Optional[float] = None) -> float:
        self.step_count += 1
        return self.get_lr(self.step_count)

    @property
    def current_lr(self) -> float:
        return self.get_lr(self.step_count)

    def reset(self):
        self.step_count = 0

    def state_dict(self) -> Dict:
        return {k: v for k, v in self.__dict__.items() if isinstance(v, (int, float, bool, str, list, tuple, type(None)))}

    def load_state_dict(self, sd: Dict):
        self.__dict__.update(sd)


class ConstantLR(LRScheduler):
    def get_lr(self, step):
        return self.base_lr


class StepDecay(LRScheduler):
    def __init__(self, base_lr, step_size: int, gamma: float = 0.1):
        super().__init__(base_lr)
        if step_size <= 0:
            raise ValueError("step_size must be positive")
        self.step_size, self.gamma = step_size, gamma

    def get_lr(self, step):
        return self.base_lr * self.gamma ** (step // self.step_size)


class MultiStepDecay(LRScheduler):
    def __init__(self, base_lr, milestones: Sequence[int], gamma: float = 0.1):
        super().__init__(base_lr)
        self.milestones, self.gamma = sorted(milestones), gamma

    def get_lr(self, step):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if step >= m)


class ExponentialDecay(LRScheduler):
    def __init__(self, base_lr, gamma: float):
        super().__init__(base_lr)
        self.gamma = gamma

    def get_lr(self, step):
        return self.base_lr * self.gamma ** step


class CosineAnnealing(LRScheduler):
    def __init__(self, base_lr, t_max: int, eta_min: float = 0.0):
        super().__init__(base_lr)
        if t_max <= 0:
            raise ValueError("t_max must be positive")
        self.t_max, self.eta_min = t_max, eta_min

    def get_lr(self, step):
        s = min(step, self.t_max)
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * s / self.t_max)) / 2


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, base_lr, t_0: int, t_mult: int = 1, eta_min: float = 0.0):
        super().__init__(base_lr)
        if t_0 <= 0 or t_mult < 1:
            raise ValueError("t_0 must be positive and t_mult >= 1")
        self.t_0, self.t_mult, self.eta_min = t_0, t_mult, eta_min

    def get_lr(self, step):
        t_i, t_cur = self.t_0, step
        while t_cur >= t_i:
            t_cur -= t_i
            t_i *= self.t_mult
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t_cur / t_i)) / 2


class PolynomialDecay(LRScheduler):
    def __init__(self, base_lr, total_steps: int, end_lr: float = 0.0, power: float = 1.0):
        super().__init__(base_lr)
        self.total_steps, self.end_lr, self.power = total_steps, end_lr, power

    def get_lr(self, step):
        s = min(step, self.total_steps)
        return (self.base_lr - self.end_lr) * (1 - s / self.total_steps) ** self.power + self.end_lr


class OneCycle(LRScheduler):
    def __init__(self, max_lr, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0,
                 final_div_factor: float = 1e4):
        super().__init__(max_lr)
        self.total_steps, self.pct_start = total_steps, pct_start
        self.initial_lr = max_lr / div_factor
        self.min_lr = self.initial_lr / final_div_factor

    def get_lr(self, step):
        up = max(1, int(self.pct_start * self.total_steps))
        if step <= up:
            return self.initial_lr + (self.base_lr - self.initial_lr) * (1 - math.cos(math.pi * step / up)) / 2
        s = min(step, self.total_steps) - up
        down = max(1, self.total_steps - up)
        return self.min_lr + (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * s / down)) / 2


class CyclicLR(LRScheduler):
    def __init__(self, base_lr, max_lr: float, step_size_up: int, step_size_down: Optional[int] = None,
                 mode: str = "triangular", gamma: float = 1.0):
        super().__init__(base_lr)
        self.max_lr, self.up, self.down = max_lr, step_size_up, step_size_down or step_size_up
        self.mode, self.gamma = mode, gamma

    def get_lr(self, step):
        total = self.up + self.down
        cycle, pos = step // total, step % total
        x = pos / self.up if pos <= self.up else 1 - (pos - self.up) / self.down
        scale = {"triangular": 1.0, "triangular2": 1.0 / (2 ** cycle), "exp_range": self.gamma ** step}[self.mode]
        return self.base_lr + (self.max_lr - self.base_lr) * max(0.0, x) * scale


class LinearWarmup(LRScheduler):
    """Linear ramp from ``start_factor * lr`` to the wrapped scheduler's (or base) rate."""

    def __init__(self, base_lr, warmup_steps: int, after: Optional[LRScheduler] = None, start_factor: float = 0.0):
        super().__init__(base_lr)
        self.warmup_steps, self.after, self.start_factor = warmup_steps, after, start_factor

    def get_lr(self, step):
        if step < self.warmup_steps:
            f = self.start_factor + (1 - self.start_factor) * step / max(1, self.warmup_steps)
            return self.base_lr * f
        return self.after.get_lr(step - self.warmup_steps) if self.after else self.base_lr


class ConstantWarmup(LRScheduler):
    def __init__(self, base_lr, warmup_steps: int, warmup_lr: float, after: Optional[LRScheduler] = None):
        super().__init__(base_lr)
        self.warmup_steps, self.warmup_lr, self.after = warmup_steps, warmup_lr, after

    def get_lr(self, step):
        if step < self.warmup_steps:
            return self.warmup_lr
        return self.after.get_lr(step - self.warmup_steps) if self.after else self.base_lr


class ReduceLROnPlateau(LRScheduler):
    def __init__(self, base_lr, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4,
                 cooldown: int = 0, min_lr: float = 0.0):
        super().__init__(base_lr)
        if factor >= 1.0:
            raise ValueError("factor must be < 1")
        self.mode, self.factor, self.patience, self.threshold = mode, factor, patience, threshold
        self.cooldown, self.min_lr = cooldown, min_lr
        self.lr, self.best, self.bad, self.cool = base_lr, None, 0, 0

    def get_lr(self, step):
        return self.lr

    def step(self, metric: Optional[float] = None) -> float:
        self.step_count += 1
        if metric is None:
            return self.lr
        better = self.best is None or (metric < self.best - self.threshold if self.mode == "min" else metric > self.best + self.threshold)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
        if self.cool > 0:
            self.cool -= 1
            self.bad = 0
        if self.bad > self.patience:
            self.lr = max(self.lr * self.factor, self.min_lr)
            self.cool, self.bad = self.cooldown, 0
        return self.lr


class ChainedScheduler(LRScheduler):
    """Product of the factors ``lr_i(step) / base_i`` of every member, applied to ``base_lr``."""

    def __init__(self, base_lr, schedulers: List[LRScheduler]):
        super().__init__(base_lr)
        self.schedulers = schedulers

    def get_lr(self, step):
        lr = self.base_lr
        for s in self.schedulers:
            lr *= s.get_lr(step) / s.base_lr if s.base_lr else 0.0
        return lr


class SequentialScheduler(LRScheduler):
    def __init__(self, schedulers: List[LRScheduler], milestones: Sequence[int]):
        super().__init__(schedulers[0].base_lr)
        if len(milestones) != len(schedulers) - 1:
            raise ValueError("need len(schedulers) - 1 milestones")
        self.schedulers, self.milestones = schedulers, list(milestones)

    def get_lr(self, step):
        start = 0
        for i, m in enumerate(self.milestones):
            if step < m:
                return self.schedulers[i].get_lr(step - start)
            start = m
        return self.schedulers[-1].get_lr(step - start)


class LayerWiseLRDecay:
    """lr(layer) = base * decay ** (num_layers - 1 - layer) (deeper layers learn faster)."""

    def __init__(self, base_lr: float, num_layers: int, decay: float = 0.8):
        self.base_lr, self.num_layers, self.decay = base_lr, num_layers, decay

    def lr_for_layer(self, layer: int) -> float:
        return self.base_lr * self.decay ** (self.num_layers - 1 - layer)

    def param_groups(self, named_params, layer_of: Callable[[str], int]):
        groups: Dict[int, list] = {}
        for n, p in named_params:
            groups.setdefault(layer_of(n), []).append(p)
        return [{"params": ps, "lr": self.lr_for_layer(l)} for l, ps in sorted(groups.items())]


class DiscriminativeLR:
    """Explicit per-group multipliers by name prefix."""

    def __init__(self, base_lr: float, multipliers: Dict[str, float], default: float = 1.0):
        self.base_lr, self.multipliers, self.default = base_lr, multipliers, default

    def lr_for(self, name: str) -> float:
        best = max((k for k in self.multipliers if name.startswith(k)), key=len, default=None)
        return self.base_lr * (self.multipliers[best] if best is not None else self.default)


class Callback:
    """Training-loop callback base (src/MLFramework/Training/Callback.cs)."""

    def on_train_begin(self, ctx=None): ...
    def on_epoch_begin(self, epoch, ctx=None): ...
    def on_batch_end(self, batch, ctx=None): ...
    def on_epoch_end(self, epoch, ctx=None): ...
    def on_train_end(self, ctx=None): ...


class LRSchedulerCallback(Callback):
    def __init__(self, scheduler: LRScheduler, optimizer, per_batch: bool = True):
        self.scheduler, self.optimizer, self.per_batch = scheduler, optimizer, per_batch

    def on_batch_end(self, batch, ctx=None):
        if self.per_batch:
            self.optimizer.set_learning_rate(self.scheduler.step())

    def on_epoch_end(self, epoch, ctx=None):
        if not self.per_batch:
            metric = getattr(ctx, "val_loss", None) if ctx is not None else None
            self.optimizer.set_learning_rate(self.scheduler.step(metric))
