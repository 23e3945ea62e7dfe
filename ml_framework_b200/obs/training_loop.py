"""Training loop with phase hooks.

Reference: src/MLFramework.Visualization/Hooks/TrainingLoop.cs:76-245 drives phase callbacks (EpochStart /
End, BatchStart / End, ForwardPassStart / End, BackwardPassStart / End, OptimizerStep, OnMetricUpdate,
OnException) around placeholder bodies (``loss = 0.5f``); built-in hooks Checkpoint / EarlyStopping /
GradientClipping / LRScheduler / Visualization (Hooks/BuiltIn/*.cs). Here the bodies are real: the loop
drives a ``TrainEngine`` (or any model / optimizer pair) over a data loader.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch


class TrainingPhase(enum.Enum):
    TRAIN_START = "train_start"; TRAIN_END = "train_end"
    EPOCH_START = "epoch_start"; EPOCH_END = "epoch_end"
    BATCH_START = "batch_start"; BATCH_END = "batch_end"
    FORWARD_START = "forward_start"; FORWARD_END = "forward_end"
    BACKWARD_START = "backward_start"; BACKWARD_END = "backward_end"
    OPTIMIZER_STEP = "optimizer_step"; METRIC_UPDATE = "metric_update"; EXCEPTION = "exception"
    VALIDATION_END = "validation_end"


@dataclass
class TrainingContext:
    epoch: int = 0
    step: int = 0
    batch_index: int = 0
    loss: float = float("nan")
    metrics: Dict[str, float] = field(default_factory=dict)
    should_stop: bool = False
    model: Any = None
    optimizer: Any = None
    exception: Optional[BaseException] = None


class TrainingHook:
    def on_phase(self, phase: TrainingPhase, ctx: TrainingContext):
        pass


class EarlyStoppingHook(TrainingHook):
    def __init__(self, metric: str = "val_loss", patience: int = 3, min_delta: float = 0.0, mode: str = "min"):
        self.metric, self.patience, self.min_delta, self.mode = metric, patience, min_delta, mode
        self.best = math.inf if mode == "min" else -math.inf
        self.bad = 0
        self._seen_epoch = -1

    def on_phase(self, phase, ctx):
        if phase not in (TrainingPhase.VALIDATION_END, TrainingPhase.EPOCH_END) or self.metric not in ctx.metrics:
            return
        if ctx.epoch == self._seen_epoch:          # one evaluation per epoch, whichever phase delivers the metric first
            return
        self._seen_epoch = ctx.epoch
        v = ctx.metrics[self.metric]
        better = v < self.best - self.min_delta if self.mode == "min" else v > self.best + self.min_delta
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                ctx.should_stop = True


class GradientClippingHook(TrainingHook):
    def __init__(self, max_norm: float = 1.0):
        self.max_norm, self.last_norm = max_norm, 0.0

    def on_phase(self, phase, ctx):
        if phase == TrainingPhase.BACKWARD_END and ctx.model is not None:
            ps = [p for p in ctx.model.parameters() if p.grad is not None]
            if ps:
                self.last_norm = float(torch.nn.utils.clip_grad_norm_(ps, self.max_norm))


class LRSchedulerHook(TrainingHook):
    def __init__(self, scheduler, per: str = "step"):
        self.s, self.per = scheduler, per

    def on_phase(self, phase, ctx):
        if (self.per == "step" and phase == TrainingPhase.OPTIMIZER_STEP) or (self.per == "epoch" and phase == TrainingPhase.EPOCH_END):
            self.s.step()


class CheckpointHook(TrainingHook):
    def __init__(self, save_fn: Callable[[TrainingContext], None], every_n_steps: int = 0, every_epoch: bool = True):
        self.save_fn, self.n, self.every_epoch = save_fn, every_n_steps, every_epoch
        self.saves = 0

    def on_phase(self, phase, ctx):
        if (phase == TrainingPhase.EPOCH_END and self.every_epoch) or \
           (phase == TrainingPhase.BATCH_END and self.n and ctx.step % self.n == 0):
            self.save_fn(ctx)
            self.saves += 1


class VisualizationHook(TrainingHook):
    def __init__(self, visualizer, log_every: int = 1):
        self.v, self.k = visualizer, log_every

    def on_phase(self, phase, ctx):
        if phase == TrainingPhase.BATCH_END and ctx.step % self.k == 0:
            self.v.log_scalar("train/loss", ctx.loss, ctx.step)
        elif phase == TrainingPhase.METRIC_UPDATE:
            for k, val in ctx.metrics.items():
                self.v.log_scalar(k, val, ctx.step)


class TrainingLoop:
    """``step_fn(batch) -> loss`` runs forward, backward and the optimizer step as one call (a
    ``TrainEngine.step``); or pass ``model`` + ``optimizer`` + ``loss_fn`` and the loop does the three
    phases itself, firing the per-phase hooks between them."""

    def __init__(self, hooks: Optional[List[TrainingHook]] = None, step_fn: Optional[Callable] = None, model=None, optimizer=None,
                 loss_fn: Optional[Callable] = None):
        self.hooks, self.step_fn = list(hooks or []), step_fn
        self.model, self.optimizer, self.loss_fn = model, optimizer, loss_fn
        self.ctx = TrainingContext(model=model, optimizer=optimizer)

    def add_hook(self, h: TrainingHook):
        self.hooks.append(h)

    def _fire(self, phase: TrainingPhase):
        for h in self.hooks:
            h.on_phase(phase, self.ctx)

    def _one(self, batch) -> float:
        if self.step_fn is not None:
            self._fire(TrainingPhase.FORWARD_START)
            loss = self.step_fn(batch)
            self._fire(TrainingPhase.OPTIMIZER_STEP)
            return float(loss)
        self._fire(TrainingPhase.FORWARD_START)
        loss = self.loss_fn(self.model, batch)
        self._fire(TrainingPhase.FORWARD_END)
        self._fire(TrainingPhase.BACKWARD_START)
        self.optimizer.zero_grad()
        loss.backward()
        self._fire(TrainingPhase.BACKWARD_END)
        self.optimizer.step()
        self._fire(TrainingPhase.OPTIMIZER_STEP)
        return float(loss.detach())

    def train(self, epochs: int, loader: Iterable, val_loader: Optional[Iterable] = None, val_fn: Optional[Callable] = None) -> TrainingContext:
        ctx = self.ctx
        self._fire(TrainingPhase.TRAIN_START)
        try:
            for ep in range(epochs):
                ctx.epoch = ep
                if hasattr(loader, "set_epoch"):
                    loader.set_epoch(ep)
                self._fire(TrainingPhase.EPOCH_START)
                tot, n = 0.0, 0
                for bi, batch in enumerate(loader):
                    ctx.batch_index = bi
                    self._fire(TrainingPhase.BATCH_START)
                    ctx.loss = self._one(batch)
                    ctx.step += 1
                    tot, n = tot + ctx.loss, n + 1
                    self._fire(TrainingPhase.BATCH_END)
                    if ctx.should_stop:
                        break
                ctx.metrics["train_loss"] = tot / max(1, n)
                if val_loader is not None and val_fn is not None:
                    ctx.metrics.update(self.validate(val_loader, val_fn))
                    self._fire(TrainingPhase.VALIDATION_END)
                self._fire(TrainingPhase.METRIC_UPDATE)
                self._fire(TrainingPhase.EPOCH_END)
                if ctx.should_stop:
                    break
        except BaseException as e:
            ctx.exception = e
            self._fire(TrainingPhase.EXCEPTION)
            raise
        finally:
            self._fire(TrainingPhase.TRAIN_END)
        return ctx

    @torch.no_grad()
    def validate(self, loader: Iterable, val_fn: Callable) -> Dict[str, float]:
        tot, n = 0.0, 0
        for batch in loader:
            tot += float(val_fn(batch))
            n += 1
        return {"val_loss": tot / max(1, n)}
