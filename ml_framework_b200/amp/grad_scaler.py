"""Loss scaling for mixed-precision training.

State machine and defaults follow the reference's ``DynamicLossScaler``
(src/MLFramework/Amp/DynamicLossScaler.cs:78-269): initial scale 65536, growth x2 after
``growth_interval`` (2000) consecutive clean steps, back-off x0.5 on overflow, clamped to
[min_scale 1, max_scale 2**24]; ``GradScaler`` (src/MLFramework/Amp/GradScaler.cs:83-160) wraps
it with ``scale_loss / unscale / step / update``; presets from ``GradScalerFactory``
(src/MLFramework/Amp/GradScalerFactory.cs:14-109).

On CUDA the scale, the growth tracker and the found-inf flag live on the device: the loss
kernel multiplies its gradient by the scale, the fused optimizer reads ``1/scale`` and the
flag, and ``update()`` is a one-thread kernel, so a training step never synchronises with the
host. In multi-rank jobs the found-inf flag is all-reduced (MAX) before the optimizer step
(the reference checks overflow per rank only, src/MLFramework/Distributed/FSDP/FSDPMixedPrecision.cs:163-215).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Dict, Iterable, Optional

import torch

from ..ops import native


@dataclass
class DynamicScalerConfig:
    initial_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    min_scale: float = 1.0
    max_scale: float = float(2 ** 24)
    enabled: bool = True

    def validate(self):
        if self.initial_scale <= 0:
            raise ValueError("initial_scale must be positive")
        if self.growth_factor <= 1.0:
            raise ValueError("growth_factor must be > 1")
        if not (0.0 < self.backoff_factor < 1.0):
            raise ValueError("backoff_factor must be in (0, 1)")
        if self.growth_interval <= 0:
            raise ValueError("growth_interval must be positive")
        if not (0 < self.min_scale <= self.max_scale):
            raise ValueError("need 0 < min_scale <= max_scale")


@dataclass
class DynamicScalerStats:
    scale: float
    growth_tracker: int
    total_steps: int
    skipped_steps: int


class _LossScalerBase:
    """Gradient-side operations shared by the static and the dynamic scaler (the reference's
    ``ILossScaler``, src/MLFramework/Amp/ILossScaler.cs:9): both expose ``scale_t``,
    ``inv_scale_t`` and the ``found_inf`` flag on their device."""

    def unscale_gradients(self, grads: Iterable[torch.Tensor], sumsq: Optional[torch.Tensor] = None) -> None:
        """In place ``g *= 1/scale``; raises the found-inf flag on NaN/Inf."""
        for g in grads:
            if g is None:
                continue
            if g.is_cuda:
                native.amp_unscale_check_(g, self.found_inf, inv_scale=self.inv_scale_t, sumsq=sumsq)
            else:
                g.mul_(self.inv_scale_t.to(g.dtype))
                if not torch.isfinite(g).all():
                    self.found_inf.fill_(1)
                elif sumsq is not None:
                    sumsq.add_(g.float().pow(2).sum())

    def check_overflow(self, grads: Iterable[torch.Tensor]) -> bool:
        """Host-visible overflow test (synchronises); prefer the device flag in hot loops."""
        for g in grads:
            if g is None:
                continue
            if g.is_cuda:
                native.amp_unscale_check_(g, self.found_inf, inv_scale=None, inv_scale_host=1.0, write_back=False)
            elif not torch.isfinite(g).all():
                self.found_inf.fill_(1)
        return bool(self.found_inf.item())

    def check_overflow_flag(self) -> bool:
        return bool(self.found_inf.item())

    def sync_found_inf(self, pg) -> None:
        """Make every rank agree on overflow before anyone applies an update."""
        if pg is not None and pg.world_size > 1:
            from ..dist.process_group import ReduceOp
            pg.all_reduce(self.found_inf, op=ReduceOp.MAX)


class StaticLossScaler(_LossScalerBase):
    """Fixed scale (src/MLFramework/Amp/StaticLossScaler.cs)."""

    def __init__(self, scale: float = 1.0, device="cpu"):
        if scale <= 0:
            raise ValueError("scale must be positive")
        self.device = torch.device(device)
        self.scale_t = torch.tensor(float(scale), device=self.device)
        self.inv_scale_t = torch.tensor(1.0 / float(scale), device=self.device)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.enabled = True
        self.total_steps = 0
        self.skipped_steps = 0

    @property
    def scale(self) -> float:
        return float(self.scale_t.item())

    def scale_loss(self, loss):
        return loss * self.scale_t

    def update(self):
        """A fixed scale never changes; a skipped step is only counted."""
        self.total_steps += 1
        self.skipped_steps += int(self.found_inf.item()) if self.found_inf.device.type == "cpu" else 0
        self.found_inf.zero_()

    def get_stats(self) -> "DynamicScalerStats":
        return DynamicScalerStats(self.scale, 0, self.total_steps, self.skipped_steps)

    def state_dict(self) -> Dict:
        return {"scale": self.scale, "total_steps": self.total_steps, "skipped": self.skipped_steps}

    def load_state_dict(self, sd: Dict):
        self.scale_t.fill_(sd["scale"])
        self.inv_scale_t.fill_(1.0 / sd["scale"])
        self.total_steps = sd.get("total_steps", 0)
        self.skipped_steps = sd.get("skipped", 0)


class DynamicLossScaler(_LossScalerBase):
    def __init__(self, config: Optional[DynamicScalerConfig] = None, device="cpu", **overrides):
        cfg = config or DynamicScalerConfig()
        for k, v in overrides.items():
            setattr(cfg, k, v)
        cfg.validate()
        self.cfg = cfg
        self.enabled = cfg.enabled
        self.device = torch.device(device)
        self.scale_t = torch.tensor(float(cfg.initial_scale), device=self.device)
        self.inv_scale_t = torch.tensor(1.0 / float(cfg.initial_scale), device=self.device)
        self.tracker = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.total_steps = 0

    # ---- API
    @property
    def scale(self) -> float:
        return float(self.scale_t.item())

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.scale_t if self.enabled else loss

    def update(self) -> None:
        """Advance the state machine using the found-inf flag, then clear the flag."""
        self.total_steps += 1
        if not self.enabled:
            self.found_inf.zero_()
            return
        c = self.cfg
        if self.scale_t.is_cuda:
            native.scaler_update_(self.scale_t, self.tracker, self.found_inf, growth=c.growth_factor, backoff=c.backoff_factor,
                                  interval=c.growth_interval, min_scale=c.min_scale, max_scale=c.max_scale, skipped=self.skipped)
            torch.reciprocal(self.scale_t, out=self.inv_scale_t)
        else:
            s = float(self.scale_t)
            if int(self.found_inf) != 0:
                s *= c.backoff_factor
                self.tracker.zero_()
                self.skipped += 1
            else:
                self.tracker += 1
                if int(self.tracker) >= c.growth_interval:
                    s *= c.growth_factor
                    self.tracker.zero_()
            s = min(max(s, c.min_scale), c.max_scale)
            self.scale_t.fill_(s)
            self.inv_scale_t.fill_(1.0 / s)
            self.found_inf.zero_()

    def get_stats(self) -> DynamicScalerStats:
        return DynamicScalerStats(self.scale, int(self.tracker.item()), self.total_steps, int(self.skipped.item()))

    def state_dict(self) -> Dict:
        return {"config": asdict(self.cfg), "scale": self.scale, "tracker": int(self.tracker.item()),
                "total_steps": self.total_steps, "skipped": int(self.skipped.item())}

    def load_state_dict(self, sd: Dict):
        self.scale_t.fill_(sd["scale"])
        self.inv_scale_t.fill_(1.0 / sd["scale"])
        self.tracker.fill_(sd["tracker"])
        self.total_steps = sd["total_steps"]
        self.skipped.fill_(sd["skipped"])


class GradScaler:
    """``scale_loss -> backward -> step(optimizer) -> update`` with skip-on-overflow."""

    def __init__(self, scaler=None, device="cpu", process_group=None):
        self.scaler = scaler if scaler is not None else DynamicLossScaler(device=device)
        self.pg = process_group

    def scale_loss(self, loss):
        return self.scaler.scale_loss(loss)

    def unscale(self, grads, sumsq=None):
        self.scaler.unscale_gradients(grads, sumsq)

    def check_overflow(self, grads) -> bool:
        return self.scaler.check_overflow(grads)

    def prepare_gradients(self, grads) -> bool:
        """Unscale and test; False means the step must be skipped (GradScaler.PrepareGradients)."""
        grads = list(grads)
        self.unscale(grads)
        self.scaler.sync_found_inf(self.pg)
        return not self.scaler.check_overflow_flag()

    def step(self, optimizer, grads_already_unscaled: bool = False) -> None:
        """Runs ``optimizer.step`` with the device-resident 1/scale and found-inf flag."""
        self.scaler.sync_found_inf(self.pg)
        if grads_already_unscaled:
            optimizer.step(found_inf=self.scaler.found_inf)
        else:
            optimizer.step(inv_scale=self.scaler.inv_scale_t, found_inf=self.scaler.found_inf)

    def update(self):
        self.scaler.update()

    @property
    def scale(self):
        return self.scaler.scale


class GradScalerFactory:
    """Presets (src/MLFramework/Amp/GradScalerFactory.cs:14-109)."""

    @staticmethod
    def conservative(device="cpu"):
        return GradScaler(DynamicLossScaler(DynamicScalerConfig(initial_scale=32768.0, growth_interval=5000), device))

    @staticmethod
    def aggressive(device="cpu"):
        return GradScaler(DynamicLossScaler(DynamicScalerConfig(initial_scale=65536.0, growth_interval=1000), device))

    @staticmethod
    def fp16(device="cpu"):
        return GradScaler(DynamicLossScaler(DynamicScalerConfig(initial_scale=65536.0, growth_interval=2000), device))

    @staticmethod
    def bf16(device="cpu"):
        return GradScaler(DynamicLossScaler(DynamicScalerConfig(initial_scale=8.0, growth_interval=2000), device))

    @staticmethod
    def static(scale: float, device="cpu"):
        return GradScaler(StaticLossScaler(scale, device))
