"""Training engine: the public entry point that wires a model, flat parameter buffers, mixed
precision, the optimizer and a data-parallel strategy into one ``step(ids, targets)`` call.

Strategies
  ``"none"``  single process.
  ``"ddp"``   replicated parameters, flat gradient bucket all-reduced.
  ``"fsdp"``  fully sharded parameters / gradients / optimizer state (ZeRO-3 style, one unit per
              transformer block; see :mod:`ml_framework_b200.parallel.fsdp`).
  ``"zero2"`` gradients and optimizer state sharded, parameters replicated ("grad-op sharding").

The step is the flow of the reference's AMP training loop (src/MLFramework/Amp/GradScaler.cs:83-160,
src/MLFramework/Amp/Integrations/AmpOptimizerWrapper.cs:68-119): scale the loss, backward,
unscale + overflow check, skip or apply the update, update the scale — with the scale, the
overflow flag and the skip decision all kept on the device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from .amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig
from .obs.profiler import nvtx_range
from .optim.optimizers import AdamW
from .parallel.flat import FlatParams


@dataclass
class EngineConfig:
    strategy: str = "none"             # none | ddp | fsdp | zero2
    lr: float = 3e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    loss_scaling: bool = True
    scaler: DynamicScalerConfig = field(default_factory=DynamicScalerConfig)
    grad_dtype: Optional[torch.dtype] = None   # default: parameter dtype
    fused_comm: bool = True            # use the in-kernel NVLink paths when peers are mapped
    bucket_size_mb: float = 25.0

    def validate(self):
        if self.strategy not in ("none", "ddp", "fsdp", "zero2"):
            raise ValueError(f"unknown strategy {self.strategy!r}")
        if self.lr <= 0:
            raise ValueError("lr must be positive")
        self.scaler.validate()


class TrainEngine:
    def __init__(self, model: nn.Module, config: Optional[EngineConfig] = None, process_group=None):
        self.cfg = config or EngineConfig()
        self.cfg.validate()
        self.model = model
        self.pg = process_group
        self.world = process_group.world_size if process_group is not None else 1
        p0 = next(model.parameters())
        self.device = p0.device
        self.scaler = DynamicLossScaler(self.cfg.scaler, device=self.device) if self.cfg.loss_scaling else None
        strategy = self.cfg.strategy if self.world > 1 else ("none" if self.cfg.strategy in ("ddp", "zero2") else self.cfg.strategy)
        self.strategy = strategy
        if strategy in ("fsdp", "zero2"):
            from .parallel.fsdp import FSDP, FSDPConfig
            self.reducer = None
            self.fsdp = FSDP(model, FSDPConfig(fused_comm=self.cfg.fused_comm, sharding_strategy="full" if strategy == "fsdp" else "grad_op"), process_group,
                             optimizer_kwargs=dict(lr=self.cfg.lr, betas=self.cfg.betas, eps=self.cfg.eps,
                                                   weight_decay=self.cfg.weight_decay))
            self.flat = None
            self.optimizer = self.fsdp.optimizer
        else:
            self.fsdp = None
            params = [p for p in model.parameters() if p.requires_grad]
            # tied parameters appear once
            seen, uniq = set(), []
            for p in params:
                if id(p) not in seen:
                    seen.add(id(p))
                    uniq.append(p)
            self.reducer = None
            self.symm = None
            grad_alloc = None
            gdt = self.cfg.grad_dtype or uniq[0].dtype
            if strategy == "ddp" and self.world > 1:
                from .parallel.ddp import fused_comm_possible
                if fused_comm_possible(self.pg, self.device, self.cfg.fused_comm, gdt):
                    # the flat gradient buffer lives in symmetric memory: buckets are reduced by peer loads / stores
                    from .dist.symm import SymmetricMemory
                    self.symm = SymmetricMemory(self.pg, self.device)
                    holder = {}

                    def grad_alloc(n, dt, holder=holder):
                        holder["buf"] = self.symm.alloc(n * torch.empty(0, dtype=dt).element_size())
                        return holder["buf"].view(dt, n)
            self.flat = FlatParams(uniq, grad_dtype=self.cfg.grad_dtype, grad_alloc=grad_alloc)
            self.optimizer = AdamW(self.flat, lr=self.cfg.lr, betas=self.cfg.betas, eps=self.cfg.eps,
                                   weight_decay=self.cfg.weight_decay)
            if strategy == "ddp" and self.world > 1:
                from .parallel.ddp import FlatGradReducer
                self.pg.broadcast(self.flat.flat, src=0)
                flag = None
                if self.symm is not None:
                    flag = self.symm.alloc_flag()
                    if self.scaler is not None:
                        self.scaler.found_inf = flag.view(torch.int32, 1)   # every rank's kernels raise every rank's flag
                self.reducer = FlatGradReducer(self.flat, self.pg, self.cfg.bucket_size_mb, symm=self.symm,
                                               symm_buf=holder["buf"] if self.symm is not None else None, flag=flag)
        self.steps = 0

    # ------------------------------------------------------------------
    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimisation step on a local micro-batch; returns the (unscaled) loss tensor."""
        if self.fsdp is not None:
            loss = self.fsdp.train_step(ids, targets, self.scaler)
            self.steps += 1
            return loss
        flat = self.flat
        flat.zero_grad()
        scale_t = self.scaler.scale_t if self.scaler is not None else None
        with nvtx_range("forward"):
            loss = self.model(ids, targets, loss_scale=scale_t)
        with nvtx_range("backward"):
            loss.backward()
        flat.gather_missing_grads()
        grad_scale = 1.0
        checked = False
        if self.reducer is not None:
            # buckets were all-reduced (and averaged) from the gradient-ready hooks while backward ran;
            # this reduces what the hooks could not and waits for the communication stream
            with nvtx_range("ddp.finish_reductions"):
                self.reducer.finish()
            checked = self.symm is not None      # the in-kernel all-reduce checks every reduced value
        if self.scaler is not None:
            from .ops import native
            if not checked:
                if flat.grad.is_cuda:
                    native.amp_unscale_check_(flat.grad, self.scaler.found_inf, inv_scale=None, write_back=False)
                elif not torch.isfinite(flat.grad).all():
                    self.scaler.found_inf.fill_(1)
                if self.world > 1:
                    self.scaler.sync_found_inf(self.pg)
            self.optimizer.step(grad_scale=grad_scale, inv_scale=self.scaler.inv_scale_t, found_inf=self.scaler.found_inf)
            self.scaler.update()
        else:
            self.optimizer.step(grad_scale=grad_scale)
        self.steps += 1
        return loss

    def close(self):
        """Releases the peer-mapped buffers of the fused communication paths (collective when they exist)."""
        if self.fsdp is not None:
            self.fsdp.close()
        if getattr(self, "symm", None) is not None:
            self.symm.close()
            self.symm = None

    def state_dict(self):
        sd = {"steps": self.steps, "optimizer": self.optimizer.state_dict() if hasattr(self.optimizer, "state_dict") else None}
        if self.scaler is not None:
            sd["scaler"] = self.scaler.state_dict()
        return sd
