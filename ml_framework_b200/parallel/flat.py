"""Flat parameter / gradient buffers.

``FlatParams`` re-homes a list of parameters into one contiguous buffer (each parameter becomes
a view, 16-byte aligned) and gives every parameter a ``main_grad`` view into a matching flat
gradient buffer. Weight-gradient kernels write into ``main_grad`` directly (see
:mod:`ml_framework_b200.ops.functional`), the optimizer updates the whole buffer with one fused
kernel, and DDP / FSDP reduce or shard the buffer without per-tensor packing — the flat
equivalent of the reference's ``GradientBucket.Prepare`` / ``CopyBack``
(src/MLFramework/Distributed/GradientBucket.cs:85-156).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    def __init__(self, params: Sequence[nn.Parameter], grad_dtype: Optional[torch.dtype] = None,
                 pad_multiple: int = 1, align_elems: int = 8, alloc: Optional[Callable] = None,
                 grad_alloc: Optional[Callable] = None, with_grad: bool = True):
        params = list(params)
        if not params:
            raise ValueError("FlatParams needs at least one parameter")
        self.params = params
        self.dtype, self.device = params[0].dtype, params[0].device
        for p in params:
            if p.dtype != self.dtype or p.device != self.device:
                raise ValueError("all parameters of a flat buffer must share dtype and device")
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off = _align(off + p.numel(), align_elems)
        self.numel_unpadded = off
        self.numel = _align(off, max(pad_multiple, align_elems))
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.flat = alloc(self.numel, self.dtype)
        self.grad_dtype = grad_dtype or self.dtype
        self.grad = (grad_alloc or alloc)(self.numel, self.grad_dtype) if with_grad else None
        with torch.no_grad():
            for p, o in zip(params, self.offsets):
                view = self.flat[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                if self.grad is not None:
                    p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
                    p._main_grad_started = False

    def zero_grad(self, set_to_zero: bool = False):
        """Marks gradients as not started (the first wgrad overwrites); zero-fills on request."""
        for p in self.params:
            p._main_grad_started = False
            p.grad = None
        if set_to_zero and self.grad is not None:
            self.grad.zero_()

    def repoint(self, flat: torch.Tensor):
        """Make the parameters views of another buffer with the same layout (no copy)."""
        self.flat = flat
        for p, o in zip(self.params, self.offsets):
            p.data = flat[o:o + p.numel()].view(p.shape)

    def gather_missing_grads(self):
        """Copy autograd ``.grad`` of parameters whose kernels did not write ``main_grad``."""
        for p in self.params:
            if p.grad is not None:
                if getattr(p, "_main_grad_started", False):
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                    p._main_grad_started = True
                p.grad = None
            elif not getattr(p, "_main_grad_started", False):
                p.main_grad.zero_()
                p._main_grad_started = True
