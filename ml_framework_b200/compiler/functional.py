"""Functional transforms: vmap, pmap, jit, grad composition.

Reference: src/MLFramework/Functional/** (vmap / pmap / jit transforms over delegates). ``vmap`` and
``grad`` are ``torch.func``; ``pmap`` maps a function over the leading axis across the ranks of a process
group (each rank computes its slice, results are all-gathered); ``jit`` caches a CUDA-graph capture per
input signature (there is no tracing compiler in this framework: launch overhead is what a captured
graph removes, kernels are hand-written).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.func as tf

from ..hal.cuda_graphs import CUDAGraphManager

vmap = tf.vmap
grad = tf.grad
grad_and_value = tf.grad_and_value


def compose(*fns: Callable) -> Callable:
    def run(x):
        for f in fns:
            x = f(x)
        return x
    return run


def pmap(fn: Callable, pg=None) -> Callable:
    """``pmap(fn)(x)``: x is split along dim 0 over the ranks of ``pg``; every rank applies ``fn`` to its
    slice; the outputs are all-gathered so each rank returns the full result. With no process group
    it degenerates to a loop over the leading axis in chunks of one."""
    def run(x: torch.Tensor):
        if pg is None or pg.world_size == 1:
            return torch.cat([fn(c) for c in x.split(max(1, x.shape[0]))], 0)
        W, r = pg.world_size, pg.rank
        if x.shape[0] % W:
            raise ValueError(f"leading dimension {x.shape[0]} not divisible by world size {W}")
        n = x.shape[0] // W
        y = fn(x[r * n:(r + 1) * n]).contiguous()
        return pg.all_gather(y, dim=0)
    return run


_manager: Optional[CUDAGraphManager] = None


def jit(fn: Callable, name: Optional[str] = None) -> Callable:
    global _manager
    if _manager is None:
        _manager = CUDAGraphManager()
    mgr = _manager

    def run(*inputs: torch.Tensor):
        return mgr.run(name or getattr(fn, "__name__", "jit_fn"), fn, *inputs)
    run.__wrapped__ = fn
    return run
