"""Tensor-parallel convenience API: layer factories, rank-conditional execution, a tensor-returning group facade,
mesh-aware context set-up.

Reference: src/MLFramework/Layers/TensorParallel/{ColumnParallelLinearFactory.cs (CreateForAttention :32,
CreateForMLPHidden :51), RowParallelLinearFactory.cs, TPMLPFactory.cs:20-140, TPConv2dFactory.cs:13-124},
src/MLFramework/Distributed/TensorParallel/{TPState.cs (ExecuteOnRank :18, ExecuteOnMaster :47, ExecuteOnAll :66),
TensorParallelGroup.cs:101-192, TensorParallelContext.cs}, src/MLFramework/Distributed/Mesh/{MeshState.cs:14-70,
TensorParallelMeshContext.cs:39-58, TPMeshLayerFactory.cs (returns placeholder layers there; real layers here)}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch
import torch.nn as nn

from ..dist.mesh import DeviceMesh
from ..dist.process_group import ReduceOp
from . import tensor_parallel as tpmod
from .tensor_parallel import (ColumnParallelLinear, Conv2dInputParallel, Conv2dOutputParallel, RowParallelLinear, TPContext, TPMLP)


# ------------------------------------------------------------------ factories
class ColumnParallelLinearFactory:
    @staticmethod
    def create(in_features: int, out_features: int, bias: bool = True, gather_output: bool = False, tp: Optional[TPContext] = None, **kw) -> ColumnParallelLinear:
        return ColumnParallelLinear(in_features, out_features, bias, gather_output, tp=tp, **kw)

    @staticmethod
    def create_for_attention(d_model: int, n_heads: int, n_kv_heads: Optional[int] = None, head_dim: Optional[int] = None, bias: bool = False,
                             tp: Optional[TPContext] = None, **kw) -> ColumnParallelLinear:
        """The fused Q / K / V projection: heads are split over the ranks, so both head counts must divide."""
        ctx = tp or tpmod.get_context()
        kvh = n_kv_heads or n_heads
        hd = head_dim or d_model // n_heads
        if n_heads % ctx.world or kvh % ctx.world:
            raise ValueError(f"{n_heads} query and {kvh} key/value heads do not split over {ctx.world} ranks")
        return ColumnParallelLinear(d_model, (n_heads + 2 * kvh) * hd, bias, False, tp=ctx, **kw)

    @staticmethod
    def create_for_mlp_hidden(d_model: int, hidden: int, bias: bool = True, gated: bool = False, tp: Optional[TPContext] = None, **kw) -> ColumnParallelLinear:
        """The up projection (``gated``: gate and up stacked, as SwiGLU wants them); output stays sharded for the row layer."""
        return ColumnParallelLinear(d_model, hidden * (2 if gated else 1), bias, False, tp=tp, **kw)


class RowParallelLinearFactory:
    @staticmethod
    def create(in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = True, tp: Optional[TPContext] = None, **kw) -> RowParallelLinear:
        return RowParallelLinear(in_features, out_features, bias, input_is_parallel, tp=tp, **kw)

    @staticmethod
    def create_for_attention_output(d_model: int, n_heads: int, head_dim: Optional[int] = None, bias: bool = False, tp: Optional[TPContext] = None, **kw):
        return RowParallelLinear(n_heads * (head_dim or d_model // n_heads), d_model, bias, True, tp=tp, **kw)

    @staticmethod
    def create_for_mlp_output(hidden: int, d_model: int, bias: bool = True, tp: Optional[TPContext] = None, **kw):
        return RowParallelLinear(hidden, d_model, bias, True, tp=tp, **kw)


class TPMLPFactory:
    @staticmethod
    def create_mlp_block(d_model: int, hidden: int, activation: str = "gelu", bias: bool = True, tp: Optional[TPContext] = None, **kw) -> TPMLP:
        if activation not in ("gelu", "relu"):
            raise ValueError(f"unknown activation {activation!r}")
        return TPMLP(d_model, hidden, activation, bias, tp=tp, **kw)

    @staticmethod
    def forward_mlp(block: TPMLP, x: torch.Tensor) -> torch.Tensor:
        return block(x)


class TPConv2dFactory:
    @staticmethod
    def create_output_parallel(in_ch, out_ch, kernel_size, tp: Optional[TPContext] = None, **kw) -> Conv2dOutputParallel:
        return Conv2dOutputParallel(in_ch, out_ch, kernel_size, tp=tp, **kw)

    @staticmethod
    def create_input_parallel(in_ch, out_ch, kernel_size, tp: Optional[TPContext] = None, **kw) -> Conv2dInputParallel:
        return Conv2dInputParallel(in_ch, out_ch, kernel_size, tp=tp, **kw)

    @staticmethod
    def create_bottleneck(in_ch: int, mid_ch: int, out_ch: int, kernel_size=3, tp: Optional[TPContext] = None) -> nn.Sequential:
        """Output-parallel conv (no gather) -> ReLU -> input-parallel conv: one all-reduce for the pair."""
        return nn.Sequential(Conv2dOutputParallel(in_ch, mid_ch, kernel_size, padding=kernel_size // 2, gather_output=False, tp=tp), nn.ReLU(),
                             Conv2dInputParallel(mid_ch, out_ch, kernel_size, padding=kernel_size // 2, input_is_parallel=True, tp=tp))


# ------------------------------------------------------------------ rank-conditional execution
class TPState:
    """Run a function on one rank, on the master, or on all ranks of the tensor-parallel group."""

    def __init__(self, tp: Optional[TPContext] = None):
        self.tp = tp or tpmod.get_context()

    @property
    def rank(self) -> int:
        return self.tp.rank

    @property
    def world_size(self) -> int:
        return self.tp.world

    @property
    def is_master(self) -> bool:
        return self.tp.rank == 0

    def execute_on_rank(self, rank: int, fn: Callable[..., Any], *a, **k):
        if not (0 <= rank < self.tp.world):
            raise ValueError(f"rank {rank} is outside the group of {self.tp.world}")
        return fn(*a, **k) if self.tp.rank == rank else None

    def execute_on_master(self, fn: Callable[..., Any], *a, **k):
        return self.execute_on_rank(0, fn, *a, **k)

    def execute_on_all(self, fn: Callable[[int], Any], barrier: bool = False):
        """``fn(rank)`` everywhere; with ``barrier`` the ranks leave together."""
        out = fn(self.tp.rank)
        if barrier and self.tp.pg is not None and self.tp.world > 1:
            self.tp.pg.barrier()
        return out

    def broadcast_from_master(self, value: Any):
        """A Python object computed on the master, on every rank."""
        if self.tp.pg is None or self.tp.world == 1:
            return value
        return self.tp.pg.broadcast_object(value if self.is_master else None, 0)


class TensorParallelGroup:
    """Collectives of the tensor-parallel group that RETURN their result (the reference's async ``ICommunicator``
    surface) instead of writing in place."""

    def __init__(self, tp: Optional[TPContext] = None):
        self.tp = tp or tpmod.get_context()

    @property
    def size(self) -> int:
        return self.tp.world

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        out = t.clone()
        if self.tp.world > 1:
            self.tp.pg.all_reduce(out, op)
        return out

    def all_gather(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        return t.clone() if self.tp.world == 1 else self.tp.pg.all_gather(t, dim % t.dim())

    def reduce_scatter(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, dim: int = 0) -> torch.Tensor:
        return t.clone() if self.tp.world == 1 else self.tp.pg.reduce_scatter(t, op, dim)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        out = t.clone()
        if self.tp.world > 1:
            self.tp.pg.broadcast(out, root)
        return out

    def barrier(self):
        if self.tp.world > 1:
            self.tp.pg.barrier()


# ------------------------------------------------------------------ mesh-aware set-up
@dataclass
class MeshState:
    mesh: DeviceMesh

    def tp_world_size(self) -> int:
        return self.mesh.tp_world_size

    def dp_world_size(self) -> int:
        return self.mesh.dp_world_size

    def is_master_rank(self) -> bool:
        return self.mesh.is_master()

    def execute_on_master(self, fn: Callable[..., Any], *a, **k):
        return self.mesh.execute_on_master(fn, *a, **k)

    def describe(self) -> str:
        m = self.mesh
        return (f"rank {m.rank}: tp {m.tp_rank}/{m.tp_world_size}, dp {m.dp_rank}/{m.dp_world_size}, pp {m.pp_rank}/{m.pp_world_size}")


class TensorParallelMeshContext:
    """Tensor parallelism initialised from a device mesh: the TP group is the mesh's tensor dimension through this
    rank, the DP group its data dimension. ``groups`` may supply ready communicators (tests with simulated ranks);
    otherwise the sub-groups are created from the default process group (collective)."""

    def __init__(self, mesh: DeviceMesh, tp_group=None, dp_group=None, symm=None, fused: bool = True):
        self.mesh = mesh
        self.tp_group = tp_group if tp_group is not None else (mesh.process_group("tensor") if mesh.tp_world_size > 1 else None)
        self.dp_group = dp_group if dp_group is not None else (mesh.process_group("data") if mesh.dp_world_size > 1 else None)
        self.tp = tpmod.initialize(self.tp_group, symm, fused) if self.tp_group is not None else tpmod.initialize(None, None, False)
        self.state = MeshState(mesh)

    @classmethod
    def initialize_with_mesh(cls, mesh: DeviceMesh, **kw) -> "TensorParallelMeshContext":
        return cls(mesh, **kw)

    @property
    def tp_rank(self) -> int:
        return self.mesh.tp_rank

    @property
    def dp_rank(self) -> int:
        return self.mesh.dp_rank

    def gradient_manager(self):
        """Gradient averaging over the data-parallel group for this rank's tensor-parallel shards."""
        from .tensor_parallel import TPGradientManager
        return TPGradientManager(self.tp, self.dp_group)


class TPMeshLayerFactory:
    def __init__(self, ctx: TensorParallelMeshContext):
        self.ctx = ctx

    def column_linear(self, in_features: int, out_features: int, **kw) -> ColumnParallelLinear:
        return ColumnParallelLinear(in_features, out_features, tp=self.ctx.tp, **kw)

    def row_linear(self, in_features: int, out_features: int, **kw) -> RowParallelLinear:
        return RowParallelLinear(in_features, out_features, tp=self.ctx.tp, **kw)

    def mlp(self, d_model: int, hidden: int, **kw) -> TPMLP:
        return TPMLP(d_model, hidden, tp=self.ctx.tp, **kw)
