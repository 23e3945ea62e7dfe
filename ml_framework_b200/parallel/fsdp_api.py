"""FSDP vocabulary around the engine in :mod:`ml_framework_b200.parallel.fsdp`: sharding strategies as planners,
bucketed multi-tensor gather / scatter helpers with verification, parameter introspection, mixed-precision helpers.

Reference (src/MLFramework/Distributed/FSDP/): ShardingStrategy.cs (ParameterInfo :10, ShardingPlan :31, ShardAssignment
:52, FullShardingStrategy :89-139, LayerWiseShardingStrategy :144-196, HybridShardingStrategy :201-265, factory :270-300,
HybridConfig :305), AllGatherOperation.cs / AllGatherHelper (AllGatherMultipleAsync :21, CalculateBuckets :43),
ReduceScatterOperation.cs / ReduceScatterHelper (ReduceScatterMultipleAsync :23, VerifyReduceScatter :57),
FSDPExtensions.cs (GetParameter :55, IsParameterGathered :108, IsParameterOffloaded :133), FSDP.cs FSDPState :64-79,
FSDPMixedPrecision.cs:11-215 (own loss scaler: initial 2.0, x2 / x0.5, interval 2000, range [1, 65536]).
"""
from __future__ import annotations

import enum
import hashlib
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..dist.process_group import ReduceOp
from .fsdp import FSDP, padded_numel, shard_bounds


# ------------------------------------------------------------------ planning
@dataclass
class ParameterInfo:
    name: str
    shape: Tuple[int, ...]
    numel: int
    layer_name: str = ""
    always_gathered: bool = False          # replicated (e.g. embeddings in the reference's rule)

    @staticmethod
    def from_named(named_params: Iterable[Tuple[str, torch.Tensor]], always_gathered_patterns: Sequence[str] = ("embedding",)) -> List["ParameterInfo"]:
        return [ParameterInfo(n, tuple(p.shape), p.numel(), n.rsplit(".", 1)[0] if "." in n else "",
                              any(k in n.lower() for k in always_gathered_patterns)) for n, p in named_params]


@dataclass
class ShardAssignment:
    parameter: str
    owner_ranks: List[int]                 # every rank for a split parameter, one rank for a whole-layer owner
    shard_numel: int                       # elements each owner holds
    start: Dict[int, int] = field(default_factory=dict)       # rank -> first element of its piece (split parameters)
    replicated: bool = False


@dataclass
class ShardingPlan:
    world_size: int
    strategy: str
    assignments: Dict[str, ShardAssignment] = field(default_factory=dict)

    def elements_on_rank(self, rank: int) -> int:
        n = 0
        for a in self.assignments.values():
            if a.replicated or rank in a.owner_ranks:
                n += a.shard_numel
        return n

    def balance(self) -> float:
        """max / mean of the per-rank element counts (1.0 = perfectly even)."""
        per = [self.elements_on_rank(r) for r in range(self.world_size)]
        mean = sum(per) / len(per)
        return max(per) / mean if mean else 1.0


def stable_hash(s: str) -> int:
    """Same value in every process and run (Python's ``hash`` of a string is salted per process)."""
    return int.from_bytes(hashlib.md5(s.encode()).digest()[:8], "little")


class ShardingStrategy:
    name = "base"

    def plan(self, params: Sequence[ParameterInfo], world_size: int) -> ShardingPlan:
        raise NotImplementedError

    @staticmethod
    def _replicated(p: ParameterInfo, world: int) -> ShardAssignment:
        return ShardAssignment(p.name, list(range(world)), p.numel, replicated=True)

    @staticmethod
    def _split(p: ParameterInfo, world: int) -> ShardAssignment:
        per = padded_numel(p.numel, world) // world
        return ShardAssignment(p.name, list(range(world)), per, {r: min(r * per, p.numel) for r in range(world)})


class FullShardingStrategy(ShardingStrategy):
    """Every parameter cut into ``world_size`` equal pieces (ZeRO-3)."""
    name = "full"

    def plan(self, params, world_size):
        pl = ShardingPlan(world_size, self.name)
        for p in params:
            pl.assignments[p.name] = self._replicated(p, world_size) if p.always_gathered else self._split(p, world_size)
        return pl


class GradOpShardingStrategy(FullShardingStrategy):
    """Parameters stay whole on every rank after the first gather; gradients and optimizer state are cut (ZeRO-2). The
    plan describes the gradient / optimizer-state pieces."""
    name = "grad_op"


class LayerWiseShardingStrategy(ShardingStrategy):
    """A layer's parameters live whole on one rank, chosen by a stable hash of the layer name."""
    name = "layer_wise"

    def plan(self, params, world_size):
        pl = ShardingPlan(world_size, self.name)
        for p in params:
            if p.always_gathered:
                pl.assignments[p.name] = self._replicated(p, world_size)
            else:
                pl.assignments[p.name] = ShardAssignment(p.name, [stable_hash(p.layer_name or p.name) % world_size], p.numel)
        return pl


@dataclass
class HybridConfig:
    full_shard_patterns: Sequence[str] = ("transformer", "attention", "attn", "mlp", "blocks")
    layer_wise_patterns: Sequence[str] = ("classifier", "head")
    default: str = "full"


class HybridShardingStrategy(ShardingStrategy):
    name = "hybrid"

    def __init__(self, config: Optional[HybridConfig] = None):
        self.cfg = config or HybridConfig()
        if self.cfg.default not in ("full", "layer_wise"):
            raise ValueError("default must be 'full' or 'layer_wise'")
        self._full, self._lw = FullShardingStrategy(), LayerWiseShardingStrategy()

    def choice(self, name: str) -> str:
        low = name.lower()
        if any(k in low for k in self.cfg.full_shard_patterns):
            return "full"
        if any(k in low for k in self.cfg.layer_wise_patterns):
            return "layer_wise"
        return self.cfg.default

    def plan(self, params, world_size):
        pl = ShardingPlan(world_size, self.name)
        for p in params:
            sub = self._full if self.choice(p.name) == "full" else self._lw
            pl.assignments[p.name] = sub.plan([p], world_size).assignments[p.name]
        return pl


def create_sharding_strategy(name: str, **kw) -> ShardingStrategy:
    table = {"full": FullShardingStrategy, "grad_op": GradOpShardingStrategy, "layer_wise": LayerWiseShardingStrategy, "hybrid": HybridShardingStrategy}
    if name not in table:
        raise KeyError(f"unknown sharding strategy {name!r}; one of {sorted(table)}")
    return table[name](**kw)


# ------------------------------------------------------------------ multi-tensor helpers
def calculate_buckets(numels: Sequence[int], bucket_size_mb: float = 25.0, element_bytes: int = 2) -> List[List[int]]:
    """Indices grouped in order so that a bucket's gathered size stays within the limit (a tensor above the limit gets
    a bucket of its own)."""
    if bucket_size_mb <= 0:
        raise ValueError("bucket_size_mb must be positive")
    limit = int(bucket_size_mb * (1 << 20))
    out: List[List[int]] = []
    cur: List[int] = []
    size = 0
    for i, n in enumerate(numels):
        b = n * element_bytes
        if cur and size + b > limit:
            out.append(cur)
            cur, size = [], 0
        cur.append(i)
        size += b
    if cur:
        out.append(cur)
    return out


class AllGatherHelper:
    @staticmethod
    def all_gather_multiple(pg, shards: Sequence[torch.Tensor], numels: Sequence[int], bucket_size_mb: float = 25.0) -> List[torch.Tensor]:
        """Equal-size flat shards of several parameters -> the full flat parameters (trimmed to ``numels``), ONE collective
        per bucket."""
        if len(shards) != len(numels):
            raise ValueError("one element count per shard")
        W = pg.world_size
        out: List[Optional[torch.Tensor]] = [None] * len(shards)
        gathered_sizes = [s.numel() * W for s in shards]
        for bucket in calculate_buckets(gathered_sizes, bucket_size_mb, shards[0].element_size() if shards else 2):
            flat = torch.cat([shards[i].reshape(-1) for i in bucket])
            full = pg.all_gather(flat.view(1, -1), 0) if W > 1 else flat.view(1, -1)        # [W, sum of shard sizes]
            off = 0
            for i in bucket:
                n = shards[i].numel()
                out[i] = full[:, off:off + n].reshape(-1)[:numels[i]].clone()
                off += n
        return out


class ReduceScatterHelper:
    @staticmethod
    def reduce_scatter_multiple(pg, grads: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.AVG, bucket_size_mb: float = 25.0) -> List[torch.Tensor]:
        """Full flat gradients (any lengths) -> this rank's reduced pieces, ONE collective per bucket. A gradient is
        padded to a multiple of 8 x world elements, as the engine's shards are."""
        W, r = pg.world_size, pg.rank
        out: List[Optional[torch.Tensor]] = [None] * len(grads)
        padded = [padded_numel(g.numel(), W) for g in grads]
        for bucket in calculate_buckets(padded, bucket_size_mb, grads[0].element_size() if grads else 2):
            rows = []
            for i in bucket:
                g = torch.zeros(padded[i], dtype=grads[i].dtype, device=grads[i].device)
                g[:grads[i].numel()] = grads[i].reshape(-1)
                rows.append(g.view(W, -1))
            stacked = torch.cat(rows, 1).contiguous()                     # [W, sum of per-rank pieces]
            mine = pg.reduce_scatter(stacked, op, 0).reshape(-1) if W > 1 else stacked.reshape(-1)
            off = 0
            for i in bucket:
                n = padded[i] // W
                out[i] = mine[off:off + n].clone()
                off += n
        return out

    @staticmethod
    def verify_reduce_scatter(pg, full_grad: torch.Tensor, reduced_piece: torch.Tensor, op: ReduceOp = ReduceOp.AVG, atol: float = 1e-5) -> bool:
        """Checks a piece against an all-reduce of the full gradient (test / debug aid: costs a full all-reduce)."""
        W, r = pg.world_size, pg.rank
        ref = torch.zeros(padded_numel(full_grad.numel(), W), dtype=torch.float32, device=full_grad.device)
        ref[:full_grad.numel()] = full_grad.reshape(-1).float()
        if W > 1:
            pg.all_reduce(ref, ReduceOp.SUM)
        if op == ReduceOp.AVG:
            ref /= W
        per = ref.numel() // W
        return bool(torch.allclose(ref[r * per:(r + 1) * per], reduced_piece.float(), atol=atol))


# ------------------------------------------------------------------ introspection of a running engine
class FSDPState(enum.Enum):
    IDLE = "idle"
    FORWARD = "forward"
    BACKWARD = "backward"
    OPTIMIZER = "optimizer"


class FSDPExtensions:
    @staticmethod
    def _find(fsdp: FSDP, name: str):
        for u in fsdp.all_units():
            for sp in u.sharded:
                if sp.name == name:
                    return u, sp
        return None, None

    @classmethod
    def parameter_names(cls, fsdp: FSDP) -> List[str]:
        return [sp.name for u in fsdp.all_units() for sp in u.sharded] + [n for n, _ in fsdp.replicated]

    @classmethod
    def get_parameter(cls, fsdp: FSDP, name: str) -> torch.Tensor:
        """The full parameter, gathered if necessary (collective for sharded parameters)."""
        for n, p in fsdp.replicated:
            if n == name:
                return p.detach().clone()
        u, sp = cls._find(fsdp, name)
        if u is None:
            raise KeyError(f"no parameter named {name!r}")
        full = torch.zeros(u.full_numel, dtype=fsdp.dtype, device=fsdp.device)
        fsdp._gather_unit(u, full)
        return full[sp.full_off:sp.full_off + sp.numel].view(sp.shape).clone()

    @classmethod
    def is_parameter_sharded(cls, fsdp: FSDP, name: str) -> bool:
        return cls._find(fsdp, name)[0] is not None

    @classmethod
    def is_parameter_gathered(cls, fsdp: FSDP, name: str) -> bool:
        """True while the parameter's unit holds a full copy (between its pre-forward gather and its release), and always
        for replicated parameters."""
        if any(n == name for n, _ in fsdp.replicated):
            return True
        u, _ = cls._find(fsdp, name)
        if u is None:
            raise KeyError(f"no parameter named {name!r}")
        return u.gathered is not None

    @classmethod
    def is_parameter_offloaded(cls, fsdp: FSDP, name: str) -> bool:
        u, _ = cls._find(fsdp, name)
        if u is None:
            return False
        return bool(getattr(fsdp, "offload_params", False))

    @classmethod
    def local_shard_bounds(cls, fsdp: FSDP, name: str) -> Tuple[int, int]:
        """[start, end) of this rank's piece in the flattened parameter by the reference's ceil(N / W) rule."""
        u, sp = cls._find(fsdp, name)
        if u is None:
            raise KeyError(f"no parameter named {name!r}")
        return shard_bounds(sp.numel, fsdp.world, fsdp.rank)

    @classmethod
    def memory_summary(cls, fsdp: FSDP) -> Dict[str, int]:
        esz = torch.empty(0, dtype=fsdp.dtype).element_size()
        sharded = sum(u.shard_numel for u in fsdp.all_units())
        full = sum(u.full_numel for u in fsdp.all_units())
        return {"sharded_parameter_bytes": sharded * esz, "full_parameter_bytes": full * esz, "optimizer_state_bytes": sharded * 12,
                "largest_unit_bytes": max((u.full_numel for u in fsdp.all_units()), default=0) * esz}


# ------------------------------------------------------------------ mixed precision helpers
@dataclass
class FSDPMixedPrecisionConfig:
    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.bfloat16
    master_dtype: torch.dtype = torch.float32
    initial_loss_scale: float = 2.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    min_loss_scale: float = 1.0
    max_loss_scale: float = 65536.0

    def scaler_config(self):
        from ..amp.grad_scaler import DynamicScalerConfig
        return DynamicScalerConfig(initial_scale=self.initial_loss_scale, growth_factor=self.growth_factor, backoff_factor=self.backoff_factor,
                                   growth_interval=self.growth_interval, min_scale=self.min_loss_scale, max_scale=self.max_loss_scale)


class FSDPMixedPrecision:
    def __init__(self, config: Optional[FSDPMixedPrecisionConfig] = None):
        self.cfg = config or FSDPMixedPrecisionConfig()

    def convert_to_mixed_precision(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.cfg.param_dtype) if t.is_floating_point() else t

    def convert_gradient_to_fp32(self, g: torch.Tensor) -> torch.Tensor:
        return g.to(self.cfg.master_dtype) if g.is_floating_point() else g

    def make_scaler(self, device="cpu"):
        from ..amp.grad_scaler import DynamicLossScaler
        return DynamicLossScaler(self.cfg.scaler_config(), device)

    @staticmethod
    def check_overflow(grads: Iterable[torch.Tensor], pg=None) -> bool:
        """Non-finite value in any gradient of ANY rank (the reference's check is rank-local; agreeing across ranks is
        what keeps their parameters identical)."""
        bad = any(not bool(torch.isfinite(g).all()) for g in grads if g is not None)
        if pg is not None and pg.world_size > 1:
            f = torch.tensor([1.0 if bad else 0.0])
            pg.all_reduce(f, ReduceOp.MAX)
            bad = bool(f.item() > 0)
        return bad
