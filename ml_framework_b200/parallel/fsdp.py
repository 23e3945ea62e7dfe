"""Fully sharded data parallel (ZeRO-3) and gradient/optimizer-state sharding (ZeRO-2).

Semantics follow the reference's FSDP (src/MLFramework/Distributed/FSDP/FSDP.cs:67-233,
FSDPShardingUnit.cs:84-110, FSDPConfig.cs:8-58, ShardingStrategy.cs:89-265):

* sharding is per *parameter*: parameter p of N elements is cut into W contiguous pieces and
  rank r owns piece r (the reference uses ceil(N/W) with a short last piece; here N is padded
  to a multiple of 8W so every piece is equal and 16-byte aligned);
* parameters are all-gathered before a unit's forward and again before its backward and
  released afterwards; gradients are reduce-scattered after the unit's backward; optimizer
  state (fp32 master, Adam m and v) exists only for the owned pieces
  (FSDP/FSDPOptimizerStateManager.cs:37-245);
* some parameters stay replicated ("always gathered", FSDP.cs:223-233: embeddings in the
  reference). Here every 1-D parameter (norm scales, biases) is replicated, since the first
  kernel of a unit needs them before any gather could complete; their gradients are
  all-reduced and every rank applies the same update;
* strategies: ``full`` (every unit sharded over all ranks), ``grad_op`` (ZeRO-2: parameters
  replicated, gradients reduce-scattered, optimizer state sharded — required by the
  benchmark configurations, absent in the reference), ``layer_wise`` (a unit's parameters are
  owned whole by rank ``hash(unit) % W``: ShardingStrategy.cs:144-196), ``hybrid`` (name list:
  ShardingStrategy.cs:201-265);
* mixed precision: bf16 parameters and gradients on the wire, fp32 master weights, dynamic
  loss scale whose overflow flag is all-reduced so every rank skips together
  (FSDPMixedPrecision.cs:11-215 keeps the flag rank-local);
* CPU offload of the optimizer state shards with pinned buffers (FSDPCpuOffload.cs:13-305).

A unit is a transformer block (module list entry) rather than a single parameter, so one
gather serves all GEMMs of the block. With the peer-memory layer active the gather is done by
copy CTAs inside the block's first GEMM (``fused_comm``), and the reduce-scatter by a kernel
that reads the peers' gradient buffers directly; otherwise both are NCCL/gloo collectives
issued on a side stream one unit ahead of compute.
"""
from __future__ import annotations

import os
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..dist.process_group import ReduceOp
from ..obs.profiler import nvtx_range
from ..ops import native, reference


@dataclass
class FSDPCpuOffloadConfig:
    enabled: bool = False
    offload_optimizer_states: bool = True
    offload_gradients: bool = False
    offload_parameters: bool = False
    prefetch_steps: int = 1

    def validate(self):
        if not (0 <= self.prefetch_steps <= 10):
            raise ValueError("prefetch_steps must be in [0, 10]")
        if self.enabled and self.offload_gradients and not self.offload_optimizer_states:
            raise ValueError("offload_gradients needs offload_optimizer_states (the update then runs where the gradients are)")


@dataclass
class FSDPConfig:
    sharding_strategy: str = "full"        # full | grad_op | layer_wise | hybrid
    mixed_precision: bool = True
    offload_to_cpu: bool = False
    activation_checkpointing: bool = False
    bucket_size_mb: int = 25
    num_communication_workers: int = 2
    fused_comm: bool = True
    # tuning knobs of the fused paths; each default can be overridden from the environment (MLF_FSDP_REDUCE_CTAS,
    # MLF_FSDP_COPY_CTAS, MLF_FSDP_GATHER_PARTS) without touching the code that builds the config
    reduce_ctas: int = field(default_factory=lambda: int(os.environ.get("MLF_FSDP_REDUCE_CTAS", "64")))   # CTAs of a unit's reduce-scatter kernel (it overlaps the next unit's backward)
    gather_copy_ctas: int = field(default_factory=lambda: int(os.environ.get("MLF_FSDP_COPY_CTAS", "16")))  # CTAs a GEMM lends to the parameter gather of the next unit
    # the next unit's gather is cut into this many parts; each large GEMM of the current unit carries as many parts as
    # its copy CTAs move while it runs (1: the first GEMM carries all)
    gather_parts: int = field(default_factory=lambda: int(os.environ.get("MLF_FSDP_GATHER_PARTS", "1")))
    min_shard_numel: int = 4096            # smaller / 1-D parameters stay replicated
    hybrid_full_patterns: Sequence[str] = ("transformer", "attention", "attn", "mlp", "blocks")
    hybrid_layerwise_patterns: Sequence[str] = ("classifier", "head")
    cpu_offload: FSDPCpuOffloadConfig = field(default_factory=FSDPCpuOffloadConfig)

    def validate(self):
        if self.sharding_strategy not in ("full", "grad_op", "layer_wise", "hybrid"):
            raise ValueError(f"unknown sharding strategy {self.sharding_strategy!r}")
        if not (1 <= self.bucket_size_mb <= 1000):
            raise ValueError("bucket_size_mb must be in [1, 1000]")
        if not (1 <= self.num_communication_workers <= 16):
            raise ValueError("num_communication_workers must be in [1, 16]")
        self.cpu_offload.validate()


def shard_bounds(numel: int, world: int, rank: int):
    """The reference's rule: shard size ceil(N/W), rank r owns [r*s, min((r+1)*s, N))."""
    s = (numel + world - 1) // world
    lo = min(rank * s, numel)
    return lo, min(lo + s, numel)


def padded_numel(numel: int, world: int, mult: int = 8) -> int:
    q = world * mult
    return (numel + q - 1) // q * q


class _ShardedParam:
    def __init__(self, name: str, p: nn.Parameter, world: int, rank: int):
        self.name, self.param = name, p
        self.numel = p.numel()
        self.shape = tuple(p.shape)
        self.padded = padded_numel(self.numel, world)
        self.shard_numel = self.padded // world
        self.full_off = 0    # offset in the unit's gathered buffer
        self.shard_off = 0   # offset in the unit's shard buffer


class FSDPUnit:
    """Parameters of one module that are gathered / reduced together."""

    def __init__(self, name: str, module: nn.Module, params: List[tuple], world: int, rank: int):
        self.name, self.module = name, module
        self.sharded: List[_ShardedParam] = [_ShardedParam(n, p, world, rank) for n, p in params]
        off_f = off_s = 0
        for sp in self.sharded:
            sp.full_off, sp.shard_off = off_f, off_s
            off_f += sp.padded
            off_s += sp.shard_numel
        self.full_numel, self.shard_numel = off_f, off_s
        self.shard: Optional[torch.Tensor] = None        # bf16 owned pieces
        self.grad_shard: Optional[torch.Tensor] = None   # reduced gradient pieces
        self.gathered: Optional[torch.Tensor] = None     # current full buffer (or None)
        self.grad_full: Optional[torch.Tensor] = None
        self.state_off = 0                               # offset in the global optimizer shard
        self.gather_work: list = []
        self.rs_work: list = []
        self.owner: Optional[int] = None                 # layer_wise: owning rank


class _PreBackward(torch.autograd.Function):
    """Identity on a unit's output; its backward runs before the unit's own backward."""

    @staticmethod
    def forward(ctx, x, fsdp, idx):
        ctx.fsdp, ctx.idx = fsdp, idx
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.fsdp._pre_backward(ctx.idx)
        return g, None, None


class _PostBackward(torch.autograd.Function):
    """Identity on a unit's input; its backward runs after every gradient of the unit exists."""

    @staticmethod
    def forward(ctx, x, fsdp, idx):
        ctx.fsdp, ctx.idx = fsdp, idx
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.fsdp._post_backward(ctx.idx)
        return g, None, None


class FSDPPrefetchManager:
    """Brings offloaded parameter shards back to the device ahead of their use.

    With ``offload_parameters`` the bf16 shards a rank owns live in pinned host memory. ``request(i)`` starts the
    host -> device copy of unit i's shard on a copy stream into one of ``prefetch_steps + 2`` staging buffers;
    ``get(i)`` makes the compute stream wait for that copy only and returns the device view; ``release(i)`` gives
    the buffer back once the kernels that read it are queued (the next copy into it waits for them through an
    event). The reference does the same with a worker thread and a request queue
    (src/MLFramework/Distributed/FSDP/FSDPCpuOffload.cs:398-569, worker loop :453; OffloadParameter /
    PrefetchParameter :115-253); here the copy stream is the worker. On the CPU everything is synchronous."""

    def __init__(self, device: torch.device, dtype: torch.dtype, max_numel: int, steps: int):
        self.device, self.steps = device, steps
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None
        self.free = [torch.empty(max_numel, dtype=dtype, device=device) for _ in range(steps + 2)]
        self.resident: Dict[int, tuple] = {}     # unit index -> (buffer, event or None, numel)
        self.freed_at: Dict[int, object] = {}    # buffer address -> event after its last reader
        self.requests = self.hits = 0

    def request(self, idx: int, host_shard: torch.Tensor):
        if idx in self.resident or not self.free:
            return
        buf = self.free.pop()
        n = host_shard.numel()
        self.requests += 1
        if self.cuda:
            after = self.freed_at.pop(buf.data_ptr(), None)
            if after is not None:
                self.stream.wait_event(after)
            with torch.cuda.stream(self.stream):
                buf[:n].copy_(host_shard, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
        else:
            buf[:n].copy_(host_shard)
            ev = None
        self.resident[idx] = (buf, ev, n)

    def get(self, idx: int, host_shard: torch.Tensor) -> torch.Tensor:
        if idx in self.resident:
            self.hits += 1
        else:
            if not self.free:                     # every buffer is in use: drop the oldest prefetch nobody consumed
                self.release(next(iter(self.resident)))
            self.request(idx, host_shard)
        buf, ev, n = self.resident[idx]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        return buf[:n]

    def release(self, idx: int):
        ent = self.resident.pop(idx, None)
        if ent is None:
            return
        buf = ent[0]
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record()                            # after the readers queued on the compute stream
            self.freed_at[buf.data_ptr()] = ev
        self.free.append(buf)

    def release_all(self):
        for idx in list(self.resident):
            self.release(idx)


class FSDP:
    """Wraps ``model`` (which must expose ``embed``, ``blocks`` and a ``forward(ids, targets,
    loss_scale)`` like the models in :mod:`ml_framework_b200.models`; any module with a
    ``blocks`` ModuleList works) and owns the sharded optimizer."""

    def __init__(self, model: nn.Module, config: Optional[FSDPConfig], process_group,
                 optimizer_kwargs: Optional[dict] = None):
        self.cfg = config or FSDPConfig()
        self.cfg.validate()
        self.model = model
        self.pg = process_group
        self.world = process_group.world_size if process_group is not None else 1
        self.rank = process_group.rank if process_group is not None else 0
        self.device = next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        self.opt_kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
        self.opt_kw.update(optimizer_kwargs or {})
        self.step_count = 0
        self._rot_owner = {}
        self._pending_rs: list = []
        self._rs_done: dict = {}
        self.symm = None
        self.fused = False
        off = self.cfg.cpu_offload
        self.offload_params = bool(off.enabled and off.offload_parameters and self.cfg.sharding_strategy == "full")
        self.offload_grads = bool(off.enabled and off.offload_gradients)
        # peers read parameter shards straight out of this rank's device memory on the fused path, so shards that
        # live on the host go through process-group collectives instead
        if (self.cfg.fused_comm and self.world > 1 and self.device.type == "cuda" and not self.offload_params
                and self.cfg.sharding_strategy in ("full", "grad_op")):
            from ..dist.symm import SymmetricMemory
            self.symm = SymmetricMemory(process_group, self.device)
            self.fused = True
        self._build_units()
        self._allocate()
        if self.fused:
            self._setup_fused()
        self._install_hooks()
        self.optimizer = self  # exposes step()/state_dict() for the engine

    # ------------------------------------------------------------------ construction
    def _build_units(self):
        cfg, W = self.cfg, self.world
        blocks = getattr(self.model, "blocks", None)
        self.units: List[FSDPUnit] = []
        self.replicated: List[tuple] = []
        claimed = set()

        def split(prefix, module):
            sharded = []
            for n, p in module.named_parameters():
                if id(p) in claimed or not p.requires_grad:
                    continue
                claimed.add(id(p))
                full = f"{prefix}.{n}" if prefix else n
                if p.dim() < 2 or p.numel() < cfg.min_shard_numel:
                    self.replicated.append((full, p))
                else:
                    sharded.append((full, p))
            return sharded
        if blocks is not None:
            for i, blk in enumerate(blocks):
                sh = split(f"blocks.{i}", blk)
                if sh:
                    self.units.append(FSDPUnit(f"blocks.{i}", blk, sh, W, self.rank))
        root = split("", self.model)
        self.root_unit = FSDPUnit("root", self.model, root, W, self.rank) if root else None
        if cfg.sharding_strategy in ("layer_wise", "hybrid"):
            for u in self.all_units():
                lw = cfg.sharding_strategy == "layer_wise" or any(k in u.name for k in cfg.hybrid_layerwise_patterns)
                if cfg.sharding_strategy == "hybrid" and any(k in u.name for k in cfg.hybrid_full_patterns):
                    lw = False
                if lw:
                    u.owner = zlib.crc32(u.name.encode()) % W

    def all_units(self) -> List[FSDPUnit]:
        return self.units + ([self.root_unit] if self.root_unit is not None else [])

    def _allocate(self):
        dev, dt, W, r = self.device, self.dtype, self.world, self.rank
        keep_full = self.cfg.sharding_strategy == "grad_op"
        total_shard = 0
        for u in self.all_units():
            u.state_off = total_shard
            total_shard += u.shard_numel
        n_rep = sum(p.numel() for _, p in self.replicated)
        self.rep_off = total_shard
        rep_pad = (n_rep + 7) // 8 * 8
        total = total_shard + rep_pad
        state_dev = "cpu" if (self.cfg.offload_to_cpu or (self.cfg.cpu_offload.enabled and self.cfg.cpu_offload.offload_optimizer_states)) else dev
        self.state_device = torch.device(state_dev)
        pin = self.state_device.type == "cpu" and torch.cuda.is_available()
        mk = lambda: torch.zeros(total, dtype=torch.float32, device=self.state_device, pin_memory=pin)  # noqa: E731
        self.master, self.m, self.v = mk(), mk(), mk()
        esz = torch.empty(0, dtype=dt).element_size()
        self._symm_bufs = {}

        def symm_or_local(name, numel):
            if self.fused and numel > 0:
                b = self.symm.alloc(numel * esz)
                self._symm_bufs[name] = b
                return b.view(dt, numel)
            return torch.zeros(numel, dtype=dt, device=dev)
        pin_p = torch.cuda.is_available()
        if self.offload_params:
            # owned bf16 shards on the (pinned) host; the small replicated tail keeps a device copy of its own
            self.param_shards = torch.zeros(total, dtype=dt, device="cpu", pin_memory=pin_p)
            self._rep_dev = torch.zeros(rep_pad, dtype=dt, device=dev)
        else:
            self.param_shards = symm_or_local("param_shards", total)      # bf16 working copy of what this rank owns
            self._rep_dev = None
        self.grad_host = torch.zeros(total, dtype=dt, device="cpu", pin_memory=pin_p) if self.offload_grads else None
        # reduced gradients of what this rank owns (symmetric on the fused path: its replicated tail is all-reduced in place)
        self.grad_shards = symm_or_local("grad_shards", total)
        max_full = max([u.full_numel for u in self.units], default=0)
        # block units rotate through two gathered / gradient buffers; the root unit keeps its own
        n_rot = 2 if not keep_full else 0
        self._rot_full = [torch.zeros(max_full, dtype=dt, device=dev) for _ in range(n_rot)] if max_full else []
        self._rot_grad = [symm_or_local(f"rot_grad{k}", max_full) for k in range(2)] if max_full else []
        # One rank: a shard is the whole parameter, so block units compute on their shards and write
        # gradients into their gradient shards directly (nothing to gather, nothing to reduce).
        self._alias_shards = self.world == 1 and self.cfg.sharding_strategy == "full" and not self.offload_params
        self.prefetch = None
        if self.offload_params:
            max_shard = max([u.shard_numel for u in self.all_units()], default=0)
            self.prefetch = FSDPPrefetchManager(dev, dt, max_shard, self.cfg.cpu_offload.prefetch_steps)
            self._opt_stage = torch.zeros(max(max_shard, rep_pad, 8), dtype=dt, device=dev)
        with torch.no_grad():
            for u in self.all_units():
                u.shard = self.param_shards[u.state_off:u.state_off + u.shard_numel]
                u.grad_shard = self.grad_shards[u.state_off:u.state_off + u.shard_numel]
                persistent = keep_full or u is self.root_unit
                if u.owner is not None and u.owner == r:
                    # layer-wise ownership: this rank holds the whole unit and its optimizer state
                    u.owned_full = torch.zeros(u.full_numel, dtype=dt, device=dev)
                    u.owned_grad = torch.zeros(u.full_numel, dtype=dt, device=dev)
                    u.owned_master = torch.zeros(u.full_numel, dtype=torch.float32, device=self.state_device)
                    u.owned_m = torch.zeros_like(u.owned_master)
                    u.owned_v = torch.zeros_like(u.owned_master)
                if persistent:
                    u.gathered = torch.zeros(u.full_numel, dtype=dt, device=dev)
                    u.grad_full = symm_or_local(f"grad_full.{u.name}", u.full_numel) if u is self.root_unit else None
                for sp in u.sharded:
                    flat = torch.zeros(sp.padded, dtype=dt, device=dev)
                    flat[:sp.numel].copy_(sp.param.data.reshape(-1))
                    u.shard[sp.shard_off:sp.shard_off + sp.shard_numel].copy_(flat[r * sp.shard_numel:(r + 1) * sp.shard_numel])
                    if u.owner is not None and u.owner == r:
                        u.owned_full[sp.full_off:sp.full_off + sp.padded].copy_(flat)
                        u.owned_master[sp.full_off:sp.full_off + sp.padded].copy_(flat.float())
                    if persistent:
                        u.gathered[sp.full_off:sp.full_off + sp.padded].copy_(flat)
                        sp.param.data = u.gathered[sp.full_off:sp.full_off + sp.numel].view(sp.shape)
                    else:
                        sp.param.data = torch.empty(0, dtype=dt, device=dev)   # released until gathered
            # replicated small parameters: one flat buffer + flat gradient
            off = self.rep_off
            self.rep_grad = self.grad_shards[self.rep_off:self.rep_off + rep_pad]
            self.rep_flat = self.param_shards[self.rep_off:self.rep_off + rep_pad] if self._rep_dev is None else self._rep_dev
            for _, p in self.replicated:
                n = p.numel()
                self.param_shards[off:off + n].copy_(p.data.reshape(-1))
                ro = off - self.rep_off
                self.rep_flat[ro:ro + n].copy_(p.data.reshape(-1))
                p.data = self.rep_flat[ro:ro + n].view(p.shape)
                p.main_grad = self.grad_shards[off:off + n].view(p.shape)
                p._main_grad_started = False
                off += n
            self.master.copy_(self.param_shards.float().to(self.state_device))
        self._comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None

    def _setup_fused(self):
        """Device-resident segment tables for the peer-copy gather and the peer-read reduce-scatter."""
        from ..dist.symm import make_copy_segs, make_reduce_segs
        esz = self.param_shards.element_size()
        pb = self._symm_bufs["param_shards"]
        W, r = self.world, self.rank
        for u in self.all_units():
            copy, red = [], []
            for sp in u.sharded:
                for i in range(W):
                    src_rank = (r + i) % W          # own shard first, then the peers in ring order
                    src = pb.ptrs[src_rank] + (u.state_off + sp.shard_off) * esz
                    dst_off = (sp.full_off + src_rank * sp.shard_numel) * esz
                    copy.append((src, dst_off, sp.shard_numel * esz))
                red.append((sp.full_off + r * sp.shard_numel, u.state_off + sp.shard_off, sp.shard_numel))
            u._copy_rel = copy                       # dst is relative to the gathered buffer's base
            u._copy_tables = {}
            u._red_segs = make_reduce_segs(red, self.device)
            u._red_numel = sum(x[2] for x in red)
        self._grad_buf_of = {}
        self._flag = self.symm.alloc_flag()        # overflow flag every rank's reduction kernels raise on every rank
        self._rs_done = {}                         # gradient buffer address -> event of the reduction that last read it
        self._sync_key = "fsdp"

    def _copy_table(self, u: "FSDPUnit", full: torch.Tensor) -> torch.Tensor:
        return self._copy_parts(u, full)[0]

    def _copy_parts(self, u: "FSDPUnit", full: torch.Tensor):
        """The unit's peer-copy table for the gathered buffer ``full`` laid out as ``cfg.gather_parts`` consecutive parts of
        about equal bytes (every large segment is cut into that many 16-byte aligned slices, small ones stay whole in
        the first part): returns (table, row offsets of the parts, bytes per part). Copying all rows copies the unit;
        copying the rows of some parts copies those slices."""
        from ..dist.symm import make_copy_segs
        key = full.data_ptr()
        if key not in u._copy_tables:
            P = max(1, int(self.cfg.gather_parts))
            parts = [[] for _ in range(P)]
            for s, d, n in u._copy_rel:
                if n < P * 65536:
                    parts[0].append((s, key + d, n))
                    continue
                per = (n // 16 + P - 1) // P * 16
                for k in range(P):
                    lo, hi = min(n, k * per), min(n, (k + 1) * per)
                    if hi > lo:
                        parts[k].append((s + lo, key + d + lo, hi - lo))
            rows, nbytes, flat = [0], [], []
            for part in parts:
                flat.extend(part)
                rows.append(len(flat))
                nbytes.append(sum(x[2] for x in part))
            u._copy_tables[key] = (make_copy_segs(flat, self.device), rows, nbytes)
        return u._copy_tables[key]

    def _install_hooks(self):
        fs = self
        if self.cfg.activation_checkpointing:
            # each unit's forward keeps only its input and is recomputed in backward, inside the unit's
            # gather / reduce hooks (which stay on the module call, outside the recomputed region)
            from ..checkpoint.activation import checkpoint
            for u in self.units:
                inner = u.module.forward
                u.module.forward = (lambda *a, _f=inner: checkpoint(_f, *a))
        for i, u in enumerate(self.units):
            def pre(mod, args, i=i):
                fs._pre_forward(i)
                x = args[0]
                if torch.is_grad_enabled() and x.requires_grad:
                    return (_PostBackward.apply(x, fs, i),) + tuple(args[1:])
                return None

            def post(mod, args, out, i=i):
                fs._post_forward(i)
                if torch.is_grad_enabled() and isinstance(out, torch.Tensor) and out.requires_grad:
                    return _PreBackward.apply(out, fs, i)
                return out
            u.module.register_forward_pre_hook(pre)
            u.module.register_forward_hook(post)

    # ------------------------------------------------------------------ gather / release
    def _point_params(self, u: FSDPUnit, full: torch.Tensor, grad_full: Optional[torch.Tensor]):
        for sp in u.sharded:
            sp.param.data = full[sp.full_off:sp.full_off + sp.numel].view(sp.shape)
            if grad_full is not None:
                sp.param.main_grad = grad_full[sp.full_off:sp.full_off + sp.numel].view(sp.shape)
                sp.param._main_grad_started = False

    def _gather_unit(self, u: FSDPUnit, full: torch.Tensor):
        """All-gather every sharded parameter of the unit into ``full`` (per-parameter collectives,
        rank-major inside each parameter == row sharding)."""
        shard = self._device_shard(u)
        if self.world == 1:
            for sp in u.sharded:
                full[sp.full_off:sp.full_off + sp.padded].copy_(shard[sp.shard_off:sp.shard_off + sp.shard_numel])
            self._done_with_shard(u)
            return
        if self.fused:
            from ..ops import gemm as gemm_mod
            if getattr(u, "_prefetched_into", None) == full.data_ptr():
                u._prefetched_into = None            # already gathered by copy CTAs riding on an earlier GEMM
                return
            rest = gemm_mod.pending_piggyback((id(u), full.data_ptr()))
            if rest is not None:
                # the unit's GEMM-carried prefetch was only partly handed out: copy the parts nobody took
                tbl, first, n = rest
                self.symm.peer_copy(tbl[first:], n)
                return
            gemm_mod.clear_piggyback()               # a queued prefetch nobody picked up must not fire later
            tbl = self._copy_table(u, full)
            self.symm.peer_copy(tbl, tbl.shape[0])      # nothing else runs at this point: all SMs
            return
        if u.owner is not None:
            if self.rank == u.owner:
                full[:u.full_numel].copy_(u.owned_full)
            self.pg.broadcast(full[:u.full_numel], src=u.owner)
            return
        for sp in u.sharded:
            self.pg.all_gather_into(full[sp.full_off:sp.full_off + sp.padded],
                                    shard[sp.shard_off:sp.shard_off + sp.shard_numel])
        self._done_with_shard(u)

    # ---- offloaded parameter shards
    def _unit_index(self, u: FSDPUnit) -> int:
        return len(self.units) if u is self.root_unit else self.units.index(u)

    def _device_shard(self, u: FSDPUnit) -> torch.Tensor:
        """The unit's owned pieces on the device: the shard itself, or its prefetched copy when shards live on the host."""
        if self.prefetch is None:
            return u.shard
        return self.prefetch.get(self._unit_index(u), u.shard)

    def _done_with_shard(self, u: FSDPUnit):
        if self.prefetch is not None:
            self.prefetch.release(self._unit_index(u))

    def _prefetch_units(self, first: int, direction: int):
        """Start the host -> device copies of the next ``prefetch_steps`` units in execution order."""
        if self.prefetch is None:
            return
        for k in range(1, self.cfg.cpu_offload.prefetch_steps + 1):
            j = first + direction * k
            if 0 <= j < len(self.units):
                self.prefetch.request(j, self.units[j].shard)

    def _schedule_prefetch(self, j: int):
        """Attach the gather of unit j to the next large GEMM: its copy CTAs pull unit j's shards
        from the peers over NVLink while the tensor-core CTAs of that GEMM compute."""
        if not self.fused or not (0 <= j < len(self.units)) or self.cfg.sharding_strategy == "grad_op":
            return
        from ..ops import gemm as gemm_mod
        u = self.units[j]
        full = self._rot_full[j % 2]
        tbl, rows, nbytes = self._copy_parts(u, full)
        gemm_mod.set_piggyback(tbl, tbl.shape[0], n_copy_ctas=self.cfg.gather_copy_ctas,
                               on_attached=lambda u=u, full=full: setattr(u, "_prefetched_into", full.data_ptr()),
                               part_rows=rows, part_bytes=nbytes, tag=(id(u), full.data_ptr()))

    def _pre_forward(self, i: int):
        u = self.units[i]
        if self.cfg.sharding_strategy == "grad_op":
            self._point_params(u, u.gathered, None)
            return
        if self._alias_shards:
            u.gathered = u.shard
            self._point_params(u, u.shard, None)
            return
        full = self._rot_full[i % 2]
        self._gather_unit(u, full)
        self._rot_owner[i % 2] = i
        u.gathered = full
        self._point_params(u, full, None)
        self._schedule_prefetch(i + 1)
        self._prefetch_units(i, +1)

    def _post_forward(self, i: int):
        pass  # the rotating buffer is simply reused two units later

    def _pre_backward(self, i: int):
        u = self.units[i]
        if self._alias_shards:
            u.gathered, u._gbuf = u.shard, u.grad_shard
            self._point_params(u, u.shard, u.grad_shard)
            return
        gbuf = self._rot_grad[i % 2] if u.grad_full is None or self.cfg.sharding_strategy != "grad_op" else u.grad_full
        if self.cfg.sharding_strategy == "grad_op":
            gbuf = self._rot_grad[i % 2]
            self._wait_grad_buffer(gbuf)
            self._point_params(u, u.gathered, gbuf)
            u._gbuf = gbuf
            return
        full = self._rot_full[i % 2]
        if self._rot_owner.get(i % 2) != i:          # the last units of the forward pass are still resident
            self._gather_unit(u, full)
            self._rot_owner[i % 2] = i
        self._prefetch_units(i, -1)
        u.gathered = full
        self._wait_grad_buffer(gbuf)
        self._point_params(u, full, gbuf)
        u._gbuf = gbuf
        if self._rot_owner.get((i - 1) % 2) != i - 1:
            self._schedule_prefetch(i - 1)

    def _reduce_unit_fused(self, u: FSDPUnit, gbuf: torch.Tensor, found_inf=None):
        """Reduce-scatter by peer reads on the communication stream, overlapped with the backward of the
        next unit: ONE launch waits inside the kernel until every rank has queued it (their backward of
        this unit is then complete), sums this rank's slices of all W gradient buffers straight out of
        peer memory, raises every rank's overflow flag on a non-finite sum, and leaves once every peer
        has finished reading this rank's buffer. The compute stream waits for that launch only when the
        buffer is written again, two units later."""
        for sp in u.sharded:
            if not getattr(sp.param, "_main_grad_started", False):
                gbuf[sp.full_off:sp.full_off + sp.padded].zero_()
        name = next(k for k, b in self._symm_bufs.items() if b.local.data_ptr() == gbuf.data_ptr())
        buf = self._symm_bufs[name]
        cs = self._comm_stream
        ready = torch.cuda.Event()
        ready.record()
        cs.wait_event(ready)
        with torch.cuda.stream(cs):
            self.symm.rs_reduce_sync(buf, u._red_segs, u._red_segs.shape[0], self.grad_shards, u._red_numel, flag=self._flag,
                                     key=self._sync_key, max_ctas=self.cfg.reduce_ctas)
            done = torch.cuda.Event()
            done.record(cs)
        self._rs_done[gbuf.data_ptr()] = done

    def _wait_grad_buffer(self, gbuf: torch.Tensor):
        """Before a gradient buffer is written again: the reduction that read it (here and on the peers) must be over."""
        if self._pending_rs:
            self._drain_reductions(gbuf.data_ptr())
        ev = self._rs_done.pop(gbuf.data_ptr(), None) if self.fused else None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _reduce_unit(self, u: FSDPUnit, gbuf: torch.Tensor):
        if self.fused:
            self._reduce_unit_fused(u, gbuf, getattr(self, "_found_inf", None))
            return
        for sp in u.sharded:
            p = sp.param
            view = gbuf[sp.full_off:sp.full_off + sp.padded]
            if p.grad is not None:          # gradient came through autograd (CPU / non-native path)
                view[:sp.numel].copy_(p.grad.reshape(-1))
                view[sp.numel:].zero_()
                p.grad = None
            elif not getattr(p, "_main_grad_started", False):
                view.zero_()
            out = u.grad_shard[sp.shard_off:sp.shard_off + sp.shard_numel]
            if self.world == 1:
                if out.data_ptr() != view.data_ptr():     # a single rank writes gradients straight into its shard
                    out.copy_(view)
            elif u.owner is not None:
                self.pg.reduce(view, dst=u.owner, op=ReduceOp.SUM)
                if self.rank == u.owner:
                    u.owned_grad[sp.full_off:sp.full_off + sp.padded].copy_(view)
                out.zero_()
            else:
                # asynchronous: up to num_communication_workers units' reductions stay in flight behind the
                # backward of the following units (the reference's communication workers, FSDPConfig.cs:8-58)
                work = self.pg.reduce_scatter(view, op=ReduceOp.SUM, async_op=True)
                self._pending_rs.append((gbuf.data_ptr(), work, out))
        if self.world > 1 and u.owner is None:
            limit = self.cfg.num_communication_workers * max(1, len(u.sharded))
            while len(self._pending_rs) > limit:
                self._complete_reduction(self._pending_rs.pop(0))

    def _complete_reduction(self, ent):
        _, work, out = ent
        out.copy_(work.wait())

    def _drain_reductions(self, buffer_ptr: Optional[int] = None):
        """Completes the asynchronous reductions that read ``buffer_ptr`` (all of them when None)."""
        keep = []
        for ent in self._pending_rs:
            if buffer_ptr is None or ent[0] == buffer_ptr:
                self._complete_reduction(ent)
            else:
                keep.append(ent)
        self._pending_rs = keep

    def _post_backward(self, i: int):
        u = self.units[i]
        with nvtx_range(f"fsdp.reduce_scatter.{u.name}"):
            self._reduce_unit(u, u._gbuf)
            self._offload_unit_grads(u)

    def _offload_unit_grads(self, u: FSDPUnit):
        """``offload_gradients``: the reduced gradient pieces leave for pinned host memory as soon as they exist
        (FSDPCpuOffload.OffloadGradient, FSDPCpuOffload.cs:175-214); the update then reads them there."""
        if self.grad_host is None or self.fused:
            return
        self._drain_reductions(u._gbuf.data_ptr() if hasattr(u, "_gbuf") and u is not self.root_unit else None)
        s0, n = u.state_off, u.shard_numel
        self.grad_host[s0:s0 + n].copy_(self.grad_shards[s0:s0 + n], non_blocking=True)

    # ------------------------------------------------------------------ step
    def train_step(self, ids, targets, scaler=None):
        self.zero_grad()
        if self.fused and scaler is not None:
            flag = self._flag.view(torch.int32, 1)
            if scaler.found_inf.data_ptr() != flag.data_ptr():
                scaler.found_inf = flag           # the scaler's flag is the one the reduction kernels raise on every rank
        self._found_inf = scaler.found_inf if scaler is not None else None
        self._rot_owner = {}                          # shards changed at the last optimizer step
        root = self.root_unit
        if root is not None:
            if self.cfg.sharding_strategy != "grad_op":
                self._gather_unit(root, root.gathered)
            self._point_params(root, root.gathered, root.grad_full)
        scale_t = scaler.scale_t if scaler is not None else None
        with nvtx_range("fsdp.forward"):
            loss = self.model(ids, targets, loss_scale=scale_t)
        with nvtx_range("fsdp.backward"):
            loss.backward()
        with nvtx_range("fsdp.reduce_root_and_replicated"):
            if root is not None:
                self._reduce_unit(root, root.grad_full)
                self._offload_unit_grads(root)
            self._finish_replicated()
        with nvtx_range("fsdp.optimizer"):
            self.step(scaler)
        return loss

    def _finish_replicated(self):
        self._drain_reductions()
        for _, p in self.replicated:
            if p.grad is not None:
                if getattr(p, "_main_grad_started", False):
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                p.grad = None
            elif not getattr(p, "_main_grad_started", False):
                p.main_grad.zero_()
        if self.world > 1 and self.rep_grad.numel():
            if self.fused:
                # in place over every rank's replicated tail, on the communication stream behind the unit reductions
                cs = self._comm_stream
                cs.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(cs):
                    self.symm.all_reduce_two_shot_sync(self._symm_bufs["grad_shards"], self.rep_grad.numel(), flag=self._flag,
                                                       offset_bytes=self.rep_off * self.rep_grad.element_size(),
                                                       key=self._sync_key, max_ctas=32)
            else:
                # bucket_size_mb bounds one all-reduce message (FSDPConfig.BucketSizeMB, FSDPConfig.cs:8-58)
                per = max(8, int(self.cfg.bucket_size_mb * 1024 * 1024) // self.rep_grad.element_size())
                for lo in range(0, self.rep_grad.numel(), per):
                    self.pg.all_reduce(self.rep_grad[lo:lo + per], op=ReduceOp.SUM)
        if self.fused:
            torch.cuda.current_stream().wait_stream(self._comm_stream)   # every reduction of the step is in grad_shards
            self._rs_done.clear()

    def zero_grad(self):
        for _, p in self.replicated:
            p._main_grad_started = False
            p.grad = None
        for u in self.all_units():
            for sp in u.sharded:
                sp.param.grad = None
                sp.param._main_grad_started = False

    def step(self, scaler=None):
        """Sharded AdamW over everything this rank owns (one fused kernel on the GPU)."""
        self.step_count += 1
        kw = self.opt_kw
        g = self.grad_shards
        inv_scale = found = None
        if scaler is not None:
            if self.fused:
                pass    # every reduced value was checked by the reduction kernels, which raise the flag on all ranks
            else:
                if g.is_cuda:
                    native.amp_unscale_check_(g, scaler.found_inf, inv_scale=None, write_back=False)
                elif not torch.isfinite(g.float()).all():
                    scaler.found_inf.fill_(1)
                scaler.sync_found_inf(self.pg)
            inv_scale, found = scaler.inv_scale_t, scaler.found_inf
        gscale = 1.0 / self.world
        b1, b2 = kw["betas"]
        if self.master.is_cuda and self.offload_params:
            # parameter shards live on the host: update unit by unit through a device staging buffer, each slice
            # leaving for pinned memory right behind its kernel (stream order keeps the one buffer safe)
            if self.prefetch is not None:
                self.prefetch.release_all()
            spans = [(u.state_off, u.shard_numel) for u in self.all_units() if u.shard_numel]
            rep_n = self.rep_flat.numel()
            for s0, n in spans + ([(self.rep_off, rep_n)] if rep_n else []):
                stage = self._opt_stage[:n] if s0 != self.rep_off else self.rep_flat
                native.adamw_(self.master[s0:s0 + n], self.m[s0:s0 + n], self.v[s0:s0 + n], g[s0:s0 + n], stage, lr=kw["lr"],
                              beta1=b1, beta2=b2, eps=kw["eps"], weight_decay=kw["weight_decay"], step=self.step_count,
                              grad_scale=gscale, inv_scale=inv_scale, found_inf=found)
                self.param_shards[s0:s0 + n].copy_(stage, non_blocking=True)
        elif self.master.is_cuda:
            native.adamw_(self.master, self.m, self.v, g, self.param_shards, lr=kw["lr"], beta1=b1, beta2=b2, eps=kw["eps"],
                          weight_decay=kw["weight_decay"], step=self.step_count, grad_scale=gscale, inv_scale=inv_scale,
                          found_inf=found)
        else:
            skip = found is not None and int(found.item()) != 0
            if not skip:
                if self.grad_host is not None:
                    # the sharded part arrived unit by unit during backward; the replicated tail follows now
                    rn = self.rep_grad.numel()
                    if rn:
                        self.grad_host[self.rep_off:self.rep_off + rn].copy_(self.rep_grad)
                    if g.is_cuda:
                        torch.cuda.current_stream().synchronize()
                    g = self.grad_host
                gf = g.detach().to(self.state_device).float() * gscale
                if inv_scale is not None:
                    gf = gf * float(inv_scale.item())
                p, m, v = reference.adamw_ref(self.master, self.m, self.v, gf, lr=kw["lr"], beta1=b1, beta2=b2,
                                              eps=kw["eps"], weight_decay=kw["weight_decay"], step=self.step_count)
                self.master.copy_(p); self.m.copy_(m); self.v.copy_(v)
                self.param_shards.copy_(self.master.to(self.param_shards.device, non_blocking=True).to(self.dtype))
                if self._rep_dev is not None:
                    rn = self._rep_dev.numel()
                    self._rep_dev.copy_(self.param_shards[self.rep_off:self.rep_off + rn], non_blocking=True)
            if self.prefetch is not None:
                self.prefetch.release_all()
        for u in self.all_units():
            if u.owner is not None and u.owner == self.rank and self.world > 1:
                self._step_owned(u, gscale, inv_scale, found)
        if scaler is not None:
            scaler.update()
        if self.fused:
            self.symm.barrier()      # peers may read the updated shards only after every rank's update
        if self.cfg.sharding_strategy == "grad_op":
            for u in self.all_units():
                self._gather_unit(u, u.gathered)

    def _step_owned(self, u: FSDPUnit, gscale, inv_scale, found):
        kw = self.opt_kw
        b1, b2 = kw["betas"]
        if u.owned_master.is_cuda:
            native.adamw_(u.owned_master, u.owned_m, u.owned_v, u.owned_grad, u.owned_full, lr=kw["lr"], beta1=b1, beta2=b2,
                          eps=kw["eps"], weight_decay=kw["weight_decay"], step=self.step_count, grad_scale=gscale,
                          inv_scale=inv_scale, found_inf=found)
            return
        if found is not None and int(found.item()) != 0:
            return
        gf = u.owned_grad.detach().to(self.state_device).float() * gscale
        if inv_scale is not None:
            gf = gf * float(inv_scale.item())
        p, m, v = reference.adamw_ref(u.owned_master, u.owned_m, u.owned_v, gf, lr=kw["lr"], beta1=b1, beta2=b2,
                                      eps=kw["eps"], weight_decay=kw["weight_decay"], step=self.step_count)
        u.owned_master.copy_(p); u.owned_m.copy_(m); u.owned_v.copy_(v)
        u.owned_full.copy_(u.owned_master.to(u.owned_full.device).to(self.dtype))

    def close(self):
        """Unmaps and frees the symmetric buffers (parameters, gradients and shards living in them become invalid)."""
        if self.symm is not None:
            if self.pg is not None and self.world > 1:
                torch.cuda.synchronize()
                self.pg.barrier()          # nobody may still be reading this rank's buffers
            self.symm.close()
            self.symm = None

    # ------------------------------------------------------------------ state
    def set_learning_rate(self, lr: float):
        self.opt_kw["lr"] = lr

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Gathers every parameter in full precision of the working dtype (all ranks get a copy)."""
        out = {}
        for u in self.all_units():
            full = torch.zeros(u.full_numel, dtype=self.dtype, device=self.device)
            self._gather_unit(u, full)
            for sp in u.sharded:
                out[sp.name] = full[sp.full_off:sp.full_off + sp.numel].view(sp.shape).clone()
        for n, p in self.replicated:
            out[n] = p.detach().clone()
        return out

    def local_state(self) -> Dict[str, torch.Tensor]:
        """This rank's shard of parameters and optimizer state (for multi-shard checkpoints)."""
        return {"param_shards": self.param_shards, "master": self.master, "m": self.m, "v": self.v,
                "step": torch.tensor(self.step_count)}

    def load_local_state(self, sd):
        self.param_shards.copy_(sd["param_shards"])
        self.master.copy_(sd["master"]); self.m.copy_(sd["m"]); self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])

    def state_dict(self):
        return {k: (v.detach().cpu().clone() if isinstance(v, torch.Tensor) else v) for k, v in self.local_state().items()}
