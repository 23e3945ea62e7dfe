"""FSDP state utilities: gather / scatter of the sharded optimizer state, gather-to-rank-0 checkpoints,
gradient accumulation over micro-batches.

Reference: ``FSDPOptimizerStateManager.GatherOptimizerState / ScatterOptimizerState / GatherAdamState /
ScatterAdamState`` (src/MLFramework/Distributed/FSDP/FSDPOptimizerStateManager.cs:120-245), ``FSDPCheckpoint``
(FSDPCheckpoint.cs:62-331: gather to rank 0, files ``{prefix}_epoch{e}_step{s}_metadata.json`` /
``_parameters.bin`` / ``_optimizer.bin``, keep the last ``MaxCheckpoints = 5``), ``GradientAccumulator``
(FSDP/GradientAccumulator.cs:42-140). Works for the full-shard and grad-op strategies.
"""
from __future__ import annotations

import glob
import json
import os
import re
import time
from typing import Dict, List, Optional

import torch


def _piece(buf: torch.Tensor, u, sp) -> torch.Tensor:
    return buf[u.state_off + sp.shard_off:u.state_off + sp.shard_off + sp.shard_numel]


def gather_optimizer_state(fsdp, dst: Optional[int] = 0) -> Optional[Dict[str, Dict[str, torch.Tensor]]]:
    """Full (unsharded) fp32 master weights and Adam moments per parameter name. ``dst`` = the rank that keeps
    the result (None: every rank)."""
    out: Dict[str, Dict[str, torch.Tensor]] = {}
    keep = dst is None or fsdp.rank == dst
    for u in fsdp.all_units():
        for sp in u.sharded:
            entry = {}
            for key, buf in (("master", fsdp.master), ("exp_avg", fsdp.m), ("exp_avg_sq", fsdp.v)):
                local = _piece(buf, u, sp).to(fsdp.device)
                full = fsdp.pg.all_gather(local.contiguous(), dim=0) if fsdp.world > 1 else local
                if keep:
                    entry[key] = full[:sp.numel].view(sp.shape).cpu().clone()
            if keep:
                out[sp.name] = entry
    off = fsdp.rep_off
    for n, p in fsdp.replicated:
        k = p.numel()
        if keep:
            out[n] = {"master": fsdp.master[off:off + k].view(p.shape).cpu().clone(), "exp_avg": fsdp.m[off:off + k].view(p.shape).cpu().clone(),
                      "exp_avg_sq": fsdp.v[off:off + k].view(p.shape).cpu().clone()}
        off += k
    if keep:
        out["__step__"] = {"step": torch.tensor(fsdp.step_count)}
    return out if keep else None


def scatter_optimizer_state(fsdp, full: Dict[str, Dict[str, torch.Tensor]]):
    """Every rank slices its own piece out of the full state (``full`` must be available on every rank: load the
    file on each rank, or broadcast it first) and refreshes its working parameter shard from the master weights."""
    W, r = fsdp.world, fsdp.rank
    with torch.no_grad():
        for u in fsdp.all_units():
            for sp in u.sharded:
                e = full[sp.name]
                for key, buf in (("master", fsdp.master), ("exp_avg", fsdp.m), ("exp_avg_sq", fsdp.v)):
                    flat = torch.zeros(sp.padded, dtype=torch.float32)
                    flat[:sp.numel] = e[key].reshape(-1).float()
                    _piece(buf, u, sp).copy_(flat[r * sp.shard_numel:(r + 1) * sp.shard_numel])
                u.shard[sp.shard_off:sp.shard_off + sp.shard_numel].copy_(_piece(fsdp.master, u, sp).to(fsdp.device).to(fsdp.dtype))
                if u.gathered is not None:                  # persistent (grad-op strategy / root unit): refresh the full copy too
                    u.gathered[sp.full_off:sp.full_off + sp.numel].copy_(e["master"].reshape(-1).to(fsdp.device).to(fsdp.dtype))
        off = fsdp.rep_off
        for n, p in fsdp.replicated:
            k = p.numel()
            e = full[n]
            fsdp.master[off:off + k].copy_(e["master"].reshape(-1).float())
            fsdp.m[off:off + k].copy_(e["exp_avg"].reshape(-1).float())
            fsdp.v[off:off + k].copy_(e["exp_avg_sq"].reshape(-1).float())
            fsdp.param_shards[off:off + k].copy_(e["master"].reshape(-1).to(fsdp.device).to(fsdp.dtype))
            off += k
        if "__step__" in full:
            fsdp.step_count = int(full["__step__"]["step"])


class FSDPCheckpoint:
    def __init__(self, fsdp, directory: str, prefix: str = "fsdp", max_checkpoints: int = 5):
        self.fsdp, self.dir, self.prefix, self.max = fsdp, directory, prefix, max_checkpoints
        os.makedirs(directory, exist_ok=True)

    def _base(self, epoch: int, step: int) -> str:
        return os.path.join(self.dir, f"{self.prefix}_epoch{epoch}_step{step}")

    def save(self, epoch: int, step: int, extra: Optional[Dict] = None) -> Optional[str]:
        f = self.fsdp
        params = f.full_state_dict()                               # collective
        opt = gather_optimizer_state(f, dst=0)                     # collective
        base = self._base(epoch, step)
        if f.rank == 0:
            torch.save({k: v.cpu() for k, v in params.items()}, base + "_parameters.bin.tmp")
            os.replace(base + "_parameters.bin.tmp", base + "_parameters.bin")
            torch.save(opt, base + "_optimizer.bin.tmp")
            os.replace(base + "_optimizer.bin.tmp", base + "_optimizer.bin")
            meta = {"epoch": epoch, "step": step, "world_size": f.world, "timestamp": time.time(), "strategy": f.cfg.sharding_strategy,
                    "parameters": {k: list(v.shape) for k, v in params.items()}, "extra": extra or {}}
            with open(base + "_metadata.json.tmp", "w") as fh:
                json.dump(meta, fh, indent=1)
            os.replace(base + "_metadata.json.tmp", base + "_metadata.json")       # the manifest appears last: its presence marks a complete save
            self._prune()
        f.pg.barrier() if f.world > 1 else None
        return base if f.rank == 0 else None

    def list(self) -> List[tuple]:
        out = []
        for p in glob.glob(os.path.join(self.dir, f"{self.prefix}_epoch*_step*_metadata.json")):
            m = re.search(r"_epoch(\d+)_step(\d+)_metadata\.json$", p)
            if m:
                out.append((int(m[1]), int(m[2])))
        return sorted(out)

    def _prune(self):
        for e, s in self.list()[:-self.max] if self.max > 0 else []:
            for suffix in ("_metadata.json", "_parameters.bin", "_optimizer.bin"):
                try:
                    os.remove(self._base(e, s) + suffix)
                except FileNotFoundError:
                    pass

    def load(self, epoch: Optional[int] = None, step: Optional[int] = None) -> Dict:
        """Loads the given (or the latest) checkpoint at the CURRENT world size: the files hold full tensors, every
        rank slices what it owns."""
        have = self.list()
        if not have:
            raise FileNotFoundError(f"no checkpoints with prefix {self.prefix!r} in {self.dir}")
        e, s = (epoch, step) if epoch is not None else have[-1]
        base = self._base(e, s)
        with open(base + "_metadata.json") as fh:
            meta = json.load(fh)
        opt = torch.load(base + "_optimizer.bin", map_location="cpu", weights_only=True)
        scatter_optimizer_state(self.fsdp, opt)
        return meta


class FSDPGradientAccumulator:
    """Accumulates the reduced gradient shards of several micro-batches before the optimizer step
    (the sum lives in fp32; ``apply`` writes the average back to the gradient shard buffer)."""

    def __init__(self, fsdp, accumulation_steps: int):
        if accumulation_steps <= 0:
            raise ValueError("accumulation_steps must be positive")
        self.fsdp, self.n, self.count = fsdp, accumulation_steps, 0
        self._acc = torch.zeros(fsdp.grad_shards.numel(), dtype=torch.float32, device=fsdp.grad_shards.device)

    def add_gradients(self) -> bool:
        self._acc += self.fsdp.grad_shards.float()
        self.count += 1
        return self.is_complete()

    def is_complete(self) -> bool:
        return self.count >= self.n

    def apply(self):
        self.fsdp.grad_shards.copy_((self._acc / max(1, self.count)).to(self.fsdp.grad_shards.dtype))
        self._acc.zero_()
        self.count = 0
