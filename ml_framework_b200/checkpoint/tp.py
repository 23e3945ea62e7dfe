"""Checkpoints of tensor-parallel models and checkpoint validation.

Reference: ``DistributedTPCheckpoint`` (one file per TP rank in a directory, src/MLFramework/Checkpoint/
DistributedTPCheckpoint.cs:44-240), ``CentralizedTPCheckpoint`` (shards gathered to one file on rank 0,
CentralizedTPCheckpoint.cs:31-252), ``TPCheckpointManager`` (:19-178), ``TPCheckpointMetadata`` (ModelName, SavedAt,
TPWorldSize, MeshShape, Version :10-39); ``CheckpointValidator`` with integrity (checksum, size) and compatibility
(schema, version) checkers (src/MLFramework/Checkpointing/Validation/CheckpointValidator.cs:36-132).
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

VERSION = "1.0.0"


@dataclass
class TPCheckpointMetadata:
    model_name: str
    tp_world_size: int
    mesh_shape: Sequence[int] = ()
    saved_at: float = field(default_factory=time.time)
    version: str = VERSION
    shard_dims: Dict[str, Optional[int]] = field(default_factory=dict)     # parameter -> dimension split over TP (None = replicated)
    checksums: Dict[str, str] = field(default_factory=dict)                # file -> sha256


def _sha(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for c in iter(lambda: f.read(1 << 20), b""):
            h.update(c)
    return h.hexdigest()


def default_shard_dim(name: str, tensor: torch.Tensor) -> Optional[int]:
    """Which dimension of a parameter of this package's TP layers is split: column-parallel weights and the
    vocabulary-parallel tables on dim 0, row-parallel weights on dim 1, norms replicated."""
    if tensor.dim() < 2:
        return None if "norm" in name else 0
    if any(k in name for k in (".o.", ".down.", "row")):
        return 1
    return 0


class DistributedTPCheckpoint:
    """Every TP rank writes ``rank_{r}.pt`` into the checkpoint directory; rank 0 adds ``tp_metadata.json``."""

    def __init__(self, directory: str, pg=None):
        self.dir, self.pg = directory, pg
        self.rank = pg.rank if pg is not None else 0
        self.world = pg.world_size if pg is not None else 1

    def save(self, state: Dict[str, torch.Tensor], model_name: str = "model", mesh_shape: Sequence[int] = (),
             shard_dim: Callable[[str, torch.Tensor], Optional[int]] = default_shard_dim) -> str:
        os.makedirs(self.dir, exist_ok=True)
        path = os.path.join(self.dir, f"rank_{self.rank}.pt")
        torch.save({k: v.detach().cpu() for k, v in state.items()}, path + ".tmp")
        os.replace(path + ".tmp", path)
        sums = self.pg.all_gather_object((f"rank_{self.rank}.pt", _sha(path))) if self.pg is not None else [(f"rank_0.pt", _sha(path))]
        if self.rank == 0:
            meta = TPCheckpointMetadata(model_name, self.world, list(mesh_shape), shard_dims={k: shard_dim(k, v) for k, v in state.items()},
                                        checksums=dict(sums))
            with open(os.path.join(self.dir, "tp_metadata.json"), "w") as f:
                json.dump(asdict(meta), f, indent=1)
        if self.pg is not None:
            self.pg.barrier()
        return path

    def load_metadata(self) -> TPCheckpointMetadata:
        with open(os.path.join(self.dir, "tp_metadata.json")) as f:
            return TPCheckpointMetadata(**json.load(f))

    def load(self, verify: bool = True) -> Dict[str, torch.Tensor]:
        meta = self.load_metadata()
        if meta.tp_world_size != self.world:
            raise ValueError(f"checkpoint was written at TP = {meta.tp_world_size}, loading at TP = {self.world}; use CentralizedTPCheckpoint "
                             "or load_full() and re-split")
        path = os.path.join(self.dir, f"rank_{self.rank}.pt")
        if verify and meta.checksums.get(f"rank_{self.rank}.pt") not in (None, _sha(path)):
            raise IOError(f"{path}: checksum mismatch")
        return torch.load(path, map_location="cpu", weights_only=True)

    def load_full(self) -> Dict[str, torch.Tensor]:
        """Reassembles full tensors from all rank files (any process can do this)."""
        meta = self.load_metadata()
        shards = [torch.load(os.path.join(self.dir, f"rank_{r}.pt"), map_location="cpu", weights_only=True) for r in range(meta.tp_world_size)]
        return merge_tp_shards(shards, meta.shard_dims)


def merge_tp_shards(shards: Sequence[Dict[str, torch.Tensor]], shard_dims: Dict[str, Optional[int]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in shards[0]:
        d = shard_dims.get(k)
        out[k] = shards[0][k].clone() if d is None else torch.cat([s[k] for s in shards], dim=d)
    return out


def split_tp_state(full: Dict[str, torch.Tensor], shard_dims: Dict[str, Optional[int]], world: int, rank: int) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in full.items():
        d = shard_dims.get(k)
        if d is None:
            out[k] = v.clone()
        else:
            if v.shape[d] % world:
                raise ValueError(f"{k}: dimension {d} of size {v.shape[d]} is not divisible by TP = {world}")
            out[k] = v.chunk(world, dim=d)[rank].contiguous().clone()
    return out


class CentralizedTPCheckpoint:
    """Rank 0 gathers every rank's shards and writes ONE file with full tensors; loading re-splits for the current TP size."""

    def __init__(self, path: str, pg=None):
        self.path, self.pg = path, pg
        self.rank = pg.rank if pg is not None else 0
        self.world = pg.world_size if pg is not None else 1

    def save(self, state: Dict[str, torch.Tensor], model_name: str = "model",
             shard_dim: Callable[[str, torch.Tensor], Optional[int]] = default_shard_dim):
        dims = {k: shard_dim(k, v) for k, v in state.items()}
        cpu = {k: v.detach().cpu() for k, v in state.items()}
        shards = self.pg.all_gather_object(cpu) if self.pg is not None else [cpu]
        if self.rank == 0:
            full = merge_tp_shards(shards, dims)
            meta = asdict(TPCheckpointMetadata(model_name, self.world, shard_dims=dims))
            torch.save({"state": full, "metadata": meta}, self.path + ".tmp")
            os.replace(self.path + ".tmp", self.path)
        if self.pg is not None:
            self.pg.barrier()

    def load(self) -> Tuple[Dict[str, torch.Tensor], TPCheckpointMetadata]:
        blob = torch.load(self.path, map_location="cpu", weights_only=False)
        meta = TPCheckpointMetadata(**blob["metadata"])
        return split_tp_state(blob["state"], meta.shard_dims, self.world, self.rank), meta


class TPCheckpointManager:
    def __init__(self, root: str, pg=None, centralized: bool = False, max_to_keep: int = 5):
        self.root, self.pg, self.centralized, self.max = root, pg, centralized, max_to_keep
        os.makedirs(root, exist_ok=True)

    def _tags(self) -> List[str]:
        return sorted(d for d in os.listdir(self.root) if d.startswith("step_"))

    def save(self, step: int, state: Dict[str, torch.Tensor], **kw):
        tag = f"step_{step:09d}"
        if self.centralized:
            CentralizedTPCheckpoint(os.path.join(self.root, tag + ".pt"), self.pg).save(state, **kw)
        else:
            DistributedTPCheckpoint(os.path.join(self.root, tag), self.pg).save(state, **kw)
        if (self.pg is None or self.pg.rank == 0) and self.max > 0:
            import shutil
            for old in self._tags()[:-self.max]:
                p = os.path.join(self.root, old)
                shutil.rmtree(p) if os.path.isdir(p) else os.remove(p)

    def latest_step(self) -> Optional[int]:
        t = self._tags()
        return int(t[-1].split("_")[1].split(".")[0]) if t else None

    def load(self, step: Optional[int] = None) -> Dict[str, torch.Tensor]:
        step = self.latest_step() if step is None else step
        if step is None:
            raise FileNotFoundError(f"no checkpoints under {self.root}")
        tag = f"step_{step:09d}"
        if self.centralized:
            return CentralizedTPCheckpoint(os.path.join(self.root, tag + ".pt"), self.pg).load()[0]
        return DistributedTPCheckpoint(os.path.join(self.root, tag), self.pg).load()


# ------------------------------------------------------------------ validation
@dataclass
class ValidationResult:
    ok: bool
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)


class CheckpointValidator:
    """Integrity (files present, sizes, SHA-256) and compatibility (format version, world size, tensor shapes against a
    model) of a multi-shard checkpoint written by ``checkpoint.distributed``."""

    def __init__(self, supported_major: int = 1):
        self.supported_major = supported_major

    def validate(self, prefix: str, model_state: Optional[Dict[str, torch.Tensor]] = None, world_size: Optional[int] = None) -> ValidationResult:
        from .distributed import CheckpointLoader, ShardFileVerifier
        res = ValidationResult(True)
        try:
            meta = CheckpointLoader().load_metadata(prefix)
        except Exception as e:
            return ValidationResult(False, [f"manifest unreadable: {e}"])
        try:
            major = int(str(meta.Version).split(".")[0])
            if major != self.supported_major:
                res.errors.append(f"format version {meta.Version} is not supported (major {self.supported_major})")
        except ValueError:
            res.errors.append(f"malformed version {meta.Version!r}")
        ok, errs = ShardFileVerifier.verify_checkpoint(prefix)
        if not ok:
            res.errors += errs
        if world_size is not None and meta.WorldSize != world_size:
            res.warnings.append(f"checkpoint world size {meta.WorldSize} != current {world_size}: loading will reshard")
        if model_state is not None:
            names = {t.Name for s in meta.Shards for t in s.Tensors}
            for k in model_state:
                if k not in names and not any(n.endswith("." + k) or n.startswith(k + ".") for n in names):
                    res.errors.append(f"tensor {k!r} missing from the checkpoint")
        res.ok = not res.errors
        return res
