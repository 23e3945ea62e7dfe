"""Checks and helpers around the distributed checkpoint: integrity, compatibility, typed state, per-strategy collection.

Reference (src/MLFramework/Checkpointing/): Validation/CheckpointValidator.cs:36-132, Integrity/{Checksum,Size}IntegrityChecker.cs,
Compatibility/{Schema,Version}CompatibilityChecker.cs, State/{StateCompatibilityChecker.cs, DistributedStateCollector.cs,
ModelStateDict.cs, OptimizerStateDict.cs}, Integration/{FSDPCheckpointHelper.cs:32-52, DDPCheckpointHelper.cs:32,
TensorParallelCheckpointHelper.cs:32}, Resharding/ReshardingStrategy.cs (SimpleReshardingStrategy :162-290 reads every shard
and cuts, ParallelReshardingStrategy :292-496 reads only what overlaps), API/{CheckpointEnums.cs, CheckpointOptions.cs,
DistributedCheckpointFactory.cs}.
"""
from __future__ import annotations

import enum
import hashlib
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .distributed import (FORMAT_VERSION, CheckpointError, CheckpointMetadata, DistributedCheckpoint, LoadOptions, MetadataValidator, MultiShardCheckpointFormat, ReshardingStrategy, SaveOptions, manifest_path)


class CheckpointFormat(enum.Enum):
    MULTI_SHARD = "multishard"
    SINGLE_FILE = "singlefile"


class CheckpointCompressionLevel(enum.Enum):
    NONE = "none"
    FAST = "fast"
    BALANCED = "balanced"
    MAX = "max"


# ------------------------------------------------------------------ results
@dataclass
class ValidationIssue:
    check: str
    message: str
    severity: str = "error"          # error | warning


@dataclass
class ValidationReport:
    issues: List[ValidationIssue] = field(default_factory=list)

    @property
    def is_valid(self) -> bool:
        return not any(i.severity == "error" for i in self.issues)

    def errors(self) -> List[str]:
        return [f"{i.check}: {i.message}" for i in self.issues if i.severity == "error"]

    def warnings(self) -> List[str]:
        return [f"{i.check}: {i.message}" for i in self.issues if i.severity == "warning"]

    def add(self, check: str, message: str, severity: str = "error"):
        self.issues.append(ValidationIssue(check, message, severity))

    def extend(self, other: "ValidationReport"):
        self.issues.extend(other.issues)


def _shard_file(prefix: str, s) -> str:
    return os.path.join(os.path.dirname(prefix) or ".", s.FilePath)


# ------------------------------------------------------------------ integrity
class SizeIntegrityChecker:
    name = "size"

    def check(self, prefix: str, meta: CheckpointMetadata) -> ValidationReport:
        r = ValidationReport()
        for s in meta.Shards:
            p = _shard_file(prefix, s)
            if not os.path.exists(p):
                r.add(self.name, f"shard file {s.FilePath} is missing")
            elif os.path.getsize(p) != s.FileSize:
                r.add(self.name, f"{s.FilePath}: {os.path.getsize(p)} bytes on disk, manifest says {s.FileSize}")
            data = sum(t.Size for t in s.Tensors)
            if data > s.FileSize:
                r.add(self.name, f"{s.FilePath}: tensors need {data} bytes, file has {s.FileSize}")
        return r


class ChecksumIntegrityChecker:
    """Recomputes every shard's payload checksum (the shard reader verifies SHA-256 while it reads)."""
    name = "checksum"

    def check(self, prefix: str, meta: CheckpointMetadata) -> ValidationReport:
        r = ValidationReport()
        for s in meta.Shards:
            p = _shard_file(prefix, s)
            if not os.path.exists(p):
                continue                       # the size check reports missing files
            try:
                MultiShardCheckpointFormat.read_shard(p, s, verify=True, names=[])
            except CheckpointError as e:
                r.add(self.name, f"{s.FilePath}: {e}")
        return r


# ------------------------------------------------------------------ compatibility
class VersionCompatibilityChecker:
    """Same major version required; a newer minor version than this reader's is a warning (fields may be ignored)."""
    name = "version"

    def __init__(self, reader_version: str = FORMAT_VERSION):
        self.reader = self._parse(reader_version)

    @staticmethod
    def _parse(v: str) -> Tuple[int, int, int]:
        parts = (v.split(".") + ["0", "0"])[:3]
        try:
            return tuple(int(x) for x in parts)
        except ValueError:
            raise ValueError(f"not a version: {v!r}")

    def check(self, meta: CheckpointMetadata) -> ValidationReport:
        r = ValidationReport()
        try:
            v = self._parse(meta.Version)
        except ValueError as e:
            r.add(self.name, str(e))
            return r
        if v[0] != self.reader[0]:
            r.add(self.name, f"checkpoint format {meta.Version} is not readable by format {'.'.join(map(str, self.reader))}")
        elif v[:2] > self.reader[:2]:
            r.add(self.name, f"checkpoint format {meta.Version} is newer than this reader; unknown fields are ignored", "warning")
        return r


class SchemaCompatibilityChecker:
    """The manifest has what a loader needs: shards for every rank, tensor entries with dtype / shape / extent that
    agree with each other, consistent slice descriptions of sharded tensors across ranks."""
    name = "schema"
    _ITEM = {"float32": 4, "float16": 2, "bfloat16": 2, "float64": 8, "int64": 8, "int32": 4, "int16": 2, "int8": 1, "uint8": 1, "bool": 1}

    def check(self, meta: CheckpointMetadata) -> ValidationReport:
        r = ValidationReport()
        for e in MetadataValidator.validate(meta):
            r.add(self.name, e)
        slices: Dict[str, List] = {}
        for s in meta.Shards:
            for t in s.Tensors:
                n = 1
                for d in t.Shape:
                    n *= d
                isz = self._ITEM.get(t.DataType)
                if isz is None:
                    r.add(self.name, f"{t.Name}: unknown data type {t.DataType!r}")
                elif n * isz != t.Size:
                    r.add(self.name, f"{t.Name} in shard {s.Rank}: shape {t.Shape} x {isz} bytes != {t.Size}")
                if t.ShardDim is not None:
                    slices.setdefault(t.Name, []).append(t)
        for name, ts in slices.items():
            g = ts[0].GlobalShape
            if any(t.GlobalShape != g or t.ShardDim != ts[0].ShardDim for t in ts):
                r.add(self.name, f"{name}: ranks disagree on the global shape or the sharded dimension")
                continue
            if g is not None and sum(t.Shape[t.ShardDim] for t in ts) < g[ts[0].ShardDim]:
                r.add(self.name, f"{name}: slices cover {sum(t.Shape[t.ShardDim] for t in ts)} of {g[ts[0].ShardDim]} along dim {ts[0].ShardDim}")
            if sorted(t.ShardIndex for t in ts) != list(range(len(ts))):
                r.add(self.name, f"{name}: slice indices are not 0..{len(ts) - 1}")
        return r


class CheckpointValidator:
    """Everything at once: manifest present and parseable, schema, version, sizes and (unless ``quick``) checksums."""

    def __init__(self, quick: bool = False):
        self.quick = quick

    def validate(self, prefix: str) -> ValidationReport:
        r = ValidationReport()
        if not os.path.exists(manifest_path(prefix)):
            r.add("manifest", f"no manifest at {manifest_path(prefix)}")
            return r
        try:
            meta = CheckpointMetadata.from_json(open(manifest_path(prefix)).read())
        except Exception as e:           # noqa: BLE001 - an unreadable manifest is the finding
            r.add("manifest", f"manifest cannot be parsed: {e}")
            return r
        r.extend(VersionCompatibilityChecker().check(meta))
        r.extend(SchemaCompatibilityChecker().check(meta))
        r.extend(SizeIntegrityChecker().check(prefix, meta))
        if not self.quick and r.is_valid:
            r.extend(ChecksumIntegrityChecker().check(prefix, meta))
        return r


# ------------------------------------------------------------------ typed state
class StateDict(dict):
    """Name -> tensor with a few conveniences; ``kind`` is ``"model"`` or ``"optimizer"``."""
    kind = "state"

    def total_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.values() if isinstance(v, torch.Tensor))

    def fingerprint(self) -> str:
        """A digest of names, dtypes and shapes (not values): equal for states that can be loaded into each other."""
        h = hashlib.sha256()
        for k in sorted(self):
            v = self[k]
            if isinstance(v, torch.Tensor):
                h.update(f"{k}|{v.dtype}|{tuple(v.shape)};".encode())
        return h.hexdigest()[:16]

    def with_prefix(self, prefix: str) -> "StateDict":
        return type(self)({prefix + k: v for k, v in self.items()})

    def strip_prefix(self, prefix: str) -> "StateDict":
        return type(self)({k[len(prefix):]: v for k, v in self.items() if k.startswith(prefix)})


class ModelStateDict(StateDict):
    kind = "model"

    @classmethod
    def from_module(cls, m: torch.nn.Module) -> "ModelStateDict":
        return cls(m.state_dict())


class OptimizerStateDict(StateDict):
    """Flat view of an optimizer's tensors: ``state.<param index>.<key>``; scalars and hyper-parameters in ``extras``."""
    kind = "optimizer"

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.extras: Dict[str, object] = {}

    @classmethod
    def from_optimizer(cls, opt) -> "OptimizerStateDict":
        sd = opt.state_dict()
        out = cls()
        for pid, st in sd.get("state", {}).items():
            for key, v in st.items():
                if isinstance(v, torch.Tensor):
                    out[f"state.{pid}.{key}"] = v
                else:
                    out.extras[f"state.{pid}.{key}"] = v
        out.extras["param_groups"] = sd.get("param_groups", [])
        return out

    def to_optimizer_state(self) -> Dict[str, object]:
        state: Dict[int, Dict[str, object]] = {}
        for k, v in list(self.items()) + [(k, v) for k, v in self.extras.items() if k.startswith("state.")]:
            _, pid, key = k.split(".", 2)
            state.setdefault(int(pid), {})[key] = v
        return {"state": state, "param_groups": self.extras.get("param_groups", [])}


@dataclass
class StateCompatibility:
    missing: List[str] = field(default_factory=list)          # expected by the target, absent in the checkpoint
    unexpected: List[str] = field(default_factory=list)
    shape_mismatches: List[Tuple[str, tuple, tuple]] = field(default_factory=list)
    dtype_mismatches: List[Tuple[str, str, str]] = field(default_factory=list)

    def is_compatible(self, strict: bool = True) -> bool:
        if self.shape_mismatches:
            return False
        return not (strict and (self.missing or self.unexpected))

    def describe(self) -> str:
        parts = []
        if self.missing: parts.append(f"missing: {self.missing}")
        if self.unexpected: parts.append(f"unexpected: {self.unexpected}")
        parts += [f"{n}: checkpoint {a}, target {b}" for n, a, b in self.shape_mismatches]
        parts += [f"{n}: dtype {a} -> {b} (cast on load)" for n, a, b in self.dtype_mismatches]
        return "; ".join(parts) or "compatible"


class StateCompatibilityChecker:
    def check(self, checkpoint: Dict[str, torch.Tensor], target: Dict[str, torch.Tensor]) -> StateCompatibility:
        c = StateCompatibility()
        c.missing = sorted(k for k in target if k not in checkpoint)
        c.unexpected = sorted(k for k in checkpoint if k not in target)
        for k in sorted(set(checkpoint) & set(target)):
            a, b = checkpoint[k], target[k]
            if tuple(a.shape) != tuple(b.shape):
                c.shape_mismatches.append((k, tuple(a.shape), tuple(b.shape)))
            elif a.dtype != b.dtype:
                c.dtype_mismatches.append((k, str(a.dtype), str(b.dtype)))
        return c

    def load_checked(self, module: torch.nn.Module, checkpoint: Dict[str, torch.Tensor], strict: bool = True) -> StateCompatibility:
        c = self.check(checkpoint, module.state_dict())
        if not c.is_compatible(strict):
            raise CheckpointError("state does not fit the model: " + c.describe())
        own = module.state_dict()
        with torch.no_grad():
            for k, v in checkpoint.items():
                if k in own:
                    own[k].copy_(v.to(own[k].dtype))
        return c


# ------------------------------------------------------------------ per-strategy collection
def _slice_entry(global_shape: Sequence[int], dim: int, index: int, count: int) -> dict:
    return {"GlobalShape": list(global_shape), "ShardDim": dim, "ShardIndex": index, "ShardCount": count}


class DDPCheckpointHelper:
    """Replicated state: rank 0 writes everything, the others write nothing (their shard files are empty)."""

    @staticmethod
    def collect_full_state(state: Dict[str, torch.Tensor], rank: int) -> Tuple[Dict[str, torch.Tensor], Dict[str, dict]]:
        return (dict(state) if rank == 0 else {}), {}


class FSDPCheckpointHelper:
    """Flat shards: every rank writes its piece of each flattened parameter with the slice description a loader at
    another world size needs."""

    @staticmethod
    def collect_local_shard(local: Dict[str, torch.Tensor], global_numel: Dict[str, int], rank: int, world: int):
        info = {k: _slice_entry([global_numel[k]], 0, rank, world) for k in local}
        return dict(local), info

    @staticmethod
    def load_local_shard(tensors: Dict[str, torch.Tensor], targets: Dict[str, torch.Tensor]) -> List[str]:
        """Copies loaded flat pieces into the rank's shard buffers (shorter pieces fill a prefix: the padded tail of a
        last shard stays as it is); returns the names that had no counterpart."""
        missing = []
        with torch.no_grad():
            for k, dst in targets.items():
                src = tensors.get(k)
                if src is None:
                    missing.append(k)
                    continue
                n = min(src.numel(), dst.numel())
                dst.reshape(-1)[:n].copy_(src.reshape(-1)[:n].to(dst.dtype))
        return missing


class TensorParallelCheckpointHelper:
    @staticmethod
    def collect_tp_shard(local: Dict[str, torch.Tensor], shard_dims: Dict[str, Optional[int]], rank: int, world: int):
        """``shard_dims[name]`` is the dimension a tensor is cut along (``None`` = replicated; written by rank 0 only)."""
        tensors, info = {}, {}
        for k, v in local.items():
            d = shard_dims.get(k)
            if d is None:
                if rank == 0:
                    tensors[k] = v
                continue
            g = list(v.shape)
            g[d] *= world
            tensors[k] = v
            info[k] = _slice_entry(g, d, rank, world)
        return tensors, info


class DistributedStateCollector:
    """One entry point for the three layouts; returns what ``CheckpointCoordinator.coordinate_save`` takes."""

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world

    def collect(self, strategy: str, state: Dict[str, torch.Tensor], **kw):
        if strategy == "ddp":
            return DDPCheckpointHelper.collect_full_state(state, self.rank)
        if strategy == "fsdp":
            return FSDPCheckpointHelper.collect_local_shard(state, kw["global_numel"], self.rank, self.world)
        if strategy == "tp":
            return TensorParallelCheckpointHelper.collect_tp_shard(state, kw["shard_dims"], self.rank, self.world)
        raise KeyError(f"unknown strategy {strategy!r}")


# ------------------------------------------------------------------ resharding strategies by name
class ParallelReshardingStrategy:
    """Every target rank reads only the byte ranges of the source shards that overlap its own slice."""
    name = "parallel"

    def load(self, meta: CheckpointMetadata, prefix: str, target_world: int, target_rank: int, device="cpu", verify: bool = True):
        plan = ReshardingStrategy.create_plan(meta, target_world, target_rank)
        return ReshardingStrategy.execute(plan, meta, prefix, device, verify)


class SimpleReshardingStrategy:
    """Reads ALL source shards, rebuilds every full tensor and cuts the target rank's slice out of it. Needs memory
    for the whole checkpoint on every rank; the reference's default for small models and the oracle for the parallel
    strategy in tests."""
    name = "simple"

    def load(self, meta: CheckpointMetadata, prefix: str, target_world: int, target_rank: int, device="cpu", verify: bool = True):
        parts: Dict[str, List] = {}
        for s in meta.Shards:
            data = MultiShardCheckpointFormat.read_shard(_shard_file(prefix, s), s, verify)
            for t in s.Tensors:
                parts.setdefault(t.Name, []).append((t, data[t.Name]))
        out = {}
        for name, lst in parts.items():
            t0 = lst[0][0]
            if t0.ShardDim is None or t0.GlobalShape is None:
                out[name] = lst[0][1].to(device)
                continue
            full = torch.cat([x for _, x in sorted(lst, key=lambda e: e[0].ShardIndex)], dim=t0.ShardDim)
            G = t0.GlobalShape[t0.ShardDim]
            full = full.narrow(t0.ShardDim, 0, min(G, full.shape[t0.ShardDim]))
            per = (G + target_world - 1) // target_world
            lo, hi = min(target_rank * per, G), min((target_rank + 1) * per, G)
            out[name] = full.narrow(t0.ShardDim, lo, hi - lo).contiguous().to(device)
        return out


def resharding_strategy(name: str):
    if name == "parallel":
        return ParallelReshardingStrategy()
    if name == "simple":
        return SimpleReshardingStrategy()
    raise KeyError(f"unknown resharding strategy {name!r}")


# ------------------------------------------------------------------ factory
@dataclass
class CheckpointOptions:
    directory: str = "./checkpoints"
    format: CheckpointFormat = CheckpointFormat.MULTI_SHARD
    compression: CheckpointCompressionLevel = CheckpointCompressionLevel.NONE
    max_to_keep: int = 5
    validate_after_save: bool = False
    resharding_strategy: str = "parallel"

    def save_options(self, **kw) -> SaveOptions:
        return SaveOptions(format=self.format.value, compression=self.compression.value, **kw)

    def load_options(self, **kw) -> LoadOptions:
        return LoadOptions(resharding_strategy=self.resharding_strategy, **kw)


class DistributedCheckpointFactory:
    @staticmethod
    def create(options: Optional[CheckpointOptions] = None, pg=None) -> DistributedCheckpoint:
        o = options or CheckpointOptions()
        if o.max_to_keep < 0:
            raise ValueError("max_to_keep must be non-negative")
        resharding_strategy(o.resharding_strategy)
        return DistributedCheckpoint(o.directory, pg, o.max_to_keep)

    @staticmethod
    def create_validated(options: Optional[CheckpointOptions] = None, pg=None):
        """A checkpoint object whose ``save`` validates what it wrote (rank 0) and raises when the result is unreadable."""
        ck = DistributedCheckpointFactory.create(options, pg)
        inner = ck.save

        def save(tag, *a, **k):
            meta = inner(tag, *a, **k)
            if ck.coord.rank == 0 and meta.Format == "multishard":
                rep = CheckpointValidator().validate(ck._prefix(tag))
                if not rep.is_valid:
                    raise CheckpointError("checkpoint failed validation after save: " + "; ".join(rep.errors()))
            return meta
        ck.save = save
        return ck
