"""Distributed checkpointing: multi-shard and single-file formats, save coordination, resharding on
load, async / incremental saving, validation and fault tolerance.

On-disk layout (field names as in the reference's manifest,
src/MLFramework/Checkpointing/Metadata/CheckpointMetadata.cs:6-127, Integration/ShardData.cs:6-78):

    {prefix}_shard_{rank}.shard     binary, written by the native layer (csrc/ckpt/shard_io.cpp)
    {prefix}.metadata.json          {Version, Timestamp, WorldSize, DdpRank, Sharding{Strategy,
                                     ShardCount, Precision, StrategySpecificInfo}, Shards[{Rank,
                                     FilePath, FileSize, Tensors[{Name, Shape, DataType, Offset, Size,
                                     + GlobalShape, ShardDim, ShardIndex, ShardCount}], Checksum}],
                                     Training{Epoch, Step, LearningRate, OptimizerType}, CustomFields,
                                     Format}

Save flow = ``CheckpointCoordinator.CoordinateSaveAsync`` (Coordinator/CheckpointCoordinator.cs:27-104):
barrier, every rank writes its own shard (no gather to rank 0) with a SHA-256 of the payload,
shard descriptions are gathered, rank 0 writes the manifest atomically, barrier. Load verifies
magic / rank / checksum / tensor count and, when the world size changed, re-slices tensors that
were sharded along a dimension (Resharding/ReshardingStrategy.cs:63-496).
"""
from __future__ import annotations

import ctypes as C
import enum
import gzip
import hashlib
import io
import json
import os
import queue
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib

FORMAT_VERSION = "1.0.0"
SHARD_EXT = ".shard"
MAGIC = 0x53484152

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "int64": torch.int64,
           "int32": torch.int32, "uint8": torch.uint8, "float64": torch.float64, "bool": torch.bool, "int8": torch.int8}
_DT_NAMES = {v: k for k, v in _DTYPES.items()}


class CheckpointError(RuntimeError):
    pass


class CheckpointCorruptError(CheckpointError):
    pass


# ------------------------------------------------------------------ metadata
@dataclass
class TensorMetadata:
    Name: str
    Shape: List[int]
    DataType: str
    Offset: int
    Size: int
    GlobalShape: Optional[List[int]] = None   # full tensor shape when this entry is one slice of it
    ShardDim: Optional[int] = None
    ShardIndex: int = 0
    ShardCount: int = 1


@dataclass
class ShardMetadata:
    Rank: int
    FilePath: str
    FileSize: int
    Tensors: List[TensorMetadata]
    Checksum: str


@dataclass
class ShardingMetadata:
    Strategy: str = "ddp"
    ShardCount: int = 1
    Precision: str = "fp32"
    StrategySpecificInfo: Dict[str, str] = field(default_factory=dict)


@dataclass
class TrainingMetadata:
    Epoch: int = 0
    Step: int = 0
    LearningRate: float = 0.0
    OptimizerType: str = ""
    OptimizerState: Dict = field(default_factory=dict)


@dataclass
class CheckpointMetadata:
    Version: str = FORMAT_VERSION
    Timestamp: float = 0.0
    WorldSize: int = 1
    DdpRank: int = 0
    Sharding: ShardingMetadata = field(default_factory=ShardingMetadata)
    Shards: List[ShardMetadata] = field(default_factory=list)
    Training: TrainingMetadata = field(default_factory=TrainingMetadata)
    CustomFields: Dict[str, str] = field(default_factory=dict)
    Format: str = "multishard"

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_json(cls, text: str) -> "CheckpointMetadata":
        d = json.loads(text)
        shards = [ShardMetadata(Rank=s["Rank"], FilePath=s["FilePath"], FileSize=s["FileSize"], Checksum=s["Checksum"],
                                Tensors=[TensorMetadata(**t) for t in s["Tensors"]]) for s in d.get("Shards", [])]
        return cls(Version=d.get("Version", FORMAT_VERSION), Timestamp=d.get("Timestamp", 0.0), WorldSize=d["WorldSize"],
                   DdpRank=d.get("DdpRank", 0), Sharding=ShardingMetadata(**d.get("Sharding", {})), Shards=shards,
                   Training=TrainingMetadata(**d.get("Training", {})), CustomFields=d.get("CustomFields", {}),
                   Format=d.get("Format", "multishard"))


class MetadataValidator:
    @staticmethod
    def validate(meta: CheckpointMetadata) -> List[str]:
        errs = []
        if meta.WorldSize <= 0:
            errs.append("WorldSize must be positive")
        if meta.Format == "multishard" and len(meta.Shards) != meta.WorldSize:
            errs.append(f"expected {meta.WorldSize} shards, manifest lists {len(meta.Shards)}")
        if sorted(s.Rank for s in meta.Shards) != list(range(len(meta.Shards))):
            errs.append("shard ranks are not 0..W-1")
        major = meta.Version.split(".")[0]
        if major != FORMAT_VERSION.split(".")[0]:
            errs.append(f"incompatible format version {meta.Version}")
        for s in meta.Shards:
            end = 0
            for t in s.Tensors:
                if t.Offset < end:
                    errs.append(f"tensor {t.Name} overlaps its predecessor in shard {s.Rank}")
                end = t.Offset + t.Size
        return errs


# ------------------------------------------------------------------ storage
class LocalFileSystemStorage:
    """``ICheckpointStorage`` over a directory (Checkpointing/Storage/LocalFileSystemStorage.cs)."""

    def __init__(self, root: str = "."):
        self.root = root

    def path(self, key: str) -> str:
        return key if os.path.isabs(key) else os.path.join(self.root, key)

    def write(self, key: str, data: bytes):
        p = self.path(key)
        os.makedirs(os.path.dirname(os.path.abspath(p)), exist_ok=True)
        tmp = p + ".tmp"
        with open(tmp, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, p)

    def read(self, key: str) -> bytes:
        with open(self.path(key), "rb") as f:
            return f.read()

    def exists(self, key: str) -> bool:
        return os.path.exists(self.path(key))

    def delete(self, key: str):
        try:
            os.remove(self.path(key))
        except FileNotFoundError:
            pass

    def get_metadata(self, key: str) -> Dict:
        st = os.stat(self.path(key))
        return {"size": st.st_size, "mtime": st.st_mtime}

    def list(self, prefix: str = "") -> List[str]:
        d = self.root
        return sorted(f for f in os.listdir(d) if f.startswith(prefix)) if os.path.isdir(d) else []


class StorageFactory:
    @staticmethod
    def create(kind: str = "local", **kw):
        if kind != "local":
            raise ValueError(f"unknown storage backend {kind!r}")
        return LocalFileSystemStorage(**kw)


# ------------------------------------------------------------------ shard format
def _hex() -> C.Array:
    return (C.c_char * 65)()


def shard_path(prefix: str, rank: int) -> str:
    return f"{prefix}_shard_{rank}{SHARD_EXT}"


def manifest_path(prefix: str) -> str:
    return f"{prefix}.metadata.json"


class MultiShardCheckpointFormat:
    extension = SHARD_EXT
    magic = MAGIC

    @staticmethod
    def write_shard(path: str, rank: int, tensors: Dict[str, torch.Tensor],
                    slice_info: Optional[Dict[str, dict]] = None) -> ShardMetadata:
        """Writes ``tensors`` (any device) as one shard file; returns its manifest entry."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        metas, hosts, off = [], [], 0
        for name, t in tensors.items():
            h = t.detach().contiguous().cpu()
            nbytes = h.numel() * h.element_size()
            info = (slice_info or {}).get(name, {})
            metas.append(TensorMetadata(Name=name, Shape=list(h.shape), DataType=_DT_NAMES[h.dtype], Offset=off, Size=nbytes,
                                        GlobalShape=info.get("GlobalShape"), ShardDim=info.get("ShardDim"),
                                        ShardIndex=info.get("ShardIndex", 0), ShardCount=info.get("ShardCount", 1)))
            hosts.append(h)
            off += nbytes
        n = len(hosts)
        ptrs = (C.c_void_p * max(n, 1))(*[C.c_void_p(h.data_ptr()) for h in hosts])
        sizes = (C.c_longlong * max(n, 1))(*[m.Size for m in metas])
        cs, fsize = _hex(), C.c_longlong()
        rc = _lib.get().mlf_ckpt_write_shard(path.encode(), rank, n, ptrs, sizes, n, cs, C.byref(fsize))
        _lib.check(rc, "mlf_ckpt_write_shard")
        return ShardMetadata(Rank=rank, FilePath=os.path.basename(path), FileSize=fsize.value, Tensors=metas,
                             Checksum=cs.value.decode())

    @staticmethod
    def read_header(path: str, expected_rank: int = -1):
        rank, tc, dl, do = C.c_int(), C.c_int(), C.c_longlong(), C.c_longlong()
        cs = _hex()
        rc = _lib.get().mlf_ckpt_read_header(path.encode(), expected_rank, C.byref(rank), cs, C.byref(tc), C.byref(dl), C.byref(do))
        if rc in (-10, -11, -12):
            raise CheckpointCorruptError(_lib.get().mlf_last_error().decode())
        _lib.check(rc, "mlf_ckpt_read_header")
        return rank.value, cs.value.decode(), tc.value, dl.value, do.value

    @staticmethod
    def read_shard(path: str, meta: ShardMetadata, verify: bool = True, names: Optional[Sequence[str]] = None,
                   device="cpu") -> Dict[str, torch.Tensor]:
        rank, cs, tc, dl, do = MultiShardCheckpointFormat.read_header(path, meta.Rank)
        if meta.Checksum and cs != meta.Checksum:
            raise CheckpointCorruptError(f"shard checksum mismatch for rank {meta.Rank}")
        if tc != len(meta.Tensors):
            raise CheckpointCorruptError(f"tensor count mismatch for shard {meta.Rank}: expected {len(meta.Tensors)}, found {tc}")
        if verify:
            h = _hex()
            _lib.check(_lib.get().mlf_ckpt_payload_sha256(path.encode(), C.c_longlong(do), C.c_longlong(dl), h), "payload sha256")
            if h.value.decode() != cs:
                raise CheckpointCorruptError(f"payload of shard {meta.Rank} does not match its checksum")
        out = {}
        for t in meta.Tensors:
            if names is not None and t.Name not in names:
                continue
            dt = _DTYPES[t.DataType]
            host = torch.empty(t.Shape, dtype=dt)
            if t.Size:
                rc = _lib.get().mlf_ckpt_read_data(path.encode(), C.c_longlong(do), C.c_longlong(t.Offset), C.c_longlong(t.Size),
                                                   C.c_void_p(host.data_ptr()))
                _lib.check(rc, "mlf_ckpt_read_data")
            out[t.Name] = host.to(device) if str(device) != "cpu" else host
        return out


class SingleFileCheckpointFormat:
    """Everything in one file: JSON header length, JSON header, raw tensors (Formats/SingleFileCheckpointFormat.cs)."""

    @staticmethod
    def save(path: str, tensors: Dict[str, torch.Tensor], extra: Optional[Dict] = None):
        metas, blobs, off = [], [], 0
        for n, t in tensors.items():
            h = t.detach().contiguous().cpu()
            b = h.view(torch.uint8).numpy().tobytes() if h.numel() else b""
            metas.append({"Name": n, "Shape": list(h.shape), "DataType": _DT_NAMES[h.dtype], "Offset": off, "Size": len(b)})
            blobs.append(b)
            off += len(b)
        header = json.dumps({"Format": "singlefile", "Version": FORMAT_VERSION, "Tensors": metas, "Extra": extra or {}}).encode()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(len(header).to_bytes(8, "little"))
            f.write(header)
            for b in blobs:
                f.write(b)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)

    @staticmethod
    def load(path: str, device="cpu"):
        with open(path, "rb") as f:
            n = int.from_bytes(f.read(8), "little")
            try:
                header = json.loads(f.read(n))
            except Exception as e:  # noqa: BLE001
                raise CheckpointCorruptError(f"unreadable header in {path}") from e
            base = 8 + n
            out = {}
            for m in header["Tensors"]:
                f.seek(base + m["Offset"])
                raw = bytearray(f.read(m["Size"]))
                if len(raw) != m["Size"]:
                    raise CheckpointCorruptError(f"truncated tensor {m['Name']} in {path}")
                t = torch.frombuffer(raw, dtype=_DTYPES[m["DataType"]]).reshape(m["Shape"]) if m["Size"] else torch.empty(m["Shape"], dtype=_DTYPES[m["DataType"]])
                out[m["Name"]] = t.to(device)
        return out, header.get("Extra", {})


# ------------------------------------------------------------------ coordination
class _SoloCoordinator:
    rank, world_size = 0, 1

    def barrier(self): ...
    def all_gather_object(self, o): return [o]
    def broadcast_object(self, o, src=0): return o


@dataclass
class SaveOptions:
    format: str = "multishard"
    compression: str = "none"
    include_optimizer: bool = True
    include_rng_state: bool = True
    timeout_s: float = 600.0
    custom_metadata: Dict[str, str] = field(default_factory=dict)


@dataclass
class LoadOptions:
    load_optimizer: bool = True
    load_rng_state: bool = True
    resharding_strategy: str = "parallel"
    skip_validation: bool = False
    strict: bool = True


@dataclass
class CheckpointLoadResult:
    tensors: Dict[str, torch.Tensor]
    metadata: CheckpointMetadata
    was_resharded: bool
    source_world_size: int
    target_world_size: int


class CheckpointCoordinator:
    def __init__(self, pg=None):
        self.pg = pg if pg is not None else _SoloCoordinator()

    @property
    def rank(self):
        return self.pg.rank

    @property
    def world_size(self):
        return self.pg.world_size

    def coordinate_save(self, prefix: str, local_tensors: Dict[str, torch.Tensor], slice_info: Optional[Dict[str, dict]] = None,
                        sharding: Optional[ShardingMetadata] = None, training: Optional[TrainingMetadata] = None,
                        custom: Optional[Dict[str, str]] = None) -> CheckpointMetadata:
        self.pg.barrier()
        sm = MultiShardCheckpointFormat.write_shard(shard_path(prefix, self.rank), self.rank, local_tensors, slice_info)
        all_sm = self.pg.all_gather_object(asdict(sm))
        meta = CheckpointMetadata(Timestamp=time.time(), WorldSize=self.world_size, DdpRank=self.rank,
                                  Sharding=sharding or ShardingMetadata(ShardCount=self.world_size),
                                  Shards=[ShardMetadata(Rank=s["Rank"], FilePath=s["FilePath"], FileSize=s["FileSize"],
                                                        Checksum=s["Checksum"], Tensors=[TensorMetadata(**t) for t in s["Tensors"]])
                                          for s in sorted(all_sm, key=lambda s: s["Rank"])],
                                  Training=training or TrainingMetadata(), CustomFields=custom or {})
        if self.rank == 0:
            LocalFileSystemStorage().write(manifest_path(prefix), meta.to_json().encode())
        self.pg.barrier()
        return meta


# ------------------------------------------------------------------ resharding
@dataclass
class TensorSlice:
    source_rank: int
    name: str
    src_start: int
    src_end: int
    dst_start: int


@dataclass
class ReshardingPlan:
    source_world: int
    target_world: int
    target_rank: int
    # tensor name -> (global shape, shard dim, target [lo, hi), slices to read)
    tensors: Dict[str, Tuple[List[int], Optional[int], Tuple[int, int], List[TensorSlice]]] = field(default_factory=dict)


class ReshardingStrategy:
    """Plans which pieces of which source shards a target rank must read so that a tensor cut
    into ``source_world`` equal slices along one dimension comes out cut into ``target_world``."""

    @staticmethod
    def create_plan(meta: CheckpointMetadata, target_world: int, target_rank: int) -> ReshardingPlan:
        plan = ReshardingPlan(meta.WorldSize, target_world, target_rank)
        by_name: Dict[str, List[Tuple[int, TensorMetadata]]] = {}
        for s in meta.Shards:
            for t in s.Tensors:
                by_name.setdefault(t.Name, []).append((s.Rank, t))
        for name, entries in by_name.items():
            t0 = entries[0][1]
            if t0.ShardDim is None or t0.GlobalShape is None:
                # replicated: read it from the first shard that has it
                plan.tensors[name] = (t0.Shape, None, (0, 0), [TensorSlice(entries[0][0], name, 0, 0, 0)])
                continue
            dim, gshape = t0.ShardDim, t0.GlobalShape
            G = gshape[dim]
            per_t = (G + target_world - 1) // target_world
            lo, hi = min(target_rank * per_t, G), min((target_rank + 1) * per_t, G)
            slices, pos = [], 0
            for rank, tm in sorted(entries, key=lambda e: e[1].ShardIndex):
                n = tm.Shape[dim]
                a, b = max(lo, pos), min(hi, pos + n)
                if a < b:
                    slices.append(TensorSlice(rank, name, a - pos, b - pos, a - lo))
                pos += n
            plan.tensors[name] = (gshape, dim, (lo, hi), slices)
        return plan

    @staticmethod
    def execute(plan: ReshardingPlan, meta: CheckpointMetadata, prefix: str, device="cpu", verify=True) -> Dict[str, torch.Tensor]:
        cache: Dict[int, Dict[str, torch.Tensor]] = {}
        shard_meta = {s.Rank: s for s in meta.Shards}

        def shard(rank):
            if rank not in cache:
                cache[rank] = MultiShardCheckpointFormat.read_shard(
                    os.path.join(os.path.dirname(prefix) or ".", shard_meta[rank].FilePath), shard_meta[rank], verify)
            return cache[rank]
        out = {}
        for name, (gshape, dim, (lo, hi), slices) in plan.tensors.items():
            if dim is None:
                out[name] = shard(slices[0].source_rank)[name].to(device)
                continue
            shape = list(gshape)
            shape[dim] = hi - lo
            first = shard(slices[0].source_rank)[name] if slices else None
            dst = torch.zeros(shape, dtype=first.dtype if first is not None else torch.float32)
            for sl in slices:
                src = shard(sl.source_rank)[name]
                n = sl.src_end - sl.src_start
                dst.narrow(dim, sl.dst_start, n).copy_(src.narrow(dim, sl.src_start, n))
            out[name] = dst.to(device)
        return out


class CheckpointLoader:
    def __init__(self, pg=None):
        self.pg = pg if pg is not None else _SoloCoordinator()

    def load_metadata(self, prefix: str) -> CheckpointMetadata:
        p = manifest_path(prefix)
        if not os.path.exists(p):
            raise CheckpointError(f"no manifest at {p}")
        meta = CheckpointMetadata.from_json(open(p).read())
        errs = MetadataValidator.validate(meta)
        if errs:
            raise CheckpointCorruptError("; ".join(errs))
        return meta

    def coordinate_load(self, prefix: str, options: Optional[LoadOptions] = None, device="cpu") -> CheckpointLoadResult:
        opt = options or LoadOptions()
        meta = self.load_metadata(prefix)
        W, r = self.pg.world_size, self.pg.rank
        verify = not opt.skip_validation
        if meta.WorldSize == W:
            sm = next(s for s in meta.Shards if s.Rank == r)
            tensors = MultiShardCheckpointFormat.read_shard(os.path.join(os.path.dirname(prefix) or ".", sm.FilePath), sm, verify,
                                                            device=device)
            return CheckpointLoadResult(tensors, meta, False, meta.WorldSize, W)
        if opt.resharding_strategy == "simple":
            from .validation import SimpleReshardingStrategy       # reads every shard; the parallel plan reads overlaps only
            tensors = SimpleReshardingStrategy().load(meta, prefix, W, r, device, verify)
        else:
            plan = ReshardingStrategy.create_plan(meta, W, r)
            tensors = ReshardingStrategy.execute(plan, meta, prefix, device, verify)
        return CheckpointLoadResult(tensors, meta, True, meta.WorldSize, W)


class ShardFileVerifier:
    @staticmethod
    def verify_checkpoint(prefix: str) -> Tuple[bool, List[str]]:
        errs = []
        try:
            meta = CheckpointLoader().load_metadata(prefix)
        except CheckpointError as e:
            return False, [str(e)]
        for s in meta.Shards:
            p = os.path.join(os.path.dirname(prefix) or ".", s.FilePath)
            if not os.path.exists(p):
                errs.append(f"missing shard file {s.FilePath}")
                continue
            if os.path.getsize(p) != s.FileSize:
                errs.append(f"size mismatch for {s.FilePath}")
            try:
                MultiShardCheckpointFormat.read_shard(p, s, verify=True, names=[])
            except CheckpointError as e:
                errs.append(str(e))
        return not errs, errs


# ------------------------------------------------------------------ high-level API
class DistributedCheckpoint:
    """Save / load / list / delete (Checkpointing/Integration/DistributedCheckpoint.cs:93-270)."""

    def __init__(self, directory: str, pg=None, max_to_keep: int = 5):
        self.dir, self.pg = directory, pg
        self.coord = CheckpointCoordinator(pg)
        self.loader = CheckpointLoader(pg)
        self.max_to_keep = max_to_keep

    def _prefix(self, tag: str) -> str:
        return os.path.join(self.dir, tag)

    def save(self, tag: str, model_state: Dict[str, torch.Tensor], optimizer_state: Optional[Dict[str, torch.Tensor]] = None,
             slice_info: Optional[Dict[str, dict]] = None, options: Optional[SaveOptions] = None, step: int = 0, epoch: int = 0,
             lr: float = 0.0, strategy: str = "ddp", rng_state: Optional[Dict[str, torch.Tensor]] = None) -> CheckpointMetadata:
        opt = options or SaveOptions()
        tensors = {f"model.{k}": v for k, v in model_state.items()}
        info = {f"model.{k}": v for k, v in (slice_info or {}).items()}
        if opt.include_optimizer and optimizer_state:
            tensors.update({f"optim.{k}": v for k, v in optimizer_state.items() if isinstance(v, torch.Tensor)})
        if opt.include_rng_state and rng_state:
            tensors.update({f"rng.{k}": v for k, v in rng_state.items()})
        world = self.coord.world_size
        if opt.format == "singlefile":
            if self.coord.rank == 0:
                SingleFileCheckpointFormat.save(self._prefix(tag) + ".ckpt", tensors, {"step": step, "epoch": epoch})
            self.coord.pg.barrier()
            return CheckpointMetadata(WorldSize=world, Format="singlefile", Training=TrainingMetadata(epoch, step, lr))
        meta = self.coord.coordinate_save(self._prefix(tag), tensors, info,
                                          ShardingMetadata(Strategy=strategy, ShardCount=world, Precision="mixed"),
                                          TrainingMetadata(Epoch=epoch, Step=step, LearningRate=lr), opt.custom_metadata)
        if self.coord.rank == 0 and self.max_to_keep > 0:
            for old in self.list_checkpoints()[:-self.max_to_keep]:
                self.delete(old)
        return meta

    def save_model_only(self, tag: str, model_state, **kw):
        return self.save(tag, model_state, None, options=SaveOptions(include_optimizer=False, include_rng_state=False), **kw)

    def load(self, tag: str, options: Optional[LoadOptions] = None, device="cpu") -> CheckpointLoadResult:
        single = self._prefix(tag) + ".ckpt"
        if os.path.exists(single) and not os.path.exists(manifest_path(self._prefix(tag))):
            tensors, extra = SingleFileCheckpointFormat.load(single, device)
            return CheckpointLoadResult(tensors, CheckpointMetadata(Format="singlefile"), False, 1, self.coord.world_size)
        res = self.loader.coordinate_load(self._prefix(tag), options, device)
        opt = options or LoadOptions()
        if not opt.load_optimizer:
            res.tensors = {k: v for k, v in res.tensors.items() if not k.startswith("optim.")}
        if not opt.load_rng_state:
            res.tensors = {k: v for k, v in res.tensors.items() if not k.startswith("rng.")}
        return res

    def list_checkpoints(self) -> List[str]:
        if not os.path.isdir(self.dir):
            return []
        tags = [f[:-len(".metadata.json")] for f in os.listdir(self.dir) if f.endswith(".metadata.json")]
        return sorted(tags, key=lambda t: os.path.getmtime(manifest_path(self._prefix(t))))

    def delete(self, tag: str):
        p = self._prefix(tag)
        base = os.path.basename(p)
        for f in os.listdir(self.dir):
            if f == os.path.basename(manifest_path(p)) or f == base + ".ckpt" or (f.startswith(base + "_shard_") and f.endswith(SHARD_EXT)):
                os.remove(os.path.join(self.dir, f))


# ------------------------------------------------------------------ async / incremental / fault tolerance
class CheckpointTaskType(enum.Enum):
    FULL = "full"                   # model and optimizer
    MODEL_ONLY = "model_only"


class CheckpointTaskStatus(enum.Enum):
    QUEUED = "queued"
    RUNNING = "running"
    COMPLETED = "completed"
    FAILED = "failed"
    CANCELLED = "cancelled"


class CheckpointQueueFullError(CheckpointError):
    def __init__(self, max_queue_size: int):
        super().__init__(f"the checkpoint queue is full ({max_queue_size} pending saves)")
        self.max_queue_size = max_queue_size


@dataclass
class CheckpointTaskResult:
    checkpoint_id: str
    success: bool
    value: object = None            # what ``DistributedCheckpoint.save`` returned
    error: Optional[BaseException] = None
    duration_s: float = 0.0
    bytes_snapshotted: int = 0


@dataclass
class CheckpointTaskInfo:
    """A task as the outside sees it (no tensors)."""
    id: str
    type: CheckpointTaskType
    status: CheckpointTaskStatus
    queued_at: float
    started_at: Optional[float]
    completed_at: Optional[float]

    @property
    def duration_s(self) -> Optional[float]:
        return None if self.started_at is None or self.completed_at is None else self.completed_at - self.started_at


@dataclass
class CheckpointTask:
    id: str
    type: CheckpointTaskType
    model_state: Dict[str, torch.Tensor]
    optimizer_state: Dict[str, torch.Tensor]
    options: Dict[str, object]
    queued_at: float
    started_at: Optional[float] = None
    completed_at: Optional[float] = None
    status: CheckpointTaskStatus = CheckpointTaskStatus.QUEUED
    result: Optional[CheckpointTaskResult] = None
    done: threading.Event = field(default_factory=threading.Event)

    def info(self) -> CheckpointTaskInfo:
        return CheckpointTaskInfo(self.id, self.type, self.status, self.queued_at, self.started_at, self.completed_at)


class AsyncCheckpointManager:
    """Background save queue: tensors are snapshotted to host memory on the caller's thread (the
    only part on the training step's critical path), files are written by a worker thread. Every save is
    a tracked task: queued, running, then completed, failed or cancelled
    (Checkpointing/Async/AsyncCheckpointManager.cs:9-421, CheckpointTask.cs, CheckpointTaskInfo.cs,
    CheckpointTaskResult.cs)."""

    def __init__(self, checkpoint: DistributedCheckpoint, max_pending: int = 2, keep_finished: int = 64):
        self.ckpt = checkpoint
        self.max_queue_size = max_pending
        self._q: "queue.Queue" = queue.Queue(maxsize=max_pending)
        self._results: Dict[str, object] = {}
        self._tasks: Dict[str, CheckpointTask] = {}
        self._keep = keep_finished
        self._cancelled = set()
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._worker, daemon=True)
        self._thread.start()

    @property
    def queue_size(self) -> int:
        return self._q.qsize()

    @property
    def active_task_count(self) -> int:
        with self._lock:
            return sum(t.status in (CheckpointTaskStatus.QUEUED, CheckpointTaskStatus.RUNNING) for t in self._tasks.values())

    def queue_save(self, tag: str, model_state: Dict[str, torch.Tensor], optimizer_state=None, block: bool = True, **kw) -> str:
        """Snapshots the tensors and queues the write. With ``block=False`` a full queue raises
        ``CheckpointQueueFullError`` instead of waiting for room."""
        with self._lock:
            live = self._tasks.get(tag)
            if live is not None and live.status in (CheckpointTaskStatus.QUEUED, CheckpointTaskStatus.RUNNING):
                raise CheckpointError(f"a save named {tag!r} is still in flight")
        if not block and self._q.full():
            raise CheckpointQueueFullError(self.max_queue_size)
        snap = {k: v.detach().to("cpu", copy=True) for k, v in model_state.items()}
        osnap = {k: v.detach().to("cpu", copy=True) for k, v in (optimizer_state or {}).items() if isinstance(v, torch.Tensor)}
        task = CheckpointTask(tag, CheckpointTaskType.FULL if osnap else CheckpointTaskType.MODEL_ONLY, snap, osnap, kw, time.time())
        with self._lock:
            self._tasks[tag] = task                       # a name that was cancelled stays cancelled: the worker drops it
        try:
            self._q.put(task, block=block)
        except queue.Full:
            with self._lock:
                self._tasks.pop(tag, None)
            raise CheckpointQueueFullError(self.max_queue_size) from None
        return tag

    def _finish(self, task: CheckpointTask, status: CheckpointTaskStatus, value=None, error=None):
        task.completed_at = time.time()
        task.status = status
        nbytes = sum(t.numel() * t.element_size() for t in (*task.model_state.values(), *task.optimizer_state.values()))
        task.result = CheckpointTaskResult(task.id, status is CheckpointTaskStatus.COMPLETED, value, error,
                                           task.completed_at - (task.started_at or task.completed_at), nbytes)
        task.model_state, task.optimizer_state = {}, {}          # the snapshot is no longer needed
        with self._lock:
            self._results[task.id] = value if error is None else error
            finished = [t for t in self._tasks.values() if t.done.is_set()]
            for old in sorted(finished, key=lambda t: t.completed_at or 0)[:max(0, len(finished) + 1 - self._keep)]:
                self._tasks.pop(old.id, None)
        task.done.set()

    def _worker(self):
        while True:
            task = self._q.get()
            if task is None:
                return
            try:
                if task.id in self._cancelled:
                    self._finish(task, CheckpointTaskStatus.CANCELLED, error=CheckpointError("cancelled"))
                    continue
                task.started_at, task.status = time.time(), CheckpointTaskStatus.RUNNING
                try:
                    value = self.ckpt.save(task.id, task.model_state, task.optimizer_state or None, **task.options)
                    self._finish(task, CheckpointTaskStatus.COMPLETED, value=value)
                except Exception as e:  # noqa: BLE001 - delivered through the task's result
                    self._finish(task, CheckpointTaskStatus.FAILED, error=e)
            finally:
                self._q.task_done()

    def cancel_checkpoint(self, tag: str) -> bool:
        """Cancels a save that has not started; ``False`` when it is unknown, running or finished."""
        with self._lock:
            t = self._tasks.get(tag)
            if t is None:
                self._cancelled.add(tag)                      # a save queued under this name later is dropped
                return False
            if t.status is not CheckpointTaskStatus.QUEUED:
                return False
            self._cancelled.add(tag)
            return True

    def get_task_status(self, tag: str) -> Optional[CheckpointTaskStatus]:
        with self._lock:
            t = self._tasks.get(tag)
            return t.status if t is not None else None

    def get_task_info(self, tag: str) -> Optional[CheckpointTaskInfo]:
        with self._lock:
            t = self._tasks.get(tag)
            return t.info() if t is not None else None

    def get_active_tasks(self) -> List[CheckpointTaskInfo]:
        with self._lock:
            return [t.info() for t in self._tasks.values() if t.status in (CheckpointTaskStatus.QUEUED, CheckpointTaskStatus.RUNNING)]

    def wait_for(self, tag: str, timeout_s: float = 600.0) -> CheckpointTaskResult:
        """Blocks until that save has finished one way or the other."""
        with self._lock:
            t = self._tasks.get(tag)
        if t is None:
            raise KeyError(f"no save named {tag!r}")
        if not t.done.wait(timeout_s):
            raise CheckpointError(f"save {tag!r} did not finish within {timeout_s} s")
        return t.result

    def wait_for_completion(self, timeout_s: float = 600.0):
        t0 = time.time()
        while self._q.unfinished_tasks:
            if time.time() - t0 > timeout_s:
                raise CheckpointError("async checkpoint did not finish in time")
            time.sleep(0.01)
        errs = {t: r for t, r in self._results.items() if isinstance(r, Exception) and t not in self._cancelled}
        if errs:
            raise CheckpointError(f"async saves failed: {errs}")
        return dict(self._results)

    def shutdown(self):
        self._q.put(None)


class IncrementalCheckpointManager:
    """Baseline + deltas: a delta stores only tensors whose SHA-256 changed, gzip-compressed
    (Checkpointing/Incremental/IncrementalCheckpointManager.cs:31-95)."""

    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self._hashes: Dict[str, str] = {}
        self._chain: List[str] = []

    @staticmethod
    def _hash(t: torch.Tensor) -> str:
        return hashlib.sha256(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()

    def save_baseline(self, tag: str, state: Dict[str, torch.Tensor]) -> str:
        SingleFileCheckpointFormat.save(os.path.join(self.dir, tag + ".base"), state)
        self._hashes = {k: self._hash(v) for k, v in state.items()}
        self._chain = [tag + ".base"]
        return tag

    def save_incremental(self, tag: str, state: Dict[str, torch.Tensor]) -> List[str]:
        if not self._chain:
            raise CheckpointError("save a baseline first")
        changed = {}
        for k, v in state.items():
            h = self._hash(v)
            if self._hashes.get(k) != h:
                changed[k] = v
                self._hashes[k] = h
        buf = io.BytesIO()
        torch.save({k: v.detach().cpu() for k, v in changed.items()}, buf)
        with gzip.open(os.path.join(self.dir, tag + ".delta.gz"), "wb") as f:
            f.write(buf.getvalue())
        self._chain.append(tag + ".delta.gz")
        return sorted(changed)

    def load(self) -> Dict[str, torch.Tensor]:
        state, _ = SingleFileCheckpointFormat.load(os.path.join(self.dir, self._chain[0]))
        for name in self._chain[1:]:
            with gzip.open(os.path.join(self.dir, name), "rb") as f:
                state.update(torch.load(io.BytesIO(f.read()), map_location="cpu"))
        return state


@dataclass
class RetryPolicy:
    """Checkpointing/FaultTolerance/RetryPolicy.cs:8-54: 3 retries, 1 s -> 30 s, x2."""
    max_retries: int = 3
    initial_delay_s: float = 1.0
    max_delay_s: float = 30.0
    backoff: float = 2.0

    def delay(self, attempt: int) -> float:
        return min(self.initial_delay_s * self.backoff ** attempt, self.max_delay_s)


class CircuitBreaker:
    """Opens after ``threshold`` consecutive failures (default 5); half-opens after ``reset_s``."""

    def __init__(self, threshold: int = 5, reset_s: float = 60.0, clock: Callable[[], float] = time.time):
        self.threshold, self.reset_s, self.clock = threshold, reset_s, clock
        self.failures, self.opened_at = 0, None

    @property
    def state(self) -> str:
        if self.opened_at is None:
            return "closed"
        return "half_open" if self.clock() - self.opened_at >= self.reset_s else "open"

    def allow(self) -> bool:
        return self.state != "open"

    def record_success(self):
        self.failures, self.opened_at = 0, None

    def record_failure(self):
        self.failures += 1
        if self.failures >= self.threshold:
            self.opened_at = self.clock()


class FaultToleranceHandler:
    def __init__(self, policy: Optional[RetryPolicy] = None, breaker: Optional[CircuitBreaker] = None,
                 sleep: Callable[[float], None] = time.sleep):
        self.policy, self.breaker, self.sleep = policy or RetryPolicy(), breaker or CircuitBreaker(), sleep
        self.attempts = 0

    def execute_with_retry(self, fn: Callable, *a, **k):
        last = None
        for attempt in range(self.policy.max_retries + 1):
            if not self.breaker.allow():
                raise CheckpointError("circuit breaker is open") from last
            self.attempts += 1
            try:
                r = fn(*a, **k)
                self.breaker.record_success()
                return r
            except Exception as e:  # noqa: BLE001
                last = e
                self.breaker.record_failure()
                if attempt < self.policy.max_retries:
                    self.sleep(self.policy.delay(attempt))
        raise CheckpointError(f"operation failed after {self.policy.max_retries + 1} attempts: {last}") from last

    def execute_with_timeout(self, fn: Callable, timeout_s: float, *a, **k):
        box: Dict[str, object] = {}

        def run():
            try:
                box["r"] = fn(*a, **k)
            except Exception as e:  # noqa: BLE001
                box["e"] = e
        t = threading.Thread(target=run, daemon=True)
        t.start()
        t.join(timeout_s)
        if t.is_alive():
            raise CheckpointError(f"operation timed out after {timeout_s}s")
        if "e" in box:
            raise box["e"]  # type: ignore
        return box.get("r")


class CheckpointRollbackManager:
    """Keeps the last good tag; ``rollback`` reloads it after a failed or corrupt save."""

    def __init__(self, checkpoint: DistributedCheckpoint):
        self.ckpt, self.last_good = checkpoint, None

    def mark_good(self, tag: str):
        ok, errs = ShardFileVerifier.verify_checkpoint(self.ckpt._prefix(tag))
        if not ok:
            raise CheckpointCorruptError("; ".join(errs))
        self.last_good = tag

    def rollback(self, device="cpu") -> CheckpointLoadResult:
        if self.last_good is None:
            raise CheckpointError("no verified checkpoint to roll back to")
        return self.ckpt.load(self.last_good, device=device)
