"""Model weight files: one self-describing binary format with a writer, a reader and partial (per-tensor) reads.

Reference: src/ModelZoo/Serialization/{FileFormatSpec.cs, ModelSerializer.cs:39-118, ModelDeserializer.cs,
SerializerOptions.cs}. Layout (little endian):

    8 bytes   magic "MLFMODL1"
    u32       header length H
    H bytes   JSON header: {"version", "metadata", "compression", "tensors": [{"name", "dtype", "shape", "offset",
              "nbytes", "stored_nbytes", "crc32"}]}  - offsets are relative to the data section
    padding   to a multiple of 64 bytes
    data      tensors back to back, each starting on a 64-byte boundary (so a reader can map the file and hand the
              bytes to a pinned staging buffer or a direct-storage read without re-alignment)

``SerializerOptions.dtype`` casts floating-point tensors on the way out (e.g. fp32 checkpoints stored as bf16);
``compression="zlib"`` deflates each tensor separately so that single tensors stay addressable.
"""
from __future__ import annotations

import io
import json
import struct
import zlib
from dataclasses import dataclass, field
from typing import Any, BinaryIO, Dict, Iterable, List, Optional

import torch

MAGIC = b"MLFMODL1"
ALIGN = 64
FORMAT_VERSION = 1


class ModelFormatError(RuntimeError):
    pass


@dataclass
class SerializerOptions:
    dtype: Optional[torch.dtype] = None          # cast floating-point tensors to this type when writing
    compression: str = "none"                    # none | zlib
    compression_level: int = 3
    include: Optional[Iterable[str]] = None      # tensor-name prefixes to write (default: all)
    metadata: Dict[str, Any] = field(default_factory=dict)

    def validate(self):
        if self.compression not in ("none", "zlib"):
            raise ValueError(f"unknown compression {self.compression!r}")


def _dtype_name(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def _bytes_of(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def _pad(n: int) -> int:
    return (-n) % ALIGN


class ModelSerializer:
    def __init__(self, options: Optional[SerializerOptions] = None):
        self.options = options or SerializerOptions()
        self.options.validate()

    def _tensors(self, state: Dict[str, torch.Tensor], o: SerializerOptions):
        inc = tuple(o.include) if o.include is not None else None
        for k, v in state.items():
            if not isinstance(v, torch.Tensor) or (inc is not None and not k.startswith(inc)):
                continue
            if o.dtype is not None and v.is_floating_point():
                v = v.to(o.dtype)
            yield k, v

    def serialize(self, model_or_state, out: BinaryIO, options: Optional[SerializerOptions] = None) -> int:
        o = options or self.options
        o.validate()
        state = model_or_state.state_dict() if hasattr(model_or_state, "state_dict") else model_or_state
        entries, blobs, off = [], [], 0
        for k, v in self._tensors(state, o):
            raw = _bytes_of(v)
            stored = zlib.compress(raw, o.compression_level) if o.compression == "zlib" else raw
            entries.append({"name": k, "dtype": _dtype_name(v.dtype), "shape": list(v.shape), "offset": off, "nbytes": len(raw),
                            "stored_nbytes": len(stored), "crc32": zlib.crc32(raw)})
            blobs.append(stored)
            off += len(stored) + _pad(len(stored))
        header = json.dumps({"version": FORMAT_VERSION, "metadata": o.metadata, "compression": o.compression, "tensors": entries}).encode()
        n = out.write(MAGIC) + out.write(struct.pack("<I", len(header))) + out.write(header)
        n += out.write(b"\0" * _pad(n))
        for b in blobs:
            n += out.write(b) + out.write(b"\0" * _pad(len(b)))
        return n

    def serialize_to_file(self, model_or_state, path: str, options: Optional[SerializerOptions] = None) -> int:
        with open(path, "wb") as f:
            return self.serialize(model_or_state, f, options)

    def serialized_size(self, model_or_state, options: Optional[SerializerOptions] = None) -> int:
        buf = io.BytesIO()
        return self.serialize(model_or_state, buf, options)


class ModelDeserializer:
    def __init__(self, verify_checksums: bool = True):
        self.verify = verify_checksums

    @staticmethod
    def read_header(f: BinaryIO) -> Dict[str, Any]:
        if f.read(len(MAGIC)) != MAGIC:
            raise ModelFormatError("not a model file (bad magic)")
        raw = f.read(4)
        if len(raw) < 4:
            raise ModelFormatError("truncated header")
        n, = struct.unpack("<I", raw)
        body = f.read(n)
        if len(body) < n:
            raise ModelFormatError("truncated header")
        h = json.loads(body)
        if h.get("version") != FORMAT_VERSION:
            raise ModelFormatError(f"unsupported format version {h.get('version')}")
        pos = len(MAGIC) + 4 + n
        h["_data_start"] = pos + _pad(pos)
        return h

    def _read_tensor(self, f: BinaryIO, h: Dict[str, Any], e: Dict[str, Any]) -> torch.Tensor:
        f.seek(h["_data_start"] + e["offset"])
        stored = f.read(e["stored_nbytes"])
        if len(stored) < e["stored_nbytes"]:
            raise ModelFormatError(f"tensor {e['name']!r} is truncated")
        raw = zlib.decompress(stored) if h["compression"] == "zlib" else stored
        if len(raw) != e["nbytes"] or (self.verify and zlib.crc32(raw) != e["crc32"]):
            raise ModelFormatError(f"tensor {e['name']!r} failed its checksum")
        dt = getattr(torch, e["dtype"])
        if not raw:
            return torch.empty(e["shape"], dtype=dt)
        return torch.frombuffer(bytearray(raw), dtype=dt).reshape(e["shape"])

    def deserialize(self, f: BinaryIO, names: Optional[Iterable[str]] = None) -> Dict[str, torch.Tensor]:
        h = self.read_header(f)
        want = set(names) if names is not None else None
        out = {e["name"]: self._read_tensor(f, h, e) for e in h["tensors"] if want is None or e["name"] in want}
        if want is not None and want - set(out):
            raise KeyError(f"tensors not in the file: {sorted(want - set(out))}")
        return out

    def deserialize_file(self, path: str, names: Optional[Iterable[str]] = None) -> Dict[str, torch.Tensor]:
        with open(path, "rb") as f:
            return self.deserialize(f, names)

    def metadata(self, path: str) -> Dict[str, Any]:
        with open(path, "rb") as f:
            h = self.read_header(f)
        return {"metadata": h["metadata"], "compression": h["compression"],
                "tensors": {e["name"]: (e["dtype"], tuple(e["shape"])) for e in h["tensors"]},
                "total_bytes": sum(e["nbytes"] for e in h["tensors"])}

    def load_into(self, model: torch.nn.Module, path: str, strict: bool = True) -> List[str]:
        """Loads the file into ``model``; returns the names the file did not provide (raises on them when ``strict``)."""
        state = self.deserialize_file(path)
        own = model.state_dict()
        missing = [k for k in own if k not in state]
        unexpected = [k for k in state if k not in own]
        if strict and (missing or unexpected):
            raise KeyError(f"missing {missing}, unexpected {unexpected}")
        for k, v in state.items():
            if k in own:
                if tuple(own[k].shape) != tuple(v.shape):
                    raise ModelFormatError(f"tensor {k!r}: file has {tuple(v.shape)}, model has {tuple(own[k].shape)}")
                own[k].copy_(v.to(own[k].dtype))
        return missing
