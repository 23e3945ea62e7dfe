"""``.mob`` model container: a compact operator list with tensors, read and written without pickling.

Reference: src/MobileRuntime/Serialization/MobileModelFormat.cs (header with magic / version, operator
table, tensor table), MobileModelWriter.cs, ModelSerializer.cs; operator types from
src/MobileRuntime/Backends/Metal/Models/OperatorType.cs.

Layout (little endian):
  magic "MOB1" | u32 version | u32 header_len | header JSON (utf-8) | tensor payload (64-byte aligned blobs)
The header lists inputs, outputs, operators ``{type, inputs, outputs, attrs}`` and tensors
``{name, dtype, shape, offset, nbytes, scale?, zero_point?}``; ``sha256`` covers the payload.
"""
from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np
import torch

MAGIC = b"MOB1"
VERSION = 1
_DTYPES = {"float32": torch.float32, "float16": torch.float16, "int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64}
_NP = {"float32": np.float32, "float16": np.float16, "int8": np.int8, "uint8": np.uint8, "int32": np.int32, "int64": np.int64}

OPERATOR_TYPES = ("conv2d", "fully_connected", "relu", "max_pool2d", "avg_pool2d", "batch_norm", "softmax", "add", "mul", "flatten",
                  "reshape", "concat", "sigmoid", "tanh", "global_avg_pool",
                  # the reference runtime's tensor operator set (src/MobileRuntime/Tensors/TensorOperations.cs:19-434)
                  "sub", "div", "abs", "sqrt", "square", "log", "exp", "sum", "mean", "max", "min", "matmul", "transpose", "cast", "copy")


@dataclass
class MobOperator:
    type: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class MobTensor:
    name: str
    data: torch.Tensor
    scale: Optional[float] = None          # set when the tensor is stored quantised (int8 / uint8)
    zero_point: Optional[int] = None


@dataclass
class MobModel:
    inputs: List[Dict[str, Any]]           # {"name", "shape"}
    outputs: List[str]
    operators: List[MobOperator]
    tensors: Dict[str, MobTensor]
    metadata: Dict[str, Any] = field(default_factory=dict)

    def validate(self) -> List[str]:
        errs = []
        known = {i["name"] for i in self.inputs} | set(self.tensors)
        for k, op in enumerate(self.operators):
            if op.type not in OPERATOR_TYPES:
                errs.append(f"operator #{k}: unknown type {op.type!r}")
            for n in op.inputs:
                if n not in known:
                    errs.append(f"operator #{k} ({op.type}): input {n!r} is not defined before use")
            known.update(op.outputs)
        errs += [f"output {o!r} is never produced" for o in self.outputs if o not in known]
        return errs


def _dtype_name(t: torch.dtype) -> str:
    for k, v in _DTYPES.items():
        if v == t:
            return k
    raise ValueError(f"dtype {t} is not storable in a .mob file")


def save_mob(model: MobModel, path: str):
    errs = model.validate()
    if errs:
        raise ValueError("invalid model: " + "; ".join(errs))
    payload = bytearray()
    table = []
    for name, t in model.tensors.items():
        while len(payload) % 64:
            payload.append(0)
        raw = t.data.detach().cpu().contiguous().numpy().tobytes()
        e = {"name": name, "dtype": _dtype_name(t.data.dtype), "shape": list(t.data.shape), "offset": len(payload), "nbytes": len(raw)}
        if t.scale is not None:
            e["scale"], e["zero_point"] = t.scale, t.zero_point or 0
        table.append(e)
        payload += raw
    header = {"inputs": model.inputs, "outputs": model.outputs, "metadata": model.metadata,
              "operators": [{"type": o.type, "inputs": o.inputs, "outputs": o.outputs, "attrs": o.attrs} for o in model.operators],
              "tensors": table, "sha256": hashlib.sha256(bytes(payload)).hexdigest()}
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", VERSION, len(hj)) + hj + bytes(payload))


def load_mob(path: str, verify: bool = True) -> MobModel:
    with open(path, "rb") as f:
        blob = f.read()
    if blob[:4] != MAGIC:
        raise ValueError(f"{path}: not a .mob file")
    ver, hl = struct.unpack("<II", blob[4:12])
    if ver > VERSION:
        raise ValueError(f"{path}: format version {ver} is newer than this reader ({VERSION})")
    h = json.loads(blob[12:12 + hl])
    payload = blob[12 + hl:]
    if verify and hashlib.sha256(payload).hexdigest() != h["sha256"]:
        raise IOError(f"{path}: payload checksum mismatch")
    tensors = {}
    for e in h["tensors"]:
        arr = np.frombuffer(payload, dtype=_NP[e["dtype"]], count=int(np.prod(e["shape"])) if e["shape"] else 1, offset=e["offset"])
        tensors[e["name"]] = MobTensor(e["name"], torch.from_numpy(arr.copy()).view(*e["shape"]) if e["shape"] else torch.tensor(arr[0]),
                                       e.get("scale"), e.get("zero_point"))
    ops = [MobOperator(o["type"], o["inputs"], o["outputs"], o.get("attrs", {})) for o in h["operators"]]
    return MobModel(h["inputs"], h["outputs"], ops, tensors, h.get("metadata", {}))
