"""Core types: the data-type enumeration with its facts, the shape validator, tensor / HAL conveniences.

Reference: src/RitterFramework.Core/DataType.cs:8-20 and src/MLFramework/Core/{DataType.cs, DataTypeInfo.cs:13-163
(size, name, limits, epsilon, NaN / infinity support, decimal precision, dynamic range), ShapeValidator.cs:17-222
(matmul, conv2d, concat, broadcast, dispatch by operation)}, src/MLFramework/HAL/TensorHALExtensions.cs:43-176
(device pointer, zeros / from-array on a device, moving a tensor to a device).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


class DataType(enum.Enum):
    FLOAT32 = "float32"
    FLOAT64 = "float64"
    FLOAT16 = "float16"
    BFLOAT16 = "bfloat16"
    FLOAT8_E4M3 = "float8_e4m3fn"
    FLOAT8_E5M2 = "float8_e5m2"
    INT8 = "int8"
    UINT8 = "uint8"
    INT16 = "int16"
    INT32 = "int32"
    INT64 = "int64"
    BOOL = "bool"

    @property
    def torch(self) -> torch.dtype:
        return getattr(torch, self.value)

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DataType":
        return DataType(str(dt).replace("torch.", ""))


class DataTypeInfo:
    @staticmethod
    def size_of(dt: DataType) -> int:
        return torch.empty(0, dtype=dt.torch).element_size()

    @staticmethod
    def name(dt: DataType) -> str:
        return dt.value

    @staticmethod
    def is_floating_point(dt: DataType) -> bool:
        return dt.torch.is_floating_point

    @staticmethod
    def is_integer(dt: DataType) -> bool:
        return not dt.torch.is_floating_point and dt != DataType.BOOL

    @staticmethod
    def max_value(dt: DataType) -> float:
        if dt == DataType.BOOL:
            return 1.0
        return float(torch.finfo(dt.torch).max if dt.torch.is_floating_point else torch.iinfo(dt.torch).max)

    @staticmethod
    def min_value(dt: DataType) -> float:
        if dt == DataType.BOOL:
            return 0.0
        return float(torch.finfo(dt.torch).min if dt.torch.is_floating_point else torch.iinfo(dt.torch).min)

    @staticmethod
    def epsilon(dt: DataType) -> float:
        return float(torch.finfo(dt.torch).eps) if dt.torch.is_floating_point else 1.0

    @staticmethod
    def smallest_normal(dt: DataType) -> float:
        return float(torch.finfo(dt.torch).tiny) if dt.torch.is_floating_point else 1.0

    @staticmethod
    def supports_nan(dt: DataType) -> bool:
        return dt.torch.is_floating_point

    @staticmethod
    def supports_infinity(dt: DataType) -> bool:
        return dt.torch.is_floating_point and dt != DataType.FLOAT8_E4M3       # e4m3fn spends the infinity encodings on values

    @staticmethod
    def precision(dt: DataType) -> int:
        """Decimal digits that survive a round trip."""
        if not dt.torch.is_floating_point:
            return len(str(int(DataTypeInfo.max_value(dt)))) - 1 if dt != DataType.BOOL else 1
        return max(1, int(math.floor(-math.log10(DataTypeInfo.epsilon(dt)))))

    @staticmethod
    def dynamic_range_db(dt: DataType) -> float:
        """20 log10(largest / smallest positive normal) for floating-point types, 20 log10(max) for integers."""
        if dt.torch.is_floating_point:
            return 20.0 * math.log10(DataTypeInfo.max_value(dt) / DataTypeInfo.smallest_normal(dt))
        return 20.0 * math.log10(max(DataTypeInfo.max_value(dt), 1.0))

    @staticmethod
    def tensor_core_input(dt: DataType) -> bool:
        """Operand types of the Blackwell tensor cores this package's GEMMs use or could use."""
        return dt in (DataType.BFLOAT16, DataType.FLOAT16, DataType.FLOAT8_E4M3, DataType.FLOAT8_E5M2, DataType.INT8)

    @staticmethod
    def can_cast_losslessly(src: DataType, dst: DataType) -> bool:
        if src == dst:
            return True
        s, d = src.torch, dst.torch
        if s.is_floating_point and not d.is_floating_point:
            return False
        if not s.is_floating_point and d.is_floating_point:
            return DataTypeInfo.max_value(src) <= 2.0 ** (1 - math.log2(DataTypeInfo.epsilon(dst)))
        if s.is_floating_point:
            fs, fd = torch.finfo(s), torch.finfo(d)
            return fd.eps <= fs.eps and fd.max >= fs.max and fd.tiny <= fs.tiny
        return DataTypeInfo.min_value(dst) <= DataTypeInfo.min_value(src) and DataTypeInfo.max_value(dst) >= DataTypeInfo.max_value(src)


# ------------------------------------------------------------------ shape validation
@dataclass
class ValidationResult:
    is_valid: bool
    message: str = ""
    suggestions: List[str] = field(default_factory=list)

    @staticmethod
    def ok() -> "ValidationResult":
        return ValidationResult(True)

    def __bool__(self):
        return self.is_valid


class ShapeValidator:
    @staticmethod
    def validate_matrix_multiply(a: Sequence[int], b: Sequence[int]) -> ValidationResult:
        if len(a) < 2 or len(b) < 2:
            return ValidationResult(False, f"matmul needs operands of rank >= 2, got {len(a)} and {len(b)}", ["add a dimension with unsqueeze"])
        if a[-1] != b[-2]:
            s = [f"make the inner dimensions agree ({a[-1]} vs {b[-2]})"]
            if a[-1] == b[-1]:
                s.insert(0, "transpose the second operand")
            return ValidationResult(False, f"inner dimensions differ: {list(a)} x {list(b)}", s)
        for x, y in zip(reversed(a[:-2]), reversed(b[:-2])):
            if x != y and x != 1 and y != 1:
                return ValidationResult(False, f"batch dimensions {list(a[:-2])} and {list(b[:-2])} do not broadcast", ["make the batch sizes equal or 1"])
        return ValidationResult.ok()

    @staticmethod
    def validate_conv2d(x: Sequence[int], w: Sequence[int], stride=1, padding=0, dilation=1, groups: int = 1) -> ValidationResult:
        if len(x) != 4 or len(w) != 4:
            return ValidationResult(False, f"conv2d needs [N, C, H, W] and [O, I, kh, kw], got ranks {len(x)} and {len(w)}")
        if x[1] != w[1] * groups:
            return ValidationResult(False, f"input has {x[1]} channels, weight expects {w[1]} x {groups} groups", [f"use in_channels = {x[1]}"])
        if w[0] % groups:
            return ValidationResult(False, f"{w[0]} output channels do not split into {groups} groups")
        two = lambda v: (v, v) if isinstance(v, int) else tuple(v)      # noqa: E731
        s, p, d = two(stride), two(padding), two(dilation)
        for i, nm in ((0, "height"), (1, "width")):
            out = (x[2 + i] + 2 * p[i] - d[i] * (w[2 + i] - 1) - 1) // s[i] + 1
            if out <= 0:
                return ValidationResult(False, f"output {nm} would be {out}: kernel {w[2 + i]} (dilation {d[i]}) exceeds the padded input {x[2 + i] + 2 * p[i]}",
                                        ["increase the padding", "use a smaller kernel"])
        return ValidationResult.ok()

    @staticmethod
    def validate_concat(shapes: Sequence[Sequence[int]], axis: int) -> ValidationResult:
        if not shapes:
            return ValidationResult(False, "nothing to concatenate")
        r = len(shapes[0])
        if not (-r <= axis < r):
            return ValidationResult(False, f"axis {axis} out of range for rank {r}")
        ax = axis % r
        for k, s in enumerate(shapes[1:], 1):
            if len(s) != r:
                return ValidationResult(False, f"input {k} has rank {len(s)}, input 0 has rank {r}")
            bad = [i for i in range(r) if i != ax and s[i] != shapes[0][i]]
            if bad:
                return ValidationResult(False, f"input {k} {list(s)} differs from input 0 {list(shapes[0])} outside axis {ax} (dimensions {bad})",
                                        ["only the concatenation axis may differ"])
        return ValidationResult.ok()

    @staticmethod
    def validate_broadcast(a: Sequence[int], b: Sequence[int]) -> ValidationResult:
        for i, (x, y) in enumerate(zip(reversed(a), reversed(b)), 1):
            if x != y and x != 1 and y != 1:
                return ValidationResult(False, f"dimension -{i}: {x} and {y} do not broadcast", ["sizes must be equal, or one of them 1"])
        return ValidationResult.ok()

    @classmethod
    def validate(cls, operation: str, *shapes: Sequence[int], **attrs) -> ValidationResult:
        op = operation.lower()
        if op in ("matmul", "matrixmultiply", "mm", "bmm"):
            return cls.validate_matrix_multiply(*shapes[:2])
        if op in ("conv2d",):
            return cls.validate_conv2d(*shapes[:2], **attrs)
        if op in ("concat", "cat"):
            return cls.validate_concat(list(shapes), attrs.get("axis", 0))
        if op in ("add", "sub", "mul", "div", "broadcast", "maximum", "minimum"):
            return cls.validate_broadcast(*shapes[:2])
        return ValidationResult(False, f"no shape rule for operation {operation!r}")


# ------------------------------------------------------------------ tensor / device conveniences
def device_pointer(t: torch.Tensor) -> int:
    """Address of the first element (device memory for CUDA tensors); what the C ABI of the native library takes."""
    return t.data_ptr()


def with_data_pointer(t: torch.Tensor, fn: Callable[[int], object]):
    """Calls ``fn(address)`` with the tensor kept alive and contiguous for the duration of the call."""
    c = t.contiguous()
    return fn(c.data_ptr())


def zeros_on(shape: Sequence[int], device, dtype: DataType = DataType.FLOAT32) -> torch.Tensor:
    return torch.zeros(tuple(shape), dtype=dtype.torch, device=_torch_device(device))


def from_array(data, device="cpu", dtype: DataType = DataType.FLOAT32, shape: Optional[Sequence[int]] = None) -> torch.Tensor:
    t = torch.as_tensor(data, dtype=dtype.torch)
    if shape is not None:
        t = t.reshape(tuple(shape))
    return t.to(_torch_device(device))


def to_device(t: torch.Tensor, device, non_blocking: bool = False) -> torch.Tensor:
    return t.to(_torch_device(device), non_blocking=non_blocking)


def _torch_device(device) -> torch.device:
    return device.torch if hasattr(device, "torch") else torch.device(device)
