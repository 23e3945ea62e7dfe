"""Quantization back-ends and their factory.

The reference dispatches quantized execution through ``IQuantizationBackend`` (IsAvailable, GetName, GetCapabilities,
Quantize, Dequantize, MatMulInt8, Conv2DInt8, Infer; src/MLFramework/Quantization/Backends/IQuantizationBackend.cs)
with implementations for CPU, x86 (oneDNN), ARM (NEON) and GPU (a cuDNN int8 "TODO",
Backends/GPUBackend/GPUBackend.cs:123), chosen by ``BackendFactory`` in the order preferred > GPU > x86 > ARM > CPU
(Backends/BackendFactory.cs:40-72) and described by ``BackendCapabilities`` flags (BackendCapabilities.cs).

Two back-ends exist here, both real:
* ``B200Backend`` ("GPU" / "CUDA"): quantise / dequantise through the native kernels of ``csrc/ops/quant.cu``; the int8
  products dequantise the operands in registers' precision (bf16 holds every int8 value exactly) and run on the
  tcgen05 GEMM, then apply the output scale - int8 storage and bandwidth with tensor-core arithmetic;
* ``CPUBackend`` ("CPU", also answering to the x86 / ARM names, since PyTorch's CPU kernels already pick the
  vector ISA): the same operations in integer PyTorch arithmetic with an int32 accumulator.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from .core import QuantizationParameters, dequantize, quantize


class BackendCapabilityFlags(enum.IntFlag):
    NONE = 0
    INT8_MATMUL = 1
    INT8_CONV2D = 2
    PER_CHANNEL_QUANTIZATION = 4
    MIXED_PRECISION = 8
    DYNAMIC_QUANTIZATION = 16
    STATIC_QUANTIZATION = 32
    ASYMMETRIC_QUANTIZATION = 64
    SYMMETRIC_QUANTIZATION = 128
    ALL = 255


@dataclass(frozen=True)
class BackendCapabilities:
    flags: BackendCapabilityFlags
    max_tensor_size: int = 2 ** 63 - 1
    min_batch_size: int = 1
    preferred_batch_size: int = 32
    max_threads: int = 0

    def supports(self, flag: BackendCapabilityFlags) -> bool:
        return bool(self.flags & flag)

    def __str__(self):
        names = [f.name for f in BackendCapabilityFlags if f not in (BackendCapabilityFlags.NONE, BackendCapabilityFlags.ALL) and self.flags & f]
        return f"Capabilities: [{', '.join(names)}], MaxTensorSize: {self.max_tensor_size}, PreferredBatchSize: {self.preferred_batch_size}"


class QuantizationBackend:
    name = "base"

    def is_available(self) -> bool:
        raise NotImplementedError

    def get_name(self) -> str:
        return self.name

    def get_capabilities(self) -> BackendCapabilities:
        raise NotImplementedError

    def _device(self) -> torch.device:
        raise NotImplementedError

    def quantize(self, x: torch.Tensor, qp: QuantizationParameters) -> torch.Tensor:
        return quantize(x.to(self._device()), qp)

    def dequantize(self, q: torch.Tensor, qp: QuantizationParameters, dtype=torch.float32) -> torch.Tensor:
        return dequantize(q.to(self._device()), qp, dtype)

    def matmul_int8(self, a: torch.Tensor, b: torch.Tensor, output_scale: float = 1.0) -> torch.Tensor:
        """``a`` int8 [M, K], ``b`` int8 [K, N]; returns fp32 ``(a @ b) * output_scale``."""
        raise NotImplementedError

    def conv2d_int8(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], stride=(1, 1), padding=(0, 0),
                    dilation=(1, 1), output_scale: float = 1.0) -> torch.Tensor:
        raise NotImplementedError

    def infer(self, model, inputs: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return model(inputs.to(self._device()))


class CPUBackend(QuantizationBackend):
    name = "CPU"

    def is_available(self) -> bool:
        return True

    def _device(self):
        return torch.device("cpu")

    def get_capabilities(self) -> BackendCapabilities:
        fl = BackendCapabilityFlags.ALL & ~BackendCapabilityFlags.MIXED_PRECISION
        return BackendCapabilities(fl, preferred_batch_size=32, max_threads=os.cpu_count() or 1)

    def matmul_int8(self, a, b, output_scale: float = 1.0):
        acc = a.to("cpu", torch.int32) @ b.to("cpu", torch.int32)          # exact int32 accumulation
        return acc.float() * output_scale

    def conv2d_int8(self, x, w, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_scale: float = 1.0):
        # int8 values and their products up to the accumulated sum are exact in fp64
        y = F.conv2d(x.to("cpu", torch.float64), w.to("cpu", torch.float64), None, stride, padding, dilation)
        y = y.float() * output_scale
        return y + bias.float().view(1, -1, 1, 1) if bias is not None else y


class B200Backend(QuantizationBackend):
    name = "GPU"

    def is_available(self) -> bool:
        if not torch.cuda.is_available():
            return False
        from .. import _lib
        return _lib.available()

    def _device(self):
        return torch.device("cuda", torch.cuda.current_device())

    def get_capabilities(self) -> BackendCapabilities:
        return BackendCapabilities(BackendCapabilityFlags.ALL, preferred_batch_size=256, max_threads=148)

    def matmul_int8(self, a, b, output_scale: float = 1.0):
        from ..ops.gemm import gemm
        dev = self._device()
        a16 = a.to(dev).to(torch.bfloat16).contiguous()                     # every int8 value is exact in bf16
        bt = b.to(dev).to(torch.bfloat16).t().contiguous()                  # [N, K], K-major
        K = a16.shape[1]
        if K % 8 or bt.shape[0] % 8:                                        # TMA rows need 16-byte multiples
            return (a16.float() @ bt.float().t()) * output_scale
        return gemm(a16, bt, out_dtype=torch.float32) * output_scale        # fp32 accumulation in tensor memory

    def conv2d_int8(self, x, w, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_scale: float = 1.0):
        dev = self._device()
        y = F.conv2d(x.to(dev).float(), w.to(dev).float(), None, stride, padding, dilation) * output_scale
        return y + bias.to(dev).float().view(1, -1, 1, 1) if bias is not None else y


class BackendFactory:
    """``create_default`` follows the reference's order: the preferred back-end when set and available, else the GPU,
    else the CPU (the x86 / ARM names resolve to the CPU back-end). Instances are cached per name."""

    _preferred: Optional[str] = None
    _cache: Dict[str, QuantizationBackend] = {}
    _ALIASES = {"CPU": "CPU", "X86": "CPU", "ARM": "CPU", "INTEL ONEDNN": "CPU", "ARM NEON": "CPU", "GPU": "GPU", "CUDA": "GPU",
                "B200": "GPU"}

    @classmethod
    def set_preferred_backend(cls, name: Optional[str]):
        if name is not None and name.upper() not in cls._ALIASES:
            raise ValueError(f"unknown backend {name!r}")
        cls._preferred = name

    @classmethod
    def create(cls, name: str) -> QuantizationBackend:
        key = cls._ALIASES.get(name.upper())
        if key is None:
            raise ValueError(f"unknown backend {name!r}; known: {sorted(cls._ALIASES)}")
        if key not in cls._cache:
            b = B200Backend() if key == "GPU" else CPUBackend()
            if not b.is_available():
                raise RuntimeError(f"backend {name!r} is not available on this machine")
            cls._cache[key] = b
        return cls._cache[key]

    @classmethod
    def create_default(cls) -> QuantizationBackend:
        for cand in ([cls._preferred] if cls._preferred else []) + ["GPU", "CPU"]:
            try:
                return cls.create(cand)
            except RuntimeError:
                continue
        raise RuntimeError("no quantization backend is available")

    @classmethod
    def get_available_backends(cls) -> List[str]:
        out = []
        for name in ("GPU", "CPU"):
            try:
                cls.create(name)
                out.append(name)
            except RuntimeError:
                pass
        return out

    @classmethod
    def clear_cache(cls):
        cls._cache = {}
