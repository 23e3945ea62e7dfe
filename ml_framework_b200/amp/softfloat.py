"""Software half-precision types: bit-exact conversion between fp32 and IEEE binary16 / bfloat16 on the host.

The reference carries its own ``Half`` and ``BFloat16`` structs for machines without native support
(src/MLFramework/Amp/Half.cs, BFloat16.cs: conversion from / to ``float`` with round-to-nearest-even, comparison,
arithmetic through fp32) and an optimizer wrapper that keeps fp32 state for low-precision parameters. On B200 the
device types are native; these routines exist for host-side tooling that must not depend on a tensor library's
rounding: writing checkpoints in a 16-bit format from Python lists, checking a kernel's rounding against an
independent statement of it, and decoding raw 16-bit payloads. They work on plain ints / floats and on numpy arrays.
"""
from __future__ import annotations

import struct
from typing import Iterable, List, Union

import numpy as np

Number = Union[int, float]


def _f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _bits_f32(b: int) -> float:
    return struct.unpack("<f", struct.pack("<I", b & 0xFFFFFFFF))[0]


# ------------------------------------------------------------------ bfloat16
def float_to_bfloat16_bits(x: float) -> int:
    """fp32 -> bfloat16 bit pattern, round to nearest even; NaN stays a quiet NaN, overflow rounds to infinity."""
    b = _f32_bits(float(np.float32(x)))
    if (b & 0x7F800000) == 0x7F800000 and (b & 0x007FFFFF):
        return ((b >> 16) | 0x0040) & 0xFFFF                       # NaN: keep the sign and payload top, force quiet
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF


def bfloat16_bits_to_float(h: int) -> float:
    return _bits_f32((h & 0xFFFF) << 16)


# ------------------------------------------------------------------ IEEE binary16
def float_to_half_bits(x: float) -> int:
    """fp32 -> binary16 bit pattern, round to nearest even, gradual underflow, overflow to infinity."""
    b = _f32_bits(float(np.float32(x)))
    sign = (b >> 16) & 0x8000
    exp = (b >> 23) & 0xFF
    man = b & 0x007FFFFF
    if exp == 0xFF:                                                  # infinity / NaN
        return sign | 0x7C00 | (0x0200 if man else 0) | (man >> 13)
    e = exp - 127 + 15
    if e >= 0x1F:
        return sign | 0x7C00                                         # too large: infinity
    if e <= 0:                                                       # subnormal half or zero
        if e < -10:
            return sign
        man |= 0x00800000
        shift = 14 - e
        half = man >> shift
        rem = man & ((1 << shift) - 1)
        halfway = 1 << (shift - 1)
        if rem > halfway or (rem == halfway and (half & 1)):
            half += 1
        return sign | half
    half = (e << 10) | (man >> 13)
    rem = man & 0x1FFF
    if rem > 0x1000 or (rem == 0x1000 and (half & 1)):
        half += 1                                                    # may carry into the exponent, up to infinity: correct
    return sign | half


def half_bits_to_float(h: int) -> float:
    h &= 0xFFFF
    sign = (h & 0x8000) << 16
    exp = (h >> 10) & 0x1F
    man = h & 0x03FF
    if exp == 0:
        if man == 0:
            return _bits_f32(sign)
        # subnormal: normalise
        e = -1
        while not (man & 0x0400):
            man <<= 1
            e += 1
        man &= 0x03FF
        return _bits_f32(sign | ((127 - 15 - e) << 23) | (man << 13))
    if exp == 0x1F:
        return _bits_f32(sign | 0x7F800000 | (man << 13))
    return _bits_f32(sign | ((exp - 15 + 127) << 23) | (man << 13))


# ------------------------------------------------------------------ value types
class _Soft16:
    __slots__ = ("bits",)
    _enc = staticmethod(lambda x: 0)
    _dec = staticmethod(lambda b: 0.0)

    def __init__(self, value: Number = 0.0, *, bits: int = None):
        self.bits = (bits & 0xFFFF) if bits is not None else type(self)._enc(float(value))

    def __float__(self) -> float:
        return type(self)._dec(self.bits)

    def _bin(self, other, op):
        return type(self)(op(float(self), float(other)))

    def __add__(self, o): return self._bin(o, lambda a, b: a + b)
    def __sub__(self, o): return self._bin(o, lambda a, b: a - b)
    def __mul__(self, o): return self._bin(o, lambda a, b: a * b)
    def __truediv__(self, o): return self._bin(o, lambda a, b: a / b)
    def __neg__(self): return type(self)(bits=self.bits ^ 0x8000)
    def __eq__(self, o): return float(self) == float(o)
    def __lt__(self, o): return float(self) < float(o)
    def __le__(self, o): return float(self) <= float(o)
    def __hash__(self): return hash(self.bits)
    def __repr__(self): return f"{type(self).__name__}({float(self)!r})"

    def is_nan(self) -> bool:
        return float(self) != float(self)

    def is_inf(self) -> bool:
        return float(self) in (float("inf"), float("-inf"))


class Half(_Soft16):
    """IEEE binary16 value held as its bit pattern; arithmetic goes through fp32 and rounds once."""
    _enc = staticmethod(float_to_half_bits)
    _dec = staticmethod(half_bits_to_float)
    MAX, EPSILON, MIN_NORMAL = 65504.0, 2.0 ** -10, 2.0 ** -14


class BFloat16(_Soft16):
    """bfloat16 value (fp32 range, 8 bits of significand) held as its bit pattern."""
    _enc = staticmethod(float_to_bfloat16_bits)
    _dec = staticmethod(bfloat16_bits_to_float)
    MAX, EPSILON, MIN_NORMAL = 3.3895313892515355e38, 2.0 ** -7, 2.0 ** -126


# ------------------------------------------------------------------ arrays
def to_bfloat16_bits(a: Iterable[float]) -> np.ndarray:
    """Vectorised fp32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    b = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = ((b & 0x7F800000) == 0x7F800000) & ((b & 0x007FFFFF) != 0)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF
    r = np.where(nan, ((b >> 16) | 0x0040) & 0xFFFF, r)
    return r.astype(np.uint16)


def from_bfloat16_bits(h: Iterable[int]) -> np.ndarray:
    return (np.asarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_half_bits(a: Iterable[float]) -> np.ndarray:
    flat = np.asarray(a, dtype=np.float32).ravel()
    return np.fromiter((float_to_half_bits(float(x)) for x in flat), dtype=np.uint16, count=flat.size).reshape(np.shape(a))


def from_half_bits(h: Iterable[int]) -> np.ndarray:
    flat = np.asarray(h, dtype=np.uint16).ravel()
    return np.fromiter((half_bits_to_float(int(x)) for x in flat), dtype=np.float32, count=flat.size).reshape(np.shape(h))


def round_trip_error(values: List[float], kind: str = "bfloat16") -> float:
    """Largest relative error of fp32 -> 16 bit -> fp32 over ``values`` (finite, non-zero)."""
    enc, dec = (float_to_bfloat16_bits, bfloat16_bits_to_float) if kind == "bfloat16" else (float_to_half_bits, half_bits_to_float)
    worst = 0.0
    for v in values:
        if v == 0 or v != v or v in (float("inf"), float("-inf")):
            continue
        worst = max(worst, abs(dec(enc(v)) - v) / abs(v))
    return worst
