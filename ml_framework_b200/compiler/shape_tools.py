"""Shape utilities around the symbolic shape system: comparison and reshape checks, lazily broadcast tensors, dimension
bindings, symbolic tensors, constraint building / validation, factories, an inference context.

Reference (src/MLFramework/): Shapes/ShapeComparer.cs:14-178, Shapes/BroadcastedTensor.cs:39-159 (strides of a broadcast
view, whether it must be materialised, which dimensions were broadcast), Shapes/BroadcastingRule.cs,
Shapes/ConstraintValidator.cs:31-173, Shapes/ShapeConstraintBuilder.cs:27-116, Shapes/SymbolicShapeFactory.cs,
Shapes/SymbolicDimensionFactory.cs, Shapes/Inference/InferenceContext.cs:36-165, Tensors/SymbolicTensor.cs:62-187,
Tensors/TensorShapeRegistry.cs:44-148 (dimension-name bindings).
"""
from __future__ import annotations

import enum
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .shapes import (Constraint, Dim, EqualityConstraint, ModuloConstraint, RangeConstraint, ShapeMismatchException, SymbolicDimension,
                     SymbolicShape, broadcast_shapes)


# ------------------------------------------------------------------ factories
class SymbolicDimensionFactory:
    @staticmethod
    def create(name: str, value: Optional[int] = None) -> SymbolicDimension:
        return SymbolicDimension(name, value) if value is None else SymbolicDimension(name, value, value, value)

    @staticmethod
    def bounded(name: str, lo: int, hi: Optional[int] = None) -> SymbolicDimension:
        if lo < 0 or (hi is not None and hi < lo):
            raise ValueError("bounds must satisfy 0 <= lo <= hi")
        return SymbolicDimension(name, None, lo, hi)

    @staticmethod
    def batch(max_batch: Optional[int] = None) -> SymbolicDimension:
        return SymbolicDimension("batch", None, 1, max_batch)

    @staticmethod
    def sequence(max_len: Optional[int] = None) -> SymbolicDimension:
        return SymbolicDimension("seq", None, 1, max_len)


class SymbolicShapeFactory:
    @staticmethod
    def scalar() -> SymbolicShape:
        return SymbolicShape([])

    @staticmethod
    def vector(n: Dim) -> SymbolicShape:
        return SymbolicShape([n])

    @staticmethod
    def matrix(rows: Dim, cols: Dim) -> SymbolicShape:
        return SymbolicShape([rows, cols])

    @staticmethod
    def from_concrete(*dims: int) -> SymbolicShape:
        return SymbolicShape(list(dims))

    @staticmethod
    def batched(*inner: Dim, max_batch: Optional[int] = None) -> SymbolicShape:
        return SymbolicShape([SymbolicDimensionFactory.batch(max_batch), *inner])

    @staticmethod
    def tokens(hidden: int, max_batch: Optional[int] = None, max_len: Optional[int] = None) -> SymbolicShape:
        """``[batch, seq, hidden]`` with symbolic batch and sequence."""
        return SymbolicShape([SymbolicDimensionFactory.batch(max_batch), SymbolicDimensionFactory.sequence(max_len), hidden])

    @staticmethod
    def image(channels: int, height: Dim = None, width: Dim = None) -> SymbolicShape:
        return SymbolicShape([SymbolicDimensionFactory.batch(), channels, height if height is not None else SymbolicDimension("height"),
                              width if width is not None else SymbolicDimension("width")])


# ------------------------------------------------------------------ comparison
def _dims_compatible(a: SymbolicDimension, b: SymbolicDimension) -> bool:
    if a.is_known and b.is_known:
        return a.value == b.value
    if a.is_known or b.is_known:
        k, s = (a, b) if a.is_known else (b, a)
        return s.min_value <= k.value and (s.max_value is None or k.value <= s.max_value)
    lo, hi = max(a.min_value, b.min_value), min(x for x in (a.max_value, b.max_value, float("inf")) if x is not None)
    return lo <= hi


class ShapeComparer:
    @staticmethod
    def are_equal(a: SymbolicShape, b: SymbolicShape) -> bool:
        return a == b

    @staticmethod
    def are_compatible(a: SymbolicShape, b: SymbolicShape) -> bool:
        """Could the two describe the same tensor? Same rank, and every pair of dimensions can take a common value."""
        return a.rank == b.rank and all(_dims_compatible(x, y) for x, y in zip(a, b))

    @staticmethod
    def can_broadcast(a: SymbolicShape, b: SymbolicShape) -> bool:
        try:
            broadcast_shapes(a, b)
            return True
        except ShapeMismatchException:
            return False

    @staticmethod
    def broadcast_shape(a: SymbolicShape, b: SymbolicShape) -> SymbolicShape:
        return broadcast_shapes(a, b)

    @staticmethod
    def numel(s: SymbolicShape) -> Optional[int]:
        if not s.is_fully_known:
            return None
        n = 1
        for d in s.concrete():
            n *= d
        return n

    @classmethod
    def can_reshape(cls, src: SymbolicShape, dst: Sequence[int]) -> bool:
        """Known element counts must agree (one ``-1`` is inferred); with unknown dimensions the known factor of the
        source must at least be divisible by the known factor of the target."""
        dst = list(dst)
        if dst.count(-1) > 1:
            return False
        known_dst = 1
        for d in dst:
            if d != -1:
                if d < 0:
                    return False
                known_dst *= d
        n = cls.numel(src)
        if n is not None:
            if -1 in dst:
                return known_dst != 0 and n % known_dst == 0
            return known_dst == n
        known_src = 1
        for d in src:
            if d.is_known:
                known_src *= d.value
        return -1 in dst or known_dst % max(known_src, 1) == 0 or known_src % max(known_dst, 1) == 0

    @classmethod
    def reshape(cls, src: SymbolicShape, dst: Sequence[int]) -> SymbolicShape:
        if not cls.can_reshape(src, dst):
            raise ShapeMismatchException("reshape", [src], f"cannot view {src} as {list(dst)}", ["use -1 for one target dimension"])
        dst = list(dst)
        n = cls.numel(src)
        if -1 in dst:
            if n is None:
                dst[dst.index(-1)] = SymbolicDimension("inferred")
            else:
                known = 1
                for d in dst:
                    if d != -1:
                        known *= d
                dst[dst.index(-1)] = n // known
        return SymbolicShape(dst)


# ------------------------------------------------------------------ lazily broadcast tensor
class BroadcastedTensor:
    """A tensor viewed at a broadcast shape without copying: stride 0 along every broadcast dimension."""

    def __init__(self, source: torch.Tensor, target_shape: Sequence[int]):
        target = tuple(int(d) for d in target_shape)
        src = tuple(source.shape)
        if len(src) > len(target):
            raise ShapeMismatchException("broadcast", [src, target], "source has more dimensions than the target")
        pad = (1,) * (len(target) - len(src)) + src
        for s, t in zip(pad, target):
            if s != t and s != 1:
                raise ShapeMismatchException("broadcast", [src, target], f"dimension of size {s} cannot become {t}",
                                             ["sizes must be equal, or 1 in the source"])
        self.source, self.target_shape, self._padded = source, target, pad

    @property
    def shape(self) -> Tuple[int, ...]:
        return self.target_shape

    def broadcast_sources(self) -> List[int]:
        """Target dimensions along which the source is repeated (including the leading dimensions it lacks)."""
        return [i for i, (s, t) in enumerate(zip(self._padded, self.target_shape)) if s == 1 and t != 1]

    def strides(self) -> Tuple[int, ...]:
        st = (0,) * (len(self.target_shape) - self.source.dim()) + tuple(self.source.stride())
        return tuple(0 if i in set(self.broadcast_sources()) else s for i, s in enumerate(st))

    def requires_materialization(self) -> bool:
        """False while a strided (zero-stride) view is enough; consumers that write in place or need contiguous memory
        must materialise."""
        return bool(self.broadcast_sources())

    def view(self) -> torch.Tensor:
        return self.source.expand(self.target_shape)

    def materialize(self) -> torch.Tensor:
        return self.view().contiguous()

    @property
    def expansion_factor(self) -> int:
        n = 1
        for d in self.target_shape:
            n *= d
        return n // max(self.source.numel(), 1)

    def __repr__(self):
        return f"BroadcastedTensor({tuple(self.source.shape)} -> {self.target_shape}, broadcast dims {self.broadcast_sources()})"


# ------------------------------------------------------------------ bindings, symbolic tensors
class DimensionBindings:
    """Values of named dimensions (``batch = 8``); shapes are instantiated against them."""

    def __init__(self, initial: Optional[Dict[str, int]] = None):
        self._b: Dict[str, int] = {}
        for k, v in (initial or {}).items():
            self.register_binding(k, v)

    def register_binding(self, name: str, value: int):
        if not name:
            raise ValueError("dimension name must not be empty")
        if value < 0:
            raise ValueError("a dimension cannot be negative")
        if name in self._b and self._b[name] != value:
            raise ValueError(f"dimension {name!r} is already bound to {self._b[name]}")
        self._b[name] = int(value)

    def get_binding(self, name: str) -> Optional[int]:
        return self._b.get(name)

    def has_binding(self, name: str) -> bool:
        return name in self._b

    def remove_binding(self, name: str) -> bool:
        return self._b.pop(name, None) is not None

    def clear_bindings(self):
        self._b.clear()

    def bound_names(self) -> List[str]:
        return sorted(self._b)

    def clone(self) -> "DimensionBindings":
        return DimensionBindings(dict(self._b))

    def merge_from(self, other: "DimensionBindings"):
        for k, v in other._b.items():
            self.register_binding(k, v)

    def as_dict(self) -> Dict[str, int]:
        return dict(self._b)

    def infer_from(self, shape: SymbolicShape, concrete: Sequence[int]):
        """Binds the shape's symbolic dimensions to the sizes of a concrete tensor (checking the known ones)."""
        if len(concrete) != shape.rank:
            raise ShapeMismatchException("bind", [shape, list(concrete)], "rank differs")
        for d, v in zip(shape, concrete):
            if d.is_known:
                if d.value != v:
                    raise ShapeMismatchException("bind", [shape, list(concrete)], f"dimension {d} is fixed, tensor has {v}")
            else:
                self.register_binding(d.name, v)

    def __repr__(self):
        return "DimensionBindings(" + ", ".join(f"{k}={v}" for k, v in sorted(self._b.items())) + ")"


class TensorFillType(enum.Enum):
    NONE = "none"
    ZEROS = "zeros"
    ONES = "ones"
    RANDOM = "random"


class SymbolicTensor:
    """A tensor known by its symbolic shape only; ``to_concrete`` instantiates it once the sizes are given."""

    def __init__(self, shape: SymbolicShape, fill: TensorFillType = TensorFillType.NONE, dtype: torch.dtype = torch.float32, name: str = ""):
        self.shape, self.fill, self.dtype, self.name = shape, fill, dtype, name

    def validate_shape(self) -> bool:
        return all((d.value is None or d.value >= 0) and (d.max_value is None or d.min_value <= d.max_value) for d in self.shape)

    def free_dimensions(self) -> List[str]:
        seen, out = set(), []
        for d in self.shape:
            if not d.is_known and d.name not in seen:
                seen.add(d.name)
                out.append(d.name)
        return out

    def concrete_shape(self, *values: int, bindings: Optional[DimensionBindings] = None) -> Tuple[int, ...]:
        """``values`` fill the free dimensions in order of first appearance; ``bindings`` fill them by name."""
        env = dict(bindings.as_dict()) if bindings is not None else {}
        free = [n for n in self.free_dimensions() if n not in env]
        if len(values) != len(free):
            raise ValueError(f"{len(free)} free dimensions {free}, {len(values)} values given")
        env.update(zip(free, values))
        return self.shape.bind(env).concrete()

    def can_instantiate_with(self, *dims: int) -> bool:
        if len(dims) != self.shape.rank:
            return False
        seen: Dict[str, int] = {}
        for d, v in zip(self.shape, dims):
            if d.is_known:
                if d.value != v:
                    return False
            else:
                if v < d.min_value or (d.max_value is not None and v > d.max_value) or seen.setdefault(d.name, v) != v:
                    return False
        return True

    def to_concrete(self, *values: int, bindings: Optional[DimensionBindings] = None, device="cpu", generator: Optional[torch.Generator] = None) -> torch.Tensor:
        shp = self.concrete_shape(*values, bindings=bindings)
        if self.fill == TensorFillType.ONES:
            return torch.ones(shp, dtype=self.dtype, device=device)
        if self.fill == TensorFillType.RANDOM:
            return torch.randn(shp, dtype=torch.float32, generator=generator).to(self.dtype).to(device)
        if self.fill == TensorFillType.ZEROS:
            return torch.zeros(shp, dtype=self.dtype, device=device)
        return torch.empty(shp, dtype=self.dtype, device=device)

    def __repr__(self):
        return f"SymbolicTensor({self.name or 'tensor'}: {self.shape}, {str(self.dtype).replace('torch.', '')})"


# ------------------------------------------------------------------ constraints
class ShapeConstraintBuilder:
    """Constraints for ONE named dimension, fluently: ``ShapeConstraintBuilder("seq").min(1).max(4096).modulo(8).build()``."""

    def __init__(self, name: str):
        self.name = name
        self._lo: Optional[int] = None
        self._hi: Optional[int] = None
        self._extra: List[Constraint] = []

    def min(self, v: int):
        if self._hi is not None and v > self._hi:
            raise ValueError("minimum above the maximum")
        self._lo = v
        return self

    def max(self, v: int):
        if self._lo is not None and v < self._lo:
            raise ValueError("maximum below the minimum")
        self._hi = v
        return self

    def range(self, lo: int, hi: int):
        if lo > hi:
            raise ValueError("empty range")
        self._lo, self._hi = lo, hi
        return self

    def equal(self, v: int):
        return self.range(v, v)

    def equal_to(self, other: str):
        self._extra.append(EqualityConstraint(self.name, other))
        return self

    def modulo(self, divisor: int, remainder: int = 0):
        if divisor <= 0:
            raise ValueError("divisor must be positive")
        self._extra.append(ModuloConstraint(self.name, divisor, remainder))
        return self

    def add_constraint(self, c: Constraint):
        self._extra.append(c)
        return self

    def build(self) -> List[Constraint]:
        out: List[Constraint] = []
        if self._lo is not None or self._hi is not None:
            out.append(RangeConstraint(self.name, self._lo if self._lo is not None else 0, self._hi if self._hi is not None else 2 ** 62))
        return out + list(self._extra)

    def reset(self):
        self._lo = self._hi = None
        self._extra.clear()
        return self


def describe_constraint(c: Constraint) -> str:
    if isinstance(c, RangeConstraint):
        return f"{c.lo} <= {c.name} <= {c.hi}"
    if isinstance(c, ModuloConstraint):
        return f"{c.name} % {c.modulus} == {c.remainder}"
    if isinstance(c, EqualityConstraint):
        return f"{c.a} == {c.b}"
    return repr(c)


class ConstraintValidator:
    """Checks dimension values against constraints; results per (value assignment, constraint set) are cached because
    serving validates the same few shapes over and over."""

    def __init__(self):
        self._cache: Dict[tuple, List[str]] = {}
        self.hits = self.misses = 0

    def violations(self, env: Dict[str, int], constraints: Sequence[Constraint]) -> List[str]:
        key = (tuple(sorted(env.items())), tuple(id(c) for c in constraints))
        if key in self._cache:
            self.hits += 1
            return list(self._cache[key])
        self.misses += 1
        out = [f"{describe_constraint(c)} violated by " + ", ".join(f"{k}={v}" for k, v in sorted(env.items()) if k in describe_constraint(c))
               for c in constraints if not c.check(env)]
        self._cache[key] = out
        return list(out)

    def validate_all(self, env: Dict[str, int], constraints: Sequence[Constraint]) -> bool:
        return not self.violations(env, constraints)

    def validate_dimension(self, dim: SymbolicDimension, constraints: Sequence[Constraint]) -> bool:
        return True if not dim.is_known else self.validate_all({dim.name: dim.value}, constraints)

    def validate_shape(self, shape: SymbolicShape, concrete: Sequence[int], constraints: Sequence[Constraint]) -> List[str]:
        b = DimensionBindings()
        b.infer_from(shape, concrete)
        return self.violations(b.as_dict(), constraints)

    def clear_cache(self):
        self._cache.clear()
        self.hits = self.misses = 0


# ------------------------------------------------------------------ inference context
class InferenceContext:
    """Shapes of named tensors and the results already inferred per operation id, for a pass that walks a graph once
    and is asked about the same values again later."""

    def __init__(self, initial: Optional[Dict[str, SymbolicShape]] = None):
        self._shapes: Dict[str, SymbolicShape] = dict(initial or {})
        self._results: Dict[str, List[SymbolicShape]] = {}

    def get_shape(self, name: str) -> Optional[SymbolicShape]:
        return self._shapes.get(name)

    def set_shape(self, name: str, shape: SymbolicShape):
        if not name:
            raise ValueError("tensor name must not be empty")
        self._shapes[name] = shape

    def has_shape(self, name: str) -> bool:
        return name in self._shapes

    def record_inference(self, op_id: str, outputs: Sequence[SymbolicShape]):
        self._results[op_id] = list(outputs)

    def get_operation_results(self, op_id: str) -> Optional[List[SymbolicShape]]:
        r = self._results.get(op_id)
        return None if r is None else list(r)

    def has_operation_results(self, op_id: str) -> bool:
        return op_id in self._results

    def clear_tensor_shapes(self):
        self._shapes.clear()

    def clear_operation_results(self):
        self._results.clear()

    def clear(self):
        self._shapes.clear()
        self._results.clear()

    def clone(self) -> "InferenceContext":
        c = InferenceContext(self._shapes)
        c._results = {k: list(v) for k, v in self._results.items()}
        return c

    def infer(self, engine, op_id: str, op: str, inputs: Sequence[str], output: str, **attrs) -> SymbolicShape:
        """Inference through ``engine`` with memoisation by ``op_id``; the result is stored under ``output``."""
        if op_id in self._results:
            return self._results[op_id][0]
        missing = [n for n in inputs if n not in self._shapes]
        if missing:
            raise KeyError(f"no shape recorded for {missing}")
        s = engine.infer(op, [self._shapes[n] for n in inputs], **attrs)
        self._results[op_id] = [s]
        self._shapes[output] = s
        return s
