"""Symbolic shapes, shape inference, broadcasting, constraints and shape-mismatch diagnostics.

Reference: src/MLFramework/Shapes/SymbolicDimension.cs, SymbolicShape.cs, Inference/ShapeInferenceEngine.cs:8
with rules Conv2D / ElementWise / MatMul / Reshape / Transpose, SymbolicBroadcastingEngine.cs, constraints
Equality / Modulo / Range, StaticShapeChecker.cs; diagnostics with fix suggestions from
src/RitterFramework.Core/Diagnostics/* and Exceptions/ShapeMismatchException.cs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union


@dataclass(frozen=True)
class SymbolicDimension:
    name: str
    value: Optional[int] = None
    min_value: int = 1
    max_value: Optional[int] = None

    @property
    def is_known(self) -> bool:
        return self.value is not None

    def with_value(self, v: int) -> "SymbolicDimension":
        if v < self.min_value or (self.max_value is not None and v > self.max_value):
            raise ValueError(f"{v} outside [{self.min_value}, {self.max_value}] for dimension {self.name}")
        return SymbolicDimension(self.name, v, self.min_value, self.max_value)

    def __str__(self):
        return str(self.value) if self.is_known else self.name


Dim = Union[int, SymbolicDimension]


def _d(x: Dim) -> SymbolicDimension:
    return x if isinstance(x, SymbolicDimension) else SymbolicDimension(str(x), int(x), int(x), int(x))


class SymbolicShape:
    def __init__(self, dims: Sequence[Dim]):
        self.dims: Tuple[SymbolicDimension, ...] = tuple(_d(d) for d in dims)

    @property
    def rank(self) -> int:
        return len(self.dims)

    @property
    def is_fully_known(self) -> bool:
        return all(d.is_known for d in self.dims)

    def concrete(self) -> Tuple[int, ...]:
        if not self.is_fully_known:
            raise ValueError(f"shape {self} has unknown dimensions")
        return tuple(d.value for d in self.dims)

    def bind(self, env: Dict[str, int]) -> "SymbolicShape":
        return SymbolicShape([d if d.is_known or d.name not in env else d.with_value(env[d.name]) for d in self.dims])

    def __iter__(self):
        return iter(self.dims)

    def __getitem__(self, i):
        return self.dims[i]

    def __eq__(self, o):
        return isinstance(o, SymbolicShape) and [str(d) for d in self.dims] == [str(d) for d in o.dims]

    def __repr__(self):
        return "[" + ", ".join(str(d) for d in self.dims) + "]"


# ---- constraints
class Constraint:
    def check(self, env: Dict[str, int]) -> bool:
        raise NotImplementedError


@dataclass
class EqualityConstraint(Constraint):
    a: str
    b: str

    def check(self, env):
        return self.a not in env or self.b not in env or env[self.a] == env[self.b]


@dataclass
class ModuloConstraint(Constraint):
    name: str
    modulus: int
    remainder: int = 0

    def check(self, env):
        return self.name not in env or env[self.name] % self.modulus == self.remainder


@dataclass
class RangeConstraint(Constraint):
    name: str
    lo: int
    hi: int

    def check(self, env):
        return self.name not in env or self.lo <= env[self.name] <= self.hi


class ShapeMismatchException(ValueError):
    def __init__(self, op: str, shapes: Sequence, message: str, suggestions: Sequence[str] = ()):
        self.op, self.shapes, self.suggestions = op, list(shapes), list(suggestions)
        text = f"{op}: {message}; inputs " + ", ".join(str(s) for s in shapes)
        if suggestions:
            text += "\n  suggestions:\n" + "\n".join(f"    - {s}" for s in suggestions)
        super().__init__(text)


def _same(a: SymbolicDimension, b: SymbolicDimension) -> bool:
    return (a.is_known and b.is_known and a.value == b.value) or (not a.is_known and not b.is_known and a.name == b.name)


def broadcast_shapes(a: SymbolicShape, b: SymbolicShape) -> SymbolicShape:
    out: List[SymbolicDimension] = []
    for i in range(1, max(a.rank, b.rank) + 1):
        da = a.dims[-i] if i <= a.rank else _d(1)
        db = b.dims[-i] if i <= b.rank else _d(1)
        if da.is_known and da.value == 1:
            out.append(db)
        elif db.is_known and db.value == 1:
            out.append(da)
        elif _same(da, db):
            out.append(da)
        elif not da.is_known or not db.is_known:
            out.append(da if da.is_known else db)      # assume the symbol equals the known extent
        else:
            raise ShapeMismatchException("broadcast", [a, b], f"dimension -{i}: {da} vs {db}",
                                         [f"reshape one operand so that dimension -{i} is 1 or {da}"])
    return SymbolicShape(list(reversed(out)))


class ShapeInferenceEngine:
    """Rule table op-name -> fn(input shapes, attrs) -> output shape; users may register more."""

    def __init__(self):
        self.rules: Dict[str, Callable[[Sequence[SymbolicShape], dict], SymbolicShape]] = {}
        for n in ("add", "sub", "mul", "div", "maximum", "minimum"):
            self.rules[n] = lambda s, a: broadcast_shapes(s[0], s[1])
        for n in ("relu", "gelu", "sigmoid", "tanh", "exp", "log", "sqrt", "neg", "cast", "softmax", "layer_norm", "rms_norm", "dropout", "batchnorm"):
            self.rules[n] = lambda s, a: s[0]
        self.rules["matmul"] = self._matmul
        self.rules["linear"] = self._linear
        self.rules["conv2d"] = self._conv2d
        self.rules["maxpool2d"] = self._pool
        self.rules["avgpool2d"] = self._pool
        self.rules["reshape"] = self._reshape
        self.rules["transpose"] = self._transpose
        self.rules["concat"] = self._concat
        self.rules["slice"] = self._slice
        self.rules["broadcast_to"] = lambda s, a: SymbolicShape(list(a["shape"]))
        self.rules["sum"] = self._reduce
        self.rules["mean"] = self._reduce
        self.rules["max"] = self._reduce

    def register(self, op: str, fn):
        self.rules[op] = fn

    def infer(self, op: str, shapes: Sequence[Union[SymbolicShape, Sequence[Dim]]], **attrs) -> SymbolicShape:
        if op not in self.rules:
            raise KeyError(f"no shape rule for op {op!r}")
        shapes = [s if isinstance(s, SymbolicShape) else SymbolicShape(s) for s in shapes]
        return self.rules[op](shapes, attrs)

    @staticmethod
    def _slice(s, a):
        """``starts`` / ``ends`` / optional ``steps`` per leading dimension (missing trailing dimensions are kept whole)."""
        x = s[0]
        starts, ends = list(a["starts"]), list(a["ends"])
        steps = list(a.get("steps", [1] * len(starts)))
        if not (len(starts) == len(ends) == len(steps)) or len(starts) > x.rank:
            raise ShapeMismatchException("slice", s, f"{len(starts)} starts, {len(ends)} ends, {len(steps)} steps for rank {x.rank}")
        dims: List[Dim] = []
        for i, d in enumerate(x.dims):
            if i >= len(starts):
                dims.append(d)
                continue
            if steps[i] <= 0:
                raise ShapeMismatchException("slice", s, f"step {steps[i]} of dimension {i} must be positive")
            if not d.is_known:
                dims.append(SymbolicDimension(f"slice({d.name})"))
                continue
            lo, hi, _ = slice(starts[i], ends[i], steps[i]).indices(d.value)
            dims.append(max(0, -(-(hi - lo) // steps[i])))
        return SymbolicShape(dims)

    @staticmethod
    def _matmul(s, a):
        x, y = s
        if x.rank < 2 or y.rank < 2:
            raise ShapeMismatchException("matmul", s, "operands must have rank >= 2")
        if x[-1].is_known and y[-2].is_known and x[-1].value != y[-2].value:
            sug = [f"transpose the second operand (its last dimension is {y[-1]})"] if y[-1].is_known and y[-1].value == x[-1].value else []
            sug.append(f"make the contraction sizes agree: {x[-1]} vs {y[-2]}")
            raise ShapeMismatchException("matmul", s, f"inner dimensions differ ({x[-1]} vs {y[-2]})", sug)
        batch = broadcast_shapes(SymbolicShape(x.dims[:-2]), SymbolicShape(y.dims[:-2]))
        return SymbolicShape(list(batch.dims) + [x[-2], y[-1]])

    @staticmethod
    def _linear(s, a):
        x, w = s[0], s[1]                                  # w: [out, in]
        if x[-1].is_known and w[1].is_known and x[-1].value != w[1].value:
            raise ShapeMismatchException("linear", s, f"input features {x[-1]} != weight in_features {w[1]}",
                                         [f"use a layer with in_features = {x[-1]}", f"project the input to {w[1]} features first"])
        return SymbolicShape(list(x.dims[:-1]) + [w[0]])

    @staticmethod
    def _out_hw(h: SymbolicDimension, k: int, stride: int, pad: int, dil: int = 1) -> Dim:
        if not h.is_known:
            return SymbolicDimension(f"({h.name}+{2 * pad - dil * (k - 1) - 1})//{stride}+1")
        return (h.value + 2 * pad - dil * (k - 1) - 1) // stride + 1

    @classmethod
    def _conv2d(cls, s, a):
        x, w = s[0], s[1]                                  # NCHW, [O, I/groups, kh, kw]
        g = a.get("groups", 1)
        if x[1].is_known and w[1].is_known and x[1].value != w[1].value * g:
            raise ShapeMismatchException("conv2d", s, f"input channels {x[1]} != weight channels {w[1]} x groups {g}",
                                         [f"use in_channels = {x[1]}"])
        st, pd, dl = a.get("stride", 1), a.get("padding", 0), a.get("dilation", 1)
        return SymbolicShape([x[0], w[0], cls._out_hw(x[2], w[2].value, st, pd, dl), cls._out_hw(x[3], w[3].value, st, pd, dl)])

    @classmethod
    def _pool(cls, s, a):
        x = s[0]
        k = a.get("kernel", 2)
        st, pd = a.get("stride", k), a.get("padding", 0)
        return SymbolicShape([x[0], x[1], cls._out_hw(x[2], k, st, pd), cls._out_hw(x[3], k, st, pd)])

    @staticmethod
    def _reshape(s, a):
        tgt = list(a["shape"])
        x = s[0]
        if x.is_fully_known:
            n = 1
            for d in x.concrete():
                n *= d
            known = 1
            for t in tgt:
                if t != -1:
                    known *= t
            if -1 in tgt:
                if known == 0 or n % known:
                    raise ShapeMismatchException("reshape", s, f"cannot infer -1: {n} elements into {tgt}")
                tgt[tgt.index(-1)] = n // known
            elif known != n:
                raise ShapeMismatchException("reshape", s, f"{n} elements do not fit {tgt} ({known} elements)",
                                             ["use -1 for one target dimension"])
        return SymbolicShape(tgt)

    @staticmethod
    def _transpose(s, a):
        d = list(s[0].dims)
        i, j = a.get("dim0", -2), a.get("dim1", -1)
        d[i], d[j] = d[j], d[i]
        return SymbolicShape(d)

    @staticmethod
    def _concat(s, a):
        ax = a.get("dim", 0)
        base = list(s[0].dims)
        tot = 0
        for x in s:
            if x.rank != len(base):
                raise ShapeMismatchException("concat", s, "ranks differ")
            for i, (p, q) in enumerate(zip(base, x.dims)):
                if i != ax % len(base) and p.is_known and q.is_known and p.value != q.value:
                    raise ShapeMismatchException("concat", s, f"dimension {i} differs ({p} vs {q})")
            tot = tot + x[ax].value if x[ax].is_known and tot is not None else None
        base[ax] = _d(tot) if tot is not None else SymbolicDimension("concat")
        return SymbolicShape(base)

    @staticmethod
    def _reduce(s, a):
        d = list(s[0].dims)
        if "dim" not in a:
            return SymbolicShape([])
        axes = sorted({ax % len(d) for ax in ((a["dim"],) if isinstance(a["dim"], int) else a["dim"])}, reverse=True)
        for ax in axes:                                    # from the back, so that earlier positions stay valid
            if a.get("keepdim", False):
                d[ax] = _d(1)
            else:
                d.pop(ax)
        return SymbolicShape(d)


class StaticShapeChecker:
    """Walks a list of (op, input names, output name, attrs) and reports every mismatch with the op index."""

    def __init__(self, engine: Optional[ShapeInferenceEngine] = None, constraints: Sequence[Constraint] = ()):
        self.engine, self.constraints = engine or ShapeInferenceEngine(), list(constraints)

    def check(self, inputs: Dict[str, SymbolicShape], program: Sequence[Tuple[str, Sequence[str], str, dict]],
              env: Optional[Dict[str, int]] = None) -> Tuple[Dict[str, SymbolicShape], List[str]]:
        env = env or {}
        errors = [f"constraint violated: {c}" for c in self.constraints if not c.check(env)]
        shapes = {k: (v if isinstance(v, SymbolicShape) else SymbolicShape(v)).bind(env) for k, v in inputs.items()}
        for i, (op, ins, out, attrs) in enumerate(program):
            try:
                shapes[out] = self.engine.infer(op, [shapes[n] for n in ins], **attrs)
            except (ShapeMismatchException, KeyError) as e:
                errors.append(f"op #{i} ({op}): {e}")
                break
        return shapes, errors


class ShapeReportFormatter:
    @staticmethod
    def text(e: ShapeMismatchException) -> str:
        return str(e)

    @staticmethod
    def json(e: ShapeMismatchException) -> str:
        import json
        return json.dumps({"operation": e.op, "shapes": [str(s) for s in e.shapes], "suggestions": e.suggestions})

    @staticmethod
    def html(e: ShapeMismatchException) -> str:
        items = "".join(f"<li>{s}</li>" for s in e.suggestions)
        return f"<div class='shape-error'><b>{e.op}</b>: {', '.join(str(s) for s in e.shapes)}<ul>{items}</ul></div>"
