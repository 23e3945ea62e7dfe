"""Per-operation shape diagnostics and the error-reporting service.

Reference: ``IOperationDiagnosticsHandler`` (validate / error message / suggestions / detected issues) with handlers for
matrix multiply, conv1d, conv2d, concat and pooling, a registry keyed by operation type, and ``ErrorReportingService``
(capture the executing operation's context, build a ``ShapeMismatchException`` from it, keep a log)
(src/RitterFramework.Core/Diagnostics/IOperationDiagnosticsHandler.cs, MatrixMultiplyDiagnosticsHandler.cs,
Conv2DDiagnosticsHandler.cs, ConcatDiagnosticsHandler.cs, PoolingDiagnosticsHandler.cs,
OperationDiagnosticsRegistry.cs, ErrorReportingService.cs:20-130, ValidationResult.cs).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .shapes import ShapeMismatchException, ShapeReportFormatter


@dataclass
class ValidationResult:
    is_valid: bool
    message: str = ""

    @classmethod
    def success(cls):
        return cls(True)

    @classmethod
    def failure(cls, msg: str):
        return cls(False, msg)


class OperationDiagnosticsHandler:
    op = "op"

    def validate(self, shapes: Sequence[Sequence[int]], params: Dict) -> ValidationResult:
        return ValidationResult.success()

    def generate_suggestions(self, shapes, params) -> List[str]:
        return []

    def detect_issues(self, shapes, params) -> List[str]:
        return []

    def generate_error_message(self, shapes, params, layer_name: str = "") -> str:
        r = self.validate(shapes, params)
        where = f" in layer '{layer_name}'" if layer_name else ""
        return f"{self.op}{where}: {r.message or 'shapes are valid'}; inputs " + ", ".join(str(list(s)) for s in shapes)


class MatMulDiagnosticsHandler(OperationDiagnosticsHandler):
    op = "matmul"

    def validate(self, shapes, params):
        if len(shapes) != 2:
            return ValidationResult.failure("matrix multiplication requires exactly 2 input tensors")
        a, b = list(shapes[0]), list(shapes[1])
        if len(a) < 2 or len(b) < 2:
            return ValidationResult.failure("both tensors must have at least 2 dimensions")
        if a[-1] != b[-2]:
            return ValidationResult.failure(f"inner dimensions mismatch: {a[-1]} != {b[-2]}")
        if len(a) == len(b) and len(a) > 2:
            for i in range(len(a) - 2):
                if a[i] != b[i] and 1 not in (a[i], b[i]):
                    return ValidationResult.failure(f"batch dimension {i} mismatch: {a[i]} != {b[i]}")
        return ValidationResult.success()

    def generate_suggestions(self, shapes, params):
        if len(shapes) != 2 or len(shapes[0]) < 2 or len(shapes[1]) < 2:
            return ["pass two tensors of rank 2 or more"]
        a, b = list(shapes[0]), list(shapes[1])
        out = []
        if a[-1] != b[-2]:
            if a[-1] == b[-1]:
                out.append(f"transpose the second operand: {b} -> {b[:-2] + [b[-1], b[-2]]} (a linear layer stores its weight as [out, in])")
            if a[-2] == b[-2]:
                out.append(f"transpose the first operand: {a} -> {a[:-2] + [a[-1], a[-2]]}")
            out.append(f"make the contraction sizes equal: the first operand's last dimension ({a[-1]}) must equal the second's "
                       f"second-to-last ({b[-2]})")
        return out

    def detect_issues(self, shapes, params):
        out = []
        if len(shapes) == 2 and len(shapes[0]) >= 2 and len(shapes[1]) >= 2:
            k = shapes[0][-1]
            if k % 8:
                out.append(f"contraction size {k} is not a multiple of 8: the tensor-core path needs 16-byte rows (pad to {(k + 7) // 8 * 8})")
            if shapes[1][-1] % 8:
                out.append(f"output width {shapes[1][-1]} is not a multiple of 8: stores fall back to narrow writes")
        return out


class _ConvHandler(OperationDiagnosticsHandler):
    nd = 2

    def validate(self, shapes, params):
        if len(shapes) < 2:
            return ValidationResult.failure("convolution needs an input and a weight")
        x, w = list(shapes[0]), list(shapes[1])
        if len(x) != self.nd + 2 or len(w) != self.nd + 2:
            return ValidationResult.failure(f"input and weight must have rank {self.nd + 2} (batch, channels, spatial...)")
        groups = int(params.get("groups", 1))
        if x[1] != w[1] * groups:
            return ValidationResult.failure(f"input has {x[1]} channels, weight expects {w[1] * groups} (in_channels / groups = {w[1]}, groups = {groups})")
        pad, dil, stride = self._t(params.get("padding", 0)), self._t(params.get("dilation", 1)), self._t(params.get("stride", 1))
        for i in range(self.nd):
            eff = dil[i] * (w[2 + i] - 1) + 1
            if x[2 + i] + 2 * pad[i] < eff:
                return ValidationResult.failure(f"kernel extent {eff} exceeds the padded input size {x[2 + i] + 2 * pad[i]} in spatial dimension {i}")
            if stride[i] <= 0:
                return ValidationResult.failure("stride must be positive")
        return ValidationResult.success()

    def _t(self, v):
        return tuple(v) if isinstance(v, (tuple, list)) else (int(v),) * self.nd

    def generate_suggestions(self, shapes, params):
        out = []
        if len(shapes) >= 2 and len(shapes[0]) == self.nd + 2 and len(shapes[1]) == self.nd + 2:
            x, w = shapes[0], shapes[1]
            if x[1] != w[1] * int(params.get("groups", 1)):
                if x[-1] == w[1]:
                    out.append("the input looks channels-last: permute it to (batch, channels, spatial...)")
                out.append(f"build the layer with in_channels = {x[1]}")
            pad = self._t(params.get("padding", 0))
            if any(x[2 + i] + 2 * pad[i] < w[2 + i] for i in range(self.nd)):
                out.append("add padding or use a smaller kernel")
        return out


class Conv2DDiagnosticsHandler(_ConvHandler):
    op, nd = "conv2d", 2


class Conv1DDiagnosticsHandler(_ConvHandler):
    op, nd = "conv1d", 1


class ConcatDiagnosticsHandler(OperationDiagnosticsHandler):
    op = "concat"

    def validate(self, shapes, params):
        if not shapes:
            return ValidationResult.failure("concat needs at least one tensor")
        rank = len(shapes[0])
        dim = int(params.get("dim", 0)) % max(rank, 1)
        for i, s in enumerate(shapes[1:], 1):
            if len(s) != rank:
                return ValidationResult.failure(f"tensor {i} has rank {len(s)}, tensor 0 has rank {rank}")
            for d in range(rank):
                if d != dim and s[d] != shapes[0][d]:
                    return ValidationResult.failure(f"tensor {i} has size {s[d]} in dimension {d}, tensor 0 has {shapes[0][d]} (only dimension {dim} may differ)")
        return ValidationResult.success()

    def generate_suggestions(self, shapes, params):
        r = self.validate(shapes, params)
        if r.is_valid:
            return []
        out = ["all tensors must agree in every dimension except the concatenation dimension"]
        if len({len(s) for s in shapes}) == 1:
            rank = len(shapes[0])
            ok = [d for d in range(rank) if all(all(s[e] == shapes[0][e] for e in range(rank) if e != d) for s in shapes)]
            if ok:
                out.append(f"concatenating along dimension {ok[0]} would work for these shapes")
        return out


class PoolingDiagnosticsHandler(OperationDiagnosticsHandler):
    op = "pool2d"

    def validate(self, shapes, params):
        if len(shapes) != 1 or len(shapes[0]) != 4:
            return ValidationResult.failure("pooling takes one tensor of rank 4 (batch, channels, height, width)")
        k = params.get("kernel", 2)
        k = tuple(k) if isinstance(k, (tuple, list)) else (int(k), int(k))
        p = params.get("padding", 0)
        p = tuple(p) if isinstance(p, (tuple, list)) else (int(p), int(p))
        for i in range(2):
            if shapes[0][2 + i] + 2 * p[i] < k[i]:
                return ValidationResult.failure(f"window {k[i]} exceeds the padded input size {shapes[0][2 + i] + 2 * p[i]} in spatial dimension {i}")
            if p[i] > k[i] // 2:
                return ValidationResult.failure(f"padding {p[i]} is larger than half the window {k[i]}")
        return ValidationResult.success()

    def generate_suggestions(self, shapes, params):
        return [] if self.validate(shapes, params).is_valid else ["use a smaller window, add padding, or pool fewer times before this layer"]


class OperationDiagnosticsRegistry:
    def __init__(self, defaults: bool = True):
        self._h: Dict[str, OperationDiagnosticsHandler] = {}
        if defaults:
            for h in (MatMulDiagnosticsHandler(), Conv2DDiagnosticsHandler(), Conv1DDiagnosticsHandler(), ConcatDiagnosticsHandler(),
                      PoolingDiagnosticsHandler()):
                self.register(h.op, h)
            self._h["linear"] = self._h["matmul"]
            self._h["maxpool2d"] = self._h["avgpool2d"] = self._h["pool2d"]

    def register(self, op: str, handler: OperationDiagnosticsHandler):
        self._h[op] = handler

    def get_handler(self, op: str) -> Optional[OperationDiagnosticsHandler]:
        return self._h.get(op)

    def has_handler(self, op: str) -> bool:
        return op in self._h


@dataclass
class OperationExecutionContext:
    op: str
    layer_name: str = ""
    input_shapes: List[Sequence[int]] = field(default_factory=list)
    parameters: Dict = field(default_factory=dict)
    previous_layer: str = ""


class ErrorReportingService:
    """Keeps the context of the operation being executed (per thread) and turns a failure into a
    ``ShapeMismatchException`` carrying the handler's message, detected issues and fix suggestions; every report is
    also appended to a bounded log with counts per operation."""

    def __init__(self, registry: Optional[OperationDiagnosticsRegistry] = None, max_log: int = 1000):
        self.registry = registry or OperationDiagnosticsRegistry()
        self._ctx = threading.local()
        self.log: List[Dict] = []
        self.max_log = max_log
        self.counts: Dict[str, int] = {}

    def capture_context(self, ctx: OperationExecutionContext):
        self._ctx.c = ctx

    def get_current_context(self) -> Optional[OperationExecutionContext]:
        return getattr(self._ctx, "c", None)

    def clear_context(self):
        self._ctx.c = None

    def validate_current(self) -> ValidationResult:
        c = self.get_current_context()
        h = self.registry.get_handler(c.op) if c else None
        return h.validate(c.input_shapes, c.parameters) if h else ValidationResult.success()

    def generate_shape_mismatch_exception(self, problem: str = "") -> ShapeMismatchException:
        c = self.get_current_context()
        if c is None:
            return ShapeMismatchException("unknown", [], problem or "shape mismatch outside any captured operation")
        h = self.registry.get_handler(c.op)
        msg, sugg = problem, []
        if h is not None:
            r = h.validate(c.input_shapes, c.parameters)
            msg = problem or r.message or "shape mismatch"
            sugg = h.generate_suggestions(c.input_shapes, c.parameters) + h.detect_issues(c.input_shapes, c.parameters)
        if c.layer_name:
            msg = f"layer '{c.layer_name}'" + (f" (after '{c.previous_layer}')" if c.previous_layer else "") + f": {msg}"
        e = ShapeMismatchException(c.op, [tuple(s) for s in c.input_shapes], msg or "shape mismatch", sugg)
        self.log_shape_mismatch(c.op, c.input_shapes, msg)
        return e

    def log_shape_mismatch(self, op: str, shapes, message: str):
        self.counts[op] = self.counts.get(op, 0) + 1
        self.log.append({"time": time.time(), "operation": op, "shapes": [list(s) for s in shapes], "message": message})
        if len(self.log) > self.max_log:
            del self.log[: len(self.log) - self.max_log]

    def check(self, op: str, shapes, layer_name: str = "", **params):
        """Validate an operation before running it; raises the full report when the shapes cannot work."""
        self.capture_context(OperationExecutionContext(op, layer_name, [list(s) for s in shapes], params))
        try:
            if not self.validate_current().is_valid:
                raise self.generate_shape_mismatch_exception()
        finally:
            self.clear_context()

    def report(self, e: ShapeMismatchException, fmt: str = "text") -> str:
        return {"text": ShapeReportFormatter.text, "json": ShapeReportFormatter.json, "html": ShapeReportFormatter.html}[fmt](e)
