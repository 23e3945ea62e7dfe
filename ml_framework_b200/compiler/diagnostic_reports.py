"""Shape-error reporting: per-operation formatters, report generator, fix suggestions,
declarative shape requirements and a small operation graph for whole-model checks.

Reference: src/MLFramework/Diagnostics/{IDiagnosticFormatter.cs, DiagnosticFormatterRegistry.cs,
MatrixMultiplyDiagnosticFormatter.cs, Conv2DDiagnosticFormatter.cs, ConcatDiagnosticFormatter.cs,
BroadcastDiagnosticFormatter.cs, ErrorReportGenerator.cs:8-258} and
src/RitterFramework.Core/Diagnostics/{FixSuggestionGenerator.cs:8-354, SuggestionTemplates.cs,
ShapeDiagnosticsInfo.cs:8-141, DimensionConstraint.cs, OperationShapeRequirements.cs,
DefaultOperationMetadataRegistry.cs, ComputationGraph.cs:7-116, OperationNode.cs,
DefaultShapeInferenceEngine.cs}.

The formatters explain one failed (or passed) check in words; the generator lays a
``ShapeMismatchException`` out as text, Markdown or HTML; the suggestion generator looks for the
usual causes (a missing batch axis, NHWC against NCHW, a transposed operand, feature counts of
adjacent layers); requirements state an operation's shape rules as data; the graph runs the
rules over a model description and says where the first mismatch sits.
"""
from __future__ import annotations

import enum
import html as _html
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .diagnostics import ValidationResult
from .shapes import ShapeMismatchException

__all__ = [
    "OperationType", "DiagnosticFormatter", "MatrixMultiplyDiagnosticFormatter", "Conv2DDiagnosticFormatter",
    "ConcatDiagnosticFormatter", "BroadcastDiagnosticFormatter", "DiagnosticFormatterRegistry", "ErrorReportFormat",
    "ErrorReportGenerator", "SuggestionTemplates", "FixSuggestionGenerator", "ConstraintType", "DimensionConstraint",
    "OperationShapeRequirements", "OperationMetadataRegistry", "ShapeDiagnosticsInfo", "OperationNode",
    "ComputationGraph", "GraphShapeInference",
]

Shape = Sequence[int]


class OperationType(enum.Enum):
    MATRIX_MULTIPLY = "matmul"
    LINEAR = "linear"
    CONV2D = "conv2d"
    CONV1D = "conv1d"
    CONCAT = "concat"
    BROADCAST = "broadcast"
    POOLING = "pooling"
    RESHAPE = "reshape"
    TRANSPOSE = "transpose"
    ELEMENTWISE = "elementwise"
    INPUT = "input"


def _fmt(shape: Shape) -> str:
    return "[" + ", ".join(str(int(d)) if isinstance(d, (int,)) or str(d).lstrip("-").isdigit() else str(d) for d in shape) + "]"


def _pad(shape: Shape, n: int) -> List[int]:
    return [1] * (n - len(shape)) + list(shape)


# ------------------------------------------------------------------ formatters
class DiagnosticFormatter:
    supported_operation: OperationType = OperationType.ELEMENTWISE

    def format_error(self, result: ValidationResult, *input_shapes: Shape) -> str:
        raise NotImplementedError

    def generate_suggestions(self, result: ValidationResult) -> List[str]:
        return []


class MatrixMultiplyDiagnosticFormatter(DiagnosticFormatter):
    supported_operation = OperationType.MATRIX_MULTIPLY

    def format_error(self, result, *input_shapes):
        if len(input_shapes) < 2:
            return f"Matrix multiplication: insufficient input shapes provided. {result.message}"
        a, b = input_shapes[0], input_shapes[1]
        msg = f"Matrix multiplication: shape {_fmt(a)} x {_fmt(b)} invalid\n"
        if len(a) >= 1 and len(b) >= 2 and a[-1] != b[-2]:
            return msg + f"Problem: inner dimensions {a[-1]} and {b[-2]} must match"
        return msg + f"Problem: {result.message}"

    def generate_suggestions(self, result):
        out = ["Check layer configurations: the output features of the previous layer must equal the input features of this one",
               "Verify tensor shapes before the matrix multiplication",
               "Consider transposing one of the matrices if its dimensions are swapped"]
        nums = [w for w in (result.message or "").replace(",", " ").split() if w.isdigit()]
        if len(nums) >= 2 and nums[0] != nums[1]:
            out.append(f"Previous layer outputs {nums[0]} features, but this layer expects {nums[1]}: adjust one of them")
        return out


class Conv2DDiagnosticFormatter(DiagnosticFormatter):
    supported_operation = OperationType.CONV2D

    def format_error(self, result, *input_shapes):
        if len(input_shapes) < 2:
            return f"Conv2D: insufficient input shapes provided. {result.message}"
        x, k = input_shapes[0], input_shapes[1]
        msg = f"Conv2D: input {_fmt(x)} with kernel {_fmt(k)}\n"
        if len(x) == 4 and len(k) == 4:
            if x[1] == k[1]:
                msg += f"Status: input channels ({x[1]}) match kernel channels ({k[1]})\n"
                oh, ow = x[2] - k[2] + 1, x[3] - k[3] + 1
                if oh > 0 and ow > 0 and result.is_valid:
                    return msg + f"Output shape (stride 1, no padding): [{x[0]}, {k[0]}, {oh}, {ow}]"
                if oh <= 0 or ow <= 0:
                    return msg + f"Problem: kernel {k[2]}x{k[3]} is larger than the input {x[2]}x{x[3]}"
                return msg + f"Problem: {result.message}"
            return msg + f"Problem: input channels ({x[1]}) do not match kernel channels ({k[1]})"
        return msg + f"Problem: {result.message}"

    def generate_suggestions(self, result):
        out = ["Check channel configurations: input channels must match kernel in-channels",
               "Verify kernel parameters (out-channels, in-channels, height, width)",
               "Ensure the input tensor is NCHW: [batch, channels, height, width]",
               "Check padding and stride settings if the output shape is wrong"]
        m = (result.message or "").lower()
        if "channel" in m:
            out.append("Adjust either the input tensor's channels or the kernel's in-channels so that they match")
        if "shape" in m or "larger" in m:
            out.append("Verify that the input's spatial size is compatible with the kernel size")
        return out


class ConcatDiagnosticFormatter(DiagnosticFormatter):
    supported_operation = OperationType.CONCAT

    @staticmethod
    def compatible_axis(a: Shape, b: Shape) -> Optional[int]:
        """The single axis on which the shapes may differ (0 when they are equal); ``None`` if there is none."""
        if len(a) != len(b):
            return None
        diff = [i for i, (x, y) in enumerate(zip(a, b)) if x != y]
        return 0 if not diff else (diff[0] if len(diff) == 1 else None)

    def format_error(self, result, *input_shapes):
        if len(input_shapes) < 2:
            return f"Concat: insufficient input shapes provided. {result.message}"
        a, b = input_shapes[0], input_shapes[1]
        msg = f"Concat: {_fmt(a)} + {_fmt(b)}\n"
        ax = self.compatible_axis(a, b)
        if ax is not None and result.is_valid:
            out = list(a)
            out[ax] = a[ax] + b[ax]
            return msg + f"Valid: all dimensions match except on axis {ax}\nOutput shape: {_fmt(out)}"
        if ax is not None:
            return msg + f"Problem: {result.message} (the shapes could be joined on axis {ax})"
        return msg + f"Problem: {result.message}"

    def generate_suggestions(self, result):
        out = ["Check tensor shapes: all dimensions must match except the concatenation axis",
               "Consider reshaping the tensors to compatible dimensions before concatenating",
               "Verify that the right concatenation axis is given"]
        m = (result.message or "").lower()
        if "axis" in m:
            out.append("Try another axis, or reshape the inputs so that the other dimensions agree")
        if "dimension" in m:
            out.append("Batch sizes and the other non-concatenated dimensions must be identical")
        return out


class BroadcastDiagnosticFormatter(DiagnosticFormatter):
    supported_operation = OperationType.BROADCAST

    @staticmethod
    def problematic_dimension(a: Shape, b: Shape) -> Optional[int]:
        n = max(len(a), len(b))
        for i, (x, y) in enumerate(zip(_pad(a, n), _pad(b, n))):
            if x != y and x != 1 and y != 1:
                return i
        return None

    def format_error(self, result, *input_shapes):
        if len(input_shapes) < 2:
            return f"Broadcast: insufficient input shapes provided. {result.message}"
        a, b = input_shapes[0], input_shapes[1]
        msg = f"Broadcast: {_fmt(a)} -> {_fmt(b)}\n"
        bad = self.problematic_dimension(a, b)
        if bad is None:
            return msg + "Valid: the shapes are compatible for broadcasting"
        n = max(len(a), len(b))
        return msg + (f"Problem: cannot broadcast dimension {bad} ({_pad(a, n)[bad]} against {_pad(b, n)[bad]}): "
                      "sizes must be equal or one of them 1")

    def generate_suggestions(self, result):
        out = ["Check the broadcasting rule: aligned from the right, dimensions must be equal or one of them 1",
               "Consider an explicit reshape or expand instead of relying on broadcasting",
               "Verify that the smaller tensor can be broadcast to the larger tensor's shape"]
        m = (result.message or "").lower()
        if "dimension" in m:
            out.append("Make the offending dimensions equal, or one of them 1")
        if "batch" in m:
            out.append("Batch sizes must match or one must be 1")
        return out


class DiagnosticFormatterRegistry:
    """Formatter per operation type, with a generic fall-back (DiagnosticFormatterRegistry.cs)."""

    _instance: Optional["DiagnosticFormatterRegistry"] = None

    def __init__(self, defaults: bool = True):
        self._f: Dict[OperationType, DiagnosticFormatter] = {}
        if defaults:
            for f in (MatrixMultiplyDiagnosticFormatter(), Conv2DDiagnosticFormatter(), ConcatDiagnosticFormatter(),
                      BroadcastDiagnosticFormatter()):
                self.register(f)

    @classmethod
    def instance(cls) -> "DiagnosticFormatterRegistry":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def register(self, formatter: DiagnosticFormatter) -> None:
        if formatter is None:
            raise ValueError("the formatter is required")
        self._f[formatter.supported_operation] = formatter

    def get(self, type: OperationType) -> Optional[DiagnosticFormatter]:
        return self._f.get(type)

    def format_error(self, type: OperationType, result: ValidationResult, *input_shapes: Shape) -> str:
        f = self._f.get(type)
        if f is not None:
            return f.format_error(result, *input_shapes)
        shapes = ", ".join(_fmt(s) for s in input_shapes) if input_shapes else "N/A"
        return f"{type.value}: validation failed for input shapes {shapes}. {result.message}"

    def get_suggestions(self, type: OperationType, result: ValidationResult) -> List[str]:
        f = self._f.get(type)
        return f.generate_suggestions(result) if f is not None else []


# ------------------------------------------------------------------ report generator
class ErrorReportFormat(enum.Enum):
    TEXT = "text"
    MARKDOWN = "markdown"
    HTML = "html"


class ErrorReportGenerator:
    """Lays a ``ShapeMismatchException`` out for a terminal, a ticket or a page."""

    LINE = 64

    @staticmethod
    def _parts(e: ShapeMismatchException):
        expected = list(getattr(e, "expected_shapes", ()) or ())
        details = getattr(e, "details", "") or ""
        first = str(e).split("\n", 1)[0]
        problem = first.split("; inputs ")[0]
        problem = problem[len(e.op) + 2:] if problem.startswith(e.op + ": ") else problem
        return expected, details, problem

    @classmethod
    def generate_report(cls, e: ShapeMismatchException, format: ErrorReportFormat = ErrorReportFormat.TEXT) -> str:
        if e is None:
            raise ValueError("the exception is required")
        if format is ErrorReportFormat.TEXT:
            return cls._text(e)
        if format is ErrorReportFormat.MARKDOWN:
            return cls._markdown(e)
        if format is ErrorReportFormat.HTML:
            return cls._html(e)
        raise ValueError(f"unsupported report format {format!r}")

    @classmethod
    def _text(cls, e):
        expected, details, problem = cls._parts(e)
        bar = "=" * cls.LINE
        out = [bar, "Shape mismatch", bar, "", f"Operation: {e.op}", ""]
        if e.shapes:
            out += ["INPUT SHAPES:"] + [f"  Tensor {i + 1}: {_fmt(s)}" for i, s in enumerate(e.shapes)] + [""]
        if expected:
            out += ["EXPECTED SHAPES:"] + [f"  Tensor {i + 1}: {_fmt(s)}" for i, s in enumerate(expected)] + [""]
        out += ["PROBLEM:", f"  {problem}", ""]
        if details:
            out += ["CONTEXT:", f"  {details}", ""]
        if e.suggestions:
            out += ["SUGGESTED FIXES:"] + [f"  {i + 1}. {s}" for i, s in enumerate(e.suggestions)] + [""]
        return "\n".join(out + [bar]) + "\n"

    @classmethod
    def _markdown(cls, e):
        expected, details, problem = cls._parts(e)
        out = ["# Shape mismatch", "", "## Operation", e.op, ""]
        if e.shapes:
            out += ["### Input shapes"] + [f"- Tensor {i + 1}: `{_fmt(s)}`" for i, s in enumerate(e.shapes)] + [""]
        if expected:
            out += ["### Expected shapes"] + [f"- Tensor {i + 1}: `{_fmt(s)}`" for i, s in enumerate(expected)] + [""]
        out += ["## Problem", problem, ""]
        if details:
            out += ["### Context", details, ""]
        if e.suggestions:
            out += ["## Suggested fixes"] + [f"{i + 1}. {s}" for i, s in enumerate(e.suggestions)] + [""]
        return "\n".join(out)

    @classmethod
    def _html(cls, e):
        expected, details, problem = cls._parts(e)
        esc = _html.escape

        def shapes(title, rows):
            if not rows:
                return ""
            body = "".join(f'<div class="shape">Tensor {i + 1}: {esc(_fmt(s))}</div>' for i, s in enumerate(rows))
            return f'<div class="section"><span class="label">{title}:</span><br>{body}</div>'
        fixes = ""
        if e.suggestions:
            fixes = ('<div class="section"><span class="label">Suggested fixes:</span><ol>'
                     + "".join(f"<li>{esc(s)}</li>" for s in e.suggestions) + "</ol></div>")
        ctx = f'<div class="section"><span class="label">Context:</span><br>{esc(details)}</div>' if details else ""
        return ("<!DOCTYPE html><html><head><style>.error-report{font-family:monospace;padding:20px;background:#ffeeee;margin:20px}"
                ".header{font-size:18px;font-weight:bold;margin-bottom:10px}.section{margin:10px 0}"
                ".shape{background:#ffffee;padding:5px;margin:2px 0}.problem{color:red;font-weight:bold}.label{font-weight:bold}"
                '</style></head><body><div class="error-report"><div class="header">Shape mismatch</div>'
                f'<div class="section"><span class="label">Operation:</span> {esc(e.op)}</div>'
                + shapes("Input shapes", e.shapes) + shapes("Expected shapes", expected)
                + f'<div class="section"><span class="label">Problem:</span><br><span class="problem">{esc(problem)}</span></div>'
                + ctx + fixes + "</div></body></html>")


# ------------------------------------------------------------------ fix suggestions
class SuggestionTemplates:
    MISSING_BATCH_DIM = "Input missing batch dimension. Add unsqueeze(0) or reshape to [1, {0}]"
    CHANNEL_ORDER_MISMATCH = "Channel order mismatch. Permute from {0} to {1}"
    FEATURE_SIZE_MISMATCH = "Previous layer outputs {0} features, but this layer expects {1}. Adjust layer configuration"
    TRANSPOSE_REQUIRED = "Consider transposing {0} to {1}"
    CONCATENATION_DIMENSION_MISMATCH = "Cannot concatenate on axis {0} with different sizes. Use axis {1} or reshape inputs"
    BROADCASTING_FAILURE = "Cannot broadcast shapes {0} and {1}. Batch sizes must match or be 1"
    GENERIC_SHAPE_MISMATCH = "Shape mismatch for {0}: {1} vs expected {2}"
    RESHAPE_SUGGESTION = "Try reshaping from {0} to {1}"
    SQUEEZE_SUGGESTION = "Consider squeezing dimension {0} to remove size-1 dimension"
    UNSQUEEZE_SUGGESTION = "Consider unsqueezing at dimension {0} to add size-1 dimension"


def _numel(s: Shape) -> int:
    n = 1
    for d in s:
        n *= int(d)
    return n


class FixSuggestionGenerator:
    """Recognises the usual causes of a shape error from the shapes alone (FixSuggestionGenerator.cs:17-354)."""

    def generate_suggestions(self, operation_type: OperationType, input_shapes: Sequence[Shape],
                             expected_shapes: Optional[Sequence[Shape]] = None) -> List[str]:
        if not input_shapes:
            return []
        exp = list(expected_shapes or [])
        T = OperationType
        by_type: Dict[OperationType, Callable] = {
            T.LINEAR: self._linear, T.CONV2D: self._conv2d, T.CONCAT: lambda i, e: self._concat(i),
            T.BROADCAST: lambda i, e: self._broadcast(i), T.MATRIX_MULTIPLY: self._matmul}
        out = by_type.get(operation_type, self._generic)(list(input_shapes), exp)
        out += self._common(list(input_shapes), exp)
        seen, uniq = set(), []
        for s in out:
            if s not in seen:
                seen.add(s)
                uniq.append(s)
        return uniq

    def _linear(self, ins, exp):
        out = []
        x = ins[0]
        if len(ins) >= 2 and len(ins[1]) == 2:              # weight [out_features, in_features]
            w = ins[1]
            if x[-1] != w[1]:
                out.append(SuggestionTemplates.FEATURE_SIZE_MISMATCH.format(x[-1], w[1]))
                if x[-1] == w[0]:
                    out.append(SuggestionTemplates.TRANSPOSE_REQUIRED.format(_fmt(w), _fmt(w[::-1])))
                if len(x) > 2 and _numel(x[1:]) == w[1]:
                    out.append(SuggestionTemplates.RESHAPE_SUGGESTION.format(_fmt(x), _fmt([x[0], w[1]])))
        elif exp and x[-1] != exp[0][-1]:
            out.append(SuggestionTemplates.FEATURE_SIZE_MISMATCH.format(x[-1], exp[0][-1]))
        return out

    @staticmethod
    def is_channel_order_mismatch(a: Shape, b: Shape) -> bool:
        """One shape is the NHWC reading of the other's NCHW."""
        if len(a) != 4 or len(b) != 4:
            return False
        return (a[1] == b[2] and a[2] == b[3] and a[3] == b[1]) or (b[1] == a[2] and b[2] == a[3] and b[3] == a[1])

    def _conv2d(self, ins, exp):
        out = []
        x = ins[0]
        if len(x) == 3:
            out.append(SuggestionTemplates.MISSING_BATCH_DIM.format(", ".join(map(str, x))))
        if len(ins) >= 2 and len(x) == 4 and len(ins[1]) == 4:
            k = ins[1]
            if x[1] != k[1] and x[3] == k[1]:
                out.append(SuggestionTemplates.CHANNEL_ORDER_MISMATCH.format("NHWC " + _fmt(x), "NCHW " + _fmt([x[0], x[3], x[1], x[2]])))
            elif x[1] != k[1]:
                out.append(SuggestionTemplates.FEATURE_SIZE_MISMATCH.format(x[1], k[1]).replace("features", "channels"))
        if exp and len(x) == 4 and len(exp[0]) == 4 and self.is_channel_order_mismatch(x, exp[0]) and list(x) != list(exp[0]):
            out.append(SuggestionTemplates.CHANNEL_ORDER_MISMATCH.format(_fmt(x), _fmt(exp[0])))
        return out

    def _concat(self, ins):
        if len(ins) < 2:
            return []
        a, b = ins[0], ins[1]
        if len(a) != len(b):
            small = a if len(a) < len(b) else b
            return [SuggestionTemplates.UNSQUEEZE_SUGGESTION.format(0) + f" on {_fmt(small)} so that both tensors have the same rank"]
        diff = [i for i, (x, y) in enumerate(zip(a, b)) if x != y]
        if len(diff) == 1:
            return [f"The shapes differ only on axis {diff[0]}: concatenate on that axis"]
        if len(diff) > 1:
            return [SuggestionTemplates.CONCATENATION_DIMENSION_MISMATCH.format(diff[0], diff[-1])]
        return []

    def _broadcast(self, ins):
        if len(ins) < 2:
            return []
        a, b = ins[0], ins[1]
        bad = BroadcastDiagnosticFormatter.problematic_dimension(a, b)
        if bad is None:
            return []
        out = [SuggestionTemplates.BROADCASTING_FAILURE.format(_fmt(a), _fmt(b))]
        if len(a) != len(b):
            short, long = (a, b) if len(a) < len(b) else (b, a)
            for pos in range(len(short) + 1):
                cand = list(short[:pos]) + [1] * (len(long) - len(short)) + list(short[pos:])
                if BroadcastDiagnosticFormatter.problematic_dimension(cand, long) is None:
                    out.append(SuggestionTemplates.RESHAPE_SUGGESTION.format(_fmt(short), _fmt(cand)))
                    break
        return out

    def _matmul(self, ins, exp):
        if len(ins) < 2 or len(ins[0]) < 1 or len(ins[1]) < 2:
            return []
        a, b = ins[0], ins[1]
        if a[-1] == b[-2]:
            return []
        out = []
        if a[-1] == b[-1]:
            out.append(SuggestionTemplates.TRANSPOSE_REQUIRED.format(_fmt(b), _fmt(list(b[:-2]) + [b[-1], b[-2]])))
        if len(a) >= 2 and a[-2] == b[-2]:
            out.append(SuggestionTemplates.TRANSPOSE_REQUIRED.format(_fmt(a), _fmt(list(a[:-2]) + [a[-1], a[-2]])))
        if not out:
            out.append(SuggestionTemplates.FEATURE_SIZE_MISMATCH.format(a[-1], b[-2]))
        return out

    def _generic(self, ins, exp):
        out = []
        for i, (s, e) in enumerate(zip(ins, exp)):
            if list(s) == list(e):
                continue
            if _numel(s) == _numel(e):
                out.append(SuggestionTemplates.RESHAPE_SUGGESTION.format(_fmt(s), _fmt(e)))
            else:
                out.append(SuggestionTemplates.GENERIC_SHAPE_MISMATCH.format(f"input {i}", _fmt(s), _fmt(e)))
        return out

    def _common(self, ins, exp):
        out = []
        x = ins[0]
        if exp and len(x) + 1 == len(exp[0]) and list(x) == list(exp[0][1:]):
            out.append(SuggestionTemplates.MISSING_BATCH_DIM.format(", ".join(map(str, x))))
        if exp and len(x) == len(exp[0]) + 1 and 1 in list(x):
            out.append(SuggestionTemplates.SQUEEZE_SUGGESTION.format(list(x).index(1)))
        return out


# ------------------------------------------------------------------ declarative requirements
class ConstraintType(enum.Enum):
    MUST_MATCH = "must_match"               # equals dimension (target_input_index, target_dimension_index)
    MUST_EQUAL = "must_equal"               # equals fixed_value
    MUST_BE_POSITIVE = "must_be_positive"
    MUST_BE_MULTIPLE_OF = "must_be_multiple_of"
    MUST_DIVIDE = "must_divide"             # divides fixed_value
    ANY = "any"


@dataclass
class DimensionConstraint:
    type: ConstraintType = ConstraintType.ANY
    target_input_index: Optional[int] = None
    target_dimension_index: Optional[int] = None
    fixed_value: Optional[int] = None
    multiple_of: Optional[int] = None

    def check(self, value: int, shapes: Sequence[Shape]) -> Optional[str]:
        """``None`` when satisfied, else what is wrong."""
        T = ConstraintType
        if self.type is T.MUST_MATCH:
            other = shapes[self.target_input_index][self.target_dimension_index]
            if value != other:
                return f"{value} must match dimension {self.target_dimension_index} of input {self.target_input_index} ({other})"
        elif self.type is T.MUST_EQUAL and value != self.fixed_value:
            return f"{value} must equal {self.fixed_value}"
        elif self.type is T.MUST_BE_POSITIVE and value <= 0:
            return f"{value} must be positive"
        elif self.type is T.MUST_BE_MULTIPLE_OF and value % self.multiple_of != 0:
            return f"{value} must be a multiple of {self.multiple_of}"
        elif self.type is T.MUST_DIVIDE and (value == 0 or self.fixed_value % value != 0):
            return f"{value} must divide {self.fixed_value}"
        return None


@dataclass
class OperationShapeRequirements:
    input_count: int = 1
    expected_dimensions: Optional[Sequence[Optional[int]]] = None        # rank per input; None = any
    dimension_constraints: Dict[int, Dict[int, DimensionConstraint]] = field(default_factory=dict)
    description: str = ""
    error_message_format: str = "{op}: {problem}"
    custom_validator: Optional[Callable[[Sequence[Shape], Dict], ValidationResult]] = None

    def validate(self, op: str, shapes: Sequence[Shape], params: Optional[Dict] = None) -> ValidationResult:
        if self.input_count >= 0 and len(shapes) != self.input_count:
            return ValidationResult.failure(self.error_message_format.format(op=op, problem=f"expects {self.input_count} inputs, got {len(shapes)}"))
        for i, rank in enumerate(self.expected_dimensions or ()):
            if rank is not None and len(shapes[i]) != rank:
                return ValidationResult.failure(self.error_message_format.format(
                    op=op, problem=f"input {i} must have {rank} dimensions, got {len(shapes[i])} ({_fmt(shapes[i])})"))
        for i, dims in self.dimension_constraints.items():
            for d, c in dims.items():
                bad = c.check(shapes[i][d], shapes)
                if bad:
                    return ValidationResult.failure(self.error_message_format.format(op=op, problem=f"dimension {d} of input {i}: {bad}"))
        if self.custom_validator is not None:
            return self.custom_validator(shapes, params or {})
        return ValidationResult.success()


class OperationMetadataRegistry:
    """Shape requirements per operation type (DefaultOperationMetadataRegistry.cs)."""

    def __init__(self, defaults: bool = True):
        self._r: Dict[OperationType, OperationShapeRequirements] = {}
        if defaults:
            C, T = DimensionConstraint, ConstraintType
            self.register(OperationType.MATRIX_MULTIPLY, OperationShapeRequirements(
                2, (2, 2), {0: {1: C(T.MUST_MATCH, 1, 0)}}, "[m, k] x [k, n] -> [m, n]"))
            self.register(OperationType.LINEAR, OperationShapeRequirements(
                2, (None, 2), {}, "[..., in] with weight [out, in] -> [..., out]",
                custom_validator=lambda s, p: ValidationResult.success() if s[0][-1] == s[1][1] else ValidationResult.failure(
                    f"linear: input features {s[0][-1]} do not match the weight's in-features {s[1][1]}")))
            self.register(OperationType.CONV2D, OperationShapeRequirements(
                2, (4, 4), {0: {1: C(T.MUST_MATCH, 1, 1)}}, "[n, c, h, w] with kernel [o, c, kh, kw]"))
            self.register(OperationType.CONV1D, OperationShapeRequirements(
                2, (3, 3), {0: {1: C(T.MUST_MATCH, 1, 1)}}, "[n, c, l] with kernel [o, c, k]"))
            self.register(OperationType.CONCAT, OperationShapeRequirements(
                -1, None, {}, "all dimensions equal except the concatenation axis", custom_validator=self._concat))
            self.register(OperationType.BROADCAST, OperationShapeRequirements(
                2, None, {}, "aligned from the right, dimensions equal or 1", custom_validator=self._broadcast))

    @staticmethod
    def _concat(shapes, params):
        axis = params.get("axis", 0)
        first = shapes[0]
        for s in shapes[1:]:
            if len(s) != len(first):
                return ValidationResult.failure(f"concat: ranks differ ({_fmt(first)} and {_fmt(s)})")
            for d, (x, y) in enumerate(zip(first, s)):
                if d != axis % len(first) and x != y:
                    return ValidationResult.failure(f"concat: dimension {d} differs ({x} and {y}) and is not the concatenation axis {axis}")
        return ValidationResult.success()

    @staticmethod
    def _broadcast(shapes, params):
        bad = BroadcastDiagnosticFormatter.problematic_dimension(shapes[0], shapes[1])
        return ValidationResult.success() if bad is None else ValidationResult.failure(
            f"broadcast: dimension {bad} is incompatible ({_fmt(shapes[0])} and {_fmt(shapes[1])})")

    def register(self, type: OperationType, req: OperationShapeRequirements) -> None:
        self._r[type] = req

    def get_requirements(self, type: OperationType) -> Optional[OperationShapeRequirements]:
        return self._r.get(type)

    def is_registered(self, type: OperationType) -> bool:
        return type in self._r

    def validate(self, type: OperationType, shapes: Sequence[Shape], params: Optional[Dict] = None) -> ValidationResult:
        r = self._r.get(type)
        return r.validate(type.value, shapes, params) if r is not None else ValidationResult.success()


@dataclass
class ShapeDiagnosticsInfo:
    """Everything known about one operation's shapes, for a report (ShapeDiagnosticsInfo.cs)."""
    operation_type: OperationType = OperationType.ELEMENTWISE
    layer_name: str = ""
    input_shapes: List[Shape] = field(default_factory=list)
    expected_shapes: List[Shape] = field(default_factory=list)
    actual_output_shape: Optional[Shape] = None
    is_valid: bool = True
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)
    requirements_description: str = ""
    previous_layer_name: str = ""
    previous_layer_shape: Optional[Shape] = None

    def get_formatted_report(self) -> str:
        out = [f"Operation: {self.operation_type.value}" + (f" (layer '{self.layer_name}')" if self.layer_name else ""),
               f"Status: {'valid' if self.is_valid else 'INVALID'}"]
        out += [f"  input {i}: {_fmt(s)}" for i, s in enumerate(self.input_shapes)]
        out += [f"  expected {i}: {_fmt(s)}" for i, s in enumerate(self.expected_shapes)]
        if self.actual_output_shape is not None:
            out.append(f"  output: {_fmt(self.actual_output_shape)}")
        if self.requirements_description:
            out.append(f"Requirements: {self.requirements_description}")
        if self.previous_layer_name:
            shape = f" -> {_fmt(self.previous_layer_shape)}" if self.previous_layer_shape is not None else ""
            out.append(f"Previous layer: {self.previous_layer_name}{shape}")
        out += [f"Error: {e}" for e in self.errors] + [f"Warning: {w}" for w in self.warnings]
        return "\n".join(out)

    def to_exception(self, suggestions: Sequence[str] = ()) -> ShapeMismatchException:
        e = ShapeMismatchException(self.operation_type.value, [tuple(s) for s in self.input_shapes],
                                   "; ".join(self.errors) or "shape mismatch", list(suggestions))
        e.expected_shapes = [tuple(s) for s in self.expected_shapes]
        where = f"layer '{self.layer_name}'" if self.layer_name else ""
        if self.previous_layer_name:
            where += f" after '{self.previous_layer_name}'"
        e.details = where.strip()
        return e


# ------------------------------------------------------------------ graph of operations
@dataclass
class OperationNode:
    name: str = ""
    operation_type: OperationType = OperationType.ELEMENTWISE
    input_names: Tuple[str, ...] = ()
    parameters: Dict[str, object] = field(default_factory=dict)

    @property
    def input_count(self) -> int:
        return len(self.input_names)

    def __str__(self):
        return f"{self.name} = {self.operation_type.value}({', '.join(self.input_names)})"


class ComputationGraph:
    """Named operation nodes and the edges between them (ComputationGraph.cs:7-116)."""

    def __init__(self):
        self.nodes: Dict[str, OperationNode] = {}
        self.edges: List[Tuple[str, str]] = []

    def add_node(self, node: OperationNode) -> None:
        if node is None or not node.name:
            raise ValueError("a node needs a name")
        if node.name in self.nodes:
            raise ValueError(f"node {node.name!r} already exists")
        self.nodes[node.name] = node
        for src in node.input_names:
            if src in self.nodes:
                self.edges.append((src, node.name))

    def add_edge(self, from_node: str, to_node: str) -> None:
        for n in (from_node, to_node):
            if n not in self.nodes:
                raise KeyError(f"node {n!r} is not in the graph")
        if (from_node, to_node) not in self.edges:
            self.edges.append((from_node, to_node))

    def get_input_nodes(self) -> List[str]:
        have_in = {t for _, t in self.edges}
        return [n for n in self.nodes if n not in have_in]

    def get_output_nodes(self) -> List[str]:
        have_out = {f for f, _ in self.edges}
        return [n for n in self.nodes if n not in have_out]

    def topological_order(self) -> List[str]:
        indeg = {n: 0 for n in self.nodes}
        for _, t in self.edges:
            indeg[t] += 1
        ready = [n for n in self.nodes if indeg[n] == 0]
        out = []
        while ready:
            n = ready.pop(0)
            out.append(n)
            for f, t in self.edges:
                if f == n:
                    indeg[t] -= 1
                    if indeg[t] == 0:
                        ready.append(t)
        if len(out) != len(self.nodes):
            raise ValueError("the graph has a cycle")
        return out


class GraphShapeInference:
    """Pushes shapes through a ``ComputationGraph`` and reports the first node whose inputs break its
    requirements, with the layer before it (the part of DefaultShapeInferenceEngine.cs that whole-model
    checks use). Output shapes: matmul / linear / conv (stride, padding, dilation parameters) / concat /
    broadcast; other operations pass their first input's shape on."""

    def __init__(self, metadata: Optional[OperationMetadataRegistry] = None,
                 suggestions: Optional[FixSuggestionGenerator] = None):
        self.metadata = metadata or OperationMetadataRegistry()
        self.suggestions = suggestions or FixSuggestionGenerator()

    @staticmethod
    def _conv_out(n: int, k: int, p: Dict, i: int) -> int:
        def pick(key, default):
            v = p.get(key, default)
            return v[i] if isinstance(v, (tuple, list)) else v
        s, pad, d = pick("stride", 1), pick("padding", 0), pick("dilation", 1)
        return (n + 2 * pad - d * (k - 1) - 1) // s + 1

    def output_shape(self, node: OperationNode, shapes: Sequence[Shape]) -> Shape:
        T, p = OperationType, node.parameters
        if node.operation_type is T.MATRIX_MULTIPLY:
            return [*shapes[0][:-1], shapes[1][-1]]
        if node.operation_type is T.LINEAR:
            return [*shapes[0][:-1], shapes[1][0]]
        if node.operation_type is T.CONV2D:
            x, k = shapes
            return [x[0], k[0], self._conv_out(x[2], k[2], p, 0), self._conv_out(x[3], k[3], p, 1)]
        if node.operation_type is T.CONV1D:
            x, k = shapes
            return [x[0], k[0], self._conv_out(x[2], k[2], p, 0)]
        if node.operation_type is T.CONCAT:
            ax = int(p.get("axis", 0)) % len(shapes[0])
            out = list(shapes[0])
            out[ax] = sum(s[ax] for s in shapes)
            return out
        if node.operation_type is T.BROADCAST:
            n = max(len(s) for s in shapes)
            return [max(d) for d in zip(*(_pad(s, n) for s in shapes))]
        if node.operation_type is T.RESHAPE:
            return list(p["shape"])
        if node.operation_type is T.TRANSPOSE:
            out = list(shapes[0])
            a, b = p.get("dim0", -2), p.get("dim1", -1)
            out[a], out[b] = out[b], out[a]
            return out
        return list(shapes[0])

    def infer(self, graph: ComputationGraph, input_shapes: Dict[str, Shape]) -> Tuple[Dict[str, Shape], Optional[ShapeDiagnosticsInfo]]:
        """(shape per node, diagnostics of the first failing node or ``None``). Names that are not nodes
        (weights, constants) are looked up in ``input_shapes``."""
        known: Dict[str, Shape] = {k: list(v) for k, v in input_shapes.items()}
        for name in graph.topological_order():
            node = graph.nodes[name]
            if node.operation_type is OperationType.INPUT or (not node.input_names and name in known):
                if name not in known:
                    raise KeyError(f"no shape given for input {name!r}")
                continue
            try:
                ins = [known[s] for s in node.input_names]
            except KeyError as e:
                raise KeyError(f"node {name!r} reads {e.args[0]!r}, which has no shape") from None
            res = self.metadata.validate(node.operation_type, ins, node.parameters)
            if res.is_valid:
                out = self.output_shape(node, ins)
                if any(int(d) <= 0 for d in out):
                    res = ValidationResult.failure(f"{node.operation_type.value}: the output would be {_fmt(out)}")
            if not res.is_valid:
                prev = next((s for s in node.input_names if s in graph.nodes), "")
                req = self.metadata.get_requirements(node.operation_type)
                info = ShapeDiagnosticsInfo(node.operation_type, name, ins, [], None, False, [res.message], [],
                                            req.description if req else "", prev, known.get(prev))
                info.warnings = self.suggestions.generate_suggestions(node.operation_type, ins)
                return known, info
            known[name] = out
        return known, None
