"""The user-facing controls of operator fusion: options, process-wide defaults, scoped overrides,
per-function hints, and one call that fuses a graph and reports what happened.

Reference: src/MLFramework/Fusion/{FusionResult.cs (FusionOptions, FusionAggressiveness, FusionBackend,
FusionResult, FusionRejected, FusionValidationResult), GraphOptions.cs, FusionContext.cs,
FusionApiExtensions.cs, FusibleAttribute.cs, NoFusionAttribute.cs, FusedOperation.cs}.

The machinery (pattern detectors, constraint validator, graph transformer, verifier) lives in
``compiler.fusion_passes``; this module decides which of it runs. The one back end is this package's
own code generator and GEMM epilogues, so ``FusionBackend`` has two values that do something:
``NATIVE`` and ``NONE``.
"""
from __future__ import annotations

import contextlib
import dataclasses
import enum
import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from .fusion_passes import (ConvActivationPatternDetector, ConvBatchNormPatternDetector, ElementWisePatternDetector,
                            FusionDecisionLogger, FusionStatisticsCollector, FusionVerifier, GraphTransformer,
                            LinearEpiloguePatternDetector)
from .ir import HLGraph

__all__ = [
    "FusionAggressiveness", "FusionBackend", "FusionOptions", "GraphOptions", "FusionContext", "FusionRejected",
    "FusedOperation", "FusionResult", "FusionValidationResult", "fusible", "no_fusion", "fusion_hint_of", "fuse_graph",
    "validate_fusion",
]


class FusionAggressiveness(enum.Enum):
    CONSERVATIVE = "conservative"     # GEMM epilogues and conv + batch-norm folding: exact or better arithmetic only
    MEDIUM = "medium"                 # + conv activations and element-wise chains up to ``max_fusion_ops``
    AGGRESSIVE = "aggressive"         # chains as long as the kernel generator allows


class FusionBackend(enum.Enum):
    NATIVE = "native"                 # this package's generated CUDA and GEMM epilogues
    NONE = "none"


@dataclass(frozen=True)
class FusionOptions:
    enable_fusion: bool = True
    max_fusion_ops: int = 10
    fusion_backend: FusionBackend = FusionBackend.NATIVE
    min_benefit_score: int = 50       # a chain must save at least this share (per cent) of its memory traffic
    enable_batch_norm_folding: bool = True
    enable_conv_activation_fusion: bool = True
    enable_element_wise_fusion: bool = True
    enable_gemm_epilogue_fusion: bool = True
    aggressiveness: FusionAggressiveness = FusionAggressiveness.MEDIUM
    verify: bool = False              # run the fused graph against the original on random inputs

    def validate(self) -> None:
        if self.max_fusion_ops < 2:
            raise ValueError("max_fusion_ops must be at least 2: a fusion joins operations")
        if not 0 <= self.min_benefit_score <= 100:
            raise ValueError("min_benefit_score is a percentage")

    def effective_max_ops(self) -> int:
        return {FusionAggressiveness.CONSERVATIVE: 2, FusionAggressiveness.MEDIUM: self.max_fusion_ops,
                FusionAggressiveness.AGGRESSIVE: max(self.max_fusion_ops, 16)}[self.aggressiveness]


class GraphOptions:
    """Process-wide defaults (GraphOptions.cs); ``FusionContext`` overrides them per thread."""

    _lock = threading.Lock()
    _options = FusionOptions()

    @classmethod
    def get(cls) -> FusionOptions:
        return cls._options

    @classmethod
    def set(cls, options: FusionOptions) -> None:
        options.validate()
        with cls._lock:
            cls._options = options

    @classmethod
    def update(cls, **changes) -> FusionOptions:
        cls.set(dataclasses.replace(cls._options, **changes))
        return cls._options

    @classmethod
    def reset_to_defaults(cls) -> None:
        with cls._lock:
            cls._options = FusionOptions()


_local = threading.local()


def current_options() -> FusionOptions:
    stack = getattr(_local, "stack", None)
    return stack[-1] if stack else GraphOptions.get()


class FusionContext(contextlib.AbstractContextManager):
    """``with FusionContext(options):`` — graphs fused on this thread inside the block use ``options``;
    contexts nest (FusionContext.cs)."""

    def __init__(self, options: FusionOptions):
        options.validate()
        self.options = options

    def __enter__(self):
        if not hasattr(_local, "stack"):
            _local.stack = []
        _local.stack.append(self.options)
        return self

    def __exit__(self, *exc):
        _local.stack.pop()
        return False

    @classmethod
    def disable_fusion(cls) -> "FusionContext":
        return cls(dataclasses.replace(current_options(), enable_fusion=False))

    @classmethod
    def with_options(cls, **changes) -> "FusionContext":
        return cls(dataclasses.replace(current_options(), **changes))


# ---- hints on functions that build graphs (FusibleAttribute.cs, NoFusionAttribute.cs)
def fusible(fn: Optional[Callable] = None, *, max_operations: int = 0, priority: int = 0, pattern: Optional[str] = None):
    """Marks a graph-building function as worth fusing; ``max_operations`` (0 = the options' value) and a
    ``pattern`` name restrict what is tried when the function's graph goes through ``fuse_graph(hint=fn)``."""
    def mark(f):
        f.__fusion_hint__ = {"fusible": True, "max_operations": max_operations, "priority": priority, "pattern": pattern, "reason": ""}
        return f
    return mark(fn) if fn is not None else mark


def no_fusion(fn: Optional[Callable] = None, *, reason: str = "explicitly marked as non-fusible"):
    def mark(f):
        f.__fusion_hint__ = {"fusible": False, "max_operations": 0, "priority": 0, "pattern": None, "reason": reason}
        return f
    if callable(fn):
        return mark(fn)
    if isinstance(fn, str):                               # @no_fusion("reason")
        reason = fn
    return mark


def fusion_hint_of(fn) -> Optional[Dict[str, object]]:
    return getattr(fn, "__fusion_hint__", None)


@dataclass(frozen=True)
class FusionRejected:
    pattern: str
    operations: Sequence[str]
    rejection_reason: str


@dataclass(frozen=True)
class FusedOperation:
    pattern: str
    operations: Sequence[str]        # the values the fused operation replaced


@dataclass
class FusionValidationResult:
    is_valid: bool
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)


@dataclass
class FusionResult:
    fused_graph: HLGraph
    fused_operations: List[FusedOperation]
    original_op_count: int
    fused_op_count: int
    rejected_fusions: List[FusionRejected]
    options: FusionOptions
    verified: Optional[bool] = None

    @property
    def ops_removed(self) -> int:
        return self.original_op_count - self.fused_op_count

    def summary(self) -> str:
        by: Dict[str, int] = {}
        for f in self.fused_operations:
            by[f.pattern] = by.get(f.pattern, 0) + 1
        kinds = ", ".join(f"{k} x{v}" for k, v in sorted(by.items())) or "nothing fused"
        v = "" if self.verified is None else f"; verified: {'yes' if self.verified else 'NO'}"
        return f"{self.original_op_count} -> {self.fused_op_count} operations ({kinds}); {len(self.rejected_fusions)} rejected{v}"


def _detectors(o: FusionOptions, hint: Optional[Dict[str, object]]):
    ds = []
    if o.enable_gemm_epilogue_fusion:
        ds.append(LinearEpiloguePatternDetector())
    if o.enable_batch_norm_folding:
        ds.append(ConvBatchNormPatternDetector())
    if o.enable_conv_activation_fusion and o.aggressiveness is not FusionAggressiveness.CONSERVATIVE:
        ds.append(ConvActivationPatternDetector())
    if o.enable_element_wise_fusion and o.aggressiveness is not FusionAggressiveness.CONSERVATIVE:
        ds.append(ElementWisePatternDetector())
    if hint and hint.get("pattern"):
        ds = [d for d in ds if d.name == hint["pattern"]]
    return ds


def fuse_graph(graph: HLGraph, options: Optional[FusionOptions] = None, hint=None) -> FusionResult:
    """Fuses a copy of ``graph`` under ``options`` (default: the innermost ``FusionContext``, else the
    process-wide ``GraphOptions``). ``hint`` is a function marked ``@fusible`` / ``@no_fusion`` or its hint."""
    o = options or current_options()
    o.validate()
    h = fusion_hint_of(hint) if callable(hint) else hint
    n0 = len(graph.ops)
    if not o.enable_fusion or o.fusion_backend is FusionBackend.NONE or (h is not None and not h["fusible"]):
        why = "fusion is disabled" if h is None or h["fusible"] else str(h["reason"])
        return FusionResult(graph, [], n0, n0, [FusionRejected("*", [], why)], o)
    limit = o.effective_max_ops()
    if h and h.get("max_operations"):
        limit = min(limit, int(h["max_operations"]))
    logger, stats = FusionDecisionLogger(), FusionStatisticsCollector()
    t = GraphTransformer(_detectors(o, h), stats=stats, logger=logger)
    inner_detect = [d.detect for d in t.detectors]

    def capped(detect):
        def run(g):
            out = []
            for m in detect(g):
                if len(m.op_indices) > limit:
                    logger.log(m.pattern, [g.ops[i].output for i in m.op_indices], False,
                               f"{len(m.op_indices)} operations exceed the limit of {limit}")
                    continue
                out.append(m)
            return out
        return run
    for d, det in zip(t.detectors, inner_detect):
        d.detect = capped(det)
    fused = t.transform(graph)
    done = [FusedOperation(r.pattern, tuple(r.ops)) for r in logger.accepted()]
    rejected = [FusionRejected(r.pattern, tuple(r.ops), r.reason) for r in logger.rejected()]
    res = FusionResult(fused, done, n0, len(fused.ops), rejected, o)
    if o.verify and done:
        v = FusionVerifier().verify(graph, fused)
        res.verified = bool(v.passed)
        if not res.verified:
            return FusionResult(graph, [], n0, n0, rejected + [FusionRejected("*", [], "the fused graph disagreed with the original")], o, False)
    return res


def validate_fusion(original: HLGraph, fused: HLGraph) -> FusionValidationResult:
    """Structural checks of a fused graph against its source: same interface, well-formed, not larger."""
    errors, warnings = [], []
    if [original.values[n].shape for n in original.inputs] != [fused.values[n].shape for n in fused.inputs]:
        errors.append("the inputs differ")
    if [original.values[n].shape for n in original.outputs] != [fused.values[n].shape for n in fused.outputs]:
        errors.append("the outputs differ")
    errors += fused.verify()
    if len(fused.ops) > len(original.ops):
        warnings.append(f"the fused graph has more operations ({len(fused.ops)}) than the original ({len(original.ops)})")
    if len(fused.ops) == len(original.ops):
        warnings.append("nothing was fused")
    return FusionValidationResult(not errors, errors, warnings)
