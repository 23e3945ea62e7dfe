"""Process-wide diagnostics switchboard and the shape registry it feeds.

Reference: src/MLFramework/MLFramework.cs:8-110 (``EnableDiagnostics``, ``EnableShapeTracking``, ``EnableDebugMode``,
their ``Disable`` / ``Is...`` counterparts), src/MLFramework/Core/DiagnosticsConfiguration.cs (singleton: enhanced error
reporting, suggestions, shape tracking, context depth, debug mode, shape logging), Shapes/Tensors/TensorShapeRegistry.cs.

What the switches do here:

* shape tracking - ``TensorShapeRegistry.attach(model)`` installs forward hooks that record every module's input and
  output shapes (with the chain of enclosing modules up to ``context_tracking_depth``) while tracking is on; a shape
  error raised inside a tracked forward is re-raised with the shapes that led to it;
* debug mode - autograd anomaly detection, and after every tracked module call the native library's device status
  word is read so that a kernel that recorded an error is reported at the module that launched it, not steps later;
* enhanced error reporting / suggestions - ``format_exception`` renders an exception with the recorded context and,
  for shape mismatches, the fix suggestions.
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn


@dataclass
class DiagnosticsConfiguration:
    enhanced_error_reporting: bool = False
    include_suggestions: bool = True
    enable_shape_tracking: bool = False
    context_tracking_depth: int = 1
    debug_mode: bool = False
    log_shape_information: bool = False

    def reset_to_defaults(self):
        for f in fields(self):
            setattr(self, f.name, f.default)

    def validate(self):
        if self.context_tracking_depth < 0:
            raise ValueError("context_tracking_depth must be non-negative")


_CONFIG = DiagnosticsConfiguration()
_ENABLED = False
_LOCK = threading.Lock()


def configuration() -> DiagnosticsConfiguration:
    """The singleton every component reads."""
    return _CONFIG


def enable_diagnostics(config: Optional[DiagnosticsConfiguration] = None):
    global _ENABLED
    cfg = config or DiagnosticsConfiguration(enhanced_error_reporting=True)
    cfg.validate()
    with _LOCK:
        for f in fields(cfg):
            setattr(_CONFIG, f.name, getattr(cfg, f.name))
        if config is None:
            _CONFIG.enhanced_error_reporting = True
        _ENABLED = True
    _apply_debug(_CONFIG.debug_mode)


def disable_diagnostics():
    global _ENABLED
    with _LOCK:
        _CONFIG.reset_to_defaults()
        _ENABLED = False
    _apply_debug(False)


def is_diagnostics_enabled() -> bool:
    return _ENABLED


def enable_shape_tracking(depth: int = 1, log: bool = False):
    if depth < 0:
        raise ValueError("depth must be non-negative")
    _CONFIG.enable_shape_tracking, _CONFIG.context_tracking_depth, _CONFIG.log_shape_information = True, depth, log


def disable_shape_tracking():
    _CONFIG.enable_shape_tracking = _CONFIG.log_shape_information = False


def is_shape_tracking_enabled() -> bool:
    return _CONFIG.enable_shape_tracking


def enable_debug_mode():
    _CONFIG.debug_mode = True
    _apply_debug(True)


def disable_debug_mode():
    _CONFIG.debug_mode = False
    _apply_debug(False)


def is_debug_mode() -> bool:
    return _CONFIG.debug_mode


def _apply_debug(on: bool):
    torch.autograd.set_detect_anomaly(bool(on), check_nan=bool(on))


# ------------------------------------------------------------------ shape registry
@dataclass
class ShapeRecord:
    module: str
    module_type: str
    inputs: List[Tuple[int, ...]]
    outputs: List[Tuple[int, ...]]
    context: Tuple[str, ...] = ()
    calls: int = 1


def _shapes(x) -> List[Tuple[int, ...]]:
    if isinstance(x, torch.Tensor):
        return [tuple(x.shape)]
    if isinstance(x, (tuple, list)):
        return [s for y in x for s in _shapes(y)]
    if isinstance(x, dict):
        return [s for y in x.values() for s in _shapes(y)]
    return []


class TensorShapeRegistry:
    """Shapes by name: registered explicitly (``register``) or recorded from a model's forward passes (``attach``)."""

    def __init__(self, logger: Optional[Callable[[str], None]] = None):
        self._named: Dict[str, Tuple[int, ...]] = {}
        self.records: Dict[str, ShapeRecord] = {}
        self._stack: List[str] = []
        self._handles: List[Any] = []
        self._log = logger or (lambda s: None)

    # ---- explicit registration
    def register(self, name: str, shape) -> None:
        self._named[name] = tuple(int(d) for d in shape)

    def get(self, name: str) -> Optional[Tuple[int, ...]]:
        return self._named.get(name)

    def unregister(self, name: str) -> bool:
        return self._named.pop(name, None) is not None

    def names(self) -> List[str]:
        return sorted(self._named)

    # ---- recording from a model
    def attach(self, model: nn.Module, check_device_status: bool = True) -> "TensorShapeRegistry":
        names = {m: n or "<root>" for n, m in model.named_modules()}

        def pre(mod, inp):
            if _CONFIG.enable_shape_tracking:
                self._stack.append(names[mod])

        def post(mod, inp, out):
            if not _CONFIG.enable_shape_tracking:
                return
            name = names[mod]
            if self._stack and self._stack[-1] == name:
                self._stack.pop()
            depth = _CONFIG.context_tracking_depth
            ctx = tuple(self._stack[-depth:]) if depth else ()
            r = self.records.get(name)
            if r is None:
                self.records[name] = ShapeRecord(name, type(mod).__name__, _shapes(inp), _shapes(out), ctx)
            else:
                r.inputs, r.outputs, r.context, r.calls = _shapes(inp), _shapes(out), ctx, r.calls + 1
            if _CONFIG.log_shape_information:
                self._log(f"{name} ({type(mod).__name__}): {_shapes(inp)} -> {_shapes(out)}")
            if _CONFIG.debug_mode and check_device_status:
                _check_device_status(name)
        for m in model.modules():
            self._handles.append(m.register_forward_pre_hook(pre))
            self._handles.append(m.register_forward_hook(post))
        return self

    def detach(self):
        for h in self._handles:
            h.remove()
        self._handles.clear()
        self._stack.clear()

    def active_context(self) -> Tuple[str, ...]:
        """Modules whose forward is running right now, outermost first (what a failing op was called from)."""
        return tuple(self._stack)

    def describe(self, name: str) -> str:
        r = self.records.get(name)
        if r is None:
            return f"{name}: not recorded"
        ctx = f" (inside {' > '.join(r.context)})" if r.context else ""
        return f"{name} [{r.module_type}]{ctx}: {r.inputs} -> {r.outputs}, {r.calls} calls"

    def clear(self):
        self._named.clear()
        self.records.clear()
        self._stack.clear()


def _check_device_status(where: str):
    from . import _lib
    if torch.cuda.is_available() and _lib.available():
        try:
            _lib.raise_on_status()
        except Exception as e:       # noqa: BLE001 - re-raised with the module that launched the failing kernel
            raise type(e)(f"{e} (reported after module {where!r})") from e


@contextlib.contextmanager
def tracked(model: nn.Module, depth: int = 2, registry: Optional[TensorShapeRegistry] = None):
    """Shape tracking for the block: a shape error raised by a forward inside it carries the recorded context."""
    reg = (registry or TensorShapeRegistry()).attach(model)
    was = (_CONFIG.enable_shape_tracking, _CONFIG.context_tracking_depth)
    enable_shape_tracking(depth, _CONFIG.log_shape_information)
    try:
        yield reg
    except RuntimeError as e:
        ctx = reg.active_context()
        msg = str(e).lower()
        if ctx and ("shape" in msg or "size" in msg or "mat1 and mat2" in msg):
            last = [reg.describe(n) for n in list(reg.records)[-3:]]
            raise RuntimeError(f"{e}\n  while running: {' > '.join(ctx) or '<unknown>'}\n  last recorded shapes:\n    " + "\n    ".join(last)) from e
        raise
    finally:
        _CONFIG.enable_shape_tracking, _CONFIG.context_tracking_depth = was
        reg.detach()


def format_exception(e: BaseException, registry: Optional[TensorShapeRegistry] = None) -> str:
    """One report for an exception according to the configuration: plain message; with enhanced reporting the type,
    the recorded module context and - for shape mismatches when suggestions are on - the fix suggestions."""
    if not _CONFIG.enhanced_error_reporting:
        return str(e)
    lines = [f"{type(e).__name__}: {e}"]
    if registry is not None and registry.active_context():
        lines.append("context: " + " > ".join(registry.active_context()))
    sugg = getattr(e, "suggestions", None)
    if _CONFIG.include_suggestions and sugg:
        lines.append("suggestions:")
        lines += [f"  - {s}" for s in sugg]
    return "\n".join(lines)
