"""Diagnostics switchboard, shape registry recorded from forward passes, error formatting."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200 import diagnostics as D
from ml_framework_b200.compiler.shapes import ShapeInferenceEngine, ShapeMismatchException


@pytest.fixture(autouse=True)
def _reset():
    D.disable_diagnostics()
    yield
    D.disable_diagnostics()


def test_switchboard_copies_settings_and_resets():
    assert not D.is_diagnostics_enabled() and not D.is_shape_tracking_enabled() and not D.is_debug_mode()
    D.enable_diagnostics()
    assert D.is_diagnostics_enabled() and D.configuration().enhanced_error_reporting and D.configuration().include_suggestions
    D.enable_diagnostics(D.DiagnosticsConfiguration(enable_shape_tracking=True, context_tracking_depth=3, debug_mode=True))
    c = D.configuration()
    assert c.enable_shape_tracking and c.context_tracking_depth == 3 and D.is_debug_mode() and torch.is_anomaly_enabled() and not c.enhanced_error_reporting
    D.disable_debug_mode()
    assert not torch.is_anomaly_enabled()
    D.enable_debug_mode()
    assert torch.is_anomaly_enabled()
    D.disable_diagnostics()
    assert not D.is_diagnostics_enabled() and D.configuration() == D.DiagnosticsConfiguration() and not torch.is_anomaly_enabled()
    with pytest.raises(ValueError):
        D.enable_diagnostics(D.DiagnosticsConfiguration(context_tracking_depth=-1))
    with pytest.raises(ValueError):
        D.enable_shape_tracking(-2)


def test_shape_registry_records_forward_passes_with_context():
    model = nn.Sequential(nn.Sequential(nn.Linear(4, 8), nn.ReLU()), nn.Linear(8, 2))
    lines = []
    reg = D.TensorShapeRegistry(lines.append).attach(model)
    model(torch.randn(3, 4))
    assert reg.records == {}                                  # tracking is off
    D.enable_shape_tracking(depth=2, log=True)
    model(torch.randn(3, 4))
    model(torch.randn(5, 4))
    r = reg.records["0.0"]
    assert (r.inputs, r.outputs, r.context, r.calls, r.module_type) == ([(5, 4)], [(5, 8)], ("<root>", "0"), 2, "Linear")
    assert reg.records["<root>"].context == () and "0.1 (ReLU): [(5, 8)] -> [(5, 8)]" in lines
    assert reg.describe("1") == "1 [Linear] (inside <root>): [(5, 8)] -> [(5, 2)], 2 calls" and reg.describe("9") == "9: not recorded"
    reg.detach()
    model(torch.randn(7, 4))
    assert reg.records["0.0"].calls == 2
    reg.register("tokens", [4, 2048])
    assert reg.get("tokens") == (4, 2048) and reg.names() == ["tokens"] and reg.unregister("tokens") and reg.get("tokens") is None
    reg.clear()
    assert reg.records == {}


def test_tracked_block_adds_context_to_shape_errors():
    model = nn.Sequential(nn.Linear(4, 8), nn.Linear(9, 2))
    with pytest.raises(RuntimeError) as ei:
        with D.tracked(model) as reg:
            model(torch.randn(3, 4))
    msg = str(ei.value)
    assert "while running: <root> > 1" in msg and "0 [Linear] (inside <root>): [(3, 4)] -> [(3, 8)]" in msg
    assert not D.is_shape_tracking_enabled() and reg._handles == []
    with pytest.raises(KeyError):
        with D.tracked(model):
            raise KeyError("unrelated")


def test_format_exception_follows_the_configuration():
    try:
        ShapeInferenceEngine().infer("matmul", [(2, 3), (4, 5)])
    except ShapeMismatchException as e:
        err = e
    assert D.format_exception(err) == str(err)
    D.enable_diagnostics()
    reg = D.TensorShapeRegistry()
    reg._stack[:] = ["<root>", "blocks.0"]
    text = D.format_exception(err, reg)
    assert text.startswith("ShapeMismatchException: matmul") and "context: <root> > blocks.0" in text and "suggestions:\n  - " in text
    D.configuration().include_suggestions = False
    assert "suggestions:\n  - " not in D.format_exception(err, reg).split("inputs")[0] and D.format_exception(ValueError("x")) == "ValueError: x"
