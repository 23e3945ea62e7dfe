"""Shape-error formatters, report generator, fix suggestions, declarative requirements, graph checks."""
import pytest

from ml_framework_b200.compiler import diagnostic_reports as D
from ml_framework_b200.compiler.diagnostics import ValidationResult
from ml_framework_b200.compiler.shapes import ShapeMismatchException

T = D.OperationType
FAIL = ValidationResult.failure


def test_formatters_and_registry():
    reg = D.DiagnosticFormatterRegistry.instance()
    assert reg is D.DiagnosticFormatterRegistry.instance()
    mm = reg.format_error(T.MATRIX_MULTIPLY, FAIL("inner dimensions 256 and 128 differ"), [32, 256], [128, 10])
    assert "[32, 256] x [128, 10]" in mm and "inner dimensions 256 and 128 must match" in mm
    sugg = reg.get_suggestions(T.MATRIX_MULTIPLY, FAIL("inner dimensions 256 and 128 differ"))
    assert any("outputs 256 features, but this layer expects 128" in s for s in sugg)
    conv = reg.format_error(T.CONV2D, FAIL("channel mismatch"), [8, 3, 32, 32], [16, 4, 3, 3])
    assert "input channels (3) do not match kernel channels (4)" in conv
    ok = reg.format_error(T.CONV2D, ValidationResult.success(), [8, 3, 32, 32], [16, 3, 5, 5])
    assert "Output shape (stride 1, no padding): [8, 16, 28, 28]" in ok
    assert "larger than the input" in reg.format_error(T.CONV2D, FAIL("x"), [1, 3, 2, 2], [4, 3, 5, 5])
    assert any("in-channels so that they match" in s for s in reg.get_suggestions(T.CONV2D, FAIL("channel mismatch")))
    cat = reg.format_error(T.CONCAT, ValidationResult.success(), [2, 3, 4], [2, 5, 4])
    assert "except on axis 1" in cat and "Output shape: [2, 8, 4]" in cat
    assert "could be joined on axis 1" in reg.format_error(T.CONCAT, FAIL("axis 0 sizes differ"), [2, 3, 4], [2, 5, 4])
    assert D.ConcatDiagnosticFormatter.compatible_axis([2, 3], [4, 5]) is None
    bc = reg.format_error(T.BROADCAST, FAIL("x"), [4, 3, 5], [2, 5])
    assert "cannot broadcast dimension 1 (3 against 2)" in bc
    assert "compatible for broadcasting" in reg.format_error(T.BROADCAST, FAIL("x"), [4, 1, 5], [3, 5])
    assert "insufficient input shapes" in reg.format_error(T.BROADCAST, FAIL("x"), [1])
    generic = reg.format_error(T.POOLING, FAIL("window too large"), [1, 2])
    assert generic == "pooling: validation failed for input shapes [1, 2]. window too large" and reg.get_suggestions(T.POOLING, FAIL("")) == []
    own = D.DiagnosticFormatterRegistry(defaults=False)
    assert own.get(T.CONCAT) is None
    with pytest.raises(ValueError):
        own.register(None)


def test_report_generator_three_formats():
    e = ShapeMismatchException("matmul", [(32, 256), (128, 10)], "inner dimensions 256 and 128 differ", ["transpose <b>"])
    e.expected_shapes = [(32, 128)]
    e.details = "layer 'fc2' after 'fc1'"
    text = D.ErrorReportGenerator.generate_report(e)
    assert text.startswith("=" * 64) and "Operation: matmul" in text and "  Tensor 2: [128, 10]" in text
    assert "EXPECTED SHAPES:" in text and "  inner dimensions 256 and 128 differ" in text and "CONTEXT:" in text and "1. transpose <b>" in text
    md = D.ErrorReportGenerator.generate_report(e, D.ErrorReportFormat.MARKDOWN)
    assert md.startswith("# Shape mismatch") and "- Tensor 1: `[32, 256]`" in md and "## Suggested fixes" in md
    page = D.ErrorReportGenerator.generate_report(e, D.ErrorReportFormat.HTML)
    assert page.startswith("<!DOCTYPE html>") and "transpose &lt;b&gt;" in page and "layer &#x27;fc2&#x27;" in page
    bare = D.ErrorReportGenerator.generate_report(ShapeMismatchException("op", [], "bad"))
    assert "INPUT SHAPES" not in bare and "SUGGESTED" not in bare
    with pytest.raises(ValueError):
        D.ErrorReportGenerator.generate_report(None)


def test_fix_suggestions_recognise_the_usual_causes():
    g = D.FixSuggestionGenerator()
    lin = g.generate_suggestions(T.LINEAR, [[32, 256], [10, 128]])
    assert lin == ["Previous layer outputs 256 features, but this layer expects 128. Adjust layer configuration"]
    assert any("transposing [256, 10] to [10, 256]" in s for s in g.generate_suggestions(T.LINEAR, [[32, 256], [256, 10]]))
    assert any("reshaping from [32, 16, 16] to [32, 256]" in s for s in g.generate_suggestions(T.LINEAR, [[32, 16, 16], [10, 256]]))
    nhwc = g.generate_suggestions(T.CONV2D, [[8, 32, 32, 3], [16, 3, 3, 3]])
    assert any("Permute from NHWC [8, 32, 32, 3] to NCHW [8, 3, 32, 32]" in s for s in nhwc)
    assert any("missing batch dimension" in s for s in g.generate_suggestions(T.CONV2D, [[3, 32, 32], [16, 3, 3, 3]]))
    assert g.is_channel_order_mismatch([1, 3, 8, 9], [1, 8, 9, 3]) and not g.is_channel_order_mismatch([1, 3, 8, 9], [1, 3, 8, 9])
    assert "concatenate on that axis" in g.generate_suggestions(T.CONCAT, [[2, 3, 4], [2, 5, 4]])[0]
    assert "Use axis 2" in g.generate_suggestions(T.CONCAT, [[2, 3, 4], [3, 3, 5]])[0]
    assert "same rank" in g.generate_suggestions(T.CONCAT, [[2, 3], [2, 3, 1]])[0]
    bc = g.generate_suggestions(T.BROADCAST, [[4, 3], [4, 3, 5]])
    assert "Cannot broadcast shapes [4, 3] and [4, 3, 5]" in bc[0] and "reshaping from [4, 3] to [4, 3, 1]" in bc[1]
    assert g.generate_suggestions(T.BROADCAST, [[4, 1], [4, 5]]) == []
    assert "transposing [10, 256] to [256, 10]" in g.generate_suggestions(T.MATRIX_MULTIPLY, [[32, 256], [10, 256]])[0]
    assert "outputs 7 features" in g.generate_suggestions(T.MATRIX_MULTIPLY, [[32, 7], [9, 11]])[0]
    gen = g.generate_suggestions(T.RESHAPE, [[4, 6]], [[3, 8]])
    assert gen == ["Try reshaping from [4, 6] to [3, 8]"]
    assert "Shape mismatch for input 0" in g.generate_suggestions(T.RESHAPE, [[4, 6]], [[5, 5]])[0]
    assert any("unsqueeze(0) or reshape to [1, 784]" in s for s in g.generate_suggestions(T.ELEMENTWISE, [[784]], [[1, 784]]))
    assert any("squeezing dimension 1" in s for s in g.generate_suggestions(T.ELEMENTWISE, [[4, 1, 5]], [[4, 5]]))
    assert g.generate_suggestions(T.LINEAR, []) == []


def test_dimension_constraints_and_requirements():
    C, K = D.DimensionConstraint, D.ConstraintType
    shapes = [[4, 8], [8, 3]]
    assert C(K.MUST_MATCH, 1, 0).check(8, shapes) is None and "must match" in C(K.MUST_MATCH, 1, 1).check(8, shapes)
    assert C(K.MUST_EQUAL, fixed_value=3).check(4, shapes) == "4 must equal 3" and C(K.MUST_BE_POSITIVE).check(0, shapes)
    assert C(K.MUST_BE_MULTIPLE_OF, multiple_of=8).check(12, shapes) and C(K.MUST_BE_MULTIPLE_OF, multiple_of=4).check(12, shapes) is None
    assert C(K.MUST_DIVIDE, fixed_value=12).check(5, shapes) and C(K.MUST_DIVIDE, fixed_value=12).check(4, shapes) is None and C().check(-1, shapes) is None
    reg = D.OperationMetadataRegistry()
    assert reg.validate(T.MATRIX_MULTIPLY, [[4, 8], [8, 3]]).is_valid
    assert "dimension 1 of input 0" in reg.validate(T.MATRIX_MULTIPLY, [[4, 8], [7, 3]]).message
    assert "expects 2 inputs, got 1" in reg.validate(T.MATRIX_MULTIPLY, [[4, 8]]).message
    assert "must have 4 dimensions, got 3" in reg.validate(T.CONV2D, [[3, 8, 8], [4, 3, 3, 3]]).message
    assert reg.validate(T.LINEAR, [[2, 5, 16], [4, 16]]).is_valid and "in-features 16" in reg.validate(T.LINEAR, [[2, 5, 8], [4, 16]]).message
    assert reg.validate(T.CONCAT, [[2, 3], [2, 4], [2, 1]], {"axis": 1}).is_valid
    assert "not the concatenation axis 0" in reg.validate(T.CONCAT, [[2, 3], [2, 4]], {"axis": 0}).message
    assert not reg.validate(T.BROADCAST, [[2, 3], [4, 3]]).is_valid and reg.validate(T.POOLING, [[1]]).is_valid
    custom = D.OperationShapeRequirements(1, (2,), {0: {1: C(K.MUST_BE_MULTIPLE_OF, multiple_of=16)}}, "rows of 16",
                                          error_message_format="tile rule broken in {op}: {problem}")
    reg.register(T.RESHAPE, custom)
    assert reg.is_registered(T.RESHAPE) and reg.validate(T.RESHAPE, [[4, 24]]).message.startswith("tile rule broken in reshape: dimension 1")
    assert reg.get_requirements(T.RESHAPE).description == "rows of 16"


def _mlp_graph(hidden_in=128):
    g = D.ComputationGraph()
    g.add_node(D.OperationNode("x", T.INPUT))
    g.add_node(D.OperationNode("fc1", T.LINEAR, ("x", "w1")))
    g.add_node(D.OperationNode("act", T.ELEMENTWISE, ("fc1",)))
    g.add_node(D.OperationNode("fc2", T.LINEAR, ("act", "w2")))
    return g, {"x": [32, 784], "w1": [256, 784], "w2": [10, hidden_in]}


def test_graph_inference_finds_the_first_broken_layer():
    g, shapes = _mlp_graph(256)
    assert g.get_input_nodes() == ["x"] and g.get_output_nodes() == ["fc2"] and g.topological_order() == ["x", "fc1", "act", "fc2"]
    known, info = D.GraphShapeInference().infer(g, shapes)
    assert info is None and known["fc1"] == [32, 256] and known["fc2"] == [32, 10]
    g, shapes = _mlp_graph(128)
    known, info = D.GraphShapeInference().infer(g, shapes)
    assert info is not None and info.layer_name == "fc2" and info.previous_layer_name == "act" and info.previous_layer_shape == [32, 256]
    assert not info.is_valid and "in-features 128" in info.errors[0] and any("outputs 256 features" in w for w in info.warnings)
    rep = info.get_formatted_report()
    assert "layer 'fc2'" in rep and "Status: INVALID" in rep and "Previous layer: act -> [32, 256]" in rep
    e = info.to_exception(info.warnings)
    assert e.details == "layer 'fc2' after 'act'" and "SUGGESTED FIXES" in D.ErrorReportGenerator.generate_report(e)
    with pytest.raises(KeyError, match="w2"):
        D.GraphShapeInference().infer(g, {"x": [1, 784], "w1": [256, 784]})


def test_graph_conv_concat_shapes_and_structure_errors():
    g = D.ComputationGraph()
    g.add_node(D.OperationNode("img", T.INPUT))
    g.add_node(D.OperationNode("c1", T.CONV2D, ("img", "k1"), {"stride": 2, "padding": 1}))
    g.add_node(D.OperationNode("c2", T.CONV2D, ("img", "k2"), {"stride": (2, 2), "padding": (2, 2)}))
    g.add_node(D.OperationNode("cat", T.CONCAT, ("c1", "c2"), {"axis": 1}))
    g.add_node(D.OperationNode("t", T.TRANSPOSE, ("cat",), {"dim0": 1, "dim1": 3}))
    known, info = D.GraphShapeInference().infer(g, {"img": [2, 3, 32, 32], "k1": [8, 3, 3, 3], "k2": [4, 3, 5, 5]})
    assert info is None and known["c1"] == [2, 8, 16, 16] and known["c2"] == [2, 4, 16, 16] and known["cat"] == [2, 12, 16, 16]
    assert known["t"] == [2, 16, 16, 12]
    _, bad = D.GraphShapeInference().infer(g, {"img": [2, 3, 2, 2], "k1": [8, 3, 3, 3], "k2": [4, 3, 9, 9]})
    assert bad is not None and bad.layer_name == "c2" and "the output would be" in bad.errors[0]
    with pytest.raises(ValueError):
        g.add_node(D.OperationNode("c1", T.CONV2D))
    with pytest.raises(KeyError):
        g.add_edge("c1", "nope")
    g.add_edge("t", "c1")
    with pytest.raises(ValueError, match="cycle"):
        g.topological_order()
    assert str(D.OperationNode("y", T.LINEAR, ("x", "w"))) == "y = linear(x, w)"
