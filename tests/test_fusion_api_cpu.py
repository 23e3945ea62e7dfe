"""Fusion controls: options, process-wide defaults, scoped contexts, hints, fuse_graph results."""
import pytest
import torch

from ml_framework_b200.compiler import fusion_api as FA
from ml_framework_b200.compiler.ir import HLGraph


def _graph(chain=4):
    g = HLGraph("net")
    x = g.input("x", (8, 16))
    w = g.constant(torch.randn(32, 16) * 0.1, "w")
    b = g.constant(torch.zeros(32), "b")
    h = g.op("gelu", g.op("linear", x, w, b))
    for i in range(chain):
        h = g.op(("relu", "tanh", "sigmoid", "exp", "neg")[i % 5], h)
    g.output(h)
    return g


def _same(a, b):
    x = torch.randn(8, 16)
    torch.testing.assert_close(a.run({"x": x})[0], b.run({"x": x})[0], rtol=1e-5, atol=1e-6)


def test_options_defaults_and_scoped_contexts():
    FA.GraphOptions.reset_to_defaults()
    assert FA.current_options() == FA.FusionOptions() and FA.FusionOptions().effective_max_ops() == 10
    assert FA.FusionOptions(aggressiveness=FA.FusionAggressiveness.CONSERVATIVE).effective_max_ops() == 2
    assert FA.FusionOptions(aggressiveness=FA.FusionAggressiveness.AGGRESSIVE, max_fusion_ops=4).effective_max_ops() == 16
    for bad in (FA.FusionOptions(max_fusion_ops=1), FA.FusionOptions(min_benefit_score=101)):
        with pytest.raises(ValueError):
            bad.validate()
    FA.GraphOptions.update(max_fusion_ops=6)
    assert FA.current_options().max_fusion_ops == 6
    with FA.FusionContext.with_options(max_fusion_ops=3) as outer:
        assert FA.current_options() is outer.options and FA.current_options().max_fusion_ops == 3
        with FA.FusionContext.disable_fusion():
            assert not FA.current_options().enable_fusion and FA.current_options().max_fusion_ops == 3
        assert FA.current_options().enable_fusion
    assert FA.current_options().max_fusion_ops == 6
    with pytest.raises(ValueError):
        FA.GraphOptions.update(max_fusion_ops=0)
    FA.GraphOptions.reset_to_defaults()
    assert FA.current_options().max_fusion_ops == 10


def test_fuse_graph_results_and_switches():
    FA.GraphOptions.reset_to_defaults()
    g = _graph()
    res = FA.fuse_graph(g)
    pats = sorted(f.pattern for f in res.fused_operations)
    assert pats == ["elementwise_chain", "gemm_epilogue"] and res.original_op_count == 6 and res.fused_op_count == 2 and res.ops_removed == 4
    assert "6 -> 2 operations" in res.summary() and "gemm_epilogue x1" in res.summary() and len(g.ops) == 6       # the source is untouched
    _same(g, res.fused_graph)
    v = FA.validate_fusion(g, res.fused_graph)
    assert v.is_valid and v.warnings == []
    assert "nothing was fused" in FA.validate_fusion(g, g).warnings[0]
    off = FA.fuse_graph(g, FA.FusionOptions(enable_fusion=False))
    assert off.fused_graph is g and off.fused_operations == [] and off.rejected_fusions[0].rejection_reason == "fusion is disabled"
    assert FA.fuse_graph(g, FA.FusionOptions(fusion_backend=FA.FusionBackend.NONE)).fused_op_count == 6
    with FA.FusionContext.disable_fusion():
        assert FA.fuse_graph(g).fused_op_count == 6
    only_gemm = FA.fuse_graph(g, FA.FusionOptions(enable_element_wise_fusion=False))
    assert [f.pattern for f in only_gemm.fused_operations] == ["gemm_epilogue"] and only_gemm.fused_op_count == 5
    cons = FA.fuse_graph(g, FA.FusionOptions(aggressiveness=FA.FusionAggressiveness.CONSERVATIVE))
    assert [f.pattern for f in cons.fused_operations] == ["gemm_epilogue"]
    no_epi = FA.fuse_graph(g, FA.FusionOptions(enable_gemm_epilogue_fusion=False))
    assert [f.pattern for f in no_epi.fused_operations] == ["elementwise_chain"] and no_epi.fused_op_count == 2
    _same(g, no_epi.fused_graph)
    checked = FA.fuse_graph(g, FA.FusionOptions(verify=True))
    assert checked.verified is True and "verified: yes" in checked.summary()


def test_operation_limit_and_hints():
    FA.GraphOptions.reset_to_defaults()
    g = _graph(chain=5)
    short = FA.fuse_graph(g, FA.FusionOptions(max_fusion_ops=3, enable_gemm_epilogue_fusion=False))
    assert short.fused_operations == [] and any("exceed the limit of 3" in r.rejection_reason for r in short.rejected_fusions)

    @FA.fusible(max_operations=2, pattern="gemm_epilogue")
    def build():
        return _graph()

    @FA.no_fusion("numerically delicate")
    def delicate():
        return _graph()

    @FA.no_fusion
    def bare():
        return _graph()

    assert FA.fusion_hint_of(build)["pattern"] == "gemm_epilogue" and FA.fusion_hint_of(delicate)["reason"] == "numerically delicate"
    assert FA.fusion_hint_of(bare)["fusible"] is False and FA.fusion_hint_of(len) is None
    hinted = FA.fuse_graph(build(), hint=build)
    assert [f.pattern for f in hinted.fused_operations] == ["gemm_epilogue"]
    refused = FA.fuse_graph(delicate(), hint=delicate)
    assert refused.fused_operations == [] and refused.rejected_fusions[0].rejection_reason == "numerically delicate"
