"""Fusion as a checked transformation: detectors, constraints, rewrites, verification, fall-back, statistics, run-time shapes."""
import pytest
import torch

from ml_framework_b200.compiler import fusion_passes as fp
from ml_framework_b200.compiler.ir import HLGraph, Op


def _mlp_graph(B=4, I=8, H=16):
    g = HLGraph("mlp")
    x = g.input("x", (B, I))
    r = g.input("r", (B, H))
    w = g.constant(torch.randn(H, I) * 0.3)
    b = g.constant(torch.randn(H) * 0.1)
    h = g.op("linear", x, w, b)
    a = g.op("gelu", h)
    w2 = g.constant(torch.randn(H, H) * 0.3)
    y = g.op("linear", a, w2)
    z = g.op("add", y, r)
    t = g.op("tanh", z)
    u = g.op("mul", t, r)
    v = g.op("relu", u)
    g.output(v)
    return g


def _conv_graph():
    g = HLGraph("cnn")
    x = g.input("x", (2, 3, 8, 8))
    w = g.constant(torch.randn(4, 3, 3, 3) * 0.2)
    b = g.constant(torch.randn(4) * 0.1)
    c = g.op("conv2d", x, w, b, padding=1)
    gamma, beta = g.constant(torch.rand(4) + 0.5), g.constant(torch.randn(4) * 0.1)
    mean, var = g.constant(torch.randn(4) * 0.1), g.constant(torch.rand(4) + 0.5)
    n = g.op("batchnorm", c, gamma, beta, mean, var, eps=1e-5)
    w2 = g.constant(torch.randn(4, 4, 3, 3) * 0.2)
    c2 = g.op("conv2d", n, w2, padding=1)
    r = g.op("relu", c2)
    g.output(r)
    return g


def test_analyzer_patterns_and_compatibility():
    g = _mlp_graph()
    an, chk = fp.GraphAnalyzer(), fp.OperationCompatibilityChecker()
    kinds = [an.access_pattern(o) for o in g.ops]
    P = fp.MemoryAccessPattern
    assert kinds[:2] == [P.CONTRACTION, P.ELEMENT_WISE] and an.access_pattern(Op("weird", [], "o")) == P.UNKNOWN
    ok, why = chk.can_fuse(g, g.ops[0], g.ops[1])
    assert ok and why == ""
    ok, why = chk.can_fuse(g, g.ops[1], g.ops[2])           # element-wise -> contraction
    assert not ok and "do not fuse" in why
    assert not chk.can_fuse(g, g.ops[0], g.ops[3])[0]
    idx = [4, 5, 6]
    assert an.external_inputs(g, idx) == [g.ops[3].output, "r"]
    assert an.intermediate_bytes(g, idx) == 2 * 4 * 16 * 4


def test_transformer_rewrites_and_result_matches_the_original():
    torch.manual_seed(0)
    g = _mlp_graph()
    tr = fp.GraphTransformer()
    h = tr.transform(g)
    assert [o.kind for o in h.ops] == ["linear", "linear", "fused_elementwise"]
    assert h.ops[0].attrs["epilogue"] == "gelu" and h.ops[1].attrs["epilogue"] == "residual" and h.ops[1].inputs[-1] == "r"
    assert [k for k, _ in h.ops[2].attrs["chain"]] == ["tanh", "mul", "relu"]
    assert len(g.ops) == 7                                   # the input graph is untouched
    r = fp.FusionVerifier(trials=2).verify(g, h)
    assert r.passed and r.worst_abs_error < 1e-5 and len(r.trials) == 2
    s = tr.stats.stats
    assert (s.total_ops_before, s.total_ops_after, s.fused_groups, s.fused_ops) == (7, 3, 3, 7)
    assert s.by_pattern == {"gemm_epilogue": 2, "elementwise_chain": 1} and abs(s.fusion_ratio - 1.0) < 1e-9
    assert len(tr.logger.accepted()) == 3 and "[fuse] gemm_epilogue" in tr.logger.render()


def test_conv_batchnorm_folds_and_conv_activation_merges():
    torch.manual_seed(1)
    g = _conv_graph()
    h = fp.GraphTransformer().transform(g)
    assert [o.kind for o in h.ops] == ["conv2d", "conv2d"] and h.ops[1].attrs["activation"] == "relu"
    assert fp.FusionVerifier(atol=1e-4, rtol=1e-4).verify(g, h).passed


def test_broadcast_add_is_not_taken_as_a_residual():
    g = HLGraph()
    x = g.input("x", (4, 8))
    w = g.constant(torch.randn(6, 8))
    y = g.op("linear", x, w)
    b = g.constant(torch.randn(6))
    z = g.op("add", y, b)
    g.output(z)
    assert fp.LinearEpiloguePatternDetector().detect(g) == []


def test_constraints_report_violations_and_block_the_rewrite():
    g = HLGraph()
    x = g.input("x", (8,))
    a = g.op("relu", x)
    b = g.op("tanh", a, layout="channels_last")
    c = g.op("exp", b)
    g.output(c)
    tr = fp.GraphTransformer()
    h = tr.transform(g)
    assert len(h.ops) == 3 and tr.stats.stats.rejected == 1 and tr.stats.stats.rejection_reasons == {"MemoryLayout": 1}
    assert "mixed layouts" in tr.logger.rejected()[0].reason
    ops = [Op("relu", ["x"], "a"), Op("dropout", ["a"], "b")]
    assert not fp.SideEffectConstraint().satisfies(g, ops)
    assert not fp.ControlFlowConstraint().satisfies(g, [Op("loop", [], "l")])
    g.values["i"] = fp.Value("i", (8,), torch.int32)
    g.values["d"] = fp.Value("d", (8,), torch.float64)
    assert not fp.NumericalPrecisionConstraint().satisfies(g, [Op("relu", ["x"], a), Op("cast", [a], "i")])
    assert not fp.NumericalPrecisionConstraint().satisfies(g, [Op("relu", ["x"], a), Op("cast", [a], "d")])
    v = fp.MemoryAccessPatternConstraint().violations(g, [Op("relu", [], a), Op("matmul", [], a), Op("gather", [], a)])
    assert [x.severity for x in v].count(fp.Severity.ERROR) == 2 and v[-1].severity == fp.Severity.WARNING
    lim = fp.LaunchResourceConstraint(threads=2048)
    assert any("threads" in x.message for x in lim.violations(g, [g.ops[0]]))
    small = fp.LaunchResourceConstraint(fp.LaunchLimits(shared_bytes_per_cta=1024))
    assert any("shared" in x.message for x in small.violations(g, [Op("relu", ["x"], "q", {"shared_bytes": 4096})]))
    regs = fp.LaunchResourceConstraint(fp.LaunchLimits(registers_per_sm=4096), threads=256)
    assert any("register file" in x.message for x in regs.violations(g, [g.ops[0], g.ops[1]]))


def test_verifier_catches_a_wrong_rewrite_and_the_handler_falls_back():
    g = _mlp_graph()

    class Broken(fp.GraphTransformer):
        def transform(self, graph):
            h = super().transform(graph)
            h.ops[-1].attrs["chain"][0] = ("sigmoid", False)        # not what the original computes
            return h

    handler = fp.FusionFallbackHandler(Broken(), fp.FusionVerifier())
    assert handler.compile(g) is g and handler.fallbacks == ["verify: outputs differ beyond tolerance"]

    class Raises(fp.GraphTransformer):
        def transform(self, graph):
            raise RuntimeError("boom")
    h2 = fp.FusionFallbackHandler(Raises())
    assert h2.compile(g) is g and h2.fallbacks == ["transform: boom"]

    good = fp.FusionFallbackHandler(verifier=fp.FusionVerifier())
    fused = good.compile(g)
    assert fused is not g and good.fallbacks == []
    feeds = {"x": torch.randn(4, 8), "r": torch.randn(4, 16)}
    fused.ops[-1].kind = "no_such_op"                                # fails at run time -> original runs, fused stays off
    out = good.run(g, fused, feeds)
    assert torch.allclose(out[0], g.run(feeds)[0]) and len(good.fallbacks) == 1
    good.run(g, fused, feeds)
    assert len(good.fallbacks) == 1


def test_benefit_model_and_profiler():
    g = HLGraph()
    x = g.input("x", (1 << 20,), torch.bfloat16)
    v = x
    for k in ("relu", "tanh", "exp", "neg"):
        v = g.op(k, v)
    g.output(v)
    ben = fp.FusionCandidateAnalyzer().analyze(g, [0, 1, 2, 3])
    assert ben.kernel_count_reduction == 3 and ben.memory_saved == 3 * 2 * (1 << 20)
    assert 3.0 < ben.estimated_speedup <= 4.0 and ben.should_fuse()
    assert not fp.FusionCandidateAnalyzer().analyze(g, [0]).should_fuse() and not fp.FusionBenefit.none().should_fuse()
    small = HLGraph()
    y = small.input("y", (4,))
    small.output(small.op("exp", small.op("relu", y)))
    rep = fp.FusionProfiler(fp.KernelTimingInstrument(warmup=1, iters=3)).compare(small, fp.GraphTransformer().transform(small), {"y": torch.randn(4)})
    assert rep.ops_before == 2 and rep.ops_after == 1 and rep.speedup > 0 and "2 ops -> 1 ops" in rep.render()


def test_runtime_shape_injector_specialises_and_caches_per_signature():
    built = []

    def build(shapes):
        built.append(shapes["x"])
        g = HLGraph()
        x = g.input("x", shapes["x"])
        g.output(g.op("tanh", g.op("relu", x)))
        return g

    inj = fp.RuntimeShapeInjector(build, capacity=2)
    for n in (4, 4, 8, 4, 16, 8):
        x = torch.randn(n)
        assert torch.allclose(inj(x=x)[0], torch.tanh(torch.relu(x)))
    assert built == [(4,), (8,), (16,), (8,)] and (inj.hits, inj.misses) == (2, 4)
    _, fused = inj.specialize({"x": torch.randn(16)})
    assert [o.kind for o in fused.ops] == ["fused_elementwise"]


def test_code_generator_helpers():
    g = fp.GraphTransformer().transform(_mlp_graph())
    src = fp.FusionKernelGenerator().source(g.ops[-1], torch.bfloat16, "k_chain")
    assert "k_chain" in src and "tanhf" in src and "__global__" in src
    with pytest.raises(ValueError):
        fp.FusionKernelGenerator().source(g.ops[0])
    assert fp.CudaTypeMapper.cuda_type(torch.bfloat16) == "__nv_bfloat16" and fp.CudaTypeMapper.vector_elems(torch.bfloat16) == 8
    with pytest.raises(KeyError):
        fp.CudaTypeMapper.cuda_type(torch.complex64)
    t = fp.TilingConfiguration.for_gemm(8192, 8192, 2048)
    assert (t.tile_m, t.tile_n, t.tile_k) == (128, 256, 64) and t.fits() and t.stages == 4
    assert fp.TilingConfiguration.for_gemm(256, 512, 4096).tile_n == 64
    plan = fp.SharedMemoryPlanner().plan([("a", 128, 128), ("b", 64, 100), ("stage", 128, 128)], swizzled=["stage"])
    assert plan[0].padded_row_bytes == 144 and plan[1].padded_row_bytes == 100 and plan[2].padded_row_bytes == 128
    assert plan[1].offset % 128 == 0 and plan[2].offset % 1024 == 0 and fp.SharedMemoryPlanner.total(plan) == plan[2].offset + 128 * 128
    with pytest.raises(ValueError):
        fp.SharedMemoryPlanner(limit=1000).plan([("a", 128, 128)])
    mo = fp.MemoryAccessOptimizer()
    assert mo.vector_elems(2, 4096) == 8 and mo.vector_elems(2, 4100) == 4 and mo.vector_elems(2, 4097) == 1 and mo.vector_elems(4, 1024, [0, 8]) == 2
    lu = fp.LoopUnrollingOptimizer()
    assert lu.unroll_factor(1, 8) == 4 and lu.unroll_factor(4, 8) == 2 and lu.unroll_factor(3, 4, register_budget=255) == 2
