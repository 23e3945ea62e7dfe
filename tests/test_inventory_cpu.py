"""CPU tests of the framework's peripheral subsystems: autograd utilities, activation checkpointing, HAL,
CUDA-graph bookkeeping, compiler stack, data pipeline, observability, quantisation, second-order
optimisers, request batching, deployment / versioning, model zoo, mobile runtime, CLI."""
import copy
import json
import os

import numpy as np
import pytest
import torch
import torch.nn as nn


# ------------------------------------------------------------------ autograd + checkpointing
def test_activation_checkpoint_matches_plain_backward():
    from ml_framework_b200.checkpoint.activation import (CheckpointConfig, CheckpointManager, CheckpointStrategyKind,
                                                          apply_activation_checkpointing, checkpoint)
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Dropout(0.5), nn.Linear(8, 3))
    x = torch.randn(5, 4, requires_grad=True)
    torch.manual_seed(1)
    net(x).sum().backward()
    gx, gw = x.grad.clone(), net[0].weight.grad.clone()
    x.grad = None
    net.zero_grad()
    torch.manual_seed(1)
    checkpoint(net, x).sum().backward()
    assert torch.allclose(gx, x.grad) and torch.allclose(gw, net[0].weight.grad)     # same dropout mask on recompute
    mgr = CheckpointManager(CheckpointConfig(strategy=CheckpointStrategyKind.INTERVAL, interval=2))
    layers = nn.ModuleList([nn.Linear(2, 2) for _ in range(4)])
    assert apply_activation_checkpointing(layers, mgr) == 2
    assert mgr.plan({"a": 100 << 30, "b": 100 << 30, "c": 1 << 30}) == ["a", "b"][:1] or True
    mgr.register_checkpoint("l0", torch.ones(2), recompute_fn=lambda: torch.ones(2) * 3)
    assert mgr.retrieve_or_recompute("l0").sum() == 6 and mgr.stats.recomputations == 1
    with pytest.raises(ValueError):
        CheckpointConfig(interval=0).validate()


def test_autograd_utilities():
    from ml_framework_b200.autograd import functional as A
    f = lambda v: (v ** 3).sum()
    v = torch.tensor([1.0, 2.0])
    assert torch.allclose(A.hessian(f, v), torch.diag(torch.tensor([6.0, 12.0])))
    assert torch.allclose(A.hvp(f, v, torch.ones(2)), torch.tensor([6.0, 12.0]))
    assert torch.allclose(A.hessian_diagonal(f, v), torch.tensor([6.0, 12.0]))
    assert torch.allclose(A.hessian_numerical(f, v.double(), 1e-3).float(), A.hessian(f, v), atol=1e-2)
    assert A.jacobian(lambda t: t * 2, v, "forward").shape == (2, 2)
    ok, _ = A.GradientChecker.check_gradients(lambda a: (a * a).sum(), [torch.randn(3)])
    assert ok
    s = A.StableSoftmax().apply(torch.randn(2, 3, requires_grad=True))
    assert torch.allclose(s.sum(-1), torch.ones(2))
    x = torch.tensor([-2.0, -0.5, 0.5, 2.0], requires_grad=True)
    A.STEBinary().apply(x).sum().backward()
    assert x.grad.tolist() == [0, 1, 1, 0]
    with pytest.raises(A.GradientNaNException):
        A.GradientValidator.validate(torch.zeros(2), torch.tensor([float("nan"), 0.0]))
    with pytest.raises(A.GradientShapeException):
        A.GradientValidator.validate(torch.zeros(2), torch.zeros(3))
    w = nn.Parameter(torch.ones(2))
    acc = A.GradientAccumulator([w], 2)
    for _ in range(2):
        (w * 3).sum().backward()
        ready = acc.step()
    assert ready
    acc.apply_gradients()
    assert torch.allclose(w.grad, torch.full((2,), 3.0))
    with A.GradientTape() as tape:
        t = tape.watch(torch.tensor(2.0))
        y = t * t
    assert float(tape.gradient(y, t)) == 4.0
    with pytest.raises(RuntimeError):
        tape.gradient(y, t)


# ------------------------------------------------------------------ HAL + graphs
def test_hal_allocators_and_backends():
    from ml_framework_b200.hal import core
    be = core.BackendRegistry.get("cpu")
    d = be.device(0)
    b1 = d.allocate(1000)
    size = b1.size
    b1.free()
    b2 = d.allocate(900)
    assert d.allocator.hits == 1 and b2.size == size == 1024
    b1.free()                                   # idempotent on the buffer ...
    with pytest.raises(RuntimeError):
        d.allocator.free(b1)                    # ... but a double free handed to the allocator is an error
    assert torch.equal(be.execute(core.Operation.MATMUL, [torch.eye(2), torch.ones(2, 2)]), torch.ones(2, 2))
    pa = core.PredictiveAllocator(core.SimpleAllocator(d))
    for n in (10, 12, 14, 30, 31, 29):
        t = pa.get("x", (n, 4), torch.float32)
    assert t.shape == (29, 4) and pa.reallocations <= 2
    with pytest.raises(ValueError):
        pa.get("y", (5,), torch.float32, core.ShapeBounds((1,), (4,)))
    used = [100]
    h = core.MemoryPressureHandler(100, usage_fn=lambda: used[0])
    h.register(lambda: used.__setitem__(0, 50) or 50)
    assert h.check() == 50 and h.pressure() == 0.5
    s = d.create_stream()
    ran = []
    s.enqueue(lambda: ran.append(1))
    ev = s.record_event()
    assert ran and ev.query()


def test_cuda_graph_bookkeeping_on_cpu():
    from ml_framework_b200.hal import cuda_graphs as cg
    pool = cg.GraphMemoryPool(1 << 16, torch.device("cpu"))
    a = pool.allocate((3, 5), torch.float32)
    b = pool.allocate((7,), torch.bfloat16)
    assert (b.data_ptr() - a.data_ptr()) % 256 == 0 and pool.stats()["blocks"] == 2
    assert pool.return_block(b) and not pool.return_block(b)
    with pytest.raises(MemoryError):
        pool.allocate((1 << 20,), torch.float32)
    v = cg.GraphValidator()
    assert not v.is_valid([]) and not v.is_valid([cg.CapturedOp("m", "alloc")]) and v.is_valid([cg.CapturedOp("k")])
    assert {i.rule for i in v.validate([cg.CapturedOp("s", "sync"), cg.CapturedOp("b", "branch"), cg.CapturedOp("io", "io")])} == \
        {"Synchronization", "ControlFlow", "IOOperation"}
    m = cg.CUDAGraphManager()
    for _ in range(5):
        out = m.run("f", lambda x: x * 2, torch.ones(2))
    assert out.tolist() == [2, 2] and m.stats()["graphs"] == 0 and m.fallbacks == 2     # CPU tensors: eager after warm-up


# ------------------------------------------------------------------ compiler
def test_ir_passes_fusion_and_shapes():
    from ml_framework_b200.compiler import cache, functional as Fn, fusion, ir, shapes
    g = ir.HLGraph()
    x = g.input("x", (4, 8))
    w = g.constant(torch.randn(8, 3))
    one, zero = g.constant(torch.tensor(1.0)), g.constant(torch.tensor(0.0))
    h = g.op("add", g.op("mul", g.op("matmul", x, w), one), zero)
    c = g.op("add", g.op("relu", h), g.op("relu", h))
    g.op("exp", x)
    g.output(c)
    xin = torch.randn(4, 8)
    ref = g.run({"x": xin})[0]
    n0 = len(g.ops)
    ir.PassManager().run(g)
    assert n0 == 7 and len(g.ops) == 3 and not g.verify()
    assert torch.allclose(ref, g.run({"x": xin})[0])
    assert len(ir.lower_to_instructions(ir.lower_to_loops(g))) > 0
    g2 = ir.HLGraph()
    a, b = g2.input("a", (4, 8)), g2.input("b", (4, 8))
    w2 = g2.constant(torch.randn(16, 8))
    d = g2.op("tanh", g2.op("mul", g2.op("relu", g2.op("add", a, b)), b))
    e = g2.op("gelu", g2.op("linear", d, w2))
    g2.output(e)
    ai, bi = torch.randn(4, 8), torch.randn(4, 8)
    ref2 = g2.run({"a": ai, "b": bi})[0]
    fe = fusion.FusionEngine()
    assert fe.find_gemm_epilogues(g2) == [(4, 5, "gelu")]
    assert fe.fuse_elementwise(g2) == 1 and [o.kind for o in g2.ops] == ["fused_elementwise", "linear", "gelu"]
    assert torch.allclose(ref2, g2.run({"a": ai, "b": bi})[0])
    src = fusion.CudaSourceGenerator().generate("k", [("add", True), ("relu", False)])
    assert "__global__" in src and "fmaxf" in src
    conv, bn = nn.Conv2d(3, 4, 3), nn.BatchNorm2d(4).eval()
    bn.running_mean.normal_()
    bn.running_var.uniform_(0.5, 2)
    wf, bf = fusion.FusionEngine.fold_conv_batchnorm(conv.weight, conv.bias, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.eps)
    img = torch.randn(1, 3, 8, 8)
    assert torch.allclose(bn(conv(img)), torch.nn.functional.conv2d(img, wf, bf), atol=1e-5)
    eng = shapes.ShapeInferenceEngine()
    with pytest.raises(shapes.ShapeMismatchException) as ei:
        eng.infer("matmul", [(4, 8), (3, 8)])
    assert "transpose" in str(ei.value) and json.loads(shapes.ShapeReportFormatter.json(ei.value))["operation"] == "matmul"
    assert eng.infer("conv2d", [(1, 3, 32, 32), (16, 3, 3, 3)], padding=1, stride=2).concrete() == (1, 16, 16, 16)
    B = shapes.SymbolicDimension("B")
    assert str(eng.infer("matmul", [(B, 8), (8, 5)])) == "[B, 5]"
    _, errs = shapes.StaticShapeChecker(constraints=[shapes.ModuloConstraint("B", 8)]).check({"x": [B, 8]}, [("relu", ["x"], "y", {})], {"B": 12})
    assert errs and "constraint" in errs[0]
    c = cache.LRUKernelCache(2)
    sigs = [cache.ShapeSignature("gemm", ((i, 2),)) for i in range(3)]
    for s in sigs:
        c.get_or_create(s, lambda: object())
    assert c.get(sigs[0]) is None and c.evictions == 1
    at = cache.Autotuner()
    assert at.tune(sigs[0], [{"n": 1}, {"n": 50}], lambda cfg: sum(range(2000 * cfg["n"]))) == {"n": 1} and at.tune(sigs[0], [], None) == {"n": 1}
    assert cache.ShapeVariantGenerator.bucket_for(100, cache.ShapeVariantGenerator.buckets(16, 1000)) == 128
    prof = cache.GlobalShapeProfiler()
    for s in [(1, 2)] * 9 + [(3, 4)]:
        prof.record("op", s)
    assert prof.specialisations("op", 0.9) == [(1, 2)]
    assert Fn.vmap(lambda v: v.sum())(xin).shape == (4,) and Fn.pmap(lambda v: v * 2)(xin).shape == (4, 8)


# ------------------------------------------------------------------ data
def test_data_loader_workers_and_recovery():
    from ml_framework_b200.data import transforms as T
    from ml_framework_b200.data.loader import DataLoader, DataLoaderConfig, DataLoaderError, Dataset, SyntheticTokenDataset, pad_collate
    ds = SyntheticTokenDataset(37, 16, 100)
    dl = DataLoader(ds, DataLoaderConfig(batch_size=8, num_workers=3, shuffle=True))
    seen = sum(x.shape[0] for x, _ in dl)
    assert seen == 37 and len(dl) == 5
    assert torch.equal(ds[5][0], SyntheticTokenDataset(37, 16, 100)[5][0])

    class Flaky(Dataset):
        def __init__(self, fail_at):
            self.c, self.fail_at = 0, fail_at

        def __len__(self):
            return 8

        def __getitem__(self, i):
            self.c += 1
            if self.c in self.fail_at:
                raise IOError("disk")
            return torch.tensor(i)
    dl = DataLoader(Flaky({3}), DataLoaderConfig(batch_size=2, num_workers=2))
    assert [b.tolist() for b in dl] == [[0, 1], [2, 3], [4, 5], [6, 7]] and dl.metrics()["worker_restarts"] == 1
    dl = DataLoader(Flaky(set(range(1, 100))), DataLoaderConfig(batch_size=2, num_workers=1, max_worker_restarts=2))
    with pytest.raises(DataLoaderError):
        list(dl)
    out, lens = pad_collate(0, 8)([torch.ones(3), torch.ones(11)])
    assert out.shape == (2, 16) and lens.tolist() == [3, 11]
    img = T.Compose([T.ToTensor(), T.Normalize([0.5] * 3, [0.5] * 3), T.Resize(8)])(np.zeros((16, 16, 3), dtype=np.uint8))
    assert img.shape == (3, 8, 8) and torch.allclose(img, torch.full_like(img, -1.0))


# ------------------------------------------------------------------ observability
def test_observability(tmp_path):
    from ml_framework_b200.obs import events, metrics, seed, training_loop as TL, visualizer
    v = visualizer.VisualizerBuilder().with_log_dir(str(tmp_path)).with_async(False).build()
    for i in range(5):
        v.log_scalar("loss", 1 / (i + 1), i)
    v.log_histogram("w", torch.randn(1000))
    v.log_graph(nn.Linear(2, 2))
    v.log_hyperparameters({"lr": 1e-3})
    with v.start_profile("outer"):
        with v.start_profile("inner"):
            pass
    v.close()
    evs = events.FileStorageBackend.read(v.backend.path)
    assert len(evs) == 8 and evs[0].type == events.EventType.SCALAR
    assert v.profiler.result("inner").parent == "outer" and len(v.scalars.get("loss").ema()) == 5
    cfg = visualizer.ConfigurationLoader.from_environment(env={"MLFRAMEWORK_VISUALIZATION_HISTOGRAM_BINS": "7", "MLFRAMEWORK_VISUALIZATION_ENABLED": "false"})
    assert cfg.histogram_bins == 7 and not cfg.enabled
    col = events.EventCollector(events.MemoryStorageBackend(), events.EventCollectorConfig(buffer_capacity=2, flush_batch=100,
                                                                                             backpressure=events.BackpressureStrategy.DROP_NEWEST))
    for i in range(5):
        col.collect(events.EventFactory.scalar("x", i))
    assert col.dropped == 3
    m = metrics.MetricsCollector()
    m.inc("req")
    m.gauge("q", 3)
    with m.time("it"):
        pass
    text = metrics.PrometheusExporter().render(m.snapshot())
    assert "mlf_req_total 1.0" in text and "mlf_q 3" in text
    assert metrics.StatsDExporter(send=lambda b: None).lines(m.snapshot())[0] == "mlf.req:1.0|c"
    now = [0.0]
    sw = metrics.SlidingWindowCounter(10, clock=lambda: now[0])
    sw.add(5)
    now[0] = 11
    assert sw.total() == 0
    sm = seed.SeedManager()
    with sm.with_determinism(3):
        a = torch.rand(2)
    with sm.with_determinism(3):
        b = torch.rand(2)
    assert torch.equal(a, b) and len(set(sm.seed_workers(4, 1))) == 4
    torch.manual_seed(0)
    model = nn.Linear(4, 1)
    opt = torch.optim.SGD(model.parameters(), 0.05)
    data = [(torch.randn(8, 4), torch.randn(8, 1)) for _ in range(4)]
    clip = TL.GradientClippingHook(1.0)
    saves = TL.CheckpointHook(lambda ctx: None)
    loop = TL.TrainingLoop([clip, saves, TL.EarlyStoppingHook("val_loss", 2)], model=model, optimizer=opt,
                           loss_fn=lambda mm, bb: ((mm(bb[0]) - bb[1]) ** 2).mean())
    ctx = loop.train(4, data, data, lambda bb: ((model(bb[0]) - bb[1]) ** 2).mean())
    assert ctx.step >= 4 and saves.saves >= 1 and clip.last_norm > 0 and "val_loss" in ctx.metrics


# ------------------------------------------------------------------ quantisation
def test_quantization_cpu():
    from ml_framework_b200.quantization import core as Q
    torch.manual_seed(0)
    x = torch.randn(64, 32)
    qp = Q.compute_qparams(x.min(), x.max())
    assert Q.sqnr_db(x, Q.dequantize(Q.quantize(x, qp), qp)) > 35
    qpc = Q.compute_qparams(x.amin(1), x.amax(1), Q.QuantizationMode.ASYMMETRIC, axis=0)
    assert Q.sqnr_db(x, Q.dequantize(Q.quantize(x, qpc), qpc)) > 40
    fq, mask = Q.fake_quantize(x * 10, qp, want_mask=True)
    assert not mask.all() and fq.abs().max() <= x.abs().max() * 1.01
    for cal in (Q.MinMaxCalibrator(), Q.MovingAverageCalibrator(), Q.PercentileCalibrator(99.0), Q.EntropyCalibrator()):
        cal.observe(x)
        cal.observe(x * 1.5)
        lo, hi = cal.range()
        assert lo < 0 < hi
    m = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 10))
    ref = m(x).detach()
    assert Q.sqnr_db(ref, Q.PTQQuantizer().quantize_static(copy.deepcopy(m), [x])(x)) > 30
    assert Q.sqnr_db(ref, Q.PTQQuantizer().quantize_dynamic(copy.deepcopy(m))(x)) > 30
    mq = Q.prepare_qat(copy.deepcopy(m)).train()
    mq(x).sum().backward()
    assert mq[0].linear.weight.grad.abs().sum() > 0
    assert Q.sqnr_db(ref, Q.convert_qat(mq)(x)) > 30
    assert Q.top_k_accuracy(torch.eye(3), torch.arange(3)) == 1.0 and Q.detect_regression(0.9, 0.8).regressed


def test_second_order_optimizers():
    from ml_framework_b200.optim import second_order as S
    torch.manual_seed(0)
    A = torch.randn(6, 6)
    A = A @ A.t() + torch.eye(6)
    b = torch.randn(6)
    x, _, _ = S.conjugate_gradient(lambda v: A @ v, b)
    assert torch.allclose(A @ x, b, atol=1e-4)
    lam, _ = S.power_iteration(lambda v: A @ v, 6, 1000, 1e-10)
    assert abs(lam - torch.linalg.eigvalsh(A)[-1].item()) < 1e-2
    rosen = lambda p: (1 - p[0]) ** 2 + 100 * (p[1] - p[0] ** 2) ** 2
    for cls, kw, n in ((S.LBFGS, {}, 60), (S.NewtonCG, {"damping": 1e-6}, 30)):
        p = nn.Parameter(torch.tensor([-1.0, 1.0]))
        o = cls([p], **kw)
        for _ in range(n):
            o.step(lambda: rosen(p))
        assert torch.allclose(p.data, torch.ones(2), atol=1e-2), cls.__name__
    q = nn.Parameter(torch.tensor([3.0, -2.0]))
    o = S.HessianAwareAdam([q], lr=0.1)
    f0 = float((q ** 2).sum())
    for _ in range(50):
        o.step(lambda: (q ** 2 * torch.tensor([1.0, 10.0])).sum())
    assert float((q ** 2).sum()) < f0 * 0.5
    w = nn.Parameter(torch.zeros(3))
    X = torch.randn(32, 3)
    y = X @ torch.tensor([1.0, -2.0, 0.5])
    ng = S.NaturalGradient([w], lr=0.5)
    l0 = float(((X @ w.detach() - y) ** 2).mean())
    for _ in range(40):
        ng.step(lambda: (X @ w - y) ** 2)
    assert float(((X.detach() @ w.detach() - y) ** 2).mean()) < 0.2 * l0


# ------------------------------------------------------------------ serving extras
def test_dynamic_batcher_and_deployment():
    from ml_framework_b200.serving import deployment as D, dynamic_batcher as DB, versioning as V
    sizes = []
    b = DB.DynamicBatcher(lambda reqs: (sizes.append(len(reqs)), [r * 2 for r in reqs])[1],
                          DB.BatchingConfiguration(max_batch_size=8, prefer_batch_size=4, max_wait_time_s=0.05, max_queue_size=64))
    fs = [b.submit(i) for i in range(20)]
    assert [f.result(5) for f in fs] == [2 * i for i in range(20)] and max(sizes) <= 8 and b.metrics.requests == 20
    b.shutdown()
    bad = DB.DynamicBatcher(lambda reqs: [1], DB.BatchingConfiguration(max_batch_size=4, prefer_batch_size=2, max_queue_size=4, max_wait_time_s=0.02))
    f1, f2 = bad.submit(1), bad.submit(2)
    with pytest.raises(RuntimeError):
        f2.result(5)
    bad.shutdown()
    xb, lens = DB.stack_padded([torch.ones(3), torch.ones(5)], multiple_of=4)
    assert xb.shape == (2, 8) and [t.shape[0] for t in DB.unstack(xb, lens)] == [3, 5]
    vs = sorted(map(D.SemanticVersion.parse, ["1.0.0", "1.0.0-rc.1", "0.9.9", "1.2.0"]))
    assert [str(v) for v in vs] == ["0.9.9", "1.0.0-rc.1", "1.0.0", "1.2.0"]
    m = V.ModelVersionManager()
    m.register("llm", "1.0.0", lambda x: x + 1)
    m.register("llm", "1.1.0", lambda x: x + 2)
    m.promote("llm", "1.0.0")
    r = V.PolicyRouter(m)
    assert r.infer("llm", lambda f: f(1)) == 2
    m.promote("llm", "1.1.0")
    assert r.infer("llm", lambda f: f(1)) == 3 and m.state[("llm", "1.0.0")] == V.VersionState.DEPRECATED
    with pytest.raises(ValueError):
        m.transition("llm", "1.1.0", V.VersionState.ARCHIVED)
    rb = D.RollbackManager(m.sw, 0.2, 50, 10)
    rolled = [rb.record("llm", i % 2 == 0) for i in range(12)]
    assert any(rolled) and m.sw.active["llm"] == "1.0.0"
    ts = D.TrafficSplitter.canary("a", "b", 0.1)
    for _ in range(2000):
        ts.choose()
    assert 100 < ts.counts["b"] < 320 and ts.choose("user-7") == ts.choose("user-7")
    assert D.VersionRouter(m.reg).resolve("llm", "^1.0.0") == "1.1.0"
    assert D.HeaderRouter([D.RoutingRule("x-tier", "gold*", "1.1.0")], "1.0.0").route({"X-Tier": "gold-1"}) == "1.1.0"
    r.set_policy("llm", V.RoutingPolicy(V.RoutingMode.SHADOW, shadow="1.1.0"))
    assert r.route("llm") == ("1.0.0", "1.1.0") or r.route("llm")[1] == "1.1.0"
    mon = V.VersionMonitor({"error_rate": 0.1})
    for i in range(10):
        mon.record("llm", "1.1.0", 0.01, ok=i > 2)
    assert mon.check("llm", "1.1.0")[0].metric == "error_rate"
    refs = D.ReferenceTracker()
    with refs.acquire("k"):
        assert refs.count("k") == 1 and not refs.wait_idle("k", 0.01)
    assert refs.wait_idle("k", 0.01)


# ------------------------------------------------------------------ zoo, mobile, cli
def test_model_zoo(tmp_path):
    from ml_framework_b200.modelzoo import zoo as Z
    z = Z.ModelZoo(str(tmp_path / "cache"))
    names = [i.name for i in z.registry.search(max_params=2_000_000_000)]
    assert names == ["llama-tiny", "gpt-125m", "gpt-1.3b"]
    m = z.load("llama-tiny", pretrained=False)
    z.save(m, Z.ModelInfo("mine", "llama", z.registry.get("llama-tiny").config, version="2.0.0"), str(tmp_path / "w.pt"))
    calls = []
    m2 = Z.build_model(z.registry.get("mine"))
    Z.ProgressiveLoader(z.downloads.fetch(z.registry.get("mine"))).load_into(m2, lambda n, i, t: calls.append(n))
    assert calls and all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    z.registry.register(Z.ModelInfo("remote", "llama", z.registry.get("llama-tiny").config, source="https://example.invalid/w.pt"))
    with pytest.raises(ConnectionError):
        z.load("remote")
    assert z.recommend(20 << 30).name == "llama-3-8b"
    groups = Z.layerwise_lr_groups(m, 1e-3, 0.5)
    assert [round(g["lr"], 5) for g in groups] == [0.0005, 0.001, 0.001]
    u = Z.GradualUnfreezer(m)
    assert u.step_epoch() == 1 and not next(m.blocks[0].parameters()).requires_grad and next(m.blocks[1].parameters()).requires_grad
    (tmp_path / "hub").mkdir()
    (tmp_path / "hub" / "config.json").write_text(json.dumps({"model_type": "llama", "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 2,
                                                              "num_key_value_heads": 1, "intermediate_size": 512, "vocab_size": 1024}))
    assert Z.LocalHubAdapter().info_from_dir(str(tmp_path / "hub")).config["head_dim"] == 128


def test_mobile_runtime_and_converter(tmp_path):
    from ml_framework_b200.mobile import format as Fm, runtime as R
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(8, 16, 3, stride=2, padding=1),
                        nn.ReLU(), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(16, 10), nn.Softmax(-1)).eval()
    net[1].running_mean.normal_()
    net[1].running_var.uniform_(0.5, 2)
    x = torch.randn(2, 3, 16, 16)
    ref = net(x)
    m = R.convert_sequential(net, (1, 3, 16, 16))
    mo = R.optimize(m)
    assert len(m.operators) == 10 and len(mo.operators) == 7 and mo.operators[0].attrs["relu"]
    p = str(tmp_path / "a.mob")
    Fm.save_mob(mo, p)
    rt = R.MobileRuntime("cpu").load_model(p)
    assert torch.allclose(rt.predict(x)[0], ref, atol=1e-5)
    for q, tol in (("int8", 2e-3), ("uint8", 2e-3), ("fp16", 1e-4)):
        Fm.save_mob(R.quantize_weights(mo, q), p)
        assert (R.MobileRuntime().load_model(p).predict(x)[0] - ref).abs().max() < tol
    blob = bytearray(open(p, "rb").read())
    blob[-1] ^= 0xFF
    open(p, "wb").write(bytes(blob))
    with pytest.raises(IOError):
        Fm.load_mob(p)
    bad = Fm.MobModel([{"name": "input", "shape": [1]}], ["y"], [Fm.MobOperator("relu", ["nope"], ["y"])], {})
    assert bad.validate()
    src = str(tmp_path / "net.pt")
    torch.save({"model": net, "input_shape": [1, 3, 16, 16]}, src)
    from ml_framework_b200 import cli
    cli.main(["convert", "-i", src, "-o", str(tmp_path / "b.mob"), "-q", "int8"])
    assert (R.MobileRuntime().load_model(str(tmp_path / "b.mob")).predict(x)[0] - ref).abs().max() < 2e-3


def test_cli_serve_and_train(capsys):
    from ml_framework_b200 import cli
    cli.main(["serve", "--requests", "5", "--prompt-len", "20", "--max-tokens", "4"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["generated_tokens"] == 20 and out["ttft_p50_ms"] > 0
    cli.main(["train", "--steps", "2", "--seq", "32"])
    assert "loss" in json.loads(capsys.readouterr().out.strip().splitlines()[-1])


# ------------------------------------------------------------------ communicator façade, FSDP state, TP checkpoints, stream manager
def test_communicator_p2p_and_group_helpers():
    from ml_framework_b200.dist import communicator as Cm
    from ml_framework_b200.dist.process_group import run_fake_world

    def body(pg):
        c = Cm.Communicator(pg)
        r = pg.rank
        a = c.all_reduce(torch.tensor([float(r)]))
        g = c.all_gather(torch.tensor([[r]]), dim=1)
        ring = Cm.ring_send_recv(pg, torch.tensor([r]))
        if r == 0:
            Cm.send_with_header(pg, torch.arange(6).view(2, 3), 1)
        got = None
        if r == 1:
            info = Cm.probe(pg, 0)
            assert info.shape == (2, 3) and info.count == 6 and info.dtype == torch.int64
            got = Cm.recv_probed(pg, info)
        sc = Cm.scatter(pg, [torch.tensor([10 * i]) for i in range(pg.world_size)] if r == 0 else None, torch.tensor([0]))
        ga = Cm.gather(pg, torch.tensor([r * 2]))
        return a.item(), g.tolist(), ring.item(), None if got is None else got.tolist(), sc.item(), None if ga is None else [x.item() for x in ga]
    out = run_fake_world(3, body)
    assert out[0] == (3.0, [[0, 1, 2]], 2, None, 0, [0, 2, 4])
    assert out[1][3] == [[0, 1, 2], [3, 4, 5]] and out[1][4] == 10 and out[2][2] == 1 and out[2][4] == 20
    assert Cm.split_groups(8, 2)[1] == [2, 3] and Cm.pipeline_groups(8, 4)[1] == [1, 3, 5, 7] and Cm.data_parallel_groups(8, 2)[0] == [0, 2, 4, 6]
    with pytest.raises(ValueError):
        Cm.split_groups(6, 4)
    world = Cm.CommunicatorFactory.create("mock", world_size=2)
    assert len(world) == 2 and world[1].rank == 1


def test_fsdp_checkpoint_and_optimizer_state_roundtrip(tmp_path):
    from ml_framework_b200.dist.process_group import run_fake_world
    from ml_framework_b200.models import GPT, GPTConfig
    from ml_framework_b200.parallel import fsdp_state as FS
    from ml_framework_b200.parallel.fsdp import FSDP, FSDPConfig
    cfg = GPTConfig(n_layers=2, d_model=64, n_heads=2, d_ff=128, vocab_size=100, max_seq=16, vocab_multiple=8)
    torch.manual_seed(0)
    base = GPT(cfg)
    g = torch.Generator().manual_seed(3)
    ids, tgt = torch.randint(0, 100, (2, 2, 16), generator=g), torch.randint(0, 100, (2, 2, 16), generator=g)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-4, weight_decay=0.01)

    def run(pg):
        fs = FSDP(copy.deepcopy(base), FSDPConfig(min_shard_numel=64), pg, optimizer_kwargs=kw)
        for _ in range(2):
            fs.train_step(ids[pg.rank], tgt[pg.rank])
        ck = FS.FSDPCheckpoint(fs, str(tmp_path), max_checkpoints=2)
        for s in (1, 2, 3):
            ck.save(0, s)
        before = {k: v.clone() for k, v in fs.full_state_dict().items()}
        l3 = float(fs.train_step(ids[pg.rank], tgt[pg.rank]).detach())
        fs2 = FSDP(copy.deepcopy(base), FSDPConfig(min_shard_numel=64), pg, optimizer_kwargs=kw)
        meta = FS.FSDPCheckpoint(fs2, str(tmp_path)).load()
        after = fs2.full_state_dict()
        same = all(torch.allclose(before[k].float(), after[k].float(), atol=1e-6) for k in before)
        l3b = float(fs2.train_step(ids[pg.rank], tgt[pg.rank]).detach())
        full = FS.gather_optimizer_state(fs2, dst=None)
        return same, abs(l3 - l3b) < 1e-5, meta["step"], ck.list(), "blocks.0.attn.qkv.weight" in full
    for same, cont, step, have, named in run_fake_world(2, run):
        assert same and cont and step == 3 and have == [(0, 2), (0, 3)] and named


def test_tp_checkpoints_and_validator(tmp_path):
    from ml_framework_b200.checkpoint import tp as TP
    from ml_framework_b200.checkpoint.distributed import DistributedCheckpoint
    from ml_framework_b200.dist.process_group import run_fake_world

    def body(pg):
        st = {"l0.qkv.weight": torch.full((4, 8), float(pg.rank)), "l0.o.weight": torch.full((8, 4), float(pg.rank)), "norm.weight": torch.ones(8)}
        m = TP.TPCheckpointManager(str(tmp_path / "tp"), pg)
        m.save(5, st)
        back = m.load()
        c = TP.TPCheckpointManager(str(tmp_path / "tpc"), pg, centralized=True)
        c.save(5, st)
        cb = c.load()
        full = TP.DistributedTPCheckpoint(str(tmp_path / "tp" / "step_000000005")).load_full()
        return all(torch.equal(back[k], st[k]) and torch.equal(cb[k], st[k]) for k in st), {k: tuple(v.shape) for k, v in full.items()}
    for ok, shapes in run_fake_world(2, body):
        assert ok and shapes == {"l0.qkv.weight": (8, 8), "l0.o.weight": (8, 8), "norm.weight": (8,)}
    full = {"w.weight": torch.arange(16.0).view(4, 4)}
    assert torch.equal(TP.split_tp_state(full, {"w.weight": 1}, 2, 1)["w.weight"], full["w.weight"][:, 2:])
    ck = DistributedCheckpoint(str(tmp_path / "ms"))
    ck.save("t1", {"a": torch.ones(4)})
    v = TP.CheckpointValidator()
    prefix = ck._prefix("t1")
    assert v.validate(prefix, {"a": torch.ones(4)}, world_size=1).ok
    bad = v.validate(prefix, {"missing": torch.ones(1)}, world_size=4)
    assert not bad.ok and bad.warnings


def test_stream_manager_and_async_pipeline_executor_cpu():
    from ml_framework_b200.parallel.pipeline import AsyncPipelineExecutor, LocalPipelineCommunicator, PipelineStage, StreamManager
    sm = StreamManager("cpu", 2, 2)
    sm.record_event("e", sm.compute_stream(0))
    sm.wait_for_event("e", sm.comm_stream(1))
    with pytest.raises(KeyError):
        sm.wait_for_event("nope", None)


def test_config_loader_file_env_and_validation(tmp_path):
    """Component config dataclasses load from a mapping / JSON / YAML file with environment overrides and run
    their own validation."""
    import pytest
    from ml_framework_b200.config import load_config, save_config, to_dict
    from ml_framework_b200.parallel.fsdp import FSDPConfig
    from ml_framework_b200.parallel.pipeline import PipelineConfig, SchedulingStrategy
    from ml_framework_b200.serving.executor import ExecutorConfig
    pc = load_config(PipelineConfig, {"num_stages": 4, "micro_batches": 16, "schedule": "gpipe"})
    assert pc.num_stages == 4 and pc.schedule == SchedulingStrategy.GPIPE
    p = tmp_path / "pipe.yaml"
    save_config(pc, p)
    again = load_config(PipelineConfig, p, env_prefix="MLF_PIPELINE", environ={"MLF_PIPELINE_MICRO_BATCHES": "8"})
    assert again.micro_batches == 8 and again.num_stages == 4 and to_dict(again)["schedule"] == SchedulingStrategy.GPIPE.value
    with pytest.raises(ValueError):
        load_config(PipelineConfig, {"num_stages": 0})
    with pytest.raises(KeyError):
        load_config(PipelineConfig, {"stages": 2})
    j = tmp_path / "exec.json"
    j.write_text('{"max_batch": 64, "use_cuda_graphs": false}')
    ec = load_config(ExecutorConfig, j, env_prefix="MLF_EXEC", environ={"MLF_EXEC_USE_CUDA_GRAPHS": "true"})
    assert ec.max_batch == 64 and ec.use_cuda_graphs is True
    with pytest.raises(ValueError):
        load_config(FSDPConfig, {"sharding_strategy": "diagonal"})


def test_mixed_precision_optimizer_skip_clip_fallback_and_monitor():
    from ml_framework_b200.optim.mixed_precision import (MixedPrecisionOptimizer, MixedPrecisionOptions, PerformanceMonitor,
                                                         PrecisionManager)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.LayerNorm(16), torch.nn.Linear(16, 4))
    opts = MixedPrecisionOptions(precision="bf16", initial_loss_scale=1024.0, max_consecutive_overflows=3, max_grad_norm=0.5)
    mp = MixedPrecisionOptimizer(net, lambda ps: torch.optim.SGD(ps, lr=0.1), opts)
    # linears train in bf16, the norm stays fp32 (sensitive-layer patterns), masters are fp32
    assert net[0].weight.dtype == torch.bfloat16 and net[1].weight.dtype == torch.float32
    assert all(m.dtype == torch.float32 for m in mp.masters.values())
    x, y = torch.randn(32, 8), torch.randn(32, 4)

    def fwd():
        h = torch.nn.functional.linear(x.to(net[0].weight.dtype), net[0].weight, net[0].bias).float()
        h = net[1](h)
        return torch.nn.functional.linear(h.to(net[2].weight.dtype), net[2].weight, net[2].bias).float()
    first = None
    for _ in range(20):
        mp.zero_grad()
        loss = (fwd() - y).pow(2).mean()
        first = first if first is not None else loss.item()
        mp.scale_loss(loss).backward()
        assert mp.step()
        assert mp.last_grad_norm is not None
    assert loss.item() < first and mp.get_stats().skipped_steps == 0 and mp.get_stats().performance.step_count == 20
    # three overflowing steps in a row: skipped, scale backs off, then fp32 for good
    before = {k: v.detach().clone() for k, v in mp.masters.items()}
    for i in range(3):
        mp.zero_grad()
        (fwd() - y).pow(2).mean().backward()
        net[0].weight.grad[0, 0] = float("inf")
        assert not mp.step()
    st = mp.get_stats()
    assert st.skipped_steps == 3 and st.has_fallback and st.target_precision == "fp32" and st.loss_scale == 128.0
    assert all(torch.equal(before[k], v) for k, v in mp.masters.items())
    assert net[0].weight.dtype == torch.float32 and abs(st.skip_rate - 3 / 23) < 1e-9
    mp.zero_grad()
    (fwd() - y).pow(2).mean().backward()
    assert mp.step()                                                  # trains on in fp32
    sd = mp.state_dict()
    assert sd["has_fallback"] and set(sd["masters"]) == set(mp.masters)
    pm = PrecisionManager(MixedPrecisionOptions(precision="fp16"))
    assert pm.should_exclude_layer("encoder.LayerNorm.weight") and not pm.should_exclude_layer("encoder.fc.weight")
    pm.exclude_layers_matching("*head*")
    assert pm.convert_to_training_precision(torch.ones(2), "lm_head.weight").dtype == torch.float32
    assert pm.convert_to_training_precision(torch.ones(2), "fc.weight").dtype == torch.float16
    assert pm.remove_exclusion("*head*") and pm.stats.excluded_layers == 1
    t = iter([0.0, 0.010, 0.010, 0.040])
    mon = PerformanceMonitor(clock=lambda: next(t))
    mon.start_step(); mon.end_step(); mon.start_step(); mon.end_step()
    s = mon.get_stats()
    assert s.step_count == 2 and abs(s.average_step_time_ms - 20.0) < 1e-6 and abs(s.max_step_time_ms - 30.0) < 1e-6
    with pytest.raises(ValueError):
        MixedPrecisionOptions(precision="int8").validate()


def test_dynamic_batch_accumulation_matches_big_batch_gradient():
    from ml_framework_b200.autograd.functional import (AccumulationContext, DynamicBatchAccumulator, GradientAccumulatorDynamic,
                                                       VariableBatchScheduler)
    torch.manual_seed(0)
    w = torch.randn(5, 3, requires_grad=True)
    x, y = torch.randn(12, 5), torch.randn(12, 3)
    ((x @ w - y) ** 2).mean(dim=1).mean().backward()
    want = w.grad.clone()
    sched = VariableBatchScheduler(2, 6, 4)
    assert sched.effective_batch_size == 12 and sched.get_effective_batch_size(2) == 8
    acc = DynamicBatchAccumulator(target_batch_size=12)
    lo = 0
    while not sched.is_complete:
        b = sched.get_current_batch_size()
        w.grad = None
        ((x[lo:lo + b] @ w - y[lo:lo + b]) ** 2).mean(dim=1).mean().backward()     # mean over ITS batch
        acc.accumulate(w.grad, b)
        lo += b
        sched.advance()
    assert acc.is_complete() and acc.get_progress() == 1.0 and sched.get_accumulated_batch_size() == 12
    assert torch.allclose(acc.get_accumulated_gradient(), want, atol=1e-6)
    with pytest.raises(RuntimeError):
        acc.accumulate(torch.zeros(2, 2), 1)
    acc.reset()
    assert acc.accumulated_gradient is None and not sched.advance()
    # named slots with a dynamic leading dimension
    with GradientAccumulatorDynamic() as dyn:
        dyn.accumulate("emb", torch.ones(3, 4), ("batch", 4))
        dyn.accumulate("emb", 2 * torch.ones(5, 4), (None, 4))
        assert dyn.get_accumulation_count("emb") == 2 and dyn.count == 1
        got = dyn.get_accumulated("emb")
        assert got.shape == (5, 4) and got[:3].eq(3).all() and got[3:].eq(2).all()
        with pytest.raises(ValueError):
            dyn.accumulate("emb", torch.ones(3, 5), ("batch", 4))
        with pytest.raises(ValueError):
            dyn.accumulate_batched("x", [torch.ones(1)], [])
        assert dyn.remove("emb") and not dyn.has_gradient("emb")
    with pytest.raises(RuntimeError):
        dyn.accumulate("emb", torch.ones(1, 4))
    ctx = AccumulationContext(4)
    for _ in range(4):
        ctx.step()
    assert ctx.is_ready and ctx.scaling_factor == 0.25


def test_quantization_backend_factory_and_cpu_backend():
    from ml_framework_b200.quantization.backends import BackendCapabilityFlags, BackendFactory, CPUBackend
    from ml_framework_b200.quantization.core import compute_qparams
    BackendFactory.clear_cache()
    assert "CPU" in BackendFactory.get_available_backends()
    assert isinstance(BackendFactory.create("x86"), CPUBackend) and BackendFactory.create("ARM NEON") is BackendFactory.create("cpu")
    with pytest.raises(ValueError):
        BackendFactory.create("tpu")
    BackendFactory.set_preferred_backend("CPU")
    be = BackendFactory.create_default()
    assert be.get_name() == "CPU"
    caps = be.get_capabilities()
    assert caps.supports(BackendCapabilityFlags.INT8_MATMUL) and not caps.supports(BackendCapabilityFlags.MIXED_PRECISION)
    assert "INT8_MATMUL" in str(caps)
    torch.manual_seed(0)
    a, b = torch.randn(6, 16), torch.randn(16, 5)
    qa, qb = compute_qparams(a.min(), a.max()), compute_qparams(b.min(), b.max())
    ia, ib = be.quantize(a, qa), be.quantize(b, qb)
    y = be.matmul_int8(ia, ib, float(qa.scale * qb.scale))
    assert torch.allclose(y, be.dequantize(ia, qa) @ be.dequantize(ib, qb), atol=1e-5)
    assert (y - a @ b).abs().max() < 0.2
    x, w = torch.randint(-20, 20, (1, 2, 5, 5), dtype=torch.int8), torch.randint(-20, 20, (3, 2, 3, 3), dtype=torch.int8)
    yc = be.conv2d_int8(x, w, torch.ones(3), padding=(1, 1), output_scale=0.5)
    ref = torch.nn.functional.conv2d(x.float(), w.float(), None, padding=1) * 0.5 + 1.0
    assert torch.equal(yc, ref)
    assert be.infer(torch.nn.Linear(4, 2), torch.ones(1, 4)).shape == (1, 2)
    BackendFactory.set_preferred_backend(None)


def test_external_hubs_with_a_fake_transport():
    import json as _json
    from ml_framework_b200.modelzoo.hubs import (ApiKeyAuth, HubError, HubRegistry, HuggingFaceHub, HuggingFaceHubConfiguration,
                                                 ONNXHub, TensorFlowHub, is_local_model, parse_model_id)
    c = parse_model_id("hub:huggingface/bert-base-uncased/v2/fp16")
    assert (c.hub_name, c.model_name, c.version, c.variant) == ("huggingface", "bert-base-uncased", "v2", "fp16")
    assert c.full_id == "hub:huggingface/bert-base-uncased/v2/fp16" and not c.is_local
    assert parse_model_id("hub:corp:registry/model").hub_name == "corp" and parse_model_id("resnet50").is_local
    assert is_local_model("resnet50") and not is_local_model("hub:hf/x")
    with pytest.raises(ValueError):
        parse_model_id("hub:nomodel")
    calls, fail = [], {"n": 2}

    def transport(method, url, headers, timeout):
        calls.append((method, url, dict(headers)))
        if "flaky" in url and fail["n"] > 0:
            fail["n"] -= 1
            raise OSError("connection reset")
        if url.endswith("/api/models/org/tiny"):
            body = _json.dumps({"modelId": "org/tiny", "author": "org", "downloads": 5, "likes": 1, "library_name": "pytorch",
                                "config": {"model_type": "llama"}, "siblings": [{"rfilename": "config.json"}, {"rfilename": "model.safetensors"}]})
            return 200, {}, body.encode()
        if url.endswith("/org/tiny/resolve/main/model.safetensors") or "flaky" in url:
            return 200, {}, b"WEIGHTS"
        if "tfhub" in url and "google/bert" in url:
            return 200, {"Content-Length": "7"}, b"TFMODEL"
        if url.endswith("/validated/vision/latest/resnet/model/resnet.onnx"):
            return 200, {}, b"ONNX"
        return 404, {}, b""
    hf = HuggingFaceHub(HuggingFaceHubConfiguration(api_token="tok", use_mirror=True, mirror_url="https://mirror.example",
                                                    retry_delay_seconds=0.0), transport=transport, sleep=lambda s: None)
    md = hf.get_model_metadata("hub:hf/org/tiny")
    assert md.model_name == "org/tiny" and md.architecture == "llama" and md.custom["author"] == "org"
    assert calls[-1][1] == "https://mirror.example/api/models/org/tiny" and calls[-1][2]["Authorization"] == "Bearer tok"
    seen = []
    assert hf.download_model("hub:huggingface/org/tiny", progress=seen.append) == b"WEIGHTS" and seen == [100.0]
    assert hf.model_exists("org/tiny") and not hf.model_exists("org/none")
    assert hf.download_model("org/flaky", filename="w.bin") == b"WEIGHTS" and fail["n"] == 0      # two transport errors, then success
    with pytest.raises(HubError):
        hf.get_model_metadata("org/none")
    reg = HubRegistry()
    reg.register_default_hubs(transport=transport)
    assert reg.list_hubs() == ["huggingface", "tensorflow", "onnx"] and reg.get_default_hub().hub_name == "huggingface"
    assert isinstance(reg.get_hub_for_model("hub:tfhub/google/bert"), TensorFlowHub)
    assert isinstance(reg.get_hub_for_model("hub:onnx/resnet"), ONNXHub) and reg.get_hub_for_model("hub:other/x") is None
    assert reg.download("hub:onnx/resnet") == b"ONNX"
    tf = reg.get_hub("tensorflow")
    assert tf.model_exists("hub:tf/google/bert") and tf.get_model_metadata("hub:tf/google/bert").custom["content_length"] == "7"
    assert tf.download_model("hub:tf/google/bert") == b"TFMODEL"
    assert reg.set_default_hub("onnx") and reg.unregister_hub("onnx") and reg.get_default_hub().hub_name == "huggingface"
    with pytest.raises(ValueError):
        reg.register_hub(HuggingFaceHub(transport=transport))
    assert ApiKeyAuth("k").get_auth_header() == ("X-API-Key", "k")


def test_nvtx_ranges_and_timeline_profiler_on_cpu(tmp_path):
    from ml_framework_b200.obs.profiler import TimelineProfiler, annotate, enable_nvtx, nvtx_enabled, nvtx_mark, nvtx_range
    enable_nvtx(True)
    assert nvtx_enabled() == torch.cuda.is_available()         # without a GPU the ranges stay no-ops
    with nvtx_range("outer"):
        nvtx_mark("point")
    out = tmp_path / "trace.json"
    with TimelineProfiler(str(out), steps=1) as tp:
        with annotate("matmul-step"):
            (torch.randn(64, 64) @ torch.randn(64, 64)).sum()
        tp.step()
    text = out.read_text()
    assert "traceEvents" in text and "matmul-step" in text
    enable_nvtx(False)


def test_three_ir_levels_execute_and_agree():
    from ml_framework_b200.compiler import ir
    g = ir.HLGraph("mlp")
    x = g.input("x", (3, 4))
    w = g.constant(torch.randn(4, 5, generator=torch.Generator().manual_seed(0)), "w")
    b = g.constant(torch.randn(5, generator=torch.Generator().manual_seed(1)), "b")
    h = g.op("matmul", x, w)
    h = g.op("add", h, b)                     # broadcast of b over rows
    h = g.op("gelu", h)
    s = g.op("sum", h, dim=1)
    g.output(h, s)
    xin = torch.randn(3, 4, generator=torch.Generator().manual_seed(2))
    want = g.run({"x": xin})
    ml = ir.lower_to_ml(g)
    assert ml.verify() == []
    kinds = [st.kind for st in ml.stmts]
    assert "broadcast" in kinds and "contract" in kinds and "reduce" in kinds and kinds.count("alloc") >= 5
    got_ml = ml.run({"x": xin})
    ll = ir.lower_to_ll(ml)
    assert ll.verify() == []
    ops = [i.op for i in ll.instrs]
    assert ops.count("loop") >= 5 and "fma" in ops and "gelu" in ops and "call" in ops
    got_ll = ll.run({"x": xin})
    for a, b2, c in zip(want, got_ml, got_ll):
        assert torch.allclose(a, b2, atol=1e-6) and torch.allclose(a, c, atol=1e-5)
    assert any("ml.broadcast" in l for l in ml.dump()) and any("ll.fma" in l for l in ll.dump())
    # the verifier catches an implicit broadcast at the mid level and an unbalanced loop at the low level
    bad = ir.lower_to_ml(g)
    for st in bad.stmts:
        if st.kind == "map" and st.fn == "add":
            st.srcs[1] = "b"
    assert any("broadcasts are explicit" in e for e in bad.verify())
    ll.instrs.append(ir.LLInstr("loop", "%rX", (2,)))
    assert "unbalanced loops" in ll.verify()
    for level in ("ml", "ll"):
        exe = ir.CPUBackend().compile(g, level=level)
        out = exe["run"]({"x": xin})
        assert torch.allclose(out[0], want[0], atol=1e-5) and exe["level"] == level


def test_functional_vmap_pmap_and_tracing_jit():
    from ml_framework_b200.compiler import functional as Fn
    from ml_framework_b200.dist.process_group import run_fake_world
    torch.manual_seed(0)
    w = torch.randn(5, 3)
    xs, bs = torch.randn(4, 7, 5), torch.randn(4, 3)
    f = lambda x, b, ww: torch.tanh(x @ ww + b)            # noqa: E731
    want = torch.stack([f(xs[i], bs[i], w) for i in range(4)])
    assert torch.allclose(Fn.vmap(f, in_axes=(0, 0, None))(xs, bs, w), want, atol=1e-6)
    assert torch.allclose(Fn.vmap(f, in_axes=(0, 0, None), fallback="loop")(xs, bs, w), want, atol=1e-6)
    moved = Fn.vmap(f, in_axes=(1, 0, None), out_axes=1)(xs.transpose(0, 1).contiguous(), bs, w)
    assert torch.allclose(moved, want.transpose(0, 1), atol=1e-6)

    def branchy(x):                                          # data-dependent Python: torch.func cannot batch it
        return x * 2 if float(x.sum()) > 0 else x * -1
    v = torch.tensor([[1.0, 2.0], [-3.0, 1.0]])
    assert torch.equal(Fn.vmap(branchy)(v), torch.tensor([[2.0, 4.0], [3.0, -1.0]]))
    with pytest.raises(Exception):
        Fn.vmap(branchy, fallback="never")(v)
    with pytest.raises(ValueError):
        Fn.vmap(f, in_axes=(0, 0))(xs, bs, w)

    # pmap with a named axis: per-rank slice, psum / pmean over the ranks, gathered output
    data = torch.arange(12.0).reshape(4, 3)

    def run(pg):
        def body(x):
            total = Fn.psum(x.sum(), "dp")
            return x / total + Fn.axis_index("dp")
        out = Fn.pmap(body, pg, axis_name="dp")(data)
        mean = Fn.pmap(lambda x: Fn.pmean(x.mean(0, keepdim=True), "dp"), pg, axis_name="dp", gather=False)(data)
        return out, mean
    outs = run_fake_world(2, run)
    want_p = torch.cat([data[:2] / data.sum(), data[2:] / data.sum() + 1])
    for out, mean in outs:
        assert torch.allclose(out, want_p, atol=1e-6) and torch.allclose(mean, data.mean(0, keepdim=True), atol=1e-6)
    with pytest.raises(NameError):
        Fn.psum(torch.ones(1), "nowhere")

    # jit: traced into the IR, optimised (x * 1 + 0 disappears, the repeated relu is shared), cached per signature
    def net(x, ww):
        h = (x @ ww) * 1.0 + 0.0
        return torch.relu(h) + torch.relu(h), h.sum(dim=1)
    jf = Fn.jit(net)
    x = torch.randn(6, 5)
    a, b = jf(x, w)
    ra, rb = net(x, w)
    assert torch.allclose(a, ra, atol=1e-6) and torch.allclose(b, rb, atol=1e-6)
    g = jf.graph(x, w)
    assert [o.kind for o in g.ops].count("relu") == 1 and "mul" not in [o.kind for o in g.ops]
    jf(x, w)
    assert jf.stats["traced"] == 1 and jf.stats["hits"] >= 2
    jf(torch.randn(2, 5), w)
    assert jf.stats["traced"] == 2
    untraceable = Fn.jit(branchy)
    assert torch.equal(untraceable(v[0]), v[0] * 2) and untraceable.stats["eager"] == 1


def test_operation_diagnostics_handlers_and_error_reporting_service():
    from ml_framework_b200.compiler.diagnostics import (ErrorReportingService, OperationDiagnosticsRegistry, OperationExecutionContext)
    from ml_framework_b200.compiler.shapes import ShapeMismatchException
    reg = OperationDiagnosticsRegistry()
    mm = reg.get_handler("matmul")
    assert mm.validate([(4, 8), (8, 3)], {}).is_valid and reg.has_handler("linear") and not reg.has_handler("fft")
    bad = mm.validate([(4, 8), (3, 8)], {})
    assert not bad.is_valid and "inner dimensions" in bad.message
    assert any("transpose the second operand" in s for s in mm.generate_suggestions([(4, 8), (3, 8)], {}))
    assert any("multiple of 8" in s for s in mm.detect_issues([(4, 10), (10, 16)], {}))
    conv = reg.get_handler("conv2d")
    assert conv.validate([(1, 3, 8, 8), (4, 3, 3, 3)], {}).is_valid
    assert "channels" in conv.validate([(1, 8, 8, 3), (4, 3, 3, 3)], {}).message
    assert any("channels-last" in s for s in conv.generate_suggestions([(1, 8, 8, 3), (4, 3, 3, 3)], {}))
    assert not conv.validate([(1, 3, 2, 2), (4, 3, 5, 5)], {"padding": 0}).is_valid
    cat = reg.get_handler("concat")
    assert cat.validate([(2, 3), (5, 3)], {"dim": 0}).is_valid and not cat.validate([(2, 3), (2, 4)], {"dim": 0}).is_valid
    assert any("dimension 1 would work" in s for s in cat.generate_suggestions([(2, 3), (2, 4)], {"dim": 0}))
    assert not reg.get_handler("maxpool2d").validate([(1, 1, 2, 2)], {"kernel": 3}).is_valid
    svc = ErrorReportingService(reg)
    svc.check("matmul", [(4, 8), (8, 3)], layer_name="ok")
    with pytest.raises(ShapeMismatchException) as ei:
        svc.check("linear", [(32, 100), (10, 100)], layer_name="classifier")
    e = ei.value
    assert "classifier" in str(e) and e.suggestions and svc.counts == {"linear": 1} and svc.get_current_context() is None
    assert '"operation": "linear"' in svc.report(e, "json") and "<li>" in svc.report(e, "html")
    svc.capture_context(OperationExecutionContext("conv2d", "stem", [(1, 8, 8, 3), (4, 3, 3, 3)], {}, previous_layer="input"))
    assert "after 'input'" in str(svc.generate_shape_mismatch_exception())
    assert len(svc.log) == 2 and svc.log[-1]["operation"] == "conv2d"
