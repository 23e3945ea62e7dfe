"""Remaining host-side pieces on CPU: activation-checkpoint policy and manager, model-zoo registry / plug-ins / cache
eviction / transfer-learning helpers, loss-scaler state and presets, kernel-cache helpers, metric exporters and reporter."""
import json
import os
import time

import pytest
import torch
import torch.nn as nn


def test_activation_checkpoint_policies_builder_manager_and_wrapping():
    from ml_framework_b200.checkpoint import activation as AC
    K = AC.CheckpointStrategyKind
    cfg = (AC.CheckpointConfigBuilder().with_strategy(K.SELECTIVE).with_interval(3).with_layers(["attn", "mlp"]).excluding(["mlp"])
           .with_memory_budget(0.5).build())
    assert cfg.strategy == K.SELECTIVE and cfg.interval == 3 and cfg.max_memory_percentage == 0.5
    for bad in (dict(interval=0), dict(max_memory_percentage=0.0), dict(max_memory_percentage=1.5)):
        with pytest.raises(ValueError):
            AC.CheckpointConfig(**bad).validate()
    m = AC.CheckpointManager(cfg)
    assert m.should_checkpoint("attn", 0) and not m.should_checkpoint("mlp", 1) and not m.should_checkpoint("norm", 2)
    iv = AC.CheckpointManager(AC.CheckpointConfig(K.INTERVAL, interval=2))
    assert [iv.should_checkpoint(f"l{i}", i) for i in range(4)] == [True, False, True, False]
    sz = AC.CheckpointManager(AC.CheckpointConfig(K.SIZE_BASED, min_activation_size_bytes=1000))
    assert sz.should_checkpoint("a", 0, 2000) and not sz.should_checkpoint("a", 0, 10)
    aware = AC.CheckpointManager(AC.CheckpointConfig(K.MEMORY_AWARE, max_memory_percentage=0.5, device_memory_bytes=1000))
    assert not aware.should_checkpoint("a", 0, 400)
    aware.register_checkpoint("kept", torch.zeros(100))                  # 400 bytes stored
    assert aware.should_checkpoint("a", 1, 200) and aware.stats.stored_bytes == 400 and aware.stats.peak_stored_bytes == 400
    smart = AC.CheckpointManager(AC.CheckpointConfig(K.SMART, max_memory_percentage=0.5, device_memory_bytes=1000, min_activation_size_bytes=100))
    assert not smart.should_checkpoint("a", 0, 50) and not smart.should_checkpoint("a", 0, 200)
    smart.register_checkpoint("kept", torch.zeros(50))
    assert smart.should_checkpoint("a", 0, 100)
    assert aware.plan({"a": 300, "b": 100, "c": 250}) == ["a"] and aware.plan({"a": 10}) == []
    calls = []
    aware.register_checkpoint("re", torch.zeros(10), recompute_fn=lambda: calls.append(1) or torch.ones(10))
    assert torch.equal(aware.retrieve_or_recompute("re"), torch.ones(10)) and calls == [1] and aware.stats.recomputations == 1
    assert aware.retrieve_or_recompute("kept").numel() == 100 and aware.stats.saved_bytes == 40
    with pytest.raises(KeyError):
        aware.retrieve_or_recompute("nope")
    aware.clear()
    assert aware.stats.stored_bytes == 0
    layers = nn.ModuleList([nn.Linear(4, 4) for _ in range(4)])
    assert AC.apply_activation_checkpointing(layers, iv) == 2 and isinstance(layers[0], AC.CheckpointedModuleWrapper)
    assert AC.apply_activation_checkpointing(layers, iv) == 0                # already wrapped
    x = torch.randn(2, 4, requires_grad=True)
    plain = nn.Sequential(*[l.module if isinstance(l, AC.CheckpointedModuleWrapper) else l for l in layers])
    y = x
    for l in layers:
        y = l(y)
    y.sum().backward()
    g = x.grad.clone()
    x.grad = None
    plain(x).sum().backward()
    assert torch.allclose(g, x.grad, atol=1e-6)


def test_model_zoo_versions_plugins_cache_eviction_and_transfer_helpers(tmp_path):
    from ml_framework_b200.modelzoo import zoo as Z
    reg = Z.ZooRegistry()
    tiny = Z.default_registry().get("llama-tiny").config
    reg.register(Z.ModelInfo("m", "llama", tiny, version="1.2.0"))
    reg.register(Z.ModelInfo("m", "llama", tiny, version="1.10.0", description="newest", task="causal-lm", tags=("chat",)))
    assert reg.get("m").version == "1.10.0" and reg.get("m", "1.2.0").version == "1.2.0" and len(reg.list()) == 2
    assert [i.version for i in reg.search("newest")] == ["1.10.0"] and reg.search(tags=("chat", "code")) == []
    assert reg.search(task="vision") == []
    with pytest.raises(KeyError):
        reg.get("m", "9.9.9")
    cards = tmp_path / "cards"
    cards.mkdir()
    (cards / "ext.json").write_text(json.dumps({"name": "ext", "architecture": "llama", "config": tiny, "version": "0.1.0", "tags": ["x"]}))
    reg.add_plugin(Z.RegistryPlugin(str(cards)))
    assert reg.get("ext").tags == ("x",) and reg.get("ext", "0.1.0").name == "ext"
    with pytest.raises(KeyError):
        reg.get("ext", "0.2.0")
    locked = Z.ZooRegistry()
    locked.add_plugin(Z.RegistryPlugin(str(cards), token="bad", expected_token="good"))
    with pytest.raises(PermissionError):
        locked.get("ext")
    cache = Z.ModelCacheManager(str(tmp_path / "cache"), max_bytes=2500)
    for i, name in enumerate(["a", "b", "c"]):
        with cache.lock(name, "1"):
            with open(cache.path(name, "1"), "wb") as f:
                f.write(b"x" * 1000)
        cache.touch(name, "1")
        time.sleep(0.01)
    cache.touch("a", "1")                                                  # a was used last: b is the oldest
    assert cache.evict() == ["b-1"] and cache.contains("a", "1") and not cache.contains("b", "1") and cache.evict() == []
    info = Z.ModelInfo("big", "llama", Z.default_registry().get("llama-3-8b").config)
    infer, train = Z.ModelZoo.estimate_memory_bytes(info), Z.ModelZoo.estimate_memory_bytes(info, training=True, batch_tokens=8192)
    assert infer == info.num_params() * 2 and train > infer * 8
    lat1, lat512 = Z.ModelZoo.estimate_latency_ms(info, 1), Z.ModelZoo.estimate_latency_ms(info, 4096)
    assert lat1 == pytest.approx(info.num_params() * 2 / 6.5e12 * 1e3) and lat512 > lat1    # one token is bound by the weights
    z = Z.ModelZoo(str(tmp_path / "z"))
    bench = z.benchmark("llama-tiny", batch=1, seq=16, iters=1)
    assert bench["ms"] > 0 and bench["tokens_per_s"] > 0 and z.recommend(1) is None
    m = z.load("llama-tiny", pretrained=False)
    total = sum(1 for _ in m.parameters())
    assert Z.freeze(m) == total and not any(p.requires_grad for p in m.parameters())
    n = Z.unfreeze(m, ["blocks.1", "norm_f"])
    assert 0 < n < total and all(p.requires_grad == ("blocks.1" in k or "norm_f" in k) for k, p in m.named_parameters())
    Z.replace_head(m, "norm_f", nn.Identity())
    assert isinstance(m.norm_f, nn.Identity)
    with pytest.raises(AttributeError):
        Z.replace_head(m, "no_such_head", nn.Identity())


def test_loss_scaler_state_round_trips_and_presets():
    from ml_framework_b200.amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig, GradScalerFactory, StaticLossScaler
    s = StaticLossScaler(128.0)
    s.found_inf.fill_(1)
    s.update()
    s.update()
    st = s.get_stats()
    assert (st.scale, st.total_steps, st.skipped_steps) == (128.0, 2, 1) and float(s.scale_loss(torch.tensor(2.0))) == 256.0
    t = StaticLossScaler(1.0)
    t.load_state_dict(s.state_dict())
    assert t.scale == 128.0 and float(t.inv_scale_t) == 1 / 128 and t.total_steps == 2 and t.skipped_steps == 1
    with pytest.raises(ValueError):
        StaticLossScaler(0.0)
    d = DynamicLossScaler(DynamicScalerConfig(initial_scale=1024.0, growth_interval=2))
    d.found_inf.fill_(1)
    d.update()                                                             # overflow: halve
    d.update()
    d.update()                                                             # two clean steps: double
    st = d.get_stats()
    assert d.scale == 1024.0 and st.total_steps == 3 and st.skipped_steps == 1
    e = DynamicLossScaler()
    e.load_state_dict(d.state_dict())
    assert e.scale == d.scale and e.total_steps == 3 and int(e.skipped.item()) == 1 and int(e.tracker.item()) == int(d.tracker.item())
    assert GradScalerFactory.conservative().scale == 32768.0 and GradScalerFactory.aggressive().scaler.cfg.growth_interval == 1000
    assert GradScalerFactory.fp16().scale == 65536.0 and GradScalerFactory.bf16().scale == 8.0 and GradScalerFactory.static(4.0).scale == 4.0


def test_kernel_cache_helpers_and_lazy_compilation():
    from ml_framework_b200.compiler import cache as KC
    a, b = torch.zeros(2, 3), torch.zeros(3, 4, dtype=torch.bfloat16)
    sig = KC.ShapeSignature.of("matmul", a, b, extra=("nt",))
    assert sig.shapes == ((2, 3), (3, 4)) and sig.dtype == "torch.float32" and "nt" in sig.key()
    c = KC.LRUKernelCache(2)
    sigs = [KC.ShapeSignature("op", ((i,),)) for i in range(3)]
    built = []
    for s in sigs + [sigs[2]]:
        c.get_or_create(s, lambda s=s: built.append(s) or s.key())
    st = c.stats()
    assert len(c) == 2 and st["evictions"] == 1 and st["hits"] == 1 and st["misses"] == 3 and st["hit_rate"] == 0.25 and len(built) == 3
    with pytest.raises(ValueError):
        KC.LRUKernelCache(0)
    mgr = KC.LazyCompilationManager(lambda s: f"kernel<{s.shapes[0][0]}>")
    assert mgr.get(sigs[0]) == "kernel<0>" and mgr.get(sigs[0]) == "kernel<0>" and mgr.compilations == 1
    mgr.precompile(sigs)
    assert mgr.compilations == 3 and mgr.compile_seconds >= 0
    assert KC.ShapeVariantGenerator.buckets(100, 1000) == [128, 256, 512, 1000] and KC.ShapeVariantGenerator.bucket_for(300, [128, 256, 512]) == 512
    with pytest.raises(ValueError):
        KC.ShapeVariantGenerator.bucket_for(600, [128, 256, 512])
    space = KC.gemm_search_space(8192, 4096, 2048)
    assert space and all(isinstance(d, dict) for d in space)
    prof = KC.GlobalShapeProfiler.instance()
    assert prof is KC.GlobalShapeProfiler.instance()
    for n in (128, 128, 128, 256, 512):
        prof.record("probe_op", (n, 64))
    assert prof.specialisations("probe_op", coverage=0.6)[0] == (128, 64)
    tc = KC.TuningCache()
    tuner = KC.Autotuner(tc, timer=lambda fn: (fn(), {"a": 3.0, "b": 1.0, "c": 2.0}[last[0]])[1])
    last = [None]
    best = tuner.tune(sigs[0], [{"v": "a"}, {"v": "b"}, {"v": "c"}], lambda cfg: last.__setitem__(0, cfg["v"]))
    assert best == {"v": "b"} and tuner.trials == 3 and tuner.tune(sigs[0], [{"v": "a"}], lambda cfg: None) == {"v": "b"}   # cached
    with pytest.raises(RuntimeError):
        KC.Autotuner(timer=lambda fn: (_ for _ in ()).throw(ValueError("x"))).tune(sigs[1], [{"v": 1}], lambda cfg: None)


def test_metric_exporters_and_periodic_reporter():
    from ml_framework_b200.obs import metrics as M
    col = M.MetricsCollector()
    col.inc("requests", 3)
    col.gauge("queue", 7)
    with col.time("step"):
        time.sleep(0.002)
    snap = col.snapshot()
    lines = []
    M.ConsoleExporter().export(snap, printer=lines.append)
    assert lines[0] == "[counter] requests = 3.0" and lines[1] == "[gauge] queue = 7" and lines[2].startswith("[timing] step: n=1")
    sent = []
    M.StatsDExporter(send=sent.append).export(snap)
    assert sent[0] == b"mlf.requests:3.0|c" and sent[1] == b"mlf.queue:7|g" and sent[2].endswith(b"|ms")
    out = []

    class Capture:
        def export(self, s):
            out.append(s["counters"]["requests"])
    rep = M.MetricsReporter(col, [Capture(), M.PrometheusExporter()], interval_s=0.01)
    rep.report_once()
    rep.start()
    time.sleep(0.08)
    rep.stop()
    assert len(out) >= 3 and set(out) == {3.0}
    now = [0.0]
    w = M.SlidingWindowCounter(4.0, clock=lambda: now[0])
    w.add(8)
    assert w.rate() == 2.0
