"""Model discovery (search, estimators, recommendation), benchmarking with history and reports, the weight-file format."""
import io
import json

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.modelzoo import benchmark as B
from ml_framework_b200.modelzoo import discovery as D
from ml_framework_b200.modelzoo import serialization as S
from ml_framework_b200.modelzoo.zoo import ModelInfo, ModelZoo, default_registry


def _registry():
    r = default_registry()
    r.get("gpt-125m").metrics = {"accuracy": 0.61}
    r.get("gpt-125m").license = "MIT"
    r.get("gpt-1.3b").metrics = {"accuracy": 0.72}
    r.get("gpt-1.3b").license = "Apache-2.0"
    r.get("llama-3-8b").metrics = {"accuracy": 0.83}
    return r


def test_search_filters_sorting_relevance_and_builder():
    svc = D.ModelSearchService(_registry())
    names = lambda res: [x.model.name for x in res]      # noqa: E731
    assert names(svc.search(D.ModelSearchQuery(architecture="GPT"))) == ["gpt-1.3b", "gpt-125m"]
    assert names(svc.search_by_accuracy(0.7)) == ["llama-3-8b", "gpt-1.3b"]
    assert names(svc.search_by_size(4 << 30)) == ["llama-tiny", "gpt-125m", "gpt-1.3b"]
    assert names(svc.search(D.ModelSearchQuery(min_parameters=5_000_000_000, sort_by=D.SearchSortBy.PARAMETERS))) == ["llama-3-8b", "llama-2-13b"]
    assert names(svc.search(D.ModelSearchQuery(license="mit"))) == ["gpt-125m"] and svc.search(D.ModelSearchQuery(license="gpl")) == []
    rel = svc.search(D.ModelSearchQuery(text="llama serving", sort_by=D.SearchSortBy.RELEVANCE, sort_descending=True))
    assert rel[0].model.name == "llama-3-8b" and rel[0].score > rel[-1].score and "text" in rel[0].matched
    adv = svc.advanced_search(lambda b: b.with_task("causal-lm").with_tags("llama").with_filter("deep", lambda i: i.config["n_layers"] >= 32)
                              .sort_by(D.SearchSortBy.NAME).limit(5))
    assert names(adv) == ["llama-2-13b", "llama-3-8b"] and adv[0].matched == ["task", "tags", "deep"] and adv[0].score == 1.0
    assert len(svc.search_by_task("causal-lm", limit=2)) == 2 and svc.search_by_task("vision") == []
    with pytest.raises(ValueError):
        D.ModelSearchQuery(min_accuracy=0.9, max_accuracy=0.1).validate()
    with pytest.raises(ValueError):
        D.ModelSearchQueryBuilder().limit(0).build()


def test_estimators_follow_the_roofline():
    r = _registry()
    lat, mem = D.LatencyEstimator(), D.MemoryEstimator()
    l8 = r.get("llama-3-8b")
    p = l8.num_params()
    decode = lat.estimate(l8, D.DeviceType.B200, batch_size=1, seq_len=1, context=1024)
    assert abs(decode - (p * 2 + 2 * 32 * 1024 * 1025 * 2) / 6600e9 * 1e3 - 32 * 12e-3) < 1e-6          # weight + KV streaming bound
    prefill = lat.estimate(l8, D.DeviceType.B200, batch_size=8, seq_len=2048)
    assert prefill > 2 * p * 8 * 2048 / 1400e12 * 1e3 and prefill > 20 * decode                         # compute bound
    assert lat.estimate(l8, D.DeviceType.CPU) > 30 * lat.estimate(l8, D.DeviceType.B200)
    assert lat.tokens_per_second(l8, batch_size=64, context=512) > 20 * lat.tokens_per_second(l8, batch_size=1, context=512)
    infer = mem.estimate(l8, batch_size=64, seq_len=1024)
    assert infer > p * 2 + 2 * 32 * 1024 * 64 * 1024 * 2 and mem.estimate(l8, training=True) > p * 16
    assert mem.fits(l8, D.DeviceType.B200, batch_size=64, seq_len=1024) and not mem.fits(r.get("llama-2-13b"), D.DeviceType.B200, batch_size=64, seq_len=4096, training=True)


def test_recommendation_strategies_constraints_and_alternatives():
    eng = D.ModelRecommendationEngine(_registry())
    acc = eng.recommend_with_strategy(D.ModelConstraints(task="causal-lm"), D.RecommendationStrategy.ACCURACY_FIRST)
    fast = eng.recommend_with_strategy(D.ModelConstraints(task="causal-lm"), D.RecommendationStrategy.PERFORMANCE_FIRST)
    assert acc[0].model.name == "gpt-1.3b" and fast[0].model.name in ("llama-tiny", "gpt-125m") and len(acc) == 3
    score = lambda res, n: next(x.score for x in res if x.model.name == n)      # noqa: E731
    every = D.ModelConstraints(task="causal-lm")
    assert score(eng.recommend_with_strategy(every, D.RecommendationStrategy.ACCURACY_FIRST, 9), "llama-3-8b") > \
        score(eng.recommend_with_strategy(every, D.RecommendationStrategy.PERFORMANCE_FIRST, 9), "llama-3-8b")
    assert any("strategy accuracy_first" in x for x in acc[0].reasons)
    c = D.ModelConstraints().with_task("causal-lm").with_min_accuracy(0.7).with_max_memory(8 << 30).with_batch(1, context=512)
    got = eng.recommend_for_constraints(c)
    assert [x.model.name for x in got] == ["gpt-1.3b"] and got[0].estimated_memory_bytes < 8 << 30
    rt = eng.recommend_for_constraints(D.ModelConstraints(task="causal-lm").with_environment(D.DeploymentEnv.REALTIME).with_max_latency(0.5))
    assert rt and all(x.estimated_latency_ms <= 0.5 for x in rt) and eng.strategy_for(D.DeploymentEnv.EDGE) == D.RecommendationStrategy.MEMORY_CONSTRAINED
    assert eng.recommend_for("vision") is None and eng.recommend_for("causal-lm", max_latency_ms=1e-6) is None
    assert [i.name for i in eng.alternatives("llama-3-8b", 2)] == ["llama-2-13b", "llama-tiny"]
    for bad in (lambda: D.ModelConstraints().with_max_latency(0), lambda: D.ModelConstraints().with_max_memory(-1), lambda: D.ModelConstraints().with_min_accuracy(2)):
        with pytest.raises(ValueError):
            bad()


def test_benchmark_service_history_comparison_and_reports(tmp_path):
    hist = B.BenchmarkHistory(str(tmp_path / "h" / "bench.json"))
    svc = B.ModelBenchmarkService(ModelZoo(str(tmp_path / "cache")), hist)
    o = B.BenchmarkOptions(batch_size=2, seq_len=16, warmup_iterations=1, iterations=4)
    r1 = svc.benchmark("llama-tiny", o)
    assert len(r1.latencies_ms) == 4 and r1.min_ms <= r1.p50_ms <= r1.p95_ms <= r1.p99_ms <= r1.max_ms and r1.throughput > 0 and r1.std_ms >= 0
    calls = []
    slow = svc.benchmark_model("llama-tiny", lambda: calls.append(1), B.BenchmarkOptions(batch_size=2, seq_len=16, warmup_iterations=2, iterations=3))
    assert len(calls) == 5
    slow.latencies_ms = [x * 0 + r1.p50_ms * 2 for x in slow.latencies_ms]
    cmp_ = hist.compare_with_previous(slow)
    assert cmp_ is not None and abs(cmp_.change - 1.0) < 1e-9 and cmp_.is_regression() and not B.BenchmarkComparison("m", 1.0, 1.02).is_regression()
    assert hist.total_count == 2 and hist.get_latest("llama-tiny") is slow and len(hist.get_history("llama-tiny", 1)) == 1
    again = B.BenchmarkHistory(str(tmp_path / "h" / "bench.json"))
    assert again.total_count == 2 and abs(again.get_history("llama-tiny")[0].p50_ms - r1.p50_ms) < 1e-12
    assert again.get_history_in_range("llama-tiny", 0, 1) == [] and "2 runs" in again.summary()
    hist.export_json(str(tmp_path / "out.json"))
    assert len(json.load(open(tmp_path / "out.json"))["llama-tiny"]) == 2
    fake = {"a": B.BenchmarkResult("a", "cpu", 1, 8, 2, [2.0, 2.0]), "b": B.BenchmarkResult("b", "cpu", 1, 8, 2, [1.0, 1.0])}
    c = svc.rank(fake)
    assert c.winner == "b" and c.ranking == ["b", "a"] and c.relative_to_winner() == {"a": 2.0, "b": 1.0}
    assert svc.rank(fake, "tokens_per_s", lower_is_better=False).winner == "b"
    rep = B.BenchmarkReporter()
    assert "| 1 | 8 | 2 |" in rep.render(fake["a"]) and json.loads(rep.render(fake["a"], "json"))["p50_ms"] == 2.0 and rep.render(fake["a"], "csv").count("\n") == 2
    assert "| 1 | b | 1.000 | 1.00x |" in rep.render_comparison(c) and rep.render_comparison(c, "csv").splitlines()[2].startswith("2,a,2.0")
    rep.generate_report(c, str(tmp_path / "cmp.md"))
    assert "winner: b" in open(tmp_path / "cmp.md").read()
    with pytest.raises(ValueError):
        rep.render(fake["a"], "xml")
    with pytest.raises(ValueError):
        B.BenchmarkOptions(iterations=0).validate()
    with pytest.raises(RuntimeError):
        B.ModelBenchmarkService().benchmark("x")
    hist.clear_history("llama-tiny")
    assert hist.total_count == 0
    two = svc.compare(["llama-tiny"], B.ComparisonOptions(benchmark=o))
    assert two.winner == "llama-tiny"
    hist.clear_all()


def test_weight_file_round_trip_cast_compression_partial_reads_and_damage(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    m.register_buffer("steps", torch.tensor(7))
    m.register_buffer("empty", torch.zeros(0))
    p = str(tmp_path / "m.mlfm")
    n = S.ModelSerializer(S.SerializerOptions(metadata={"arch": "mlp"})).serialize_to_file(m, p)
    assert n == (tmp_path / "m.mlfm").stat().st_size and n == S.ModelSerializer().serialized_size(m, S.SerializerOptions(metadata={"arch": "mlp"}))
    de = S.ModelDeserializer()
    sd = de.deserialize_file(p)
    assert set(sd) == set(m.state_dict()) and all(torch.equal(sd[k], v) for k, v in m.state_dict().items()) and sd["steps"].item() == 7
    meta = de.metadata(p)
    assert meta["metadata"] == {"arch": "mlp"} and meta["tensors"]["0.weight"] == ("float32", (16, 8)) and meta["total_bytes"] == sum(v.numel() * v.element_size() for v in m.state_dict().values())
    with open(p, "rb") as f:
        h = de.read_header(f)
    assert h["_data_start"] % 64 == 0 and all(e["offset"] % 64 == 0 for e in h["tensors"])
    part = de.deserialize_file(p, ["2.bias"])
    assert list(part) == ["2.bias"]
    with pytest.raises(KeyError):
        de.deserialize_file(p, ["nope"])
    m2 = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    m2.register_buffer("steps", torch.tensor(0))
    m2.register_buffer("empty", torch.zeros(0))
    assert de.load_into(m2, p) == [] and torch.equal(m2[0].weight, m[0].weight) and m2.steps.item() == 7
    pz = str(tmp_path / "z.mlfm")
    big = {"w": torch.zeros(4096), "i": torch.arange(10)}
    nz = S.ModelSerializer().serialize_to_file(big, pz, S.SerializerOptions(compression="zlib", dtype=torch.bfloat16))
    back = de.deserialize_file(pz)
    assert nz < 1024 and back["w"].dtype == torch.bfloat16 and back["i"].dtype == torch.int64 and torch.equal(back["i"], big["i"])
    only = S.ModelSerializer().serialized_size(m, S.SerializerOptions(include=["0."]))
    assert only < n
    raw = bytearray(open(p, "rb").read())
    raw[h["_data_start"] + 5] ^= 0xFF
    with pytest.raises(S.ModelFormatError, match="checksum"):
        de.deserialize(io.BytesIO(bytes(raw)))
    assert set(S.ModelDeserializer(verify_checksums=False).deserialize(io.BytesIO(bytes(raw)))) == set(sd)
    with pytest.raises(S.ModelFormatError, match="magic"):
        de.deserialize(io.BytesIO(b"garbage-garbage"))
    with pytest.raises(S.ModelFormatError, match="truncated"):
        de.deserialize(io.BytesIO(open(p, "rb").read()[:h["_data_start"] + 200]))
    with pytest.raises(KeyError):
        de.load_into(nn.Linear(2, 2), p)
    wrong = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 5))
    with pytest.raises(S.ModelFormatError, match="file has"):
        de.load_into(wrong, p, strict=False)
    with pytest.raises(ValueError):
        S.SerializerOptions(compression="lz4").validate()
