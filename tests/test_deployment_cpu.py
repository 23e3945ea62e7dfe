"""Model deployment on CPU: semantic versions, metadata, registry, checksum-verified loading, hot swap with draining
and concurrent requests, automatic rollback on error rate, header / version routing, traffic splitting, experiments."""
import threading
import time

import pytest

from ml_framework_b200.serving import deployment as D


def test_semantic_versions_metadata_and_registry():
    V = D.SemanticVersion.parse
    assert V("1.2.3") == V("1.2.3+build.7") and hash(V("1.2.3")) == hash(V("1.2.3+x")) and V("1.2.3") != V("1.2.4")
    assert V("1.0.0-alpha") < V("1.0.0-alpha.1") < V("1.0.0-beta") < V("1.0.0-rc.1") < V("1.0.0") < V("1.0.1")
    assert V("1.0.0-rc.2") < V("1.0.0-rc.10")                                   # numeric identifiers compare as numbers
    assert V("1.4.0").compatible_with(V("1.2.0")) and not V("2.0.0").compatible_with(V("1.2.0")) and not V("1.1.0").compatible_with(V("1.2.0"))
    assert str(V(" 3.1.4-rc.1+sha ")) == "3.1.4-rc.1+sha" and len({V("1.0.0"), V("1.0.0+a"), V("1.0.1")}) == 2
    assert str(V("v1.2.3")) == "1.2.3"                                            # a leading v is accepted
    for bad in ("1.2", "1.2.x", "1.2.3.4", ""):
        with pytest.raises(ValueError):
            V(bad)
    meta = D.ModelMetadata("llm", "1.0.0", tags={"team": "a"})
    back = D.ModelMetadata.from_json(meta.to_json())
    assert back == meta
    reg = D.ModelRegistry()
    for v in ("1.10.0", "1.2.0", "1.9.1"):
        reg.register(f"model-{v}", D.ModelMetadata("llm", v))
    assert reg.versions("llm") == ["1.2.0", "1.9.1", "1.10.0"] and reg.latest("llm") == "1.10.0" and reg.get("llm", "1.9.1") == "model-1.9.1"
    with pytest.raises(ValueError):
        reg.register("dup", D.ModelMetadata("llm", "1.2.0"))
    reg.unregister("llm", "1.10.0")
    reg.unregister("llm", "1.10.0")
    assert reg.latest("llm") == "1.9.1"
    with pytest.raises(KeyError):
        reg.get("llm", "1.10.0")
    with pytest.raises(KeyError):
        reg.latest("nothing")


def test_loader_verifies_the_recorded_checksum(tmp_path):
    p = tmp_path / "w.bin"
    p.write_bytes(b"weights-v1")
    loader = D.ModelLoader(lambda path: open(path, "rb").read())
    sha = D.ModelLoader.checksum(str(p))
    assert len(sha) == 64 and loader.load(str(p), D.ModelMetadata("m", "1.0.0", checksum=sha)) == b"weights-v1"
    assert loader.load(str(p)) == b"weights-v1"                                 # no metadata: nothing to verify
    p.write_bytes(b"weights-v2")
    with pytest.raises(IOError):
        loader.load(str(p), D.ModelMetadata("m", "1.0.0", checksum=sha))


def test_hot_swap_drains_in_flight_requests_and_rollback_restores_the_previous_version():
    reg = D.ModelRegistry()
    reg.register(lambda x: ("v1", x), D.ModelMetadata("llm", "1.0.0"))
    reg.register(lambda x: ("v2", x), D.ModelMetadata("llm", "2.0.0"))
    sw = D.ModelHotSwapper(reg)
    sw.activate("llm", "1.0.0")
    with pytest.raises(KeyError):
        sw.activate("llm", "9.9.9")
    started, release, results = threading.Event(), threading.Event(), []

    def slow_request():
        def call(m):
            started.set()
            release.wait(5)
            return m(1)
        results.append(sw.serve("llm", call))
    t = threading.Thread(target=slow_request)
    t.start()
    started.wait(5)
    assert not sw.swap("llm", "2.0.0", drain_timeout=0.05)                      # the old version still has a request in flight
    assert sw.serve("llm", lambda m: m(2)) == ("v2", 2)                         # new requests already see the new version
    release.set()
    t.join(5)
    assert results == [("v1", 1)]                                               # the in-flight request finished on the old one
    assert sw.swap("llm", "1.0.0", drain_timeout=1.0) and sw.swap("llm", "1.0.0")
    assert sw.swap("llm", "2.0.0", drain_timeout=1.0, unload_old=True)
    with pytest.raises(KeyError):
        reg.get("llm", "1.0.0")                                                 # drained and unloaded
    assert sw.serve("llm", lambda m: m(3), version="2.0.0") == ("v2", 3)
    reg.register(lambda x: ("v3", x), D.ModelMetadata("llm", "3.0.0"))
    sw.swap("llm", "3.0.0")
    rb = D.RollbackManager(sw, error_threshold=0.3, window=10, min_samples=5)
    outcomes = [rb.record("llm", ok) for ok in (True, True, False, False)]
    assert outcomes == [False] * 4 and rb.error_rate("llm") == 0.5              # not enough samples yet
    assert rb.record("llm", False) and sw.active["llm"] == "2.0.0" and rb.rollbacks == [("llm", "3.0.0", "2.0.0")]
    assert rb.error_rate("llm") == 0.0                                          # the window restarts after a rollback
    fresh = D.ModelHotSwapper(reg)
    fresh.activate("llm", "2.0.0")
    assert not D.RollbackManager(fresh).rollback("llm")                         # nothing to go back to


def test_header_and_version_routing_traffic_split_and_experiments():
    hr = D.HeaderRouter([D.RoutingRule("x-tier", "gold*", "2.0.0", priority=1)], default="1.0.0")
    hr.add(D.RoutingRule("X-Tier", "gold-beta", "3.0.0-rc.1", priority=5))
    assert hr.route({"X-TIER": "gold-beta"}) == "3.0.0-rc.1" and hr.route({"x-tier": "gold-7"}) == "2.0.0"
    assert hr.route({"x-tier": "silver"}) == "1.0.0" and hr.route({}) == "1.0.0" and D.HeaderRouter().route({"a": "b"}) is None
    reg = D.ModelRegistry()
    for v in ("1.0.0", "1.3.0", "2.1.0"):
        reg.register(v, D.ModelMetadata("m", v))
    vr = D.VersionRouter(reg)
    assert vr.resolve("m") == "2.1.0" and vr.resolve("m", "^1.0.0") == "1.3.0" and vr.resolve("m", "1.0.0") == "1.0.0"
    for bad in ("^3.0.0", "1.1.0"):
        with pytest.raises(KeyError):
            vr.resolve("m", bad)
    with pytest.raises(KeyError):
        vr.resolve("other")
    ts = D.TrafficSplitter({"a": 3, "b": 1}, seed=1)
    picks = [ts.choose() for _ in range(4000)]
    assert 0.70 < picks.count("a") / 4000 < 0.80 and ts.counts["a"] + ts.counts["b"] == 4000
    assert len({ts.choose("user-42") for _ in range(20)}) == 1                  # sticky
    ts.set_weights({"a": 0, "b": 1})
    assert {ts.choose() for _ in range(50)} == {"b"}
    for bad in ({"a": 0, "b": 0}, {"a": -1, "b": 2}):
        with pytest.raises(ValueError):
            D.TrafficSplitter(bad)
    ex = D.ExperimentTracker()
    for i in range(50):
        ex.record("control", "latency", 10.0 + (i % 5) * 0.1)
        ex.record("treatment", "latency", 9.0 + (i % 5) * 0.1)
    s = ex.summary("control", "latency")
    assert s["n"] == 50 and s["mean"] == pytest.approx(10.2) and s["var"] > 0
    cmp_ = ex.compare("control", "treatment", "latency")
    assert cmp_["diff"] == pytest.approx(-1.0) and cmp_["t"] < -20 and cmp_["n_a"] == cmp_["n_b"] == 50
    assert ex.summary("nobody", "latency") == {"n": 0, "mean": 0.0, "var": 0.0} and ex.compare("nobody", "nothing", "x")["t"] == 0.0
    it = D.InferenceTracker()
    with it.track("ok"):
        time.sleep(0.002)
    with pytest.raises(RuntimeError):
        with it.track("bad"):
            raise RuntimeError("boom")
    assert it.errors["bad"] == 1 and it.errors["ok"] == 0 and it.p("ok", 50) >= 0.002 and it.p("none", 99) == 0.0


def test_version_loader_lineage_monitor_and_guarded_swaps():
    import threading
    import time
    import pytest
    import torch.nn as nn
    from ml_framework_b200.serving import version_ops as V
    from ml_framework_b200.serving.deployment import ModelHotSwapper

    loader = V.VersionLoader()
    info = loader.load_version("clf", "1.0.0", lambda: nn.Linear(4, 2), source="mem://a", stage="prod")
    loader.load_version("clf", "1.1.0", lambda: nn.Linear(4, 2))
    assert info.memory_bytes == 4 * (8 + 2) and info.load_seconds >= 0 and info.source == "mem://a" and loader.loaded_versions("clf") == ["1.0.0", "1.1.0"]
    import torch
    w = loader.warm_up_version("clf", "1.1.0", [torch.zeros(1, 4)] * 3)
    assert w.warmed_up and w.warmup_requests == 3 and loader.total_memory_bytes() == 80 and not loader.get_load_info("clf", "1.0.0").warmed_up
    with pytest.raises(ValueError):
        loader.load_version("clf", "1.0.0", lambda: None)
    with pytest.raises(KeyError):
        loader.get_load_info("clf", "9.9.9")

    lin = V.ModelLineage()
    lin.tag("clf", "1.0.0", "stable"); lin.tag("clf", "1.1.0", "candidate"); lin.tag("clf", "1.1.0", "stable")
    assert lin.resolve("clf", "stable") == "1.1.0" and lin.tags_of("clf", "1.1.0") == ["candidate", "stable"] and lin.tags_of("clf", "1.0.0") == []
    lin.set_parent("clf", "1.1.0", "clf", "1.0.0"); lin.set_parent("clf", "1.2.0", "clf", "1.1.0")
    assert lin.ancestry("clf", "1.2.0") == [("clf", "1.1.0"), ("clf", "1.0.0")] and lin.children("clf", "1.0.0") == [("clf", "1.1.0")] and lin.parent("clf", "1.0.0") is None
    with pytest.raises(ValueError):
        lin.set_parent("clf", "1.0.0", "clf", "1.2.0")
    assert lin.untag("clf", "candidate") and not lin.untag("clf", "candidate")

    now = {"t": 100.0}
    mon = V.TimedVersionMonitor(min_samples=10, error_rate_threshold=0.1, latency_p99_ms_threshold=50.0, cooldown_s=30.0, clock=lambda: now["t"])
    got = []
    mon.subscribe_to_alerts(got.append)
    for i in range(20):
        now["t"] += 1.0
        mon.record("clf", "1.0.0", latency_ms=10.0 + i % 3, success=True, memory_mb=100.0)
        mon.record("clf", "1.1.0", latency_ms=8.0 if i < 15 else 200.0, success=i % 4 != 0, memory_mb=90.0)
    kinds = [(a.type, a.severity) for a in got]
    assert (V.AlertType.HIGH_ERROR_RATE, V.AlertSeverity.CRITICAL) in kinds and any(t == V.AlertType.HIGH_LATENCY for t, _ in kinds) and all(a.version == "1.1.0" for a in got)
    assert len([a for a in got if a.type == V.AlertType.HIGH_ERROR_RATE]) == 1                # cooldown
    m = mon.get_metrics("clf", "1.0.0")
    assert m.total_requests == 20 and m.error_rate == 0.0 and abs(m.throughput_rps - 1.0) < 1e-9 and m.latency_p50_ms == 11.0
    early = mon.get_metrics("clf", "1.1.0", V.TimeRange(0, 110.0))
    assert early.total_requests == 10 and early.latency_p99_ms == 8.0
    cmp_ = mon.compare_versions("clf", "1.0.0", "1.1.0")
    assert "error_rate" in cmp_.regressions() and "memory_mean_mb" not in cmp_.regressions() and cmp_.deltas["memory_mean_mb"].improved and not cmp_.v2_is_better
    assert mon.unsubscribe_from_alerts(got.append) is True and mon.unsubscribe_from_alerts(got.append) is False
    mon.clear_metrics("clf", "1.1.0")
    assert mon.get_metrics("clf", "1.1.0").total_requests == 0

    sw = ModelHotSwapper(loader.reg)
    sw.activate("clf", "1.0.0")
    g = V.GuardedVersionSwapper(sw, loader, mon, max_error_rate=0.1)
    assert g.check_version_health("clf", "1.0.0").healthy and not g.check_version_health("clf", "3.0.0").healthy
    r = g.swap_version("clf", "1.1.0", canary=lambda model: model(torch.zeros(1, 4)).shape == (1, 2))
    assert r.success and r.from_version == "1.0.0" and r.drained and sw.active["clf"] == "1.1.0" and g.get_swap_status("clf").state == V.SwapState.COMPLETED
    bad = g.swap_version("clf", "1.0.0", canary=lambda model: 1 / 0)
    assert not bad.success and "canary raised" in bad.message and sw.active["clf"] == "1.1.0" and g.get_swap_status("clf").state == V.SwapState.FAILED
    calls = {"n": 0}

    def flaky(model):                      # healthy before the switch, unhealthy on the live path
        calls["n"] += 1
        return calls["n"] == 1
    rb = g.swap_version("clf", "1.0.0", canary=flaky)
    assert not rb.success and rb.message.startswith("rolled back") and sw.active["clf"] == "1.1.0" and g.get_swap_status("clf").state == V.SwapState.ROLLED_BACK
    g.increment_in_flight("clf", "1.1.0")
    t = threading.Timer(0.05, lambda: g.decrement_in_flight("clf", "1.1.0"))
    t.start()
    assert g.get_swap_status("clf").in_flight == {"1.1.0": 1} and not g.drain_version("clf", "1.1.0", 0.01) and g.drain_version("clf", "1.1.0", 1.0)
    with pytest.raises(ValueError):
        g.decrement_in_flight("clf", "1.1.0")
    back = g.rollback_version("clf")
    assert back.success and back.to_version == "1.0.0" and sw.active["clf"] == "1.0.0"
    assert not g.rollback_version("clf", "7.7.7").success and not V.GuardedVersionSwapper(ModelHotSwapper(loader.reg)).rollback_version("other").success
    loader.unload_version("clf", "1.1.0")
    assert not loader.is_version_loaded("clf", "1.1.0") and not g.check_version_health("clf", "1.1.0").healthy


def test_request_router_split_config_experiment_metrics_and_deployment_log():
    import threading

    from ml_framework_b200.serving import deployment as D
    reg = D.ModelRegistry()
    for v in ("1.0.0", "1.1.0", "2.0.0"):
        reg.register(f"model-{v}", D.ModelMetadata("m", v))
    sw = D.ModelHotSwapper(reg)
    log = D.DeploymentLog(sw, clock=iter(range(100)).__next__)
    first = log.deploy("m", "1.0.0")
    assert first.status is D.DeploymentStatus.ACTIVE and first.previous_version is None and log.current("m") is first
    router = D.RequestRouter(reg, sw)
    assert router.route("m") == "1.0.0"                                               # the active version
    assert router.route("m", D.RoutingContext(requested_version="^1.0.0")) == "1.1.0" and router.route("m", D.RoutingContext(requested_version="latest")) == "2.0.0"
    router.add_rule("m", D.TypedRoutingRule("X-Client", "beta-", "2.0.0", D.MatchType.PREFIX, priority=5))
    router.add_rule("m", D.TypedRoutingRule("X-Client", r"^internal-\d+$", "1.1.0", D.MatchType.REGEX, priority=9))
    router.add_rule("m", D.TypedRoutingRule("X-Tier", "gold", "1.1.0"))
    router.add_rule("m", D.TypedRoutingRule("X-Region", "eu-*", "1.0.0", D.MatchType.GLOB))
    R = lambda **h: router.route("m", D.RoutingContext(headers=h))                     # noqa: E731
    assert R(**{"x-client": "beta-7"}) == "2.0.0" and R(**{"X-Client": "internal-42"}) == "1.1.0" and R(**{"X-Tier": "gold"}) == "1.1.0"
    assert R(**{"X-Tier": "golden"}) == "1.0.0" and R(**{"X-Region": "eu-west"}) == "1.0.0"
    cfg = D.TrafficSplitConfig("m", {"1.0.0": 80.0, "2.0.0": 20.0})
    router.set_traffic_split(cfg, seed=1)
    picks = [router.route("m", D.RoutingContext(user_id=f"u{i}")) for i in range(2000)]
    assert 0.15 < picks.count("2.0.0") / 2000 < 0.25
    assert len({router.route("m", D.RoutingContext(user_id="same")) for _ in range(20)}) == 1      # sticky per user
    assert router.decisions["split"] == 2020 and router.decisions["rule"] == 4 and router.clear_traffic_split("m") and not router.clear_traffic_split("m")
    for bad in ({"1.0.0": 50.0}, {"1.0.0": 120.0, "2.0.0": -20.0}, {}):
        with pytest.raises(ValueError):
            D.TrafficSplitConfig("m", bad).validate()
    with pytest.raises(KeyError):
        router.set_traffic_split(D.TrafficSplitConfig("m", {"9.9.9": 100.0}))
    with pytest.raises(D.RoutingError) as ei:
        router.route("m", D.RoutingContext(requested_version="3.0.0"))
    assert ei.value.model_name == "m" and ei.value.context.requested_version == "3.0.0"
    with pytest.raises(D.RoutingError):
        router.route("unknown")

    em = D.ExperimentMetrics.from_samples("exp1", "2.0.0", [10.0] * 18 + [50.0, 90.0], [True] * 19 + [False], {"ctr": 0.2})
    assert em.request_count == 20 and em.success_rate == 0.95 and em.error_rate == pytest.approx(0.05) and em.p95_latency_ms == 50.0
    assert em.mean_latency_ms == pytest.approx((180 + 140) / 20) and D.ExperimentMetrics("e", "v").success_rate == 0.0
    with pytest.raises(ValueError):
        D.ExperimentMetrics.from_samples("e", "v", [1.0], [])

    second = log.deploy("m", "2.0.0", note="canary won")
    assert second.previous_version == "1.0.0" and first.status is D.DeploymentStatus.RETIRED and first.retired_at is not None
    assert sw.active["m"] == "2.0.0" and [r.version for r in log.history("m")] == ["1.0.0", "2.0.0"]
    with pytest.raises(KeyError):
        log.deploy("m", "7.7.7")
    assert log.records[-1].status is D.DeploymentStatus.FAILED and log.current("m") is second
    back = log.rollback("m")
    assert back.version == "1.0.0" and second.status is D.DeploymentStatus.ROLLED_BACK and sw.active["m"] == "1.0.0" and "rollback from 2.0.0" in back.note
    # a version that still serves a request cannot be released
    started, finish = threading.Event(), threading.Event()
    t = threading.Thread(target=lambda: sw.serve("m", lambda model: (started.set(), finish.wait(10)), version="2.0.0"))
    t.start(); started.wait(5)
    with pytest.raises(D.ReferenceLeakError) as leak:
        log.release("m", "2.0.0")
    assert leak.value.count == 1
    finish.set(); t.join(5)
    log.release("m", "2.0.0")
    assert reg.versions("m") == ["1.0.0", "1.1.0"]
    with pytest.raises(ValueError):
        log.release("m", "1.0.0")
    assert D.DeploymentLog(sw).rollback("nothing") is None
