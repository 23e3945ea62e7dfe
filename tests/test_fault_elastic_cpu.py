"""Failure detection, retry, elastic rescaling - all injected on the host (a rank that raises, a
worker that stops sending heartbeats, a dropped message); nothing here touches a GPU."""
import pytest
import torch

from ml_framework_b200.dist.elastic import (AdaptiveLearningRateScheduler, DataRedistributor, ElasticCoordinator, ElasticError,
                                            ElasticTrainingConfig, ElasticWorker, LRAdaptationStrategy, RescaleType, WorkerStatus)
from ml_framework_b200.dist.fault_tolerance import (AlgorithmSelector, ChunkManager, CollectiveAlgorithm, CommunicationConfig,
                                                    ErrorRecoveryManager, FaultTolerantCommunication, HealthMonitor, NCCLConfig,
                                                    RankHealth, RecoveryStrategy, RingAllReduce, TimeoutManager,
                                                    create_data_parallel_groups, create_pipeline_groups, create_split_groups)
from ml_framework_b200.dist.process_group import (CommunicationError, CommunicationTimeout, RankMismatchError, ReduceOp,
                                                  run_fake_world)
from ml_framework_b200.data.samplers import ElasticDistributedSampler


class FlakyPG:
    rank, world_size = 0, 2

    def __init__(self, fail_times, exc):
        self.fail_times, self.exc, self.calls = fail_times, exc, 0

    def all_reduce(self, t, op=None):
        self.calls += 1
        if self.calls <= self.fail_times:
            raise self.exc
        return t * 2


def test_retry_timeout_and_abort_strategies():
    sleeps = []
    ft = FaultTolerantCommunication(FlakyPG(2, IOError("link")), CommunicationConfig(max_retries=3, retry_delay_ms=100), sleep=sleeps.append)
    assert ft.all_reduce(torch.ones(1)).item() == 2 and ft.retries == 2 and sleeps == [0.1, 0.1]
    ft = FaultTolerantCommunication(FlakyPG(5, CommunicationTimeout("slow")), CommunicationConfig(max_retries=2, retry_delay_ms=0), sleep=lambda s: None)
    with pytest.raises(CommunicationTimeout):
        ft.all_reduce(torch.ones(1))
    assert ft.pg.calls == 3
    ft = FaultTolerantCommunication(FlakyPG(1, RankMismatchError("bad")), sleep=lambda s: None)
    with pytest.raises(RankMismatchError):
        ft.all_reduce(torch.ones(1))
    assert ft.pg.calls == 1 and ft.recovery.get_statistics()["by_strategy"] == {"abort": 1}
    rec = ErrorRecoveryManager()
    assert rec.handle_error("x", KeyError("?")) == RecoveryStrategy.ABORT


def test_a_rank_that_never_joins_times_out_the_others():
    def run(pg):
        if pg.rank == 1:
            return "absent"                       # never calls the collective
        with pytest.raises(CommunicationTimeout):
            pg.all_reduce(torch.ones(2))
        return "timed out"
    assert run_fake_world(2, run, timeout_s=0.3) == ["timed out", "absent"]

    def run2(pg):                                  # a rank that raises before the collective
        if pg.rank == 0:
            pg.drop_next = True
        try:
            pg.barrier()
            return "ok"
        except CommunicationError as e:
            return type(e).__name__
    assert run_fake_world(2, run2, timeout_s=0.3) == ["CommunicationError", "CommunicationTimeout"]


def test_health_monitor_and_timeout_manager():
    now = [0.0]
    hm = HealthMonitor(3, clock=lambda: now[0])
    now[0] = 31.0
    hm.update_heartbeat(0)
    assert hm.status(0) == RankHealth.HEALTHY and hm.status(1) == RankHealth.UNRESPONSIVE
    now[0] = 61.0
    hm.update_heartbeat(0)
    assert hm.status(2) == RankHealth.FAILED and hm.get_healthy_ranks() == [0] and hm.get_failed_ranks() == [1, 2]
    tm = TimeoutManager(clock=lambda: now[0])
    h = tm.start_timeout(5)
    now[0] = 67.0
    assert tm.is_expired(h)
    tm.extend_timeout(h, 10)
    assert not tm.is_expired(h)
    tm.cancel_timeout(h)
    assert not tm.is_expired(h)


def test_ring_all_reduce_matches_sum_and_chunking():
    cm = ChunkManager(10, 4)
    assert cm.sizes == [3, 3, 2, 2] and cm.offsets == [0, 3, 6, 8]
    data = [torch.arange(10, dtype=torch.float32) * (r + 1) for r in range(4)]
    want = sum(data)

    def run(pg):
        t = data[pg.rank].clone()
        RingAllReduce(pg).all_reduce(t, ReduceOp.SUM)
        a = data[pg.rank].clone()
        RingAllReduce(pg).all_reduce(a, ReduceOp.AVG)
        return t, a
    for t, a in run_fake_world(4, run):
        assert torch.equal(t, want) and torch.allclose(a, want / 4)


def test_algorithm_selection_groups_and_nccl_env():
    s = AlgorithmSelector(nvswitch=False)
    assert s.select_all_reduce(1024, 8) == CollectiveAlgorithm.RECURSIVE_DOUBLING
    assert s.select_all_reduce(512 * 1024, 16) == CollectiveAlgorithm.RABENSEIFNER
    assert s.select_all_reduce(8 << 20, 8) == CollectiveAlgorithm.RING and s.select_all_reduce(64 << 20, 8) == CollectiveAlgorithm.TREE
    nv = AlgorithmSelector()
    assert nv.select_all_reduce(2 << 20, 8) == CollectiveAlgorithm.ONE_SHOT and nv.select_all_reduce(64 << 20, 8) == CollectiveAlgorithm.TWO_SHOT
    assert create_split_groups(8, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert create_pipeline_groups(8, 4) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    assert create_data_parallel_groups(8, 2) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    env = NCCLConfig.create_debug().apply({})
    assert env["NCCL_DEBUG"] == "INFO" and env["NCCL_BLOCKING_WAIT"] == "1" and env["NCCL_BUFFSIZE"] == str(4 << 20)


def test_elastic_lifecycle_heartbeat_failure_and_debounce():
    now = [0.0]
    cfg = ElasticTrainingConfig(min_workers=1, stability_window_ms=1000, worker_heartbeat_timeout_ms=500, failure_tolerance_percentage=50)
    coord = ElasticCoordinator(cfg, clock=lambda: now[0])
    samplers = {w: ElasticDistributedSampler(100, 1, 0, shuffle=False) for w in "abc"}

    class Opt:
        lr = 0.1
        def set_learning_rate(self, lr): self.lr = lr
    opts = {w: Opt() for w in "abc"}
    workers = {w: ElasticWorker(w, coord, samplers[w], AdaptiveLearningRateScheduler(0.1, 1), opts[w]) for w in "abc"}
    workers["a"].connect_to_cluster()
    now[0] = 0.2
    workers["b"].connect_to_cluster()              # rapid change: the window restarts, only one event fires
    assert coord.poll() is None
    now[0] = 1.0
    for w in "ab":
        workers[w].heartbeat()
    assert coord.poll() is None
    now[0] = 1.3
    for w in "ab":
        workers[w].heartbeat()
    ev = coord.poll()
    assert ev is not None and ev.kind == RescaleType.SCALE_UP and ev.new.world_size == 2 and len(coord.events) == 1
    assert workers["a"].status == WorkerStatus.ACTIVE and (workers["a"].rank, workers["b"].rank) == (0, 1)
    assert abs(opts["a"].lr - 0.2) < 1e-12 and len(samplers["b"]) == 50
    # worker b stops sending heartbeats: detected, unregistered, one scale-down event after the window
    now[0] = 1.6
    workers["a"].heartbeat()
    now[0] = 1.9
    workers["a"].heartbeat()
    assert coord.check_health() == ["b"]
    now[0] = 2.2
    workers["a"].heartbeat()
    assert coord.poll() is None
    now[0] = 2.6
    workers["a"].heartbeat()
    now[0] = 3.0
    workers["a"].heartbeat()
    ev = coord.poll()
    assert ev.kind == RescaleType.SCALE_DOWN and ev.removed == ["b"] and workers["a"].world_size == 1
    # a second failure crosses the 50 % tolerance
    workers["c"].connect_to_cluster()
    with pytest.raises(ElasticError, match="tolerance"):
        coord.unregister_worker("c", graceful=False)


def test_lr_adaptation_and_data_plan():
    s = AdaptiveLearningRateScheduler(0.1, 4, LRAdaptationStrategy.SQUARE_ROOT)
    assert abs(s.adapt_learning_rate(16) - 0.2) < 1e-12 and s.transition_learning_rate(0.1, 0.2, 5, 10) == pytest.approx(0.15)
    plan = DataRedistributor().calculate_plan(100, 4, 2)
    moved = sum(t.end - t.start for t in plan)
    assert moved == 75 and all(t.src_rank != t.dst_rank for t in plan)
    with pytest.raises(ValueError):
        ElasticTrainingConfig(min_workers=0).validate()


def test_learning_rate_transition_manager_and_health_timer():
    import time as _t
    import torch
    from ml_framework_b200.dist.elastic import ElasticCoordinator, ElasticError, ElasticTrainingConfig, LearningRateTransitionManager
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1)
    m = LearningRateTransitionManager(opt, transition_steps=4)
    assert not m.in_transition and m.step() is None and m.current_lr() == 0.1
    m.start_transition(0.5)
    lrs = [m.step() for _ in range(4)]
    assert [round(x, 6) for x in lrs] == [0.2, 0.3, 0.4, 0.5] and not m.in_transition and opt.param_groups[0]["lr"] == 0.5
    m.start_transition(0.1)
    m.step(); m.step()                                   # half way: 0.3
    m.start_transition(0.9)                              # a second rescale restarts from the rate in force
    assert m.history[:2] == [(0.1, 0.5), (0.5, 0.1)] and abs(m.history[2][0] - 0.3) < 1e-12 and m.history[2][1] == 0.9 and abs(m.step() - 0.45) < 1e-9
    cos = LearningRateTransitionManager(None, transition_steps=2, mode="cosine")
    cos.start_transition(1.0, from_lr=0.0)
    assert abs(cos.step() - 0.5) < 1e-12 and cos.step() == 1.0 and cos.current_lr() is None
    jump = LearningRateTransitionManager(opt, transition_steps=0)
    jump.start_transition(0.01)
    assert opt.param_groups[0]["lr"] == 0.01
    import pytest as _p
    with _p.raises(ElasticError):
        LearningRateTransitionManager(None).start_transition(1.0)
    with _p.raises(ValueError):
        LearningRateTransitionManager(None, mode="step")

    now = {"t": 0.0}
    co = ElasticCoordinator(ElasticTrainingConfig(min_workers=1, stability_window_ms=0, worker_heartbeat_timeout_ms=50, failure_tolerance_percentage=40),
                            clock=lambda: now["t"])
    for w in ("a", "b", "c"):
        co.register_worker(w)
    co.start_health_timer(period_s=0.01)
    _t.sleep(0.05)
    assert co.topology.world_size == 3                   # the timer's poll raised the first rescaling event
    now["t"] = 1.0                                       # every heartbeat is stale now: all three fail -> above tolerance
    _t.sleep(0.1)
    co.stop_health_timer()
    with _p.raises(ElasticError):
        co.raise_timer_error()
    co.raise_timer_error()                               # reported once


def test_elastic_state_records_sampler_state_and_transfer_manager():
    import threading
    from ml_framework_b200.data.samplers import ElasticDistributedSampler
    from ml_framework_b200.dist import elastic as E
    shards = E.DataShard.split(10, 3)
    assert [(s.start_index, s.end_index, s.size) for s in shards] == [(0, 4, 4), (4, 8, 4), (8, 10, 2)]
    wm = E.WorkerMetadata("w0", E.WorkerStatus.ACTIVE, 0.0, 100.0, rank=0, custom_attributes={"zone": "a"})
    assert wm.is_healthy(10.0, now=105.0) and not wm.is_healthy(10.0, now=120.0)
    wm.status = E.WorkerStatus.FAILED
    assert not wm.is_healthy(10.0, now=100.0)
    st = E.GlobalTrainingState(2, 500, 3e-4, 64, 4, consumed_samples=1200, optimizer_state=b"\x00\x01")
    back = E.GlobalTrainingState.from_json(st.to_json())
    assert back.current_step == 500 and back.optimizer_state == b"\x00\x01" and back.learning_rate == 3e-4
    nxt = st.after_rescale(6, lr=4.5e-4)
    assert (nxt.global_batch_size, nxt.active_worker_count, nxt.learning_rate, nxt.current_step, nxt.consumed_samples) == (96, 6, 4.5e-4, 500, 1200)
    assert st.after_rescale(2, per_worker_batch=8).global_batch_size == 16

    s = ElasticDistributedSampler(100, 4, 1, shuffle=True, seed=3)
    s.set_epoch(2)
    s.record_consumed(40)
    snap = E.SamplerState.capture(s)
    assert (snap.worker_count, snap.worker_rank, snap.epoch, snap.consumed) == (4, 1, 2, 40)
    parts = [list(snap.restore(worker_count=3, worker_rank=r)) for r in range(3)]
    s.update_topology(4, 1)
    assert sorted(i for p in parts for i in p) == sorted(list(snap.restore(4, 0)) + list(snap.restore(4, 1)) + list(snap.restore(4, 2)) + list(snap.restore(4, 3)))
    assert len({i for p in parts for i in p}) == 60 and list(snap.restore()) == list(s)

    plan = E.DataRedistributor().calculate_plan(100, 4, 2)
    mgr = E.DataTransferManager(max_concurrent_transfers=2, max_retries=1)
    attempts, lock = {}, threading.Lock()

    def copy(t):
        with lock:
            attempts[(t.src_rank, t.dst_rank)] = attempts.get((t.src_rank, t.dst_rank), 0) + 1
            n = attempts[(t.src_rank, t.dst_rank)]
        if t.src_rank == 3 and n == 1:
            raise OSError("transient")
        if t.src_rank == 2:
            raise OSError("gone")
        return (t.end - t.start) * 4
    ok = mgr.execute_plan(plan, copy)
    assert not ok and [t.src_rank for t, _ in mgr.failed] == [2] and mgr.failed[0][1] == "gone" and attempts[(3, 1)] == 2 and attempts[(2, 1)] == 2
    assert mgr.bytes_moved == sum((t.end - t.start) * 4 for t in mgr.completed) and mgr.progress(len(plan)) == 1.0
    mine = E.DataTransferManager()
    assert mine.execute_plan(plan, lambda t: 0, only_rank=0) and all(0 in (t.src_rank, t.dst_rank) for t in mine.completed)
    stop = E.DataTransferManager()
    assert not stop.execute_plan(plan, lambda t: 0, cancel=lambda: True) and all(e == "cancelled" for _, e in stop.failed)
    import pytest as _p
    with _p.raises(ValueError):
        E.DataTransferManager(0)
