"""Software all-reduce algorithms on simulated ranks of every shape, the optimiser, validated wrappers, handles, events."""
import pytest
import torch

from ml_framework_b200.dist import algorithms as A
from ml_framework_b200.dist import collective_ops as C
from ml_framework_b200.dist.fault_tolerance import AlgorithmSelector, CollectiveAlgorithm
from ml_framework_b200.dist.process_group import CommunicationError, RankMismatchError, ReduceOp, Work, run_fake_world


@pytest.mark.parametrize("world", [2, 3, 4, 5, 6, 8])
@pytest.mark.parametrize("alg", [CollectiveAlgorithm.RECURSIVE_DOUBLING, CollectiveAlgorithm.RABENSEIFNER, CollectiveAlgorithm.TREE, CollectiveAlgorithm.RING])
def test_every_algorithm_sums_on_every_world_size(world, alg):
    n = 37                                         # odd: halving produces uneven pieces

    def worker(pg):
        t = torch.arange(n, dtype=torch.float64) * (pg.rank + 1)
        A.all_reduce_with(pg, t, alg)
        m = torch.full((3, 2), float(pg.rank))
        A.all_reduce_with(pg, m, alg, ReduceOp.MAX)
        a = torch.full((5,), float(pg.rank + 1))
        A.all_reduce_with(pg, a, alg, ReduceOp.AVG)
        return t, m, a
    want = torch.arange(n, dtype=torch.float64) * (world * (world + 1) / 2)
    for t, m, a in run_fake_world(world, worker):
        assert torch.equal(t, want) and torch.equal(m, torch.full((3, 2), float(world - 1))) and torch.allclose(a, torch.full((5,), (world + 1) / 2))


def test_step_and_byte_counts_match_the_schedules():
    def worker(pg):
        out = {}
        for cls in (A.RecursiveDoublingAllReduce, A.RabenseifnerAllReduce, A.TreeAllReduce):
            alg = cls(pg)
            alg.all_reduce(torch.ones(1024, dtype=torch.float32))
            out[cls.__name__] = (alg.steps, alg.bytes_sent)
        return out
    res = run_fake_world(8, worker)
    assert all(r["RecursiveDoublingAllReduce"] == (3, 3 * 4096) for r in res)
    assert all(r["RabenseifnerAllReduce"] == (6, 2 * (512 + 256 + 128) * 4) for r in res)      # 2 (P-1)/P of the vector
    assert res[0]["TreeAllReduce"] == (6, 3 * 4096) and res[7]["TreeAllReduce"] == (2, 4096)
    single = run_fake_world(1, lambda pg: A.RabenseifnerAllReduce(pg).all_reduce(torch.ones(3)))
    assert torch.equal(single[0], torch.ones(3))


def test_optimizer_selects_by_size_and_buckets_small_tensors():
    def worker(pg):
        opt = A.CommunicationOptimizer(pg, AlgorithmSelector(nvswitch=False), native_collectives=False, bucket_bytes=64)
        small, mid, big = torch.ones(8), torch.ones(4096), torch.ones(1 << 20)
        for t in (small, mid, big):
            opt.all_reduce_optimized(t)
        grads = [torch.full((4,), 1.0), torch.full((6,), 2.0), torch.full((10,), 3.0), torch.full((3,), 4.0, dtype=torch.float64)]
        n = opt.all_reduce_many(grads)
        return opt.choices, float(small[0]), float(big[-1]), n, [float(g[0]) for g in grads]
    for choices, s, b, n, g in run_fake_world(4, worker):
        assert s == 4.0 and b == 4.0 and n == 3 and g == [4.0, 8.0, 12.0, 16.0]
        assert choices["recursive_doubling"] >= 2 and choices["rabenseifner"] >= 1 and choices["ring"] == 1
    native = run_fake_world(2, lambda pg: A.CommunicationOptimizer(pg).all_reduce_optimized(torch.ones(4)))
    assert torch.equal(native[0], torch.full((4,), 2.0))


def test_validated_wrappers():
    def worker(pg):
        out = {}
        out["ar"] = C.all_reduce_tensor(pg, torch.ones(2) * (pg.rank + 1))
        ts = C.all_reduce_tensors(pg, [torch.ones(2), torch.ones(3, 2) * 2])
        out["many"] = (ts[0].tolist(), ts[1].shape, float(ts[1][0, 0]))
        out["ag"] = C.all_gather_tensor(pg, torch.full((1, 2), float(pg.rank)), 0)
        out["bc"] = C.broadcast_to_all(pg, torch.full((2,), float(pg.rank + 5)), root=1)
        out["red"] = C.reduce_tensor(pg, torch.ones(2), root=0)
        out["rs"] = C.reduce_scatter_tensor(pg, torch.arange(4.0))
        lin = torch.nn.Linear(2, 1)
        lin.weight.grad = torch.full((1, 2), float(pg.rank))
        out["avg"] = (C.average_gradients(pg, lin.parameters()), lin.weight.grad.tolist())
        full = torch.arange(8.0).view(4, 2) if pg.rank == 0 else None
        out["sc"] = C.scatter_rows(pg, full, 0, like=torch.empty(2, 2))
        C.barrier(pg)
        return out
    r0, r1 = run_fake_world(2, worker)
    assert r0["ar"].tolist() == [3.0, 3.0] and r0["many"] == ([2.0, 2.0], (3, 2), 4.0) and r1["ag"].tolist() == [[0.0, 0.0], [1.0, 1.0]]
    assert r0["bc"].tolist() == [6.0, 6.0] and r0["red"].tolist() == [2.0, 2.0] and r0["rs"].tolist() == [0.0, 2.0] and r1["rs"].tolist() == [4.0, 6.0]
    assert r1["avg"] == (1, [[0.5, 0.5]]) and r1["sc"].tolist() == [[4.0, 5.0], [6.0, 7.0]]

    def bad(pg):
        errs = []
        for fn, exc in ((lambda: C.all_reduce_tensor(pg, torch.ones(0)), ValueError), (lambda: C.all_reduce_tensor(pg, [1.0]), TypeError),
                        (lambda: C.all_reduce_tensor(pg, torch.ones(2, dtype=torch.int32), ReduceOp.AVG), ValueError),
                        (lambda: C.all_reduce_tensor(pg, torch.ones(2, dtype=torch.bool), ReduceOp.SUM), ValueError),
                        (lambda: C.broadcast_tensor(pg, torch.ones(2), root=7), RankMismatchError),
                        (lambda: C.all_reduce_tensors(pg, [torch.ones(1), torch.ones(1, dtype=torch.float64)]), TypeError),
                        (lambda: C.all_gather_tensor(pg, torch.ones(2), dim=3), IndexError),
                        (lambda: C.reduce_scatter_tensor(pg, torch.ones(3)), ValueError),
                        (lambda: C.validate_reduce_operation("sum", torch.float32), TypeError)):
            try:
                fn()
                errs.append(None)
            except exc:
                errs.append(exc.__name__)
        return errs
    assert all(e is not None for e in run_fake_world(2, bad)[0]) and C.all_reduce_tensors(None, []) == []


class _FakeWork(Work):
    def __init__(self, fail=False):
        super().__init__(None)
        self.fail, self.done = fail, False

    def is_completed(self):
        return self.done

    def wait(self, timeout=None):
        if self.fail:
            raise CommunicationError("link down")
        self.done = True
        return "ok"


def test_handles_and_event_handler():
    done = C.CompletedOperationHandle(5)
    assert done.is_completed and done.wait() == 5 and done.try_wait() and done.get_result() == 5
    ev = C.AsyncCommunicationEventHandler()
    seen = []
    ev.on_completed.append(lambda name, s: seen.append(("ok", name)))
    ev.on_failed.append(lambda name, e: seen.append(("bad", name, str(e))))
    h = ev.track(C.PendingOperationHandle(_FakeWork(), name="ar"))
    assert not h.is_completed and not h.try_wait()
    with pytest.raises(CommunicationError):
        h.get_result()
    assert h.wait() == "ok" and h.is_completed and h.get_result() == "ok" and h.wait() == "ok" and seen == [("ok", "ar")]
    f = ev.track(C.PendingOperationHandle(_FakeWork(fail=True), name="bc"))
    with pytest.raises(CommunicationError):
        f.wait()
    with pytest.raises(CommunicationError):
        f.get_result()
    assert seen[-1] == ("bad", "bc", "link down") and ev.statistics()["completed"] == 1 and ev.statistics()["failed"] == 1 and isinstance(ev.last_error, CommunicationError)
    polled = C.PendingOperationHandle(_FakeWork())
    polled._w.done = True
    assert polled.is_completed and polled.elapsed_s is not None
    res = run_fake_world(2, lambda pg: C.all_reduce_async(pg, torch.ones(2), events=C.AsyncCommunicationEventHandler()).wait())
    assert res[0].tolist() == [2.0, 2.0]
    assert isinstance(run_fake_world(1, lambda pg: C.all_reduce_async(pg, torch.ones(2)))[0], C.CompletedOperationHandle)
    assert C.GPUDirectManager.is_supported() in (True, False) and isinstance(C.GPUDirectManager.peer_matrix(), list)


@pytest.mark.timeout(300)
def test_algorithms_over_gloo_point_to_point_three_ranks(tmp_path):
    import json
    import os
    import socket
    import sys
    from ml_framework_b200.dist.launcher import ProcessLauncher
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = ""
    for attempt in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        d = tmp_path / f"try{attempt}"
        l = ProcessLauncher(master_port=port, log_dir=str(d))
        l.launch([sys.executable, os.path.join(root, "tests", "algorithms_worker.py")], 3)
        ok = l.wait_for_all(timeout_s=120)
        log = "".join((d / f"rank_{r}.log").read_text() for r in range(3))
        if ok or not any(w in log.lower() for w in ("rendezvous", "address", "connect")):
            break
    assert ok, log[-4000:]
    res = json.loads([ln for ln in log.splitlines() if ln.startswith("{")][-1])
    assert res["world"] == 3 and all(res["ok"].values()), res
