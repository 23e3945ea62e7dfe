"""Smaller pieces of the distributed layer on CPU: device-mesh accessors, the tensor-returning communicator on simulated
ranks, named groups, error-recovery bookkeeping, communication profiler, pinned pool, operation queue, overlap helper."""
import pytest
import torch

from ml_framework_b200.dist import communicator as Cm
from ml_framework_b200.dist import fault_tolerance as FT
from ml_framework_b200.dist.mesh import DeviceMesh, DeviceMeshCoord, ParallelismDimension
from ml_framework_b200.dist.process_group import ReduceOp, run_fake_world


def test_mesh_accessors_names_and_master_helpers():
    m = DeviceMesh.create_from_rank(5, (2, 2, 2), dim_names=("dp", "tp", "pp"))
    assert m.coord == DeviceMeshCoord((1, 0, 1)) and len(m.coord) == 3 and m.coord[2] == 1
    assert m.local_rank("tp") == 0 and m.local_rank(ParallelismDimension.PIPELINE) == 1 and m.dim_size("dp") == 2
    assert m.pp_rank == 1 and m.tp_rank == 0 and m.dp_rank == 1 and m.pp_world_size == 2
    assert m.group_ranks("pp") == [4, 5] and m.group_ranks("tp", rank=0) == [0, 2] and m.group_ranks("dp") == [1, 5]
    assert not m.is_master() and m.execute_on_master(lambda: 1) is None
    m0 = DeviceMesh((4,), rank=0)
    assert m0.is_master() and m0.execute_on_master(lambda a, b=2: a + b, 1, b=5) == 6
    assert m0.tp_group_ranks() == [0] and m0.pp_group_ranks() == [0] and m0.tp_world_size == 1 and m0.pp_rank == 0
    assert m0.dim_names == ("data",) and DeviceMesh((2, 2), 0).dim_names == ("data", "tensor")
    with pytest.raises(ValueError):
        DeviceMesh((0, 2), 0)
    with pytest.raises(ValueError):
        m.rank_to_coord(8)
    with pytest.raises(ValueError):
        m.coord_to_rank((0, 0))


def test_communicator_blocking_and_async_forms_on_simulated_ranks():
    def body(pg):
        c = Cm.Communicator(pg)
        r = pg.rank
        assert c.world_size == 4 and c.rank == r
        x = torch.tensor([1.0 + r, 2.0])
        w = c.all_reduce_async(x, ReduceOp.MAX)
        w.wait()
        mx = w.result()
        assert torch.equal(x, torch.tensor([1.0 + r, 2.0]))                # out of place: the input is untouched
        rs = c.reduce_scatter(torch.arange(8, dtype=torch.float32) + r)    # sum over ranks, rank r keeps chunk r
        b = c.broadcast(torch.tensor([float(r)]), root=2)
        c.barrier_async().wait()
        rsa = c.reduce_scatter_async(torch.ones(4), ReduceOp.SUM).result()
        ba = c.broadcast_async(torch.tensor([r]), 1).result()
        return mx.tolist(), rs.tolist(), b.item(), rsa.tolist(), ba.item()
    out = run_fake_world(4, body)
    for r, (mx, rs, b, rsa, ba) in enumerate(out):
        assert mx == [4.0, 2.0] and b == 2.0 and rsa == [4.0] and ba == 1
        assert rs == [4 * (2 * r) + 6, 4 * (2 * r + 1) + 6]                # sum_r' (i + r') for i in chunk r
    with pytest.raises(ValueError):
        Cm.CommunicatorFactory.create("mpi")
    mgr = Cm.ProcessGroupManager(object())                                 # a parent without sub-group support
    assert mgr.create_group("a", [0, 1]) is None and mgr.names() == ["a"] and mgr.get("a") is None
    with pytest.raises(ValueError):
        mgr.create_group("a", [2, 3])
    with pytest.raises(KeyError):
        mgr.get("b")


def test_error_recovery_bookkeeping_config_and_named_groups():
    from ml_framework_b200.dist.process_group import CommunicationTimeout, RankMismatchError
    rec = FT.ErrorRecoveryManager()
    assert rec.handle_error("all_reduce", CommunicationTimeout("t")) == FT.RecoveryStrategy.RETRY
    assert rec.handle_error("all_reduce", RankMismatchError("r")) == FT.RecoveryStrategy.ABORT
    assert rec.handle_error("send", KeyError("k")) == FT.RecoveryStrategy.ABORT                # unknown: abort
    rec.register(KeyError, FT.RecoveryStrategy.USE_DIFFERENT_ALGORITHM)
    assert rec.handle_error("send", KeyError("k")) == FT.RecoveryStrategy.USE_DIFFERENT_ALGORITHM

    class Sub(IOError):
        pass
    assert rec.handle_error("recv", Sub("disk")) == FT.RecoveryStrategy.RETRY                  # resolved through the base class
    st = rec.get_statistics()
    assert st["total_errors"] == 5 and st["by_strategy"] == {"retry": 2, "abort": 2, "different_algorithm": 1}
    FT.CommunicationConfig().validate()
    for bad in (dict(timeout_ms=0), dict(max_retries=-1), dict(retry_delay_ms=-5)):
        with pytest.raises(ValueError):
            FT.CommunicationConfig(**bad).validate()
    sel = FT.AlgorithmSelector()
    assert sel.select_all_gather(1 << 20, 8) == FT.CollectiveAlgorithm.ONE_SHOT
    assert FT.AlgorithmSelector(nvswitch=False).select_all_gather(1 << 20, 8) == FT.CollectiveAlgorithm.RING
    assert FT.AlgorithmSelector(nvswitch=False).select_reduce_scatter(1 << 20, 8) == FT.CollectiveAlgorithm.RABENSEIFNER
    assert sel.select_reduce_scatter(1, 2) == FT.CollectiveAlgorithm.ONE_SHOT
    hp = FT.NCCLConfig.create_high_performance().apply({})
    assert hp["NCCL_NCHANNELS"] == "32" and hp["NCCL_BUFFSIZE"] == str(16 << 20) and "NCCL_DEBUG" not in hp
    assert FT.NCCLConfig.create_default().apply({}) == {"NCCL_BUFFSIZE": str(4 << 20)}
    assert FT.NCCLConfig(algorithm="Tree").apply({})["NCCL_ALGO"] == "Tree"
    pgm = FT.ProcessGroupManager(object())
    assert pgm.create_group("tp", [0, 1]) == [0, 1] and pgm.get_group("tp") == [0, 1]
    with pytest.raises(ValueError):
        pgm.create_group("tp", [2])


def test_profiler_pinned_pool_queue_and_overlap_helper():
    prof = FT.CommunicationProfiler()
    assert prof.profile("all_reduce", 1 << 20, lambda: 7, algorithm="ring") == 7
    prof.profile("all_reduce", 1 << 20, lambda: 8, algorithm="ring")
    prof.profile("barrier", 0, lambda: None)
    st = prof.get_statistics()
    assert st["all_reduce:ring"]["count"] == 2 and st["all_reduce:ring"]["bytes"] == 2 << 20 and st["all_reduce:ring"]["GBps"] > 0
    assert st["barrier"]["count"] == 1 and st["barrier"]["bytes"] == 0
    pool = FT.PinnedMemoryManager(cap_bytes=4096)
    a = pool.get(1024)
    b = pool.get(2048)
    with pytest.raises(MemoryError):
        pool.get(2048)
    pool.put(a)
    assert pool.get(1024) is a and pool.used == 3072                      # a returned buffer is reused, not counted twice
    del b

    def body(pg):
        q = FT.CommunicationOperationQueue()
        ts = [torch.tensor([float(pg.rank + i)]) for i in range(3)]
        for t in ts:
            q.enqueue(pg.all_reduce(t, ReduceOp.SUM, async_op=True))
        first = q.wait_for_any()
        q.wait_for_all()
        assert first is not None and q.wait_for_any() is None
        ov = FT.ComputeCommunicationOverlap(pg)
        res, red = ov.compute_while_communicating(torch.tensor([1.0]), lambda: "computed")
        outs = ov.pipeline([torch.tensor([float(i)]) for i in range(3)], lambda i: i * i)
        return [t.item() for t in ts], res, red.item(), outs
    out = run_fake_world(2, body)
    assert out[0] == ([1.0, 3.0, 5.0], "computed", 2.0, [0, 1, 4]) and out[1][0] == [1.0, 3.0, 5.0]


def test_mpi_style_backend_on_simulated_ranks():
    import pytest as _p
    import torch
    from ml_framework_b200.dist.communicator import MPIConfig, MPIStyleBackend
    from ml_framework_b200.dist.process_group import ReduceOp, run_fake_world

    def run(pg):
        mpi = MPIStyleBackend(pg, MPIConfig(use_cuda_aware=False))
        out = {}
        if pg.rank == 0:
            mpi.send(torch.arange(6, dtype=torch.int32).view(2, 3), 1, tag=7)
            out["echo"] = mpi.receive(1, tag=8)
        else:
            info = mpi.probe(0, tag=7)
            out["info"] = (info.shape, info.dtype, info.count)
            got = mpi.receive(0, tag=7, info=info)
            mpi.send_async(got.float() * 2, 0, tag=8).result(10)
        out["xchg"] = mpi.send_receive(torch.full((2,), float(pg.rank)), 1 - pg.rank, 1 - pg.rank)
        out["ar"] = mpi.all_reduce(torch.ones(2))
        out["ag"] = mpi.all_gather(torch.full((1,), float(pg.rank)))
        out["rs"] = mpi.reduce_scatter(torch.arange(4.0), ReduceOp.SUM)
        out["bc"] = mpi.broadcast(torch.full((1,), float(pg.rank + 3)), root=1)
        out["red"] = mpi.reduce(torch.ones(1), 0)
        mpi.barrier()
        return out
    r0, r1 = run_fake_world(2, run)
    assert r1["info"] == ((2, 3), torch.int32, 6) and r0["echo"].tolist() == [[0.0, 2.0, 4.0], [6.0, 8.0, 10.0]]
    assert r0["xchg"].tolist() == [1.0, 1.0] and r1["xchg"].tolist() == [0.0, 0.0] and r0["ar"].tolist() == [2.0, 2.0] and r0["ag"].tolist() == [0.0, 1.0]
    assert r1["rs"].tolist() == [4.0, 6.0] and r0["bc"].tolist() == [4.0] and r0["red"].tolist() == [2.0]
    with _p.raises(ValueError):
        MPIConfig(thread_level="many").validate()
    with _p.raises(ValueError):
        MPIConfig(buffer_size=0).validate()
