"""Data-parallel plumbing on CPU: bucket packing, sampler partition, launcher, and the 2-rank
gloo run whose all-reduced gradients must be identical on both ranks."""
import json
import os
import sys

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.data.samplers import BatchSampler, DistributedSampler, ElasticDistributedSampler
from ml_framework_b200.dist.launcher import DistributedTrainingError, ProcessLauncher, launch_local
from ml_framework_b200.dist.process_group import ReduceOp, run_fake_world
from ml_framework_b200.parallel.ddp import DistributedDataParallel, create_buckets

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_bucket_packing_largest_first_and_oversized_alone():
    ps = [nn.Parameter(torch.zeros(n)) for n in (10, 3000, 200, 50, 700)]
    b = create_buckets(ps, bucket_bytes=1000 * 4)
    # 3000 floats exceed the bucket: own bucket. Then 700, then 200+50+10.
    sizes = [[p.numel() for p in bk.params] for bk in b]
    assert sizes == [[3000], [700, 200, 50, 10]]
    assert b[1].offsets == [0, 700, 900, 950]
    with pytest.raises(ValueError):
        from ml_framework_b200.parallel.ddp import GradientBucketManager
        GradientBucketManager(None, ps, bucket_size_mb=0)


def test_distributed_sampler_partition():
    W, N = 3, 10
    ss = [DistributedSampler(N, W, r, shuffle=True, seed=5) for r in range(W)]
    got = sorted(i for s in ss for i in s if i >= 0)
    assert got == list(range(N))
    assert all(len(s) == 4 for s in ss)           # ceil(10 / 3) slots, padded with -1
    assert sum(1 for s in ss for i in s if i < 0) == 2
    dl = [DistributedSampler(N, W, r, shuffle=False, drop_last=True) for r in range(W)]
    assert [list(s) for s in dl] == [[0, 3, 6], [1, 4, 7], [2, 5, 8]]
    a = list(ss[0])
    ss[0].set_epoch(1)
    assert list(ss[0]) != a
    assert list(BatchSampler(dl[0], 2)) == [[0, 3], [6]]
    with pytest.raises(ValueError):
        DistributedSampler(N, 2, 2)


def test_elastic_sampler_does_not_replay_consumed_samples():
    s = ElasticDistributedSampler(100, 4, 0, shuffle=True, seed=1)
    s.record_consumed(40)
    parts = []
    for r in range(2):
        e = ElasticDistributedSampler(100, 4, 0, shuffle=True, seed=1)
        e.record_consumed(40)
        e.update_topology(2, r)
        parts.append(list(e))
    assert len(parts[0]) + len(parts[1]) == 60 and not set(parts[0]) & set(parts[1])


def test_ddp_in_simulated_world_matches_big_batch():
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    state = {k: v.clone() for k, v in ref.state_dict().items()}
    xs = torch.randn(4, 6, 8)
    ys = torch.randn(4, 6, 4)
    ((ref(xs.reshape(-1, 8)) - ys.reshape(-1, 4)) ** 2).mean().backward()
    want = [p.grad.clone() for p in ref.parameters()]

    def run(pg):
        torch.manual_seed(100 + pg.rank)
        m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
        if pg.rank == 0:
            m.load_state_dict(state)
        ddp = DistributedDataParallel(m, pg, bucket_size_mb=0.0001, reduce_op=ReduceOp.AVG)
        ((ddp(xs[pg.rank]) - ys[pg.rank]) ** 2).mean().backward()
        ddp.finish_backward()
        return [p.grad.clone() for p in m.parameters()], len(ddp.bucket_manager.buckets)
    outs = run_fake_world(4, run)
    assert outs[0][1] > 1
    for grads, _ in outs:
        for g, w in zip(grads, want):
            assert torch.allclose(g, w, atol=1e-6)


def test_launcher_env_logs_and_first_failure(tmp_path):
    script = tmp_path / "w.py"
    script.write_text("import os,sys\nprint(os.environ['RANK'], os.environ['WORLD_SIZE'], os.environ['MASTER_ADDR'], os.environ['MASTER_PORT'])\n"
                      "sys.exit(3 if os.environ['RANK']=='1' and len(sys.argv)>1 else 0)\n")
    l = launch_local(str(script), 3, log_dir=str(tmp_path / "logs"), master_port=29611)
    assert [r.exit_code for r in l.ranks] == [0, 0, 0]
    assert (tmp_path / "logs" / "rank_2.log").read_text().split() == ["2", "3", "127.0.0.1", "29611"]
    with pytest.raises(DistributedTrainingError) as e:
        launch_local(str(script), 2, ["fail"], log_dir=str(tmp_path / "logs2"), master_port=29612)
    assert e.value.rank == 1 and e.value.exit_code == 3
    from ml_framework_b200.dist.launcher import launch_multi_node
    with pytest.raises(ValueError):
        launch_multi_node(str(script), nnodes=2, node_rank=2, nproc_per_node=1, master_addr="127.0.0.1")
    with pytest.raises(ValueError):
        ProcessLauncher().launch(["true"], 2, rank_offset=3, world_size=4)


@pytest.mark.timeout(360)
def test_cpu_mlp_ddp_two_gloo_ranks(tmp_path):
    log = ""
    for attempt in range(2):          # a second rendezvous on a fresh port if the first one could not be set up
        d = tmp_path / f"try{attempt}"
        l = ProcessLauncher(master_port=_free_port(), log_dir=str(d))
        l.launch([sys.executable, os.path.join(ROOT, "baseline", "cpu_mlp_ddp.py"), "100"], 2)
        ok = l.wait_for_all(timeout_s=150)
        log = (d / "rank_0.log").read_text()
        if ok:
            break
        log += (d / "rank_1.log").read_text()
        if "rendezvous" not in log.lower() and "address" not in log.lower() and "connect" not in log.lower():
            break
    assert ok, log[-4000:]
    res = json.loads([ln for ln in log.splitlines() if ln.startswith("{")][-1])
    assert res["gradients_equal_across_ranks"] and res["parameters_in_sync"] and res["steps"] == 100

def test_ddp_no_sync_keeps_local_gradients_then_matches_big_batch():
    """One micro-step inside no_sync() plus one synchronised micro-step: inside, gradients stay local
    (nothing from an earlier step's bucket leaks in); after, they are the average over ranks of the
    accumulated two-micro-batch gradient."""
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 3))
    state = {k: v.clone() for k, v in base.state_dict().items()}
    W = 2
    xs, ys = torch.randn(W, 2, 5, 6), torch.randn(W, 2, 5, 3)

    def local_grads(rank, upto):
        m = nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 3))
        m.load_state_dict(state)
        for k in range(upto):
            ((m(xs[rank, k]) - ys[rank, k]) ** 2).mean().backward()
        return [p.grad.clone() for p in m.parameters()]
    want = [sum(g) / W for g in zip(*[local_grads(r, 2) for r in range(W)])]

    def run(pg):
        m = nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 3))
        m.load_state_dict(state)
        ddp = DistributedDataParallel(m, pg, bucket_size_mb=0.0001)
        # an earlier synchronised step leaves reduced values in the bucket buffers
        ((ddp(xs[pg.rank, 0]) - ys[pg.rank, 0]) ** 2).mean().backward()
        ddp.finish_backward()
        for p in m.parameters():
            p.grad = None
        with ddp.no_sync():
            ((ddp(xs[pg.rank, 0]) - ys[pg.rank, 0]) ** 2).mean().backward()
            ddp.finish_backward()
        inside = [p.grad.clone() for p in m.parameters()]
        ((ddp(xs[pg.rank, 1]) - ys[pg.rank, 1]) ** 2).mean().backward()
        ddp.finish_backward()
        return inside, [p.grad.clone() for p in m.parameters()]
    outs = run_fake_world(W, run)
    for r, (inside, after) in enumerate(outs):
        for g, w in zip(inside, local_grads(r, 1)):
            assert torch.allclose(g, w, atol=1e-6)
        for g, w in zip(after, want):
            assert torch.allclose(g, w, atol=1e-6)


def test_ddp_first_step_with_unused_bucket_does_not_fail():
    def run(pg):
        torch.manual_seed(0)
        used, unused = nn.Linear(4, 4), nn.Linear(4, 4)
        m = nn.ModuleList([used, unused])
        ddp = DistributedDataParallel(m, pg, bucket_size_mb=0.00001, find_unused_parameters=True)
        used(torch.ones(2, 4) * (pg.rank + 1)).sum().backward()
        ddp.finish_backward()
        return used.weight.grad.clone(), [float(p.grad.abs().sum()) for p in unused.parameters()], ddp.unused_parameters()
    outs = run_fake_world(2, run)
    assert torch.allclose(outs[0][0], torch.full((4, 4), 3.0)) and outs[0][1] == [0.0, 0.0]


def test_flat_grad_reducer_buckets_and_tied_parameter_counts():
    from ml_framework_b200.parallel.ddp import FlatGradReducer
    from ml_framework_b200.parallel.flat import FlatParams

    def run(pg):
        torch.manual_seed(0)
        ps = [nn.Parameter(torch.zeros(40)), nn.Parameter(torch.zeros(24)), nn.Parameter(torch.zeros(64))]
        flat = FlatParams(ps)
        red = FlatGradReducer(flat, pg, bucket_size_mb=64 * 4 / 2 ** 20)
        assert red.ranges == [(0, 64), (64, 128)]
        for step in range(3):
            flat.zero_grad()
            for p in reversed(ps):
                uses = 2 if p is ps[0] else 1             # a tied parameter reports once per use
                for u in range(uses):
                    if u == 0:
                        p.main_grad.fill_(float(pg.rank + 1))
                    else:
                        p.main_grad.add_(float(pg.rank + 1))
                    p._main_grad_started = True
                    p.grad_ready(p)
                    if step > 0 and p is ps[0] and u == 0:
                        assert not red.launched[0]          # not before its second use
            if step > 0:
                assert red.launched == [True, True]
            red.finish()
            assert torch.allclose(ps[0].main_grad, torch.full((40,), 3.0))     # mean of 2 and 4
            assert torch.allclose(ps[2].main_grad, torch.full((64,), 1.5))
        return True
    assert all(run_fake_world(2, run))


def test_static_grad_scaler_through_the_grad_scaler_api():
    from ml_framework_b200.amp.grad_scaler import GradScalerFactory
    gs = GradScalerFactory.static(128.0)
    p = nn.Parameter(torch.ones(3))
    loss = gs.scale_loss((p * 2).sum())
    loss.backward()
    assert torch.allclose(p.grad, torch.full((3,), 256.0))
    assert gs.prepare_gradients([p.grad]) and torch.allclose(p.grad, torch.full((3,), 2.0))
    assert not gs.check_overflow([p.grad])

    class Opt:
        def step(self, **kw):
            self.kw = kw
    o = Opt()
    gs.step(o)
    assert set(o.kw) == {"inv_scale", "found_inf"}
    gs.update()
    assert gs.scale == 128.0
    assert not gs.prepare_gradients([torch.tensor([float("nan")])])
    gs.update()
    assert gs.scaler.get_stats().skipped_steps == 1


@pytest.mark.timeout(300)
def test_two_emulated_nodes_rendezvous_and_all_reduce(tmp_path):
    """Two ``launch_multi_node`` calls on this machine stand for two nodes (two processes each): global ranks, local ranks
    and the world size come out right and a gloo all-reduce spans all four."""
    import threading
    from ml_framework_b200.dist.launcher import launch_multi_node
    script = tmp_path / "node.py"
    script.write_text(
        "import json, os, sys\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import torch\n"
        "from ml_framework_b200.dist.process_group import BackendType, destroy_process_group, init_process_group\n"
        "pg = init_process_group(BackendType.GLOO)\n"
        "t = torch.tensor([float(pg.rank)])\n"
        "pg.all_reduce(t)\n"
        "print(json.dumps({'rank': pg.rank, 'local': int(os.environ['LOCAL_RANK']), 'world': pg.world_size, 'node': int(os.environ['GROUP_RANK']), 'sum': float(t)}))\n"
        "destroy_process_group()\n")
    port = _free_port()
    errs = []

    def node(k):
        try:
            launch_multi_node(str(script), nnodes=2, node_rank=k, nproc_per_node=2, master_addr="127.0.0.1", master_port=port,
                              log_dir=str(tmp_path / f"node{k}"), timeout_s=120)
        except Exception as e:       # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=node, args=(k,)) for k in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(200)
    assert not errs, errs
    rows = []
    for k in range(2):
        for r in (2 * k, 2 * k + 1):
            log = (tmp_path / f"node{k}" / f"rank_{r}.log").read_text()
            rows.append(json.loads([ln for ln in log.splitlines() if ln.startswith("{")][-1]))
    assert sorted((x["rank"], x["local"], x["node"]) for x in rows) == [(0, 0, 0), (1, 1, 0), (2, 0, 1), (3, 1, 1)]
    assert all(x["world"] == 4 and x["sum"] == 6.0 for x in rows)
