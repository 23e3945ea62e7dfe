"""Pipeline parallelism: partitioner, micro-batch manager, GPipe / 1F1B order, and gradient
equality of a 4-stage pipeline (threads + in-process communicator, and gloo-free simulated p2p)
against the same network on one device."""
import copy
import threading

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from ml_framework_b200.dist.process_group import run_fake_world
from ml_framework_b200.parallel.pipeline import (ActivationCheckpointManager, CheckpointStrategy, GPipeScheduler,
                                                 LayerPartitioner, LocalPipelineCommunicator, MicroBatchManager,
                                                 OneFOneBScheduler, PartitionMode, PipelineConfig, PipelineStats,
                                                 PipelineValidator, ProcessGroupPipelineCommunicator, SchedulingStrategy,
                                                 build_stage, make_scheduler)


def _layers(seed=0):
    torch.manual_seed(seed)
    dims = [12, 16, 16, 16, 16, 16, 16, 8]
    out = []
    for i in range(len(dims) - 1):
        out.append(nn.Sequential(nn.Linear(dims[i], dims[i + 1]), nn.Tanh()))
    return out


def test_partitioner_modes():
    ls = _layers()
    u = LayerPartitioner(PartitionMode.UNIFORM).partition(ls, 3)
    assert u.boundaries == [(0, 3), (3, 5), (5, 7)]
    m = LayerPartitioner(PartitionMode.MANUAL, [1, 5, 1]).partition(ls, 3)
    assert m.boundaries == [(0, 1), (1, 6), (6, 7)]
    a = LayerPartitioner().partition(ls, 4)
    assert len(a.boundaries) == 4 and a.boundaries[0][0] == 0 and a.boundaries[-1][1] == 7
    assert max(a.costs) <= 2.2 * (sum(a.costs) / 4)
    with pytest.raises(ValueError):
        LayerPartitioner().partition(ls, 8)
    with pytest.raises(ValueError):
        LayerPartitioner(PartitionMode.MANUAL, [3, 3]).partition(ls, 2)


def test_micro_batch_manager_and_schedules():
    mb = MicroBatchManager(4)
    parts = mb.split_batch(torch.arange(10).reshape(10, 1))
    assert [p.shape[0] for p in parts] == [2, 2, 2, 4]          # last takes the remainder
    assert torch.equal(mb.combine_outputs(parts), torch.arange(10).reshape(10, 1))
    with pytest.raises(ValueError):
        mb.split_batch(torch.zeros(3, 1))
    p = nn.Parameter(torch.zeros(2))
    for g in (1.0, 3.0):
        p.grad = torch.full((2,), g)
        MicroBatchManager.accumulate_gradients(mb, [p])
    assert torch.equal(mb.get_accumulated_gradients()[0], torch.full((2,), 1.0))   # (1 + 3) / 4
    cfg = PipelineConfig(num_stages=4, micro_batches=8)
    stage = build_stage(_layers(), 1, 4)
    s = OneFOneBScheduler(stage, None, cfg)
    order = s.order()
    assert order[:2] == [("F", 0), ("F", 1)] and order[2:6] == [("F", 2), ("B", 0), ("F", 3), ("B", 1)]
    assert s.max_live_activations() == 3 and [o for o in order if o[0] == "B"] == [("B", i) for i in range(8)]
    g = GPipeScheduler(stage, None, cfg).order()
    assert g[:8] == [("F", i) for i in range(8)] and g[8:] == [("B", i) for i in reversed(range(8))]
    assert abs(PipelineStats(stages=4, micro_batches=16).bubble_fraction - 3 / 19) < 1e-9
    ck = ActivationCheckpointManager(CheckpointStrategy.SELECTIVE, 2)
    assert [ck.should_checkpoint(i) for i in range(4)] == [False, True, False, True]
    assert PipelineValidator.validate_configuration(PipelineConfig(num_stages=9), 7, 2) != []


def _reference(layers, x, y):
    net = nn.Sequential(*copy.deepcopy(layers))
    loss = F.mse_loss(net(x), y)
    loss.backward()
    return loss.item(), [p.grad.clone() for p in net.parameters()]


@pytest.mark.parametrize("schedule", [SchedulingStrategy.GPIPE, SchedulingStrategy.ONE_F_ONE_B])
@pytest.mark.parametrize("ckpt", [CheckpointStrategy.STORE_ALL, CheckpointStrategy.RECOMPUTE_ALL])
def test_pipeline_matches_single_device(schedule, ckpt):
    P, N = 4, 4
    layers = _layers(1)
    x, y = torch.randn(8, 12), torch.randn(8, 8)
    ref_loss, ref_grads = _reference(layers, x, y)
    comm = LocalPipelineCommunicator(P)
    cfg = PipelineConfig(num_stages=P, micro_batches=N, schedule=schedule, checkpoint_strategy=ckpt)
    results = [None] * P

    def run(r):
        stage = build_stage(copy.deepcopy(layers), r, P, LayerPartitioner(PartitionMode.UNIFORM))
        sch = make_scheduler(stage, comm.view(r), cfg, loss_fn=F.mse_loss)
        loss = sch.train_iteration(x if r == 0 else None, y if r == P - 1 else None)
        results[r] = (loss, [p.grad.clone() for p in stage.parameters()])
    ts = [threading.Thread(target=run, args=(r,)) for r in range(P)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert all(r is not None for r in results)
    grads = [g for r in results for g in r[1]]
    assert abs(results[-1][0].item() - ref_loss) < 1e-6
    assert PipelineValidator.validate_gradients(grads, ref_grads, atol=1e-6)


def test_pipeline_over_process_group_p2p():
    P, N = 2, 4
    layers = _layers(2)
    x, y = torch.randn(8, 12), torch.randn(8, 8)
    ref_loss, ref_grads = _reference(layers, x, y)

    def run(pg):
        r = pg.rank
        stage = build_stage(copy.deepcopy(layers), r, P, LayerPartitioner(PartitionMode.UNIFORM))
        comm = ProcessGroupPipelineCommunicator(pg, use_side_stream=False)
        a, b = LayerPartitioner(PartitionMode.UNIFORM).partition(layers, P).boundaries[r]
        in_dim = layers[a][0].in_features
        sch = make_scheduler(stage, comm, PipelineConfig(num_stages=P, micro_batches=N), loss_fn=F.mse_loss,
                             act_shape_fn=lambda _x: (8 // N, in_dim), act_dtype=torch.float32)
        loss = sch.train_iteration(x if r == 0 else None, y if r == P - 1 else None)
        return loss, [p.grad.clone() for p in stage.parameters()]
    outs = run_fake_world(P, run)
    grads = [g for o in outs for g in o[1]]
    assert abs(outs[-1][0].item() - ref_loss) < 1e-6 and PipelineValidator.validate_gradients(grads, ref_grads, atol=1e-6)


def test_pipeline_times_tensor_parallel_composition_gloo():
    """Two pipeline stages x two tensor-parallel ranks (four gloo processes): 1F1B with recomputation over the
    sequence-parallel Llama blocks, stage transfers over point-to-point inside the pipeline sub-groups."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
           "--master-port", "29671", "-m", "ml_framework_b200.utils.bench_pp_tp", "--model", "llama-tiny", "--layers", "4",
           "--override", "n_kv_heads=2", "--pp", "2", "--tp", "2", "--micro-batches", "4", "--seq", "64", "--steps", "2", "--warmup", "2",
           "--backend", "gloo", "--device", "cpu"]
    out = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    rec = json.loads(line)
    assert rec["config"]["parallelism"] == "pp2 x tp2" and rec["n_gpus"] == 4
    assert 0 < rec["final_loss"] < 7.2          # ln(1024) = 6.93 at initialisation, falling


def test_async_executor_two_stages_matches_single_device_gradients():
    """Two stages on two threads through the stream-aware executor (on CPU every stream is the host): forward
    activations and backward gradients cross the in-process communicator; parameter gradients equal the unsplit model's."""
    import threading
    from ml_framework_b200.parallel.pipeline import AsyncPipelineExecutor, LocalPipelineCommunicator, PipelineStage, StreamManager
    torch.manual_seed(0)
    l0, l1 = nn.Sequential(nn.Linear(6, 8), nn.Tanh()), nn.Linear(8, 3)
    ref0, ref1 = copy.deepcopy(l0), copy.deepcopy(l1)
    xs = [torch.randn(4, 6) for _ in range(3)]
    for x in xs:
        ref1(ref0(x)).pow(2).sum().backward()
    comm = LocalPipelineCommunicator(2, timeout_s=20.0)
    errs = []

    def stage0():
        try:
            ex = AsyncPipelineExecutor(PipelineStage(l0, 0, 2), comm.view(0), StreamManager("cpu"))
            for i, x in enumerate(xs):
                y = ex.forward_async(x, i)
                ex.send_async(y.detach(), i, "forward")
            for i in range(len(xs)):
                g = ex.receive_async(torch.empty(4, 8), i, "backward")
                assert ex.backward_async(g, i) is None               # the first stage's input needs no gradient
            ex.sync_compute()
            ex.sync_comm()
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))

    def stage1():
        try:
            ex = AsyncPipelineExecutor(PipelineStage(l1, 1, 2), comm.view(1), StreamManager("cpu"))
            for i in range(len(xs)):
                h = ex.receive_async(torch.empty(4, 8), i, "forward").requires_grad_(True)
                y = ex.forward_async(h, i)
                gx = ex.backward_async(2 * y.detach(), i)              # d/dy of sum(y^2)
                ex.send_async(gx, i, "backward")
            ex.streams.synchronize()
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))
    ths = [threading.Thread(target=f) for f in (stage0, stage1)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(60)
    assert not errs, errs
    for a, b in zip(list(l0.parameters()) + list(l1.parameters()), list(ref0.parameters()) + list(ref1.parameters())):
        assert torch.allclose(a.grad, b.grad, atol=1e-5)


def test_pipeline_optimizer_ties_validator_and_activation_budget():
    from ml_framework_b200.dist.process_group import run_fake_world
    from ml_framework_b200.parallel.pipeline import (ActivationCheckpointManager, CheckpointStrategy, GradientSyncMode, PipelineConfig,
                                                     PipelineOptimizer, PipelineOptimizerConfig, PipelineValidator)

    def run(pg):
        torch.manual_seed(0)
        tied = nn.Parameter(torch.ones(3) * (pg.rank + 1))              # the stages hold different copies at first
        own = nn.Parameter(torch.zeros(2))
        opt = torch.optim.SGD([tied, own], lr=0.5)
        po = PipelineOptimizer(opt, [tied], pg, PipelineOptimizerConfig(GradientSyncMode.SUM), dp_group=pg)
        po.broadcast_parameters(src=0)
        start = tied.detach().clone()
        tied.grad = torch.full((3,), float(pg.rank + 1))
        own.grad = torch.full((2,), 1.0)
        po.step([own])
        return start, tied.detach().clone(), own.detach().clone()
    out = run_fake_world(2, run)
    for start, tied, own in out:
        assert torch.equal(start, torch.ones(3))                         # broadcast from stage 0
        assert torch.equal(tied, torch.ones(3) - 0.5 * 3.0)              # gradients 1 + 2 summed over the tie group
        assert torch.equal(own, torch.zeros(2) - 0.5 * 2.0)              # data-parallel SUM over the two ranks
    none = PipelineOptimizer(torch.optim.SGD([nn.Parameter(torch.ones(1))], lr=1.0))
    none.synchronize_gradients()
    none.broadcast_parameters()
    errs = PipelineValidator.validate_configuration(PipelineConfig(num_stages=4, micro_batches=8), num_layers=2, batch=4)
    assert "more stages than layers" in errs and "batch smaller than the number of micro-batches" in errs
    assert PipelineValidator.validate_configuration(PipelineConfig(num_stages=2, micro_batches=2), 4, 8) == []
    assert PipelineValidator.validate_numerical_stability([torch.ones(2), None]) and not PipelineValidator.validate_numerical_stability([torch.tensor([float("nan")])])
    assert PipelineValidator.validate_gradients([torch.ones(2)], [torch.ones(2) + 1e-7]) and not PipelineValidator.validate_gradients([torch.ones(2)], [])
    mem = ActivationCheckpointManager(CheckpointStrategy.MEMORY_BASED, memory_budget_bytes=100)
    assert [mem.should_checkpoint(i, 40) for i in range(4)] == [False, False, True, True] and mem.stored_bytes == 80
    mem.release(40)
    assert not mem.should_checkpoint(4, 40) and mem.stored_bytes == 80
    mem.release(1000)
    assert mem.stored_bytes == 0
    sel = ActivationCheckpointManager(CheckpointStrategy.SELECTIVE, interval=3)
    assert [sel.should_checkpoint(i) for i in range(4)] == [False, True, True, False]
    assert not ActivationCheckpointManager(CheckpointStrategy.MEMORY_BASED).should_checkpoint(0, 1 << 40)    # no budget: keep everything
