"""FSDP planning strategies, bucketed gather / scatter helpers, engine introspection and mixed-precision helpers (simulated ranks)."""
import copy

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.dist.process_group import ReduceOp, run_fake_world
from ml_framework_b200.models.gpt import GPT, GPTConfig
from ml_framework_b200.parallel import fsdp_api as A
from ml_framework_b200.parallel.fsdp import FSDP, FSDPConfig


def _infos():
    m = nn.ModuleDict({"embedding": nn.Embedding(10, 4), "blocks": nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 4)), "head": nn.Linear(4, 10)})
    return A.ParameterInfo.from_named(m.named_parameters())


def test_sharding_strategies_plan_ownership():
    infos = _infos()
    assert infos[0].always_gathered and infos[1].layer_name == "blocks.0" and not infos[1].always_gathered
    full = A.create_sharding_strategy("full").plan(infos, 4)
    a = full.assignments["blocks.0.weight"]
    assert a.owner_ranks == [0, 1, 2, 3] and a.shard_numel == 8 and a.start == {0: 0, 1: 8, 2: 16, 3: 24} and full.assignments["embedding.weight"].replicated
    assert full.balance() == 1.0 and full.elements_on_rank(2) == 40 + 8 + 8 + 8 + 8 + 16 + 8
    lw = A.create_sharding_strategy("layer_wise").plan(infos, 4)
    ow, ob = lw.assignments["blocks.0.weight"].owner_ranks, lw.assignments["blocks.0.bias"].owner_ranks
    assert len(ow) == 1 and ow == ob and lw.assignments["blocks.0.weight"].shard_numel == 24 and lw.balance() >= 1.0
    assert A.stable_hash("blocks.0") == A.stable_hash("blocks.0") and A.create_sharding_strategy("layer_wise").plan(infos, 4).assignments["head.weight"].owner_ranks == lw.assignments["head.weight"].owner_ranks
    hy = A.HybridShardingStrategy()
    plan = hy.plan(infos, 4)
    assert hy.choice("blocks.1.weight") == "full" and hy.choice("head.weight") == "layer_wise" and hy.choice("other") == "full"
    assert len(plan.assignments["blocks.1.weight"].owner_ranks) == 4 and len(plan.assignments["head.weight"].owner_ranks) == 1 and plan.strategy == "hybrid"
    assert A.create_sharding_strategy("grad_op").plan(infos, 2).strategy == "grad_op"
    with pytest.raises(KeyError):
        A.create_sharding_strategy("zero9")
    with pytest.raises(ValueError):
        A.HybridShardingStrategy(A.HybridConfig(default="none"))


def test_buckets_and_multi_tensor_helpers():
    assert A.calculate_buckets([100, 100, 300, 50], bucket_size_mb=400 * 2 / (1 << 20)) == [[0, 1], [2, 3]]
    assert A.calculate_buckets([1000, 10], bucket_size_mb=1e-4) == [[0], [1]] and A.calculate_buckets([], 1.0) == []
    with pytest.raises(ValueError):
        A.calculate_buckets([1], 0)
    W = 3
    fulls = [torch.arange(10.0), torch.arange(100.0, 107.0), torch.arange(5.0) * -1]

    def run(pg):
        shards, numels = [], []
        for f in fulls:
            pad = A.padded_numel(f.numel(), W)
            p = torch.zeros(pad)
            p[:f.numel()] = f
            shards.append(p.view(W, -1)[pg.rank].clone())
            numels.append(f.numel())
        got = A.AllGatherHelper.all_gather_multiple(pg, shards, numels, bucket_size_mb=60 * 4 / (1 << 20))
        grads = [f * (pg.rank + 1) for f in fulls]
        pieces = A.ReduceScatterHelper.reduce_scatter_multiple(pg, grads, ReduceOp.AVG, bucket_size_mb=60 * 4 / (1 << 20))
        ok = [A.ReduceScatterHelper.verify_reduce_scatter(pg, g, p) for g, p in zip(grads, pieces)]
        wrong = A.ReduceScatterHelper.verify_reduce_scatter(pg, grads[0], pieces[0] + 1.0)
        return got, pieces, ok, wrong
    for rank, (got, pieces, ok, wrong) in enumerate(run_fake_world(W, run)):
        assert all(torch.equal(g, f) for g, f in zip(got, fulls)) and all(ok) and not wrong
        per = A.padded_numel(10, W) // W
        want = torch.zeros(A.padded_numel(10, W))
        want[:10] = fulls[0] * 2.0                                       # mean of (1, 2, 3) x f
        assert torch.allclose(pieces[0], want[rank * per:(rank + 1) * per])
    with pytest.raises(ValueError):
        A.AllGatherHelper.all_gather_multiple(None, [torch.zeros(1)], [])


def test_extensions_on_a_running_engine():
    cfg = GPTConfig(n_layers=2, d_model=32, n_heads=2, d_ff=64, vocab_size=64, max_seq=16)
    torch.manual_seed(0)
    base = GPT(cfg)
    ref = {n: p.detach().clone() for n, p in base.named_parameters()}

    def run(pg):
        fs = FSDP(copy.deepcopy(base), FSDPConfig(min_shard_numel=64), pg, optimizer_kwargs=dict(lr=1e-2))
        names = A.FSDPExtensions.parameter_names(fs)
        sharded = next(n for n in names if A.FSDPExtensions.is_parameter_sharded(fs, n))
        full = A.FSDPExtensions.get_parameter(fs, sharded)
        lo, hi = A.FSDPExtensions.local_shard_bounds(fs, sharded)
        mem = A.FSDPExtensions.memory_summary(fs)
        gathered = A.FSDPExtensions.is_parameter_gathered(fs, sharded)
        offl = A.FSDPExtensions.is_parameter_offloaded(fs, sharded)
        try:
            A.FSDPExtensions.get_parameter(fs, "nope")
            missing = False
        except KeyError:
            missing = True
        fs.close()
        return sharded, full, (lo, hi), mem, gathered, offl, missing, len(names)
    res = run_fake_world(2, run)
    for rank, (name, full, (lo, hi), mem, gathered, offl, missing, n) in enumerate(res):
        assert torch.allclose(full.float(), ref[name].float(), atol=1e-2) and missing and not offl and not gathered and n == len(ref)
        half = (ref[name].numel() + 1) // 2
        assert (lo, hi) == (rank * half, min((rank + 1) * half, ref[name].numel()))
        assert mem["full_parameter_bytes"] >= 2 * mem["sharded_parameter_bytes"] - 64 and mem["optimizer_state_bytes"] > 0 and mem["largest_unit_bytes"] > 0
    assert A.FSDPState.BACKWARD.value == "backward"


def test_mixed_precision_helpers():
    mp = A.FSDPMixedPrecision()
    x = torch.randn(4)
    assert mp.convert_to_mixed_precision(x).dtype == torch.bfloat16 and mp.convert_gradient_to_fp32(x.bfloat16()).dtype == torch.float32
    i = torch.ones(2, dtype=torch.int64)
    assert mp.convert_to_mixed_precision(i) is i
    sc = mp.make_scaler()
    assert float(sc.scale) == 2.0 and sc.cfg.max_scale == 65536.0 and sc.cfg.growth_interval == 2000

    def run(pg):
        g = [torch.ones(2), torch.tensor([float("inf")]) if pg.rank == 1 else torch.ones(1), None]
        return A.FSDPMixedPrecision.check_overflow(g, pg), A.FSDPMixedPrecision.check_overflow([torch.ones(1)], pg)
    assert run_fake_world(2, run) == [(True, False), (True, False)] and not A.FSDPMixedPrecision.check_overflow([torch.zeros(2)])
