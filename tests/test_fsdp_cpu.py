"""FSDP semantics on CPU with simulated ranks: sharding arithmetic, config validation, and
training equivalence (sharded run == single-process run on the concatenated batch)."""
import copy

import pytest
import torch

from ml_framework_b200.amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig
from ml_framework_b200.dist.process_group import run_fake_world
from ml_framework_b200.models import GPT, GPTConfig
from ml_framework_b200.optim.optimizers import AdamW
from ml_framework_b200.parallel.fsdp import FSDP, FSDPConfig, FSDPCpuOffloadConfig, padded_numel, shard_bounds


def test_shard_bounds_rule():
    # ceil(N / W) with a short last shard
    assert [shard_bounds(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [shard_bounds(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert padded_numel(10, 4) == 32 and padded_numel(64, 4) == 64


def test_config_validation():
    FSDPConfig().validate()
    for bad in (dict(sharding_strategy="nope"), dict(bucket_size_mb=0), dict(bucket_size_mb=1001),
                dict(num_communication_workers=0), dict(num_communication_workers=17)):
        with pytest.raises(ValueError):
            FSDPConfig(**bad).validate()
    with pytest.raises(ValueError):
        FSDPCpuOffloadConfig(prefetch_steps=11).validate()


def _reference_run(cfg, ids, tgt, steps, kw):
    torch.manual_seed(0)
    model = GPT(cfg)
    opt = AdamW(list(dict.fromkeys(model.parameters())), **kw)
    losses = []
    for s in range(steps):
        opt.zero_grad()
        loss = model(ids.reshape(-1, ids.shape[-1]), tgt.reshape(-1, tgt.shape[-1]))
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, {n: p.detach().clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("strategy", ["full", "grad_op", "layer_wise"])
def test_fsdp_matches_single_process(strategy):
    W, steps = 2, 3
    cfg = GPTConfig(n_layers=2, d_model=64, n_heads=2, d_ff=128, vocab_size=100, max_seq=16, vocab_multiple=8)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 100, (W, 2, 16), generator=g)
    tgt = torch.randint(0, 100, (W, 2, 16), generator=g)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-4, weight_decay=0.01)  # eps above fp32 noise: the key bias has a mathematically zero gradient
    ref_losses, ref_params = _reference_run(cfg, ids, tgt, steps, kw)
    torch.manual_seed(0)
    base = GPT(cfg)     # the global RNG is shared by the rank threads: build once, copy per rank

    def run(pg):
        model = copy.deepcopy(base)
        fs = FSDP(model, FSDPConfig(sharding_strategy=strategy, min_shard_numel=64), pg, optimizer_kwargs=kw)
        losses = []
        for s in range(steps):
            losses.append(fs.train_step(ids[pg.rank], tgt[pg.rank]).item())
        return losses, fs.full_state_dict(), fs.units[0].shard_numel, fs.units[0].full_numel
    outs = run_fake_world(W, run)
    for r in range(W):
        losses, params, shard_n, full_n = outs[r]
        assert shard_n * W == full_n
        for n, p in ref_params.items():
            assert torch.allclose(params[n], p, atol=2e-5), n
    # mean of the per-rank losses equals the loss on the concatenated batch
    for s in range(steps):
        assert abs(sum(outs[r][0][s] for r in range(W)) / W - ref_losses[s]) < 1e-4


def test_fsdp_overflow_skips_on_every_rank():
    W = 2
    cfg = GPTConfig(n_layers=1, d_model=64, n_heads=2, d_ff=128, vocab_size=50, max_seq=8, vocab_multiple=8)
    ids = torch.randint(0, 50, (W, 1, 8))

    torch.manual_seed(0)
    base = GPT(cfg)

    def run(pg):
        model = copy.deepcopy(base)
        fs = FSDP(model, FSDPConfig(min_shard_numel=64), pg, optimizer_kwargs=dict(lr=1e-2))
        scaler = DynamicLossScaler(DynamicScalerConfig(initial_scale=1024.0))
        before = fs.master.clone()
        if pg.rank == 1:
            # poison one gradient on one rank only: both ranks must skip
            h = model.blocks[0].mlp.fc1.weight.register_hook(lambda g: g * float("inf"))
        fs.train_step(ids[pg.rank], ids[pg.rank], scaler)
        return torch.equal(before, fs.master), scaler.scale
    outs = run_fake_world(W, run)
    assert all(o[0] for o in outs) and all(o[1] == 512.0 for o in outs)


@pytest.mark.parametrize("offload", [dict(offload_parameters=True, prefetch_steps=1),
                                     dict(offload_parameters=True, offload_gradients=True, prefetch_steps=2),
                                     dict(offload_gradients=True)])
def test_fsdp_cpu_offload_of_parameters_and_gradients_matches_plain_fsdp(offload):
    """Parameter shards on the host with a prefetch manager, gradient shards leaving for the host after each unit's
    reduction: the training result is the one of the same run without offload."""
    W, steps = 2, 3
    cfg = GPTConfig(n_layers=3, d_model=64, n_heads=2, d_ff=128, vocab_size=100, max_seq=16, vocab_multiple=8)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 100, (W, 2, 16), generator=g)
    tgt = torch.randint(0, 100, (W, 2, 16), generator=g)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-4, weight_decay=0.01)
    torch.manual_seed(0)
    base = GPT(cfg)

    def run(pg, off):
        model = copy.deepcopy(base)
        conf = FSDPConfig(min_shard_numel=64, cpu_offload=FSDPCpuOffloadConfig(enabled=off is not None, **(off or {})))
        fs = FSDP(model, conf, pg, optimizer_kwargs=kw)
        losses = [fs.train_step(ids[pg.rank], tgt[pg.rank]).item() for _ in range(steps)]
        stats = (fs.prefetch.requests, fs.prefetch.hits) if fs.prefetch is not None else None
        return losses, fs.full_state_dict(), stats, fs.param_shards.device.type
    plain = run_fake_world(W, lambda pg: run(pg, None))
    offl = run_fake_world(W, lambda pg: run(pg, offload))
    for r in range(W):
        assert all(abs(a - b) < 1e-5 for a, b in zip(plain[r][0], offl[r][0]))
        for n, p in plain[r][1].items():
            assert torch.allclose(offl[r][1][n], p, atol=1e-6), n
        if offload.get("offload_parameters"):
            req, hits = offl[r][2]
            assert req > 0 and hits > 0          # units ahead were brought in before they were asked for
            assert offl[r][3] == "cpu"
    with pytest.raises(ValueError):
        FSDPCpuOffloadConfig(enabled=True, offload_gradients=True, offload_optimizer_states=False).validate()


def test_fsdp_activation_checkpointing_and_async_reductions_match():
    W, steps = 2, 2
    cfg = GPTConfig(n_layers=3, d_model=64, n_heads=2, d_ff=128, vocab_size=100, max_seq=16, vocab_multiple=8)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 100, (W, 2, 16), generator=g)
    kw = dict(lr=1e-2, eps=1e-4)
    torch.manual_seed(0)
    base = GPT(cfg)

    def run(pg, **conf):
        model = copy.deepcopy(base)
        fs = FSDP(model, FSDPConfig(min_shard_numel=64, **conf), pg, optimizer_kwargs=kw)
        return [fs.train_step(ids[pg.rank], ids[pg.rank]).item() for _ in range(steps)], fs.full_state_dict()
    a = run_fake_world(W, lambda pg: run(pg))
    b = run_fake_world(W, lambda pg: run(pg, activation_checkpointing=True, num_communication_workers=1, bucket_size_mb=1))
    for r in range(W):
        assert all(abs(x - y) < 1e-5 for x, y in zip(a[r][0], b[r][0]))
        for n, p in a[r][1].items():
            assert torch.allclose(b[r][1][n], p, atol=1e-6), n


def test_piggyback_parts_are_spread_over_gemms_by_their_size():
    """A queued copy table in parts: every qualifying GEMM takes as many parts as its copy CTAs move while it runs,
    the callback fires with the last part, and what nobody took can be fetched back."""
    import torch
    from ml_framework_b200.ops import gemm as G
    segs = torch.zeros(10, 3, dtype=torch.int64)
    rows, nbytes = [0, 3, 4, 6, 10], [8 << 20, 8 << 20, 8 << 20, 8 << 20]
    fired = []
    G.set_piggyback(segs, 10, n_copy_ctas=16, on_attached=lambda: fired.append(1), part_rows=rows, part_bytes=nbytes, tag="u")
    assert G._take_piggyback(64, 64, 64, None) is None                    # too small a product: nothing attached
    cm = G._take_piggyback(8192, 2048, 2048, None)                        # ~57 us of product: 18 MB of copies = two parts
    assert cm.n_extra == 4 and cm.extra_segs == segs.data_ptr() and not fired
    assert G.pending_piggyback("other") is None
    cm = G._take_piggyback(8192, 8192, 2048, None)                        # a long product takes the rest
    assert cm.n_extra == 6 and cm.extra_segs == segs.data_ptr() + 4 * 24 and fired == [1]
    assert G._take_piggyback(8192, 8192, 2048, None) is None
    G.set_piggyback(segs, 10, part_rows=rows, part_bytes=nbytes, tag="u")
    G._take_piggyback(8192, 1024, 2048, None)                             # a short product: one part
    tbl, first, n = G.pending_piggyback("u")
    assert (first, n) == (3, 7) and G.pending_piggyback("u") is None
    G.set_piggyback(segs, 10)                                             # no parts: the whole table rides on one GEMM
    assert G._take_piggyback(8192, 2048, 2048, None).n_extra == 10
