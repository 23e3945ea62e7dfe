"""Sequence-sharded attention on simulated ranks against attention over the whole sequence."""
import pytest
import torch

from ml_framework_b200.dist.process_group import run_fake_world
from ml_framework_b200.ops.reference import attention_ref
from ml_framework_b200.parallel.context_parallel import (
    ContextParallelAttention, context_parallel_attention, local_positions, ring_attention,
    shard_sequence, ulysses_attention, unshard_sequence)


def _full(q, k, v, w, causal):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = attention_ref(q, k, v, causal=causal)[0]
    (out * w).sum().backward()
    return out.detach(), q.grad, k.grad, v.grad


def _data(B=2, S=32, Hq=4, Hkv=2, D=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, S, Hq, D, generator=g), torch.randn(B, S, Hkv, D, generator=g),
            torch.randn(B, S, Hkv, D, generator=g), torch.randn(B, S, Hq, D, generator=g))


def test_layouts_round_trip_and_balance():
    x = torch.arange(2 * 16 * 3).view(2, 16, 3)
    for zz in (False, True):
        shards = [shard_sequence(x, r, 4, zigzag=zz) for r in range(4)]
        assert torch.equal(unshard_sequence(shards, zigzag=zz), x)
    # zig-zag: every rank sees the same number of unmasked (query, key) pairs
    work = [int((local_positions(r, 4, 16, True)[:, None] >= torch.arange(16)[None, :]).sum()) for r in range(4)]
    assert len(set(work)) == 1
    plain = [int((local_positions(r, 4, 16, False)[:, None] >= torch.arange(16)[None, :]).sum()) for r in range(4)]
    assert plain[0] < plain[-1]
    with pytest.raises(ValueError):
        local_positions(0, 4, 12, zigzag=True)


@pytest.mark.parametrize("world,causal,zigzag", [(4, True, False), (4, True, True), (3, False, False), (2, True, True)])
def test_ring_attention_matches_full_attention_and_gradients(world, causal, zigzag):
    S = 24 if world == 3 else 32
    q, k, v, w = _data(S=S)
    ref = _full(q, k, v, w, causal)

    def run(pg):
        r = pg.rank
        ql, kl, vl, wl = (shard_sequence(t, r, world, zigzag=zigzag) for t in (q, k, v, w))
        ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
        out = ring_attention(ql, kl, vl, pg, causal=causal, zigzag=zigzag)
        (out * wl).sum().backward()
        return out.detach(), ql.grad, kl.grad, vl.grad

    res = run_fake_world(world, run)
    for i, name in enumerate(("out", "dq", "dk", "dv")):
        got = unshard_sequence([x[i] for x in res], zigzag=zigzag)
        torch.testing.assert_close(got, ref[i], rtol=1e-4, atol=1e-5, msg=lambda m, n=name: f"{n}: {m}")


def test_ulysses_attention_matches_full_attention_and_gradients():
    world = 2
    q, k, v, w = _data(S=16, Hq=4, Hkv=2)
    ref = _full(q, k, v, w, True)

    def run(pg):
        r = pg.rank
        ql, kl, vl, wl = (shard_sequence(t, r, world) for t in (q, k, v, w))
        ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
        out = ulysses_attention(ql, kl, vl, pg, causal=True)
        (out * wl).sum().backward()
        return out.detach(), ql.grad, kl.grad, vl.grad

    res = run_fake_world(world, run)
    for i in range(4):
        torch.testing.assert_close(unshard_sequence([x[i] for x in res]), ref[i], rtol=1e-4, atol=1e-5)


def test_ulysses_rejects_indivisible_heads_and_dispatcher_checks_mode():
    q, k, v, _ = _data(S=12, Hq=4, Hkv=2)

    def run(pg):
        ql, kl, vl = (shard_sequence(t, pg.rank, 3) for t in (q, k, v))
        with pytest.raises(ValueError):
            ulysses_attention(ql, kl, vl, pg)
        with pytest.raises(ValueError):
            context_parallel_attention(ql, kl, vl, pg, mode="tree")
        with pytest.raises(ValueError):
            context_parallel_attention(ql, kl, vl, pg, mode="ulysses", zigzag=True)
        return True

    assert all(run_fake_world(3, run))
    # a single rank (or no group) is ordinary attention
    torch.testing.assert_close(context_parallel_attention(q, k, v, None), attention_ref(q, k, v)[0])


@pytest.mark.parametrize("mode", ["ring", "ulysses"])
def test_module_on_shards_equals_module_on_whole_sequence(mode):
    world, hidden = 2, 32
    torch.manual_seed(3)
    whole = ContextParallelAttention(hidden, 4, 2, pg=None)
    state = {k: v.clone() for k, v in whole.state_dict().items()}
    x = torch.randn(2, 16, hidden)
    ref = whole(x)
    ref.square().sum().backward()
    ref_grad = whole.qkv.weight.grad.clone()

    def run(pg):
        m = ContextParallelAttention(hidden, 4, 2, pg=pg, mode=mode)
        m.load_state_dict(state)
        y = m(shard_sequence(x, pg.rank, world))
        y.square().sum().backward()
        g = pg.all_reduce(m.qkv.weight.grad.clone())
        return y.detach(), g

    res = run_fake_world(world, run)
    torch.testing.assert_close(unshard_sequence([r[0] for r in res]), ref.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(res[0][1], ref_grad, rtol=1e-4, atol=1e-4)
