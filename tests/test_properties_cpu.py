"""Property-based checks (hypothesis) of the pure partitioning / planning / conversion functions."""
import math

import pytest
import torch
from hypothesis import given, settings, strategies as st

from ml_framework_b200.amp import softfloat as sf
from ml_framework_b200.checkpoint.recompute import DependencyGraph, RecomputationCache
from ml_framework_b200.data.samplers import DistributedSampler, ElasticDistributedSampler
from ml_framework_b200.dist.elastic import DataRedistributor
from ml_framework_b200.dist.fault_tolerance import ChunkManager
from ml_framework_b200.dist.mesh import DeviceMesh
from ml_framework_b200.obs.histograms import QuantileCalculator
from ml_framework_b200.parallel.fsdp import padded_numel, shard_bounds
from ml_framework_b200.parallel.fsdp_api import calculate_buckets

FAST = settings(max_examples=60, deadline=None)


@FAST
@given(st.integers(0, 10_000), st.integers(1, 64))
def test_chunk_manager_partitions_exactly(n, w):
    cm = ChunkManager(n, w)
    assert sum(cm.sizes) == n and max(cm.sizes) - min(cm.sizes) <= 1 and cm.offsets == [sum(cm.sizes[:i]) for i in range(w)]
    assert sorted(cm.sizes, reverse=True) == cm.sizes                       # the first N mod W chunks carry the extra element


@FAST
@given(st.integers(1, 100_000), st.integers(1, 64))
def test_shard_bounds_cover_without_overlap_and_padding_is_minimal(n, w):
    pieces = [shard_bounds(n, w, r) for r in range(w)]
    assert pieces[0][0] == 0 and pieces[-1][1] == n and all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
    assert all(hi - lo <= math.ceil(n / w) for lo, hi in pieces)
    p = padded_numel(n, w)
    assert p >= n and p % (8 * w) == 0 and p - n < 8 * w


@FAST
@given(st.integers(1, 5000), st.integers(1, 16), st.integers(1, 16))
def test_redistribution_plan_moves_exactly_what_changes_owner(n, old, new):
    plan = DataRedistributor().calculate_plan(n, old, new)
    owner_old = lambda i: next(r for r in range(old) if DataRedistributor.shard_range(n, old, r)[0] <= i < DataRedistributor.shard_range(n, old, r)[1])      # noqa: E731
    owner_new = lambda i: next(r for r in range(new) if DataRedistributor.shard_range(n, new, r)[0] <= i < DataRedistributor.shard_range(n, new, r)[1])      # noqa: E731
    moved = set()
    for t in plan:
        assert t.src_rank != t.dst_rank and t.start < t.end
        for i in (t.start, t.end - 1):
            assert owner_old(i) == t.src_rank and owner_new(i) == t.dst_rank
        moved.update(range(t.start, t.end))
    step = max(1, n // 50)
    assert all((i in moved) == (owner_old(i) != owner_new(i)) for i in range(0, n, step))


@FAST
@given(st.integers(0, 400), st.integers(1, 9), st.booleans(), st.integers(0, 5))
def test_distributed_sampler_ranks_partition_the_epoch(n, w, shuffle, epoch):
    ss = [DistributedSampler(n, w, r, shuffle=shuffle, seed=3) for r in range(w)]
    for s in ss:
        s.set_epoch(epoch)
    got = sorted(i for s in ss for i in s if i >= 0)
    assert got == list(range(n)) and len({len(s) for s in ss}) == 1


@FAST
@given(st.integers(1, 300), st.integers(1, 6), st.integers(1, 6), st.integers(0, 300))
def test_elastic_sampler_never_replays_or_drops_after_a_rescale(n, w_old, w_new, consumed):
    consumed = min(consumed, n)
    parts = []
    for r in range(w_new):
        s = ElasticDistributedSampler(n, w_old, 0, shuffle=True, seed=1)
        s.record_consumed(consumed)
        s.update_topology(w_new, r)
        parts += list(s)
    assert len(parts) == n - consumed and len(set(parts)) == len(parts)


@FAST
@given(st.lists(st.integers(1, 4), min_size=1, max_size=4))
def test_mesh_rank_coordinate_round_trip_and_groups_partition(shape):
    size = math.prod(shape)
    m = DeviceMesh(shape, 0)
    for r in range(size):
        assert m.coord_to_rank(m.rank_to_coord(r).coords) == r
    for d in range(len(shape)):
        groups = m.all_groups(d)
        assert sorted(x for g in groups for x in g) == list(range(size)) and all(len(g) == shape[d] for g in groups)


@FAST
@given(st.lists(st.integers(1, 5000), min_size=0, max_size=30), st.integers(1, 64))
def test_buckets_keep_order_cover_everything_and_respect_the_limit(numels, kb):
    mb = kb / 1024
    buckets = calculate_buckets(numels, mb, element_bytes=2)
    assert [i for b in buckets for i in b] == list(range(len(numels)))
    limit = int(mb * (1 << 20))
    for b in buckets:
        assert len(b) == 1 or sum(numels[i] * 2 for i in b) <= limit


@FAST
@given(st.floats(allow_nan=False, allow_infinity=False, width=32))
def test_soft_bfloat16_and_half_match_torch_rounding(x):
    t = torch.tensor([x], dtype=torch.float32)
    assert sf.bfloat16_bits_to_float(sf.float_to_bfloat16_bits(x)) == float(t.to(torch.bfloat16).float())
    want = float(t.to(torch.float16).float())
    got = sf.half_bits_to_float(sf.float_to_half_bits(x))
    assert got == want or (math.isinf(got) and math.isinf(want))


@FAST
@given(st.lists(st.floats(-1e6, 1e6, allow_nan=False), min_size=1, max_size=200), st.floats(0, 1))
def test_quantile_matches_torch_linear_interpolation(values, q):
    v = torch.tensor(values, dtype=torch.float64)
    assert abs(QuantileCalculator.calculate(v, q) - float(torch.quantile(v, q))) <= 1e-6 * max(1.0, float(v.abs().max()))


@FAST
@given(st.lists(st.tuples(st.integers(0, 12), st.integers(0, 12)), max_size=30))
def test_topological_order_respects_every_edge_or_reports_the_cycle(edges):
    g = DependencyGraph()
    for a, b in edges:
        if a != b:
            g.add_dependency(f"n{a}", [f"n{b}"])
    names = [f"n{i}" for i in range(13)]
    if g.has_cycle():
        return
    order = g.topological_order(names)
    pos = {n: i for i, n in enumerate(order)}
    assert len(order) == len(set(order)) and all(pos[f"n{b}"] < pos[f"n{a}"] for a, b in edges if a != b)


@FAST
@given(st.lists(st.tuples(st.integers(0, 9), st.integers(1, 40)), max_size=60), st.integers(40, 400))
def test_recomputation_cache_never_exceeds_its_budget(ops, budget):
    c = RecomputationCache(budget * 4)
    for key, n in ops:
        c.add(f"k{key}", torch.zeros(n))
        s = c.stats()
        assert s.size_bytes <= budget * 4 and s.entries <= 10
