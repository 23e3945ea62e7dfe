"""Data pipeline on CPU: datasets and collation, samplers (sequential, random per epoch, batch, token budget, distributed
with padding / drop-last, elastic topology changes without replay), loader configuration, iterable datasets, staging
pool, transforms."""
import pytest
import torch

from ml_framework_b200.data import transforms as T
from ml_framework_b200.data.loader import (DataLoader, DataLoaderConfig, DataLoaderConfigBuilder, IterableDataset, ListDataset,
                                           PinnedMemoryPool, TensorDataset, default_collate)
from ml_framework_b200.data.samplers import (BatchSampler, DistributedSampler, DynamicBatchSampler, ElasticDistributedSampler,
                                             RandomSampler, SequentialSampler)


def test_datasets_and_collation_of_nested_structures():
    x, y = torch.arange(12.0).view(6, 2), torch.arange(6)
    ds = TensorDataset(x, y)
    assert len(ds) == 6 and torch.equal(ds[4][0], x[4]) and int(ds[4][1]) == 4
    with pytest.raises(ValueError):
        TensorDataset(x, torch.arange(5))
    with pytest.raises(ValueError):
        TensorDataset()
    items = [{"a": torch.tensor([i, i]), "b": (float(i), [i, i + 1]), "name": f"s{i}"} for i in range(3)]
    out = default_collate(items)
    assert out["a"].shape == (3, 2) and out["b"][0].tolist() == [0.0, 1.0, 2.0] and out["name"] == ["s0", "s1", "s2"]
    assert isinstance(out["b"][1], list) and out["b"][1][1].tolist() == [1, 2, 3]
    ld = ListDataset(items)
    assert len(ld) == 3 and ld[1]["name"] == "s1"
    dl = DataLoader(ds, batch_size=4)                                            # keyword configuration
    batches = list(dl)
    assert [b[0].shape[0] for b in batches] == [4, 2] and dl.metrics()["batches"] == 2 and len(dl) == 2
    dl = DataLoader(ds, DataLoaderConfig(batch_size=4, drop_last=True), transform=lambda it: (it[0] * 2, it[1]))
    (bx, by), = list(dl)
    assert torch.equal(bx, x[:4] * 2) and by.tolist() == [0, 1, 2, 3]
    moved = list(DataLoader(ds, DataLoaderConfig(batch_size=6, device="cpu")))
    assert moved[0][0].device.type == "cpu"


def test_iterable_dataset_batches_and_drop_last():
    class Stream(IterableDataset):
        def __iter__(self):
            return iter(torch.tensor(i) for i in range(7))
    assert [b.tolist() for b in DataLoader(Stream(), DataLoaderConfig(batch_size=3))] == [[0, 1, 2], [3, 4, 5], [6]]
    assert [b.tolist() for b in DataLoader(Stream(), DataLoaderConfig(batch_size=3, drop_last=True, num_workers=2))] == [[0, 1, 2], [3, 4, 5]]
    with pytest.raises(NotImplementedError):
        iter(IterableDataset())


def test_samplers_cover_every_index_once_and_reshuffle_per_epoch():
    assert list(SequentialSampler(4)) == [0, 1, 2, 3] and len(SequentialSampler(4)) == 4
    rs = RandomSampler(50, seed=3)
    e0 = list(rs)
    assert sorted(e0) == list(range(50)) and list(rs) == e0                       # same epoch, same order
    rs.set_epoch(1)
    assert sorted(rs) == list(range(50)) and list(rs) != e0
    bs = BatchSampler(SequentialSampler(10), 4)
    assert list(bs) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]] and len(bs) == 3 and len(BatchSampler(SequentialSampler(10), 4, True)) == 2
    with pytest.raises(ValueError):
        BatchSampler(SequentialSampler(3), 0)
    dl = DataLoader(ListDataset(list(range(20))), DataLoaderConfig(batch_size=5, shuffle=True, seed=9))
    first = [b.tolist() for b in dl]
    dl.set_epoch(1)
    second = [b.tolist() for b in dl]
    assert sorted(sum(first, [])) == list(range(20)) == sorted(sum(second, [])) and first != second
    dyn = DynamicBatchSampler([10, 12, 50, 8, 8, 8, 8, 60], max_tokens=64, max_batch=3)
    got = list(dyn)
    assert sum(got, []) == list(range(8))
    lens = [10, 12, 50, 8, 8, 8, 8, 60]
    assert all(max(lens[i] for i in b) * len(b) <= 64 or len(b) == 1 for b in got) and all(len(b) <= 3 for b in got)


@pytest.mark.parametrize("n,w", [(10, 4), (16, 4), (3, 4), (0, 2)])
def test_distributed_sampler_partitions_pads_and_drops(n, w):
    parts = [DistributedSampler(n, w, r, shuffle=True, seed=5) for r in range(w)]
    real = [i for p in parts for i in p if i >= 0]
    assert sorted(real) == list(range(n))                                          # every sample exactly once
    assert len({len(p) for p in parts}) == 1                                       # equal lengths (the tail is padded with -1)
    assert all(len(p) == (0 if n == 0 else -(-n // w)) for p in parts)
    if n:
        for p in parts:
            assert p.get_batch(0, len(p)) == [i for i in p.indices if i >= 0]
        seq = DistributedSampler(n, w, 0, shuffle=False)
        assert [i for i in seq if i >= 0] == list(range(0, n, w))
        p0 = parts[0]
        before = list(p0)
        p0.set_epoch(1)
        assert n < 3 or list(p0) != before or n <= w
    dropped = [DistributedSampler(n, w, r, shuffle=False, drop_last=True) for r in range(w)]
    assert all(len(d) == n // w for d in dropped) and all(i >= 0 for d in dropped for i in d)
    with pytest.raises(ValueError):
        DistributedSampler(n, w, w)
    with pytest.raises(ValueError):
        DistributedSampler(n, 0, 0)


def test_elastic_sampler_does_not_replay_after_a_topology_change():
    N = 40
    old = [ElasticDistributedSampler(N, 4, r, shuffle=True, seed=1) for r in range(4)]
    consumed = []
    for step in range(3):                                                          # three steps of one sample per rank
        consumed += [s.indices[step] for s in old]
    for s in old:
        s.record_consumed(12)
    new = [old[r] for r in range(3)]                                               # rank 3 left: three ranks go on
    for r, s in enumerate(new):
        s.update_topology(3, r)
    rest = [i for s in new for i in s]
    assert sorted(consumed + rest) == list(range(N)) and len(set(consumed) & set(rest)) == 0
    assert sum(len(s) for s in new) == N - 12 and new[0].total_size == N - 12
    with pytest.raises(ValueError):
        new[0].update_topology(2, 2)
    new[0].set_epoch(1)
    assert new[0].consumed == 0 and len(new[0]) == -(-N // 3)


def test_loader_configuration_presets_builder_and_staging_pool():
    c = DataLoaderConfigBuilder().batch_size(16).shuffle().workers(2).prefetch(3).device("cpu").drop_last().build()
    assert (c.batch_size, c.shuffle, c.num_workers, c.prefetch_batches, c.device, c.drop_last) == (16, True, 2, 3, "cpu", True)
    with pytest.raises(ValueError):
        DataLoaderConfigBuilder().batch_size(0).build()
    with pytest.raises(ValueError):
        DataLoaderConfig(prefetch_batches=0).validate()
    assert DataLoaderConfig.for_cpu_bound(6).num_workers == 6 and DataLoaderConfig.for_debugging().num_workers == 0
    g = DataLoaderConfig.for_gpu_training(32, "cuda:1")
    assert g.batch_size == 32 and g.shuffle and g.drop_last and g.device == "cuda:1"
    pool = PinnedMemoryPool(max_per_key=1)
    a = pool.get((4, 4), torch.float32)
    pool.put(a)
    pool.put(torch.empty(4, 4))                                                    # over the per-key limit: dropped
    assert pool.get((4, 4), torch.float32) is a and pool.reuses == 1 and pool.allocations == 1
    assert pool.get((4, 4), torch.float32) is not a and pool.allocations == 2


def test_transforms_lambda_crop_resize_and_normalize():
    x = torch.arange(2 * 3 * 8 * 8, dtype=torch.float32).view(2, 3, 8, 8)
    assert T.Resize((4, 6))(x).shape == (2, 3, 4, 6) and T.Resize(4, mode="nearest")(x[0]).shape == (3, 4, 4)
    c1, c2 = T.RandomCrop(5, seed=7), T.RandomCrop(5, seed=7)
    assert torch.equal(c1(x), c2(x)) and c1(x).shape == (2, 3, 5, 5)
    pipe = T.Compose([T.Lambda(lambda t: t + 1), T.Lambda(lambda t: t * 2)])
    assert torch.equal(pipe(torch.ones(2)), torch.full((2,), 4.0))
    n = T.Normalize([1.0, 2.0, 3.0], [2.0, 2.0, 2.0])(torch.ones(3, 2, 2) * torch.tensor([1.0, 2.0, 3.0]).view(3, 1, 1))
    assert torch.allclose(n, torch.zeros(3, 2, 2))
