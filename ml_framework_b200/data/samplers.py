"""Index samplers.

``DistributedSampler`` reproduces the reference's partition rule
(src/MLFramework/Data/DistributedSampler.cs:155-210): the permutation is seeded with
``seed + epoch``; rank r takes indices ``r, r + W, r + 2W, ...``; with ``drop_last`` the tail
that does not divide evenly is dropped, otherwise every rank gets ``ceil(N / W)`` slots and
slots past the end hold ``-1`` (callers skip them). ``ElasticDistributedSampler`` adds
``update_topology`` (src/MLFramework/Distributed/Data/ElasticDistributedSampler.cs:58).
"""
from __future__ import annotations

import math
from typing import Iterator, List, Optional

import torch


def _permutation(n: int, seed: int) -> List[int]:
    g = torch.Generator()
    g.manual_seed(seed)
    return torch.randperm(n, generator=g).tolist()


class SequentialSampler:
    def __init__(self, size: int):
        self.size = size

    def __iter__(self) -> Iterator[int]:
        return iter(range(self.size))

    def __len__(self):
        return self.size


class RandomSampler:
    def __init__(self, size: int, seed: int = 0):
        self.size, self.seed, self.epoch = size, seed, 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __iter__(self):
        return iter(_permutation(self.size, self.seed + self.epoch))

    def __len__(self):
        return self.size


class BatchSampler:
    def __init__(self, sampler, batch_size: int, drop_last: bool = False):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def __iter__(self):
        batch = []
        for i in self.sampler:
            if i < 0:
                continue
            batch.append(i)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else math.ceil(n / self.batch_size)


class DynamicBatchSampler:
    """Batches by a token budget: items are added until ``max_tokens`` would be exceeded."""

    def __init__(self, lengths: List[int], max_tokens: int, max_batch: Optional[int] = None):
        self.lengths, self.max_tokens, self.max_batch = lengths, max_tokens, max_batch

    def __iter__(self):
        batch, longest = [], 0
        for i, n in enumerate(self.lengths):
            new_longest = max(longest, n)
            if batch and (new_longest * (len(batch) + 1) > self.max_tokens or
                          (self.max_batch and len(batch) >= self.max_batch)):
                yield batch
                batch, new_longest = [], n
            batch.append(i)
            longest = new_longest
        if batch:
            yield batch


class DistributedSampler:
    def __init__(self, dataset_size: int, num_replicas: int, rank: int, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False):
        if num_replicas <= 0:
            raise ValueError("num_replicas must be positive")
        if not (0 <= rank < num_replicas):
            raise ValueError(f"rank {rank} out of range for {num_replicas} replicas")
        self.dataset_size, self.num_replicas, self.rank = dataset_size, num_replicas, rank
        self.shuffle, self.seed, self.drop_last, self.epoch = shuffle, seed, drop_last, 0
        self._build()

    def _build(self):
        N, W = self.dataset_size, self.num_replicas
        if N == 0:
            self.indices, self.num_samples, self.total_size = [], 0, 0
            return
        if self.drop_last:
            self.num_samples = N // W
            self.total_size = self.num_samples * W
        else:
            self.total_size = N
            self.num_samples = math.ceil(N / W)
        base = _permutation(self.total_size, self.seed + self.epoch) if self.shuffle else list(range(self.total_size))
        self.indices = []
        for i in range(self.num_samples):
            gidx = self.rank + i * W
            self.indices.append(base[gidx] if gidx < self.total_size else -1)

    def set_epoch(self, epoch: int):
        self.epoch = epoch
        self._build()

    def get_batch(self, start: int, size: int) -> List[int]:
        return [i for i in self.indices[start:start + size] if i >= 0]

    def __iter__(self):
        return iter(self.indices)

    def __len__(self):
        return self.num_samples


class ElasticDistributedSampler(DistributedSampler):
    """A distributed sampler whose world can change between epochs or mid-epoch; already
    consumed samples of the epoch are not replayed after a topology change."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.consumed = 0  # global samples consumed in the current epoch

    def record_consumed(self, global_count: int):
        self.consumed += global_count

    def update_topology(self, num_replicas: int, rank: int):
        if not (0 <= rank < num_replicas):
            raise ValueError("invalid rank for new topology")
        self.num_replicas, self.rank = num_replicas, rank
        N = self.dataset_size
        base = _permutation(N, self.seed + self.epoch) if self.shuffle else list(range(N))
        remaining = base[self.consumed:]
        self.indices = remaining[rank::num_replicas]
        self.num_samples = len(self.indices)
        self.total_size = len(remaining)

    def set_epoch(self, epoch: int):
        self.consumed = 0
        super().set_epoch(epoch)
