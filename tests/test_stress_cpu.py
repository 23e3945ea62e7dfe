"""Stress and concurrency tests of the host-side runtime pieces (native block manager, allocators, schedulers):
long allocate / free loops, rapid sequence turnover, pool exhaustion that fails gracefully, concurrent callers,
and leak checks (everything returned at the end). The reference's counterparts:
tests/MLFramework.Tests/Inference/PagedAttention/Stress/PagedAttentionStressTests.cs:44-384, tests/HAL/ConcurrencyTests.cs."""
import random
import threading

import pytest
import torch

from ml_framework_b200.serving.kv_cache import BlockShareManager, BlockTable, KVCacheBlockManager


def _mgr(total=256, bs=16):
    return KVCacheBlockManager(total, bs, head_dim=8, num_layers=1, num_kv_heads=1, device="cpu", dtype=torch.float32,
                               allocate_cache=False)


def test_rapid_sequence_turnover_leaves_no_blocks_behind():
    m = _mgr(128, 16)
    rng = random.Random(0)
    live = {}
    for it in range(4000):
        if live and (rng.random() < 0.45 or m.free_blocks < 8):
            sid = rng.choice(list(live))
            assert m.free_sequence_blocks(sid) == m.blocks_needed(live.pop(sid))
        else:
            sid, n = it + 1, rng.randint(1, 70)
            slots, _ = m.append_tokens(sid, n)
            if slots is None:                                    # exhausted: nothing may have been kept for this id
                assert m.get_sequence_length(sid) == 0 and m.get_sequence_blocks(sid) == []
                continue
            assert len(slots) == n and len(set(slots.tolist())) == n
            live[sid] = n
        used = sum(m.blocks_needed(n) for n in live.values())
        assert m.free_blocks == 128 - used
    for sid in list(live):
        m.free_sequence_blocks(sid)
    st = m.get_stats()
    assert m.free_blocks == 128 and st.allocated_blocks == 0


def test_pool_exhaustion_fails_gracefully_and_recovers():
    m = _mgr(8, 4)
    assert m.allocate_blocks(1, 6).success
    r = m.allocate_blocks(2, 3)
    assert not r.success and r.block_ids == [] and "cannot allocate" in r.error and m.free_blocks == 2
    slots, _ = m.append_tokens(3, 4 * 3)                            # needs three blocks, two are free: all or nothing
    assert slots is None and m.free_blocks == 2 and m.get_sequence_length(3) == 0
    assert m.allocate_block(4).success and m.allocate_block(4).success and not m.allocate_block(4).success
    assert not m.has_available_blocks(1)
    assert m.free_sequence_blocks(1) == 6 and m.has_available_blocks(6)
    slots, _ = m.append_tokens(3, 4 * 3)
    assert slots is not None and m.get_sequence_length(3) == 12
    with pytest.raises(KeyError):
        m.truncate(99, 0)
    assert m.free_sequence_blocks(99) <= 0                         # unknown sequence: nothing freed, no exception
    with pytest.raises(ValueError):
        KVCacheBlockManager(0, 16, allocate_cache=False)


def test_slots_of_live_sequences_never_collide_under_growth():
    m = _mgr(512, 16)
    rng = random.Random(1)
    owner = {}
    lengths = {s: 0 for s in range(1, 33)}
    for _ in range(1500):
        s = rng.choice(list(lengths))
        n = rng.randint(1, 9)
        slots, cow = m.append_tokens(s, n)
        if slots is None:
            victim = max(lengths, key=lengths.get)
            for k in [k for k, v in owner.items() if v == victim]:
                del owner[k]
            m.free_sequence_blocks(victim)
            lengths[victim] = 0
            continue
        assert cow is None
        for sl in slots.tolist():
            assert sl not in owner, "a cache slot was handed to two live sequences"
            owner[sl] = s
        lengths[s] += n
        assert m.get_sequence_length(s) == lengths[s]
        assert len(m.get_sequence_blocks(s)) == m.blocks_needed(lengths[s])
    bt = BlockTable(m)
    for s, n in lengths.items():
        if n:
            blocks = m.get_sequence_blocks(s)
            assert bt.get_block(s, n - 1) == blocks[(n - 1) // 16]


def test_long_sequence_block_list_is_complete():
    m = _mgr(5000, 1)
    slots, _ = m.append_tokens(7, 4500)                            # more blocks than the first query buffer holds
    assert slots is not None
    blocks = m.get_sequence_blocks(7)
    assert len(blocks) == 4500 and len(set(blocks)) == 4500


def test_concurrent_allocation_and_release_from_many_threads():
    m = _mgr(1024, 8)
    errors, taken = [], [set() for _ in range(8)]

    def worker(t):
        rng = random.Random(t)
        try:
            for i in range(400):
                sid = t * 100000 + i
                n = rng.randint(1, 40)
                slots, _ = m.append_tokens(sid, n)
                if slots is None:
                    continue
                got = set(m.get_sequence_blocks(sid))
                if len(got) != m.blocks_needed(n):
                    errors.append(("blocks", sid, len(got)))
                taken[t] = got
                if rng.random() < 0.3:
                    slots2, _ = m.append_tokens(sid, 5)
                if m.free_sequence_blocks(sid) <= 0:
                    errors.append(("free", sid))
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))
    ths = [threading.Thread(target=worker, args=(t,)) for t in range(8)]
    for th in ths:
        th.start()
    for th in ths:
        th.join(60)
    assert not errors, errors[:3]
    assert m.free_blocks == 1024 and m.get_stats().allocated_blocks == 0


def test_shared_prefixes_are_reference_counted_through_churn():
    m = _mgr(64, 4)
    share = BlockShareManager(m)
    slots, _ = m.append_tokens(1, 16)                               # four full blocks
    base = m.get_sequence_blocks(1)
    for child in range(2, 12):
        assert share.share_prefix(1, child, 16) == 4
    assert all(m.reference_count(b) == 11 for b in base) and m.free_blocks == 60
    # every child diverges: the first append of each copies nothing (the prefix is block-aligned) and takes one block
    for child in range(2, 12):
        s, cow = m.append_tokens(child, 1)
        assert s is not None and cow is None
    assert m.free_blocks == 50
    for child in range(2, 12):
        share.release_sequence(child)
    assert all(m.reference_count(b) == 1 for b in base) and m.free_blocks == 60
    # the share manager hands out whole blocks only: 14 tokens share three blocks, the next token opens a fresh one
    assert share.share_prefix(1, 50, 14) == 3 and m.get_sequence_length(50) == 12
    s, cow = m.append_tokens(50, 1)
    assert s is not None and cow is None and int(s[0]) % 4 == 0
    share.release_sequence(50)
    # a fork in the middle of a block shares that block too, and the first write into it copies it (copy on write)
    assert m.fork(1, 51, 14) == 4 and m.reference_count(base[3]) == 2
    s, cow = m.append_tokens(51, 1)
    assert s is not None and cow is not None and cow[0] == base[3] and cow[1] != base[3] and m.reference_count(base[3]) == 1
    assert int(s[0]) == cow[1] * 4 + 2
    m.free_sequence_blocks(51)
    m.free_sequence_blocks(1)
    assert m.free_blocks == 64


def test_allocators_stay_consistent_under_concurrent_use():
    from ml_framework_b200.hal import core
    d = core.BackendRegistry.get("cpu").device(0)
    for alloc in (core.CachingAllocator(d, max_cached_bytes=1 << 20), core.SimpleAllocator(d)):
        errors = []

        def worker(t):
            rng = random.Random(t)
            held = []
            try:
                for _ in range(300):
                    if held and rng.random() < 0.5:
                        held.pop(rng.randrange(len(held))).free()
                    else:
                        b = alloc.allocate(rng.choice([64, 500, 513, 4096, 70000]))
                        b.tensor[:8] = t                                  # the block is this thread's alone
                        held.append(b)
                    for b in held:
                        if int(b.tensor[0]) != t:
                            errors.append("a live block was handed out twice")
                for b in held:
                    b.free()
            except Exception as e:  # noqa: BLE001
                errors.append(repr(e))
        ths = [threading.Thread(target=worker, args=(t,)) for t in range(1, 9)]
        for th in ths:
            th.start()
        for th in ths:
            th.join(60)
        assert not errors, errors[:3]
        assert alloc.allocated_bytes == 0 and alloc.peak_bytes > 0 and alloc.n_allocs > 0
        if isinstance(alloc, core.CachingAllocator):
            assert alloc.cached_bytes <= 1 << 20 and alloc.hits > 0
            alloc.empty_cache()
            assert alloc.cached_bytes == 0


def test_scheduler_throughput_and_latency_under_a_burst_with_kv_accounting():
    """Two hundred requests of mixed lengths through the continuous-batching scheduler with real block accounting and a
    deterministic mock model: every request completes with exactly its tokens, batches stay within the limit, memory
    is returned, and the latency distribution is ordered (p50 <= p99 <= max)."""
    from ml_framework_b200.serving.scheduler import (BatchOutput, CompletionConfiguration, ContinuousBatchScheduler, Request,
                                                     SchedulerConfiguration)

    class Exec:
        def __init__(self, kv):
            self.kv, self.max_batch = kv, 0

        def execute_batch(self, batch):
            self.max_batch = max(self.max_batch, len(batch.requests))
            out = {}
            for r in batch.requests:
                if r.prefilled < len(r.prompt_tokens):
                    n = len(r.prompt_tokens) - r.prefilled
                    slots, _ = self.kv.append_tokens(r.id, n)
                    assert slots is not None
                    r.prefilled = len(r.prompt_tokens)
                else:
                    slots, _ = self.kv.append_tokens(r.id, 1)
                    assert slots is not None
                out[r.id] = 1000 + len(r.generated)
            return BatchOutput(out)
    kv = _mgr(2048, 16)
    ex = Exec(kv)
    s = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=16), completion=CompletionConfiguration(eos_token_id=-1))
    rng = random.Random(3)
    reqs = [Request([1] * rng.randint(1, 200), max_tokens=rng.randint(1, 24)) for _ in range(200)]
    futs = [s.enqueue(r) for r in reqs]
    s.run_until_idle()
    res = [f.result(0) for f in futs]
    assert all(len(x.tokens) == r.max_tokens and x.tokens == [1000 + i for i in range(r.max_tokens)] for x, r in zip(res, reqs))
    assert ex.max_batch <= 16 and kv.free_blocks == 2048 and kv.get_stats().allocated_blocks == 0
    lat = sorted(x.latency_s for x in res)
    assert lat[len(lat) // 2] <= lat[int(0.99 * len(lat))] <= lat[-1] and all(x.ttft_s <= x.latency_s for x in res)
    snap = s.metrics.snapshot()
    assert snap["completed"] == 200 and snap["total_tokens"] == sum(r.max_tokens for r in reqs)


def test_dynamic_batcher_under_concurrent_submitters():
    from ml_framework_b200.serving import dynamic_batcher as DB
    sizes = []
    b = DB.DynamicBatcher(lambda reqs: (sizes.append(len(reqs)), [r + 1 for r in reqs])[1],
                          DB.BatchingConfiguration(max_batch_size=16, prefer_batch_size=8, max_wait_time_s=0.005, max_queue_size=4096))
    results, errors = {}, []

    def client(t):
        try:
            fs = [(i, b.submit(t * 1000 + i)) for i in range(100)]
            for i, f in fs:
                results[(t, i)] = f.result(30)
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))
    ths = [threading.Thread(target=client, args=(t,)) for t in range(8)]
    for th in ths:
        th.start()
    for th in ths:
        th.join(60)
    b.shutdown()
    assert not errors and len(results) == 800
    assert all(v == t * 1000 + i + 1 for (t, i), v in results.items())
    assert max(sizes) <= 16 and sum(sizes) == 800 and b.metrics.requests == 800
