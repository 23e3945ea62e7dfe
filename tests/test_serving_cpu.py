"""Serving stack on CPU: native block manager / table / sharing, request queue, capacity,
completion rules, continuous-batching scheduler with a mock executor (incl. a failing one),
and the paged Llama executor against plain full-sequence greedy decoding."""
import threading
import time

import pytest
import torch

from ml_framework_b200.models import Llama, LlamaConfig
from ml_framework_b200.serving.executor import ExecutorConfig, PagedLlamaExecutor
from ml_framework_b200.serving.kv_cache import (BeamSearchBlockSharing, BlockShareManager, BlockTable, KVCacheBlockManager,
                                                SpeculativeDecodingSharing)
from ml_framework_b200.serving.scheduler import (BatchConstraints, BatchOutput, CapacityConstraints, CapacityManager,
                                                 CompletionConfiguration, CompletionDetector, CompletionReason,
                                                 ContinuousBatchScheduler, ContinuousBatchSchedulerClient,
                                                 PagedAttentionScheduler, PrefillConfiguration, PrefillHandler, Priority,
                                                 Request, RequestQueue, SchedulerConfiguration)


def test_block_manager_allocation_and_stats():
    m = KVCacheBlockManager(8, 16, allocate_cache=False)
    assert m.allocate_block(1).block_ids == [0]
    r = m.allocate_blocks(1, 3)
    assert r.success and r.block_ids == [1, 2, 3] and m.get_sequence_blocks(1) == [0, 1, 2, 3]
    bad = m.allocate_blocks(2, 5)                      # all-or-nothing
    assert not bad.success and m.free_blocks == 4 and m.get_sequence_blocks(2) == []
    assert m.free_sequence_blocks(1) == 4 and m.free_blocks == 8
    st = m.get_stats()
    assert (st.total_blocks, st.allocated_blocks, st.total_allocations, st.total_frees, st.failed_allocations) == (8, 0, 4, 4, 1)
    assert m.allocate_block(3).block_ids == [4]        # FIFO free list: freed blocks go to the back
    with pytest.raises(ValueError):
        KVCacheBlockManager(0, 16, allocate_cache=False)


def test_append_tokens_table_and_lengths():
    m = KVCacheBlockManager(6, 4, allocate_cache=False)
    slots, cow = m.append_tokens(7, 6)
    assert slots.tolist() == [0, 1, 2, 3, 4, 5] and cow is None and m.get_sequence_length(7) == 6
    slots, _ = m.append_tokens(7, 3)
    assert slots.tolist() == [6, 7, 8] and m.get_sequence_blocks(7) == [0, 1, 2]
    t = BlockTable(m)
    assert t.get_block(7, 5) == 1 and t.get_sequence_length(7) == 9
    with pytest.raises(IndexError):
        t.get_block(7, 100)
    table, lens = m.build_tables([7, 99], 4)
    assert table.tolist() == [[0, 1, 2, -1], [-1, -1, -1, -1]] and lens.tolist() == [9, 0]
    assert m.append_tokens(8, 100)[0] is None and m.get_stats().failed_allocations == 1
    assert m.truncate(7, 4) == 2 and m.get_sequence_blocks(7) == [0]


def test_prefix_sharing_copy_on_write_beams_and_speculation():
    m = KVCacheBlockManager(16, 4, head_dim=8, num_layers=1, num_kv_heads=1, device="cpu", dtype=torch.float32)
    m.append_tokens(1, 6)                               # blocks 0 (full), 1 (2 of 4 used)
    m.caches[0][1].fill_(3.0)
    sh = BlockShareManager(m)
    assert sh.share_prefix(1, 2, 6) == 1                # only the whole block is shared
    assert sh.get_reference_count(0) == 2 and m.get_sequence_length(2) == 4
    beams = BeamSearchBlockSharing(m)
    beams.initialize_beams(1, [10, 11])
    assert m.reference_count(1) == 3
    slots, cow = beams.on_beam_divergence(10)           # writes into a shared partial block -> copy first
    assert cow is not None and cow[0] == 1 and m.reference_count(1) == 2
    assert torch.equal(m.caches[0][cow[1]], m.caches[0][1]) and slots.tolist() == [cow[1] * 4 + 2]
    beams.cleanup_beams(1)
    assert m.reference_count(1) == 1
    spec = SpeculativeDecodingSharing(m)
    spec.allocate_speculative_blocks(1, 7)
    assert m.get_sequence_length(1) == 13
    spec.verify_speculation(1, 2)
    assert m.get_sequence_length(1) == 8 and len(m.get_sequence_blocks(1)) == 2
    sh.register_prefix([5, 6, 7, 8], 1)
    assert sh.find_prefix([5, 6, 7, 8, 9]) == (1, 4) and sh.find_prefix([5, 6]) is None
    free_before = m.free_blocks
    sh.release_sequence(1)
    assert m.free_blocks == free_before + 1             # block 0 is still held by sequence 2


def test_queue_capacity_completion_and_admission():
    q = RequestQueue()
    rs = [Request([1], priority=p) for p in (Priority.LOW, Priority.URGENT, Priority.NORMAL, Priority.URGENT)]
    for r in rs:
        q.enqueue(r)
    assert q.mark_cancelled(rs[3].id)
    got = q.get_requests(10, lambda r: True)
    assert [r.id for r in got] == [rs[1].id, rs[2].id, rs[0].id]
    assert rs[3].future.result(0).reason == CompletionReason.CANCELLED
    q.enqueue(Request([1] * 10)); q.enqueue(Request([1]))
    assert len(q.get_requests(5, lambda r: len(r.prompt_tokens) < 5)) == 0     # head does not fit: nobody jumps the queue
    cap = CapacityManager(CapacityConstraints(max_batch_size=2, max_memory_bytes=10_000, buffer_ratio=0.1), bytes_per_token=10)
    a, b, c = Request([0] * 100, max_tokens=300), Request([0] * 100, max_tokens=300), Request([0] * 10, max_tokens=10)
    assert cap.try_allocate(a) and cap.try_allocate(b) and not cap.try_allocate(c)   # slots exhausted
    cap.release(a.id)
    big = Request([0] * 500, max_tokens=500)
    assert not cap.try_allocate(big) and cap.try_allocate(c)                          # 9000 usable bytes
    det = CompletionDetector(CompletionConfiguration(eos_token_id=2, max_response_length=50), detokenize=lambda t: "".join(map(str, t)))
    r = Request([1, 1], max_tokens=3, stop_strings=("77",))
    assert det.check(r) is None
    r.generated = [5, 2]
    assert det.check(r) == CompletionReason.EOS
    r.generated = [7, 7]
    assert det.check(r) == CompletionReason.STOP_STRING
    r.generated = [5, 5, 5]
    assert det.check(r) == CompletionReason.MAX_TOKENS
    r.cancelled = True
    assert det.check(r) == CompletionReason.CANCELLED
    m = KVCacheBlockManager(10, 16, allocate_cache=False)
    adm = PagedAttentionScheduler(m, reserved_blocks=2)
    assert adm.can_admit(100, 28) and not adm.can_admit(100, 29)
    m.allocate_blocks(1, 8)
    assert adm.should_apply_backpressure() and adm.recommended_max_sequence_length(1) == 0
    ph = PrefillHandler(PrefillConfiguration(chunk_size=4, prompt_cache_entries=1), clock=lambda: 0.0)
    rr = Request(list(range(10)))
    assert ph.next_chunk(rr) == [0, 1, 2, 3] and ph.needs_prefill(rr)
    ph.cache_store([1, 2], "a"); ph.cache_store([3], "b")
    assert ph.cache_lookup([1, 2]) is None and ph.cache_lookup([3]) == "b"


class MockExecutor:
    """Emits prompt_len + k as the k-th token and EOS (2) after ``eos_after`` tokens."""

    def __init__(self, eos_after=4, fail_on=None):
        self.eos_after, self.fail_on, self.calls, self.batch_sizes = eos_after, fail_on, 0, []

    def execute_batch(self, batch):
        self.calls += 1
        self.batch_sizes.append(len(batch.requests))
        if self.fail_on is not None and self.calls == self.fail_on:
            raise RuntimeError("model blew up")
        out = {}
        for r in batch.requests:
            r.prefilled = len(r.prompt_tokens)
            k = len(r.generated)
            out[r.id] = 2 if k + 1 >= self.eos_after else 100 + k
        return BatchOutput(out)


class Tok:
    def encode(self, s): return [ord(c) % 50 + 3 for c in s]
    def decode(self, t): return " ".join(map(str, t))


def test_scheduler_end_to_end_with_mock_executor():
    ex = MockExecutor(eos_after=4)
    s = ContinuousBatchScheduler(ex, None, SchedulerConfiguration(max_batch_size=3))
    reqs = [Request([1, 2, 3], max_tokens=10) for _ in range(7)] + [Request([1], max_tokens=2)]
    futs = [s.enqueue(r) for r in reqs]
    s.run_until_idle()
    res = [f.result(0) for f in futs]
    assert all(r.reason == CompletionReason.EOS and r.tokens == [100, 101, 102, 2] for r in res[:7])
    assert res[7].reason == CompletionReason.MAX_TOKENS and res[7].tokens == [100, 101]
    assert max(ex.batch_sizes) == 3 and s.metrics.snapshot()["completed"] == 8
    assert s.metrics.snapshot()["reasons"] == {"eos": 7, "max_tokens": 1}
    assert all(r.ttft_s is not None and r.latency_s >= r.ttft_s for r in res)


def test_scheduler_survives_executor_failure_and_background_loop():
    ex = MockExecutor(eos_after=3, fail_on=2)
    s = ContinuousBatchScheduler(ex, None, SchedulerConfiguration(max_batch_size=2))
    client = ContinuousBatchSchedulerClient(s, Tok())
    s.start()
    try:
        a = client.submit("hello", 8)
        b = client.submit("world", 8)
        ra, rb = a.future.result(5), b.future.result(5)
        assert {ra.reason, rb.reason} == {CompletionReason.ERROR} and "blew up" in ra.error
        ok = client.generate_text("again", 8, timeout_s=5)
        assert ok.reason == CompletionReason.EOS and ok.text == "100 101 2"
        assert client.statistics()["errors"] == {"RuntimeError": 1} and client.status()["running"] == 0
        c = client.submit("x", 1000)
        assert client.cancel(c.id) and c.future.result(5).reason in (CompletionReason.CANCELLED, CompletionReason.EOS)
    finally:
        s.stop()


@pytest.mark.parametrize("torch_ops", [False, True])
def test_paged_llama_executor_matches_full_sequence_greedy(torch_ops):
    torch.manual_seed(0)
    cfg = LlamaConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128, vocab_size=50, max_seq=64, vocab_multiple=8)
    model = Llama(cfg).eval()
    kv = KVCacheBlockManager(64, 4, head_dim=16, num_layers=2, num_kv_heads=2, device="cpu", dtype=torch.float32)
    ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=8, max_seq_len=64, prefill_chunk=5, torch_ops=torch_ops))
    s = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=4), completion=CompletionConfiguration(eos_token_id=-1))
    prompts = [[3, 7, 11, 2, 9, 30, 4], [5, 6], [40, 41, 42, 43, 44, 45, 46, 47, 48, 1, 2]]
    reqs = [Request(p, max_tokens=6) for p in prompts]
    futs = [s.enqueue(r) for r in reqs]
    s.run_until_idle()
    for p, f in zip(prompts, futs):
        seq = list(p)
        for _ in range(6):
            with torch.no_grad():
                logits = model(torch.tensor([seq]))
            seq.append(int(logits[0, -1].argmax()))
        assert f.result(0).tokens == seq[len(p):], (p, f.result(0).tokens, seq[len(p):])
    assert kv.get_stats().allocated_blocks == 0          # everything released after completion


def test_iteration_level_manager_memory_aware_queue_and_cache_manager():
    from ml_framework_b200.serving.iteration import (ContinuousBatchKVCacheManager, ContinuousBatchManager, IterationScheduler,
                                                     IterationSchedulerConfig, MemoryAwareScheduler, PendingRequest)
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.scheduler import KVCacheConfiguration, PagedAttentionScheduler
    bm = KVCacheBlockManager(total_blocks=16, block_size=4, allocate_cache=False)
    mem = MemoryAwareScheduler(PagedAttentionScheduler(bm), max_queue_size=3)
    assert all(mem.enqueue_request(PendingRequest(i, estimated_max_tokens=20, prompt_tokens=8)) for i in range(3))
    assert not mem.enqueue_request(PendingRequest(9, 8))            # queue bound
    batch = ContinuousBatchManager(bm, max_batch_size=2)
    log = []

    def prefill(seqs, ranges):
        for s in seqs:
            lo, hi = ranges[s]
            bm.append_tokens(s, hi - lo)
        log.append(("prefill", list(seqs), dict(ranges)))

    def decode(seqs, lengths):
        for s in seqs:
            bm.append_tokens(s, 1)
        log.append(("decode", list(seqs), dict(lengths)))
    sch = IterationScheduler(batch, mem, prefill, decode, IterationSchedulerConfig(max_batch_size=2, max_prefill_per_iteration=4))
    st = sch.run_iteration()
    assert st.total_sequences == 2 and st.prefill_sequences == 2 and mem.queue_size() == 1
    assert log[0] == ("prefill", [0, 1], {0: (0, 8), 1: (0, 8)})
    sch.run_iteration()
    assert log[-1] == ("decode", [0, 1], {0: 8, 1: 8}) and bm.get_sequence_length(0) == 9
    batch.remove_sequence(0)
    sch.run_iteration()                                            # the queued request takes the free slot
    assert sorted(batch.current_batch()) == [1, 2] and batch.stats().utilization == 1.0
    batch.clear()
    assert bm.free_blocks == 16

    # request-level cache allocations: growth, bounded pages, compaction that returns pages
    cm = ContinuousBatchKVCacheManager(bm, KVCacheConfiguration(page_size_tokens=4, initial_pages=2, max_pages_per_request=6,
                                                                target_utilization=0.5), bytes_per_token=10)
    assert cm.allocate_cache(100, max_tokens=4) == 2 * 40           # initial pages
    assert cm.allocate_cache(101, max_tokens=100) == 6 * 40         # capped
    with pytest.raises(RuntimeError):
        cm.allocate_cache(100, 4)
    assert cm.try_extend_cache(100, 9) and cm.get_allocation(100).page_count == 5
    assert cm.try_extend_cache(100, 100) and cm.get_allocation(100).page_count == 6
    assert not cm.try_extend_cache(100, 1)                          # at the cap
    assert cm.current_usage_bytes() == 12 * 40 and bm.free_blocks == 4
    with pytest.raises(MemoryError):
        cm.allocate_cache(102, max_tokens=40)
    assert bm.free_blocks == 4                                     # nothing leaked by the failed allocation
    bm.append_tokens(100, 5)                                        # request 100 really uses 2 pages
    freed = cm.compact_cache()
    assert freed == 4 + 4 and bm.free_blocks == 12                 # 100 keeps 2 pages, 101 (no tokens) keeps its initial 2
    assert cm.get_allocation(100).page_count == 2 and cm.get_allocation(101).page_count == 2
    cm.release_cache(100)
    cm.release_cache(101)
    assert cm.allocation_count == 0 and bm.free_blocks == 16


def test_scheduler_warmup_iterations_and_iteration_timeout():
    from ml_framework_b200.serving.scheduler import (BatchOutput, ContinuousBatchScheduler, Request, SchedulerConfiguration)
    t = {"now": 0.0}

    class SlowExecutor:
        def __init__(self):
            self.warm, self.calls = [], 0

        def warm_up(self, i):
            self.warm.append(i)

        def execute_batch(self, batch):
            self.calls += 1
            t["now"] += 2.0 if self.calls == 1 else 0.001          # the first iteration overruns its budget
            for r in batch.prefill:
                r.prefilled = len(r.prompt_tokens)
            return BatchOutput({r.id: 7 for r in batch.requests})
    ex = SlowExecutor()
    s = ContinuousBatchScheduler(ex, config=SchedulerConfiguration(iteration_timeout_ms=500.0, warmup_iterations=3, max_batch_size=4),
                                 clock=lambda: t["now"])
    assert s.warm_up() == 3 and ex.warm == [0, 1, 2]
    r1 = Request([1, 2, 3], max_tokens=2)
    f1 = s.enqueue(r1)
    assert s.execute_iteration()
    assert s.timed_out_iterations == 1 and s.metrics.snapshot()["errors"].get("IterationTimeout") == 1
    f2 = s.enqueue(Request([4, 5], max_tokens=1))
    assert s.execute_iteration()                                   # after an overrun: no admission in this iteration
    assert [r.id for r in s.batch_manager.running] in ([r1.id], []) and not f2.done()
    s.run_until_idle()
    assert f1.result().tokens == [7, 7] and f2.result().tokens == [7]


def test_paged_attention_layer_prefill_chunks_and_decode_match_contiguous_attention():
    """The layer fed a prompt in two chunks and then token by token gives what one causal attention over the whole
    sequence gives (the reference's paged-vs-contiguous equivalence)."""
    import torch
    from ml_framework_b200.ops import reference
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.paged_attention_layer import AttentionPhase, PagedAttentionLayer
    torch.manual_seed(0)
    d, hq, hkv, D = 32, 4, 2, 8
    layer = PagedAttentionLayer(d, hq, hkv, D, rope_theta=10000.0)
    kv = KVCacheBlockManager(total_blocks=32, block_size=4, head_dim=D, num_layers=1, num_kv_heads=hkv, dtype=torch.float32, device="cpu")
    xs = {7: torch.randn(11, d), 9: torch.randn(6, d)}

    def contiguous(x):
        qkv = torch.nn.functional.linear(x, layer.qkv.weight)
        q, k, v = layer._split(qkv)
        pos = torch.arange(x.shape[0])
        q, k = reference.rope_ref(q, pos, 10000.0), reference.rope_ref(k, pos, 10000.0)
        o, _ = reference.attention_ref(q[None].float(), k[None].float(), v[None].float(), causal=True)
        return torch.nn.functional.linear(o[0].reshape(x.shape[0], hq * D), layer.proj.weight)
    want = {s: contiguous(x) for s, x in xs.items()}
    # first chunks of both sequences in one call, then the rest of sequence 7's prompt, then decode steps
    out = layer(torch.cat([xs[7][:5], xs[9][:4]]), kv, [7, 9], AttentionPhase.PREFILL, n_tokens=[5, 4])
    assert torch.allclose(out[:5], want[7][:5], atol=1e-5) and torch.allclose(out[5:], want[9][:4], atol=1e-5)
    out = layer(xs[7][5:9], kv, [7], AttentionPhase.PREFILL)
    assert torch.allclose(out, want[7][5:9], atol=1e-5)
    for t in range(2):
        out = layer(torch.stack([xs[7][9 + t], xs[9][4 + t]]), kv, [7, 9], AttentionPhase.DECODE)
        assert torch.allclose(out[0], want[7][9 + t], atol=1e-5) and torch.allclose(out[1], want[9][4 + t], atol=1e-5)
    assert kv.get_sequence_length(7) == 11 and kv.get_sequence_length(9) == 6
    with pytest.raises(ValueError):
        layer(xs[7][:3], kv, [7, 9], AttentionPhase.PREFILL)


def test_queue_priorities_capacity_accounting_metrics_windows_and_client_helpers():
    from ml_framework_b200.serving.scheduler import (CapacityConstraints, CapacityManager, Priority, RequestQueue, SchedulerMetricsCollector,
                                                     SlidingWindowCounter)
    q = RequestQueue(max_size=3)
    lo, hi, mid = Request([1], priority=Priority.LOW), Request([2], priority=Priority.HIGH), Request([3], priority=Priority.NORMAL)
    for r in (lo, hi, mid):
        q.enqueue(r)
    with pytest.raises(OverflowError):
        q.enqueue(Request([4]))
    mid.cancelled = True
    assert q.dequeue() is hi and q.dequeue() is lo and q.dequeue() is None       # the cancelled one is skipped and resolved
    assert mid.future.result(0).reason == CompletionReason.CANCELLED
    cap = CapacityManager(CapacityConstraints(max_batch_size=2, max_memory_bytes=1000, buffer_ratio=0.1, max_concurrent_requests=8), bytes_per_token=10)
    a, b, c = Request([0] * 10, max_tokens=20), Request([0] * 30, max_tokens=20), Request([0] * 5, max_tokens=5)
    assert cap.usable_memory == 900 and cap.estimate_required_memory(a) == 300
    assert cap.can_fit_batch([a, b]) and not cap.can_fit_batch([a, b, c])          # three requests: over the slot limit
    assert cap.try_allocate(a) and cap.active_slots == 1 and cap.utilization == pytest.approx(300 / 900)
    assert not cap.can_fit_batch([b, c]) and cap.can_fit_batch([b])
    assert cap.try_allocate(b) and not cap.try_allocate(c)                          # slots exhausted
    cap.release(a.id)
    assert cap.try_allocate(c) and cap.active_slots == 2
    big = Request([0] * 100, max_tokens=100)
    cap.release(c.id)
    assert not cap.try_allocate(big)                                                # 2000 bytes never fit 900
    assert CapacityManager().estimate_required_memory(Request([0] * 4, max_tokens=4)) == 8 * 1024
    now = [0.0]
    w = SlidingWindowCounter(10.0, clock=lambda: now[0])
    w.add(5)
    now[0] = 4.0
    w.add(3)
    assert w.total() == 8 and w.rate() == 0.8
    now[0] = 12.0
    assert w.total() == 3
    m = SchedulerMetricsCollector(capacity=4)
    for i in range(6):
        m.record_iteration(2.0 + i, 4, 4)
        m.record_batch_utilization(4, 8)
    m.record_batch_utilization(8, 8)
    m.record_error("oom")
    m.record_error("oom")
    snap = m.snapshot()
    assert snap["iterations"] == 4 and snap["mean_batch"] == 4 and snap["errors"] == {"oom": 2} and snap["total_tokens"] == 24
    assert snap["mean_batch_utilization"] == pytest.approx((0.5 * 3 + 1.0) / 4)     # the buffer keeps the last four
    ex = MockExecutor(eos_after=3)
    s = ContinuousBatchScheduler(ex, None, SchedulerConfiguration(max_batch_size=2))
    client = ContinuousBatchSchedulerClient(s, Tok())
    assert client.estimate_wait_time_s() == 0.0 and client.status()["queued"] == 0
    s.start()
    try:
        res = client.generate_batch(["ab", "cde", "f"], max_tokens=8, timeout_s=10)
        assert [r.tokens for r in res] == [[100, 101, 2]] * 3
        assert client.statistics()["completed"] == 3 and 0 < client.statistics()["mean_batch_utilization"] <= 1.0
    finally:
        s.stop()
    ph = PrefillHandler(PrefillConfiguration(chunk_size=4, prompt_cache_entries=2, prompt_cache_ttl_s=5.0), clock=lambda: now[0])
    assert ph.estimate_prefill_memory(Request(list(range(10))), 16) == 160
    ph.cache_store([1], "x")
    now[0] += 6.0
    assert ph.cache_lookup([1]) is None                                             # expired


def test_block_table_beam_and_speculative_helpers():
    from ml_framework_b200.serving.kv_cache import BeamSearchBlockSharing, BlockTable, SpeculativeDecodingSharing
    m = KVCacheBlockManager(32, 4, allocate_cache=False)
    bt = BlockTable(m)
    first = bt.allocate_and_append_block(1)
    assert bt.get_sequence_blocks(1) == [first] and bt.get_sequence_length(1) == 0
    m.append_tokens(1, 6)
    assert bt.get_sequence_length(1) == 6 and len(bt.get_sequence_blocks(1)) == 2 and bt.get_block(1, 5) == bt.get_sequence_blocks(1)[1]
    beams = BeamSearchBlockSharing(m)
    beams.initialize_beams(1, [10, 11, 12])
    shared = m.get_sequence_blocks(1)
    assert all(m.get_sequence_blocks(b) == shared for b in (10, 11, 12)) and m.reference_count(shared[0]) == 4
    slots, cow = beams.on_beam_divergence(10)
    assert cow is not None and cow[0] == shared[1] and m.get_sequence_blocks(10)[0] == shared[0]     # the half-full block is copied
    beams.replace_beam(11, 10)                                                      # beam 11 died: continue from beam 10
    assert m.get_sequence_blocks(11) == m.get_sequence_blocks(10) and m.get_sequence_length(11) == 7
    beams.cleanup_beams(1)
    assert m.reference_count(shared[0]) == 1 and beams.beams == {}
    spec = SpeculativeDecodingSharing(m)
    free0 = m.free_blocks
    slots, _ = spec.allocate_speculative_blocks(1, 7)                               # 6 + 7 = 13 tokens: two more blocks
    assert len(slots) == 7 and m.free_blocks == free0 - 2
    assert spec.verify_speculation(1, 3) >= 1 and m.get_sequence_length(1) == 9
    spec.allocate_speculative_blocks(1, 4)
    spec.reject_all_speculation(1)
    assert m.get_sequence_length(1) == 9 and m.free_blocks == free0 - 1
    assert bt.remove_sequence(1) == 3 and m.free_blocks == 32
    full = KVCacheBlockManager(1, 4, allocate_cache=False)
    BlockTable(full).allocate_and_append_block(5)
    with pytest.raises(MemoryError):
        BlockTable(full).allocate_and_append_block(6)


def test_memory_aware_queue_accessors():
    from ml_framework_b200.serving.iteration import MemoryAwareScheduler, PendingRequest
    m = KVCacheBlockManager(10, 16, allocate_cache=False)
    q = MemoryAwareScheduler(PagedAttentionScheduler(m), max_queue_size=2)
    assert q.enqueue_request(PendingRequest(1, 64, 32)) and q.enqueue_request(PendingRequest(2, 32, 16))
    assert not q.enqueue_request(PendingRequest(3, 32, 16)) and q.queue_size() == 2
    assert [p.request_id for p in q.queued_requests()] == [1, 2] and not q.should_apply_backpressure()
    m.allocate_blocks(9, 9)
    assert q.should_apply_backpressure() and q.try_admit_next_request() is None      # the head does not fit: nothing is admitted
    q.clear_queue()
    assert q.queue_size() == 0 and q.try_admit_next_request() is None


def test_tokenizers_request_tracker_and_batch_builder_pieces():
    import threading
    import time
    from concurrent.futures import Future
    from ml_framework_b200.serving import interfaces as I
    bt = I.ByteTokenizer()
    ids = bt.encode("héllo", add_eos=True)
    assert ids[0] == 1 and ids[-1] == 2 and bt.decode(ids) == "héllo" and bt.vocab_size == 259 and isinstance(bt, I.Tokenizer)
    ws = I.WhitespaceTokenizer()
    a = ws.encode("the cat sat on the mat")
    assert a[0] == a[4] and ws.decode(a) == "the cat sat on the mat" and ws.vocab_size == 8
    ws.freeze()
    assert ws.encode("the dog") == [a[0], 1] and ws.decode([a[1], 99, 2]) == "cat <unk>"
    now = {"t": 0.0}
    tr = I.RequestTracker(clock=lambda: now["t"])
    tr.start("r1", "m1"); tr.start("r2", "m2")
    now["t"] = 2.0
    assert tr.in_flight() == 2 and tr.in_flight("m1") == 1 and tr.oldest_age_s() == 2.0 and not tr.wait_idle(0.01)
    tr.finish("r1"); tr.finish("r2", ok=False, error="boom")
    st = tr.statistics()
    assert st["finished"] == 2 and st["failed"] == 1 and st["error_rate"] == 0.5 and st["mean_s"] == 2.0 and tr.wait_idle(0.01) and tr.statistics("m1")["failed"] == 0
    import pytest as _p
    with _p.raises(KeyError):
        tr.finish("r1")
    tr.start("x")
    with _p.raises(KeyError):
        tr.start("x")
    q = I.BoundedRequestQueue(3)
    assert all(q.try_enqueue(i) for i in range(3)) and not q.try_enqueue(9) and len(q) == 3
    bb = I.BatchBuilder(q, max_batch_size=2, max_wait_s=0.01)
    assert bb.build() == [0, 1] and bb.build() == [2] and bb.build(idle_wait_s=0.01) == []
    q2 = I.BoundedRequestQueue(16)
    late = threading.Timer(0.02, lambda: q2.try_enqueue("b"))
    q2.try_enqueue("a")
    late.start()
    t0 = time.monotonic()
    got = I.BatchBuilder(q2, max_batch_size=4, max_wait_s=0.2, prefer_batch_size=2).build()
    assert got == ["a", "b"] and time.monotonic() - t0 < 0.15                  # dispatched at the preferred size, not at the deadline
    fs = [Future(), Future()]
    I.ResponseScatterer.scatter(fs, ["x", "y"])
    assert [f.result() for f in fs] == ["x", "y"]
    fs = [Future(), Future()]
    with _p.raises(ValueError):
        I.ResponseScatterer.scatter(fs, ["only one"])
    assert all(isinstance(f.exception(), ValueError) for f in fs)
    fs = [Future()]
    I.ResponseScatterer.fail_all(fs, RuntimeError("down"))
    assert isinstance(fs[0].exception(), RuntimeError)
    s = I.SchedulerStatistics.from_snapshot({"requests_completed": 5, "iteration_ms_p50": 4.5, "errors": 1})
    assert s.completed_requests == 5 and s.p50_iteration_ms == 4.5 and s.errors == 1 and I.SchedulerStatus(1, 2, 3, 0.5).is_running


def test_paged_kernel_interface_and_orchestrators():
    import pytest as _p
    from ml_framework_b200.ops import reference
    from ml_framework_b200.serving import paged_kernels as PK
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.paged_attention_layer import AttentionPhase, PagedAttentionLayer
    torch.manual_seed(0)
    B, Q, C, H, Hkv, D = 2, 3, 7, 4, 2, 8
    q, k, v = torch.randn(B, Q, H, D), torch.randn(B, C, Hkv, D), torch.randn(B, C, Hkv, D)
    std, fused = PK.create_kernel("standard"), PK.create_kernel("fused")
    a = std.compute_paged_attention(q, k, v, AttentionPhase.DECODE)
    want, _ = reference.attention_ref(q.float(), k.float(), v.float(), causal=True, start_pos=C - Q)
    assert torch.allclose(a, want, atol=1e-5) and torch.allclose(fused.compute_paged_attention(q, k, v, AttentionPhase.DECODE), a, atol=1e-5)
    one = std.compute_paged_attention(q[:, :1], k, v, AttentionPhase.DECODE, scale=0.5)
    s = PK.StandardPagedAttentionKernel
    w = s.softmax(s.scale_tensor(s.matmul_query_key(q[:, :1], k), 0.5))
    assert torch.allclose(one, s.matmul_weight_value(w, v), atol=1e-6) and torch.allclose(w.sum(-1), torch.ones(B, H, 1))
    assert torch.allclose(fused.compute_paged_attention(q[:, :1], k, v, AttentionPhase.DECODE, scale=0.5), one, atol=1e-5)
    m = s.apply_causal_mask(torch.zeros(1, 1, 2, 4), start_pos=1)
    assert torch.isinf(m[0, 0, 0, 2:]).all() and torch.isfinite(m[0, 0, 1, :3]).all() and torch.isinf(m[0, 0, 1, 3])
    assert isinstance(PK.create_kernel("auto"), PK.StandardPagedAttentionKernel)
    for bad in (lambda: std.compute_paged_attention(q[0], k, v), lambda: std.compute_paged_attention(q, k, v[:, :5]), lambda: std.compute_paged_attention(torch.randn(B, Q, 3, D), k, v)):
        with _p.raises(ValueError):
            bad()
    with _p.raises(KeyError):
        PK.create_kernel("metal")

    d = 32
    layer = PagedAttentionLayer(d, 4, 2, 8, rope_theta=10000.0)
    kv = KVCacheBlockManager(total_blocks=8, block_size=4, head_dim=8, num_layers=1, num_kv_heads=2, dtype=torch.float32, device="cpu")
    pre, dec = PK.PrefillOrchestrator(kv, chunk_size=4), PK.DecodeOrchestrator(kv)
    x = torch.randn(10, d)
    assert pre.blocks_for(10) == 3 and pre.prefill_allocate_blocks(1, 10) and not pre.prefill_allocate_blocks(2, 100)
    whole = PK.PrefillOrchestrator(KVCacheBlockManager(total_blocks=8, block_size=4, head_dim=8, num_layers=1, num_kv_heads=2, dtype=torch.float32, device="cpu"))
    ref_out = whole.compute_prefill_attention(layer, x, 1)
    out = pre.compute_prefill_attention(layer, x, 1)                       # three chunks
    assert torch.allclose(out, ref_out, atol=1e-5) and kv.get_sequence_length(1) == 10
    assert not dec.needs_new_block(1) and dec.allocate_decode_block(1)
    y = dec.compute_decode_attention(layer, torch.randn(1, d), 1)
    assert y.shape == (1, d) and kv.get_sequence_length(1) == 11
    outs = pre.batch_prefill(layer, [torch.randn(3, d), torch.randn(4, d)], [5, 6])
    assert [o.shape[0] for o in outs] == [3, 4] and dec.needs_new_block(6)
    yb = dec.batch_decode(layer, torch.randn(3, d), [1, 5, 6])
    assert yb.shape == (3, d) and kv.get_sequence_length(6) == 5
    with _p.raises(MemoryError):
        pre.batch_prefill(layer, [torch.randn(20, d)], [9])
    with _p.raises(ValueError):
        dec.compute_decode_attention(layer, torch.randn(2, d), 1)
    with _p.raises(ValueError):
        pre.prefill_allocate_blocks(3, 0)


def test_block_table_and_share_statistics():
    from ml_framework_b200.serving.kv_cache import BlockShareManager, BlockTable, KVCacheBlockManager
    kv = KVCacheBlockManager(total_blocks=16, block_size=4, head_dim=8, num_layers=1, num_kv_heads=1, dtype=torch.float32, device="cpu")
    kv.append_tokens(1, 10)
    sh = BlockShareManager(kv)
    sh.register_prefix(list(range(8)), 1)
    assert sh.share_prefix(1, 2, 9) == 2                      # two whole blocks
    kv.append_tokens(2, 3)
    st = BlockTable(kv).get_stats([1, 2])
    assert (st.sequences, st.total_blocks, st.total_tokens, st.unused_slots, st.longest_sequence) == (2, 6, 21, 3, 11) and abs(st.fill_ratio - 21 / 24) < 1e-9
    ss = sh.get_stats([1, 2])
    assert (ss.shared_blocks, ss.total_references, ss.blocks_saved, ss.registered_prefixes) == (2, 4, 2, 1)
    sh.release_sequence(1)
    assert sh.get_stats([2]).shared_blocks == 0 and sh.get_stats([2]).registered_prefixes == 0
