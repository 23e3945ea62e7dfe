"""Iteration-level batching (the first-generation serving loop) and the request-level KV-cache manager.

* :class:`MemoryAwareScheduler` - bounded FIFO of pending requests admitted one at a time while the block
  manager says their estimated tokens fit (src/MLFramework/Inference/Scheduling/PagedAttentionScheduler.cs:201-311).
* :class:`PhaseManager` / :class:`ContinuousBatchManager` - which sequences are active, which are still in
  prefill and which decode; removing a sequence frees its blocks
  (src/MLFramework/Inference/Batching/ContinuousBatchManager.cs:41-189, PagedAttention/Phases/PhaseManager.cs).
* :class:`IterationScheduler` - one iteration = admit from the queue, prefill the new sequences (at most
  ``max_prefill_per_iteration``, first when ``prioritize_prefill``), decode the rest, report statistics
  (Batching/IterationScheduler.cs:37-190). The reference's ranges and lengths are placeholders (0..100); here
  they come from the block table.
* :class:`ContinuousBatchKVCacheManager` - per-request page allocations over the block manager with growth
  (``try_extend_cache``) and compaction that really returns pages: trailing pages a request no longer needs
  (ContinuousBatching/KVCache/ContinuousBatchKVCacheManager.cs:35-270, where compaction is a comment).
"""
from __future__ import annotations

import enum
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

from .kv_cache import KVCacheBlockManager
from .scheduler import KVCacheConfiguration, PagedAttentionScheduler


# ------------------------------------------------------------------ memory-aware admission queue
@dataclass
class PendingRequest:
    request_id: int
    estimated_max_tokens: int
    prompt_tokens: int = 0
    enqueued_at: float = field(default_factory=time.time)


class MemoryAwareScheduler:
    def __init__(self, paged: PagedAttentionScheduler, max_queue_size: int = 1000):
        self.paged, self.max_queue_size = paged, max_queue_size
        self._q: Deque[PendingRequest] = deque()
        self._lock = threading.Lock()

    def enqueue_request(self, req: PendingRequest) -> bool:
        with self._lock:
            if len(self._q) >= self.max_queue_size:
                return False
            self._q.append(req)
            return True

    def try_admit_next_request(self) -> Optional[PendingRequest]:
        """Head-of-line admission: the oldest request leaves the queue only when its tokens fit."""
        with self._lock:
            if not self._q:
                return None
            head = self._q[0]
            if self.paged.can_admit(head.prompt_tokens, max(0, head.estimated_max_tokens - head.prompt_tokens)):
                return self._q.popleft()
            return None

    def queue_size(self) -> int:
        with self._lock:
            return len(self._q)

    def queued_requests(self) -> List[PendingRequest]:
        with self._lock:
            return list(self._q)

    def should_apply_backpressure(self, threshold: float = 0.8) -> bool:
        return self.paged.memory_pressure() >= threshold

    def clear_queue(self):
        with self._lock:
            self._q.clear()


# ------------------------------------------------------------------ phases and the active batch
class Phase(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class PhaseManager:
    def __init__(self):
        self._phase: Dict[int, Phase] = {}

    def set_phase(self, seq_id: int, phase: Phase):
        self._phase[seq_id] = phase

    def get_phase(self, seq_id: int) -> Phase:
        return self._phase.get(seq_id, Phase.PREFILL)

    def is_prefill(self, seq_id: int) -> bool:
        return self.get_phase(seq_id) == Phase.PREFILL

    def remove_sequence(self, seq_id: int):
        self._phase.pop(seq_id, None)


@dataclass
class BatchStats:
    total_sequences: int
    prefill_sequences: int
    decode_sequences: int
    max_batch_size: int

    @property
    def utilization(self) -> float:
        return self.total_sequences / self.max_batch_size if self.max_batch_size else 0.0


class ContinuousBatchManager:
    def __init__(self, block_manager: KVCacheBlockManager, phases: Optional[PhaseManager] = None, max_batch_size: int = 32):
        self.bm, self.phases, self.max_batch_size = block_manager, phases or PhaseManager(), max_batch_size
        self._active: List[int] = []
        self._lock = threading.Lock()

    def try_add_sequence(self, seq_id: int) -> bool:
        with self._lock:
            if seq_id in self._active:
                return True
            if len(self._active) >= self.max_batch_size or self.bm.free_blocks == 0:
                return False
            self._active.append(seq_id)
            self.phases.set_phase(seq_id, Phase.PREFILL)
            return True

    def remove_sequence(self, seq_id: int):
        with self._lock:
            if seq_id in self._active:
                self._active.remove(seq_id)
            self.bm.free_sequence_blocks(seq_id)
            self.phases.remove_sequence(seq_id)

    def current_batch(self) -> List[int]:
        with self._lock:
            return list(self._active)

    def prefill_sequences(self) -> List[int]:
        with self._lock:
            return [s for s in self._active if self.phases.is_prefill(s)]

    def decode_sequences(self) -> List[int]:
        with self._lock:
            return [s for s in self._active if not self.phases.is_prefill(s)]

    def transition_to_decode(self, seq_id: int):
        with self._lock:
            if seq_id in self._active:
                self.phases.set_phase(seq_id, Phase.DECODE)

    def can_accept_more_sequences(self) -> bool:
        with self._lock:
            return len(self._active) < self.max_batch_size and self.bm.free_blocks > 0

    def stats(self) -> BatchStats:
        with self._lock:
            pre = sum(1 for s in self._active if self.phases.is_prefill(s))
            return BatchStats(len(self._active), pre, len(self._active) - pre, self.max_batch_size)

    def clear(self):
        for s in self.current_batch():
            self.remove_sequence(s)


@dataclass
class IterationSchedulerConfig:
    max_batch_size: int = 32
    min_decode_sequences: int = 1
    prioritize_prefill: bool = True
    max_prefill_per_iteration: int = 4


class IterationScheduler:
    """``prefill_fn(seq_ids, ranges)`` and ``decode_fn(seq_ids, lengths)`` run the model; ranges ``(start, end)`` are
    the tokens of a sequence not yet in the cache and lengths are the cached lengths, both read from the block
    manager."""

    def __init__(self, batch: ContinuousBatchManager, memory: MemoryAwareScheduler, prefill_fn: Callable, decode_fn: Callable,
                 config: Optional[IterationSchedulerConfig] = None, iteration_callback: Optional[Callable[[BatchStats], None]] = None,
                 prompt_lengths: Optional[Dict[int, int]] = None):
        self.batch, self.memory, self.prefill_fn, self.decode_fn = batch, memory, prefill_fn, decode_fn
        self.cfg = config or IterationSchedulerConfig(max_batch_size=batch.max_batch_size)
        self.callback = iteration_callback or (lambda stats: None)
        self.prompt_lengths = prompt_lengths if prompt_lengths is not None else {}
        self.iterations = 0

    def _admit(self):
        while self.batch.can_accept_more_sequences():
            req = self.memory.try_admit_next_request()
            if req is None:
                break
            self.prompt_lengths.setdefault(req.request_id, req.prompt_tokens)
            self.batch.try_add_sequence(req.request_id)

    def run_iteration(self) -> BatchStats:
        self._admit()
        stats = self.batch.stats()
        if stats.total_sequences == 0:
            return stats
        bm = self.batch.bm
        prefill = self.batch.prefill_sequences()[: self.cfg.max_prefill_per_iteration]
        decode = self.batch.decode_sequences()
        steps = [("prefill", prefill), ("decode", decode)]
        if not self.cfg.prioritize_prefill and len(decode) >= self.cfg.min_decode_sequences:
            steps.reverse()
        for kind, seqs in steps:
            if not seqs:
                continue
            if kind == "prefill":
                ranges = {s: (bm.get_sequence_length(s), self.prompt_lengths.get(s, bm.get_sequence_length(s))) for s in seqs}
                self.prefill_fn(seqs, ranges)
                for s in seqs:
                    self.batch.transition_to_decode(s)
            else:
                self.decode_fn(seqs, {s: bm.get_sequence_length(s) for s in seqs})
        self.iterations += 1
        self.callback(stats)
        return stats


# ------------------------------------------------------------------ request-level KV-cache allocations
@dataclass
class CachePage:
    index: int
    start_token: int
    tokens: int
    block: int


@dataclass
class CacheAllocation:
    request_id: int
    pages: List[CachePage]
    total_tokens_allocated: int
    total_bytes_allocated: int
    allocated_at: float

    @property
    def page_count(self) -> int:
        return len(self.pages)


class ContinuousBatchKVCacheManager:
    def __init__(self, block_manager: KVCacheBlockManager, config: Optional[KVCacheConfiguration] = None, bytes_per_token: int = 0):
        self.bm, self.cfg = block_manager, config or KVCacheConfiguration(page_size_tokens=block_manager.block_size)
        if self.cfg.page_size_tokens != block_manager.block_size:
            raise ValueError("page_size_tokens must equal the block manager's block size")
        self.page_bytes = bytes_per_token * self.cfg.page_size_tokens
        self._alloc: Dict[int, CacheAllocation] = {}
        self._lock = threading.Lock()

    def _pages_for(self, tokens: int) -> int:
        need = (tokens + self.cfg.page_size_tokens - 1) // self.cfg.page_size_tokens
        return min(max(self.cfg.initial_pages, need), self.cfg.max_pages_per_request)

    def _record(self, rid: int) -> CacheAllocation:
        blocks = self.bm.get_sequence_blocks(rid)
        P = self.cfg.page_size_tokens
        pages = [CachePage(i, i * P, P, b) for i, b in enumerate(blocks)]
        old = self._alloc.get(rid)
        a = CacheAllocation(rid, pages, len(pages) * P, len(pages) * self.page_bytes, old.allocated_at if old else time.time())
        self._alloc[rid] = a
        return a

    def allocate_cache(self, request_id: int, max_tokens: int) -> int:
        """Pages for ``max_tokens`` (at least ``initial_pages``, at most ``max_pages_per_request``); returns bytes.
        Nothing stays allocated when the blocks run out."""
        if max_tokens < 0:
            raise ValueError("max_tokens cannot be negative")
        with self._lock:
            if request_id in self._alloc:
                raise RuntimeError(f"cache already allocated for request {request_id}")
            n = self._pages_for(max_tokens)
            res = self.bm.allocate_blocks(request_id, n)
            if not res.success:
                self.bm.free_sequence_blocks(request_id)
                raise MemoryError(f"no room for {n} pages of request {request_id}: {res.error}")
            return self._record(request_id).total_bytes_allocated

    def release_cache(self, request_id: int):
        with self._lock:
            if self._alloc.pop(request_id, None) is not None:
                self.bm.free_sequence_blocks(request_id)

    def current_usage_bytes(self) -> int:
        with self._lock:
            return sum(a.total_bytes_allocated for a in self._alloc.values())

    def try_extend_cache(self, request_id: int, additional_tokens: int) -> bool:
        if additional_tokens <= 0:
            return False
        with self._lock:
            a = self._alloc.get(request_id)
            if a is None or a.page_count >= self.cfg.max_pages_per_request:
                return False
            want = (additional_tokens + self.cfg.page_size_tokens - 1) // self.cfg.page_size_tokens
            want = min(want, self.cfg.max_pages_per_request - a.page_count)
            if want <= 0 or not self.bm.has_available_blocks(want):
                return False
            if not self.bm.allocate_blocks(request_id, want).success:
                return False
            self._record(request_id)
            return True

    def get_allocation(self, request_id: int) -> Optional[CacheAllocation]:
        with self._lock:
            return self._alloc.get(request_id)

    def utilization(self) -> float:
        st = self.bm.get_stats()
        return st.utilization

    def compact_cache(self, used_tokens: Optional[Dict[int, int]] = None) -> int:
        """Returns pages to the pool: for every request whose cached length (``used_tokens`` or the block manager's
        own count) needs fewer pages than it holds, the trailing pages beyond ``max(needed, initial_pages)`` are
        released. Runs only when compaction is enabled and block utilisation is above ``target_utilization``
        (there is nothing to gain while the pool has room). Returns the number of pages released."""
        if not self.cfg.enable_compaction:
            return 0
        with self._lock:
            if self.utilization() < self.cfg.target_utilization:
                return 0
            P, freed = self.cfg.page_size_tokens, 0
            for rid, a in list(self._alloc.items()):
                used = (used_tokens or {}).get(rid, self.bm.get_sequence_length(rid))
                keep = max((used + P - 1) // P, min(self.cfg.initial_pages, a.page_count), 1)
                if keep < a.page_count:
                    freed += self.bm.truncate_blocks(rid, keep)
                    self._record(rid)
            return freed

    @property
    def allocation_count(self) -> int:
        with self._lock:
            return len(self._alloc)
