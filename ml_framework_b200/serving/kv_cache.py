"""KV-cache block manager, block tables and block sharing for paged attention.

``KVCacheBlockManager`` wraps the native pool (``csrc/serving/block_manager.cpp``) and owns the
device cache tensor ``[num_blocks, 2, block_size, Hkv, head_dim]`` per layer. API and behaviour
follow src/MLFramework/Inference/PagedAttention/KVCacheBlockManager.cs:39-247 (allocate one /
many (all-or-nothing) / free block / free sequence / stats / has_available_blocks),
BlockTable.cs:38-192 (per-sequence ordered blocks, token -> block, sequence length) and the
sharing managers in Sharing/ (prefix sharing with reference counts, beam search with
copy-on-divergence, speculative decoding with verify / reject).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib


@dataclass
class BlockManagerStats:
    total_blocks: int
    free_blocks: int
    allocated_blocks: int
    active_sequences: int
    total_allocations: int
    total_frees: int
    failed_allocations: int
    cow_copies: int

    @property
    def utilization(self) -> float:
        return self.allocated_blocks / self.total_blocks if self.total_blocks else 0.0


@dataclass
class BlockAllocationResult:
    success: bool
    block_ids: List[int]
    error: str = ""


class KVCacheBlockManager:
    def __init__(self, total_blocks: int, block_size: int = 16, head_dim: int = 128, num_layers: int = 1,
                 num_kv_heads: int = 1, device=None, dtype=torch.bfloat16, allocate_cache: bool = True):
        if total_blocks <= 0 or block_size <= 0:
            raise ValueError("total_blocks and block_size must be positive")
        self._L = _lib.get()
        self._L.mlf_bm_create.restype = C.c_void_p
        self._h = C.c_void_p(self._L.mlf_bm_create(total_blocks, block_size))
        if not self._h:
            raise RuntimeError("could not create the block manager")
        self.total_blocks, self.block_size = total_blocks, block_size
        self.head_dim, self.num_layers, self.num_kv_heads = head_dim, num_layers, num_kv_heads
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.caches: List[torch.Tensor] = []
        if allocate_cache:
            self.caches = [torch.zeros(total_blocks, 2, block_size, num_kv_heads, head_dim, dtype=dtype, device=self.device)
                           for _ in range(num_layers)]

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._L.mlf_bm_destroy(self._h)
                self._h = None
        except Exception:
            pass

    # ---- allocation
    def allocate_block(self, seq_id: int) -> BlockAllocationResult:
        b = self._L.mlf_bm_allocate_block(self._h, C.c_longlong(seq_id))
        return BlockAllocationResult(b >= 0, [b] if b >= 0 else [], "" if b >= 0 else "no free blocks")

    def allocate_blocks(self, seq_id: int, count: int) -> BlockAllocationResult:
        out = (C.c_int * max(count, 1))()
        n = self._L.mlf_bm_allocate_blocks(self._h, C.c_longlong(seq_id), count, out)
        if n < 0:
            return BlockAllocationResult(False, [], f"cannot allocate {count} blocks, {self.free_blocks} free")
        return BlockAllocationResult(True, list(out[:count]))

    def append_tokens(self, seq_id: int, n: int) -> Tuple[Optional[torch.Tensor], Optional[Tuple[int, int]]]:
        """Reserve cache slots for ``n`` more tokens. Returns (slots int64 [n] or None when the pool
        is exhausted, (src, dst) block copy to perform on the device for copy-on-write or None)."""
        slots = (C.c_longlong * max(n, 1))()
        cs, cd = C.c_int(-1), C.c_int(-1)
        rc = self._L.mlf_bm_append_tokens(self._h, C.c_longlong(seq_id), n, slots, C.byref(cs), C.byref(cd))
        if rc != 0:
            return None, None
        cow = (cs.value, cd.value) if cs.value >= 0 else None
        if cow is not None:
            for cache in self.caches:
                cache[cow[1]].copy_(cache[cow[0]])
        return torch.tensor(list(slots[:n]), dtype=torch.int64), cow

    def free_sequence_blocks(self, seq_id: int) -> int:
        return self._L.mlf_bm_free_sequence(self._h, C.c_longlong(seq_id))

    def truncate(self, seq_id: int, keep_tokens: int) -> int:
        r = self._L.mlf_bm_free_tail(self._h, C.c_longlong(seq_id), keep_tokens)
        if r < 0:
            raise KeyError(f"unknown sequence {seq_id} or bad length {keep_tokens}")
        return r

    def truncate_blocks(self, seq_id: int, keep_blocks: int) -> int:
        """Release reserved-but-empty blocks beyond the first ``keep_blocks`` (never blocks that hold tokens)."""
        r = self._L.mlf_bm_free_tail_blocks(self._h, C.c_longlong(seq_id), int(keep_blocks))
        if r < 0:
            raise KeyError(f"unknown sequence {seq_id}")
        return r

    def fork(self, src_seq: int, dst_seq: int, prefix_tokens: int = -1) -> int:
        r = self._L.mlf_bm_fork(self._h, C.c_longlong(src_seq), C.c_longlong(dst_seq), prefix_tokens)
        if r < 0:
            raise KeyError(f"cannot fork {src_seq} -> {dst_seq}")
        return r

    # ---- queries
    @property
    def free_blocks(self) -> int:
        return self._L.mlf_bm_free_blocks(self._h)

    def has_available_blocks(self, count: int = 1) -> bool:
        return self.free_blocks >= count

    def get_sequence_blocks(self, seq_id: int) -> List[int]:
        cap = 4096
        out = (C.c_int * cap)()
        n = self._L.mlf_bm_seq_blocks(self._h, C.c_longlong(seq_id), out, cap)
        if n > cap:                                   # a very long sequence: ask again with room for all of it
            cap = n
            out = (C.c_int * cap)()
            n = self._L.mlf_bm_seq_blocks(self._h, C.c_longlong(seq_id), out, cap)
        return [] if n < 0 else list(out[:min(n, cap)])

    def get_sequence_length(self, seq_id: int) -> int:
        n = self._L.mlf_bm_seq_tokens(self._h, C.c_longlong(seq_id))
        return max(n, 0)

    def reference_count(self, block: int) -> int:
        return self._L.mlf_bm_ref_count(self._h, block)

    def blocks_needed(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size

    def build_tables(self, seq_ids: Sequence[int], max_blocks: int, device=None):
        n = len(seq_ids)
        ids = (C.c_longlong * max(n, 1))(*seq_ids)
        table = torch.empty(n, max_blocks, dtype=torch.int32)
        lens = torch.empty(n, dtype=torch.int32)
        rc = self._L.mlf_bm_build_tables(self._h, ids, n, max_blocks, C.c_void_p(table.data_ptr()), C.c_void_p(lens.data_ptr()))
        _lib.check(rc, "mlf_bm_build_tables")
        dev = device if device is not None else self.device
        return table.to(dev, non_blocking=True), lens.to(dev, non_blocking=True)

    def get_stats(self) -> BlockManagerStats:
        s = (C.c_longlong * 8)()
        self._L.mlf_bm_stats(self._h, s)
        return BlockManagerStats(*[int(x) for x in s])


class BlockTable:
    """Per-sequence view used by attention layers (BlockTable.cs:38-192)."""

    def __init__(self, manager: KVCacheBlockManager):
        self.m = manager

    def get_block(self, seq_id: int, token_index: int) -> int:
        blocks = self.m.get_sequence_blocks(seq_id)
        i = token_index // self.m.block_size
        if token_index < 0 or i >= len(blocks):
            raise IndexError(f"token {token_index} of sequence {seq_id} has no block")
        return blocks[i]

    def get_sequence_blocks(self, seq_id: int) -> List[int]:
        return self.m.get_sequence_blocks(seq_id)

    def get_sequence_length(self, seq_id: int) -> int:
        return self.m.get_sequence_length(seq_id)

    def allocate_and_append_block(self, seq_id: int) -> int:
        r = self.m.allocate_block(seq_id)
        if not r.success:
            raise MemoryError(r.error)
        return r.block_ids[0]

    def remove_sequence(self, seq_id: int) -> int:
        return self.m.free_sequence_blocks(seq_id)

    def get_stats(self, seq_ids: Sequence[int]) -> "BlockTableStats":
        """Occupancy of the given sequences' tables: blocks held, tokens stored, slack in the last blocks."""
        blocks = tokens = 0
        longest = 0
        for s in seq_ids:
            nb, nt = len(self.m.get_sequence_blocks(s)), self.m.get_sequence_length(s)
            blocks += nb
            tokens += nt
            longest = max(longest, nt)
        cap = blocks * self.m.block_size
        return BlockTableStats(len(list(seq_ids)), blocks, tokens, cap - tokens, tokens / cap if cap else 0.0, longest)


@dataclass
class BlockTableStats:
    sequences: int
    total_blocks: int
    total_tokens: int
    unused_slots: int           # allocated but empty positions (internal fragmentation)
    fill_ratio: float
    longest_sequence: int


@dataclass
class ShareStats:
    """What sharing saves: blocks referenced by more than one sequence, and the blocks that would exist without it."""
    shared_blocks: int
    total_references: int
    blocks_saved: int
    registered_prefixes: int


class BlockShareManager:
    """Prompt-prefix sharing: sequences with a common prefix point at the same blocks."""

    def __init__(self, manager: KVCacheBlockManager):
        self.m = manager
        self._prefix_owner: Dict[tuple, int] = {}

    def share_prefix(self, src_seq: int, dst_seq: int, prefix_tokens: int) -> int:
        full = (prefix_tokens // self.m.block_size) * self.m.block_size   # only whole blocks are shared
        return self.m.fork(src_seq, dst_seq, full)

    def register_prefix(self, tokens: Sequence[int], seq_id: int):
        self._prefix_owner[tuple(tokens)] = seq_id

    def find_prefix(self, tokens: Sequence[int]) -> Optional[Tuple[int, int]]:
        """Longest registered prefix of ``tokens``: (owner sequence, length) or None."""
        best = None
        for pref, owner in self._prefix_owner.items():
            n = len(pref)
            if n <= len(tokens) and tuple(tokens[:n]) == pref and (best is None or n > best[1]):
                if self.m.get_sequence_length(owner) >= n:
                    best = (owner, n)
        return best

    def release_sequence(self, seq_id: int) -> int:
        self._prefix_owner = {k: v for k, v in self._prefix_owner.items() if v != seq_id}
        return self.m.free_sequence_blocks(seq_id)

    def get_reference_count(self, block: int) -> int:
        return self.m.reference_count(block)

    def get_stats(self, seq_ids: Sequence[int]) -> ShareStats:
        seen: Dict[int, int] = {}
        for s in seq_ids:
            for b in self.m.get_sequence_blocks(s):
                seen[b] = seen.get(b, 0) + 1
        shared = {b: n for b, n in seen.items() if n > 1}
        return ShareStats(len(shared), sum(shared.values()), sum(n - 1 for n in shared.values()), len(self._prefix_owner))


class BeamSearchBlockSharing:
    """Beams start as forks of the prompt; a beam that diverges writes into its own copy of the
    shared last block (the copy happens inside ``append_tokens``)."""

    def __init__(self, manager: KVCacheBlockManager):
        self.m = manager
        self.beams: Dict[int, List[int]] = {}

    def initialize_beams(self, prompt_seq: int, beam_ids: Sequence[int]):
        for b in beam_ids:
            self.m.fork(prompt_seq, b)
        self.beams[prompt_seq] = list(beam_ids)

    def on_beam_divergence(self, beam_id: int, n_tokens: int = 1):
        return self.m.append_tokens(beam_id, n_tokens)

    def replace_beam(self, dead_beam: int, parent_beam: int):
        self.m.free_sequence_blocks(dead_beam)
        self.m.fork(parent_beam, dead_beam)

    def cleanup_beams(self, prompt_seq: int):
        for b in self.beams.pop(prompt_seq, []):
            self.m.free_sequence_blocks(b)


class SpeculativeDecodingSharing:
    """Draft tokens get cache slots up front; verification keeps the accepted prefix and frees the rest."""

    def __init__(self, manager: KVCacheBlockManager):
        self.m = manager
        self._base: Dict[int, int] = {}

    def allocate_speculative_blocks(self, seq_id: int, n_draft: int):
        self._base[seq_id] = self.m.get_sequence_length(seq_id)
        return self.m.append_tokens(seq_id, n_draft)

    def verify_speculation(self, seq_id: int, n_accepted: int) -> int:
        base = self._base.pop(seq_id)
        return self.m.truncate(seq_id, base + n_accepted)

    def reject_all_speculation(self, seq_id: int) -> int:
        return self.verify_speculation(seq_id, 0)
