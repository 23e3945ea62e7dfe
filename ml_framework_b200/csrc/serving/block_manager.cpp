// Host-side core of paged-attention serving: KV-cache block pool, per-sequence block tables with
// reference-counted sharing, and batch table assembly. These loops sit on the per-iteration
// latency path of the continuous-batching scheduler, so they are native.
//
// Behaviour follows the reference's managers:
//   KVCacheBlockManager (src/MLFramework/Inference/PagedAttention/KVCacheBlockManager.cs:39-247): fixed pool of
//     `total_blocks` blocks of `block_size` tokens, FIFO free list, AllocateBlock / AllocateBlocks
//     (all-or-nothing) / FreeBlock / FreeSequenceBlocks, allocation counters, utilisation stats.
//   BlockTable (BlockTable.cs:38-192): ordered block list per sequence, token -> block lookup,
//     sequence length = (n - 1) * block_size + tokens in the last block.
//   BlockShareManager (Sharing/BlockShareManager.cs:34-118): a block may belong to several sequences
//     (shared prompt prefix, beam search); it returns to the pool when its last owner releases it;
//     a shared, partly filled last block is copied before being appended to (copy-on-write).
#include <stdint.h>
#include <string.h>

#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../common/host.h"

namespace mlf {

struct SeqState {
  std::vector<int> blocks;
  int tokens = 0;
};

struct BlockManager {
  int total_blocks, block_size;
  std::deque<int> free_list;
  std::vector<int> refcount;
  std::unordered_map<long long, SeqState> seqs;
  long long total_allocs = 0, total_frees = 0, failed_allocs = 0, cow_copies = 0;
  std::mutex mu;
  BlockManager(int n, int bs) : total_blocks(n), block_size(bs), refcount(n, 0) {
    for (int i = 0; i < n; ++i) free_list.push_back(i);
  }
  int take() {
    if (free_list.empty()) return -1;
    const int b = free_list.front();
    free_list.pop_front();
    refcount[b] = 1;
    ++total_allocs;
    return b;
  }
  void release(int b) {
    if (b < 0 || b >= total_blocks || refcount[b] <= 0) return;
    if (--refcount[b] == 0) {
      free_list.push_back(b);
      ++total_frees;
    }
  }
};

}  // namespace mlf

using namespace mlf;

MLF_API void* mlf_bm_create(int total_blocks, int block_size) {
  if (total_blocks <= 0 || block_size <= 0) {
    set_error("block manager needs positive total_blocks and block_size");
    return nullptr;
  }
  return new BlockManager(total_blocks, block_size);
}
MLF_API void mlf_bm_destroy(void* h) { delete static_cast<BlockManager*>(h); }

MLF_API int mlf_bm_free_blocks(void* h) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  return (int)m->free_list.size();
}

// Appends one block to the sequence; returns the block id or -1 when the pool is empty.
MLF_API int mlf_bm_allocate_block(void* h, long long seq) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  const int b = m->take();
  if (b < 0) {
    ++m->failed_allocs;
    return -1;
  }
  m->seqs[seq].blocks.push_back(b);
  return b;
}

// All-or-nothing: either `count` blocks are appended (ids written to out) or nothing changes.
MLF_API int mlf_bm_allocate_blocks(void* h, long long seq, int count, int* out) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  if (count < 0 || (int)m->free_list.size() < count) {
    ++m->failed_allocs;
    return -1;
  }
  auto& s = m->seqs[seq];
  for (int i = 0; i < count; ++i) {
    const int b = m->take();
    s.blocks.push_back(b);
    if (out) out[i] = b;
  }
  return count;
}

// Makes room for `new_tokens` more tokens of `seq` (allocating blocks as needed, copy-on-write of a
// shared partial last block) and writes their cache slots (block * block_size + offset) to slots.
// cow_src / cow_dst receive the (source, destination) block of a copy the caller must perform on the
// device, or -1. Returns 0, or -1 (nothing changed) when the pool cannot satisfy the request.
MLF_API int mlf_bm_append_tokens(void* h, long long seq, int new_tokens, long long* slots, int* cow_src, int* cow_dst) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto& s = m->seqs[seq];
  const int bs = m->block_size;
  if (cow_src) *cow_src = -1;
  if (cow_dst) *cow_dst = -1;
  const int used_in_last = s.blocks.empty() ? 0 : s.tokens - ((int)s.blocks.size() - 1) * bs;
  const int room = s.blocks.empty() ? 0 : bs - used_in_last;
  const bool last_shared = !s.blocks.empty() && room > 0 && m->refcount[s.blocks.back()] > 1;
  int need = new_tokens > room ? (new_tokens - room + bs - 1) / bs : 0;
  if (last_shared && new_tokens > 0) need += 1;
  if ((int)m->free_list.size() < need) {
    ++m->failed_allocs;
    return -1;
  }
  if (last_shared && new_tokens > 0) {
    const int old = s.blocks.back();
    const int nb = m->take();
    s.blocks.back() = nb;
    m->release(old);
    ++m->cow_copies;
    if (cow_src) *cow_src = old;
    if (cow_dst) *cow_dst = nb;
  }
  for (int i = 0; i < new_tokens; ++i) {
    const int pos = s.tokens + i;
    const int bi = pos / bs;
    while ((int)s.blocks.size() <= bi) s.blocks.push_back(m->take());
    if (slots) slots[i] = (long long)s.blocks[bi] * bs + pos % bs;
  }
  s.tokens += new_tokens;
  return 0;
}

MLF_API int mlf_bm_free_sequence(void* h, long long seq) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(seq);
  if (it == m->seqs.end()) return 0;
  const int n = (int)it->second.blocks.size();
  for (int b : it->second.blocks) m->release(b);
  m->seqs.erase(it);
  return n;
}

// Releases the last `count` blocks of a sequence (rejected speculative tokens, truncated beams).
MLF_API int mlf_bm_free_tail(void* h, long long seq, int keep_tokens) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(seq);
  if (it == m->seqs.end()) return -1;
  auto& s = it->second;
  if (keep_tokens < 0 || keep_tokens > s.tokens) return -1;
  const int keep_blocks = (keep_tokens + m->block_size - 1) / m->block_size;
  int freed = 0;
  while ((int)s.blocks.size() > keep_blocks) {
    m->release(s.blocks.back());
    s.blocks.pop_back();
    ++freed;
  }
  s.tokens = keep_tokens;
  return freed;
}

// Releases whole blocks beyond the first `keep_blocks` of a sequence that were reserved but hold no tokens
// (cache compaction): never cuts into blocks that cover the sequence's tokens. Returns the number released.
MLF_API int mlf_bm_free_tail_blocks(void* h, long long seq, int keep_blocks) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(seq);
  if (it == m->seqs.end() || keep_blocks < 0) return -1;
  auto& s = it->second;
  const int needed = (s.tokens + m->block_size - 1) / m->block_size;
  if (keep_blocks < needed) keep_blocks = needed;
  int freed = 0;
  while ((int)s.blocks.size() > keep_blocks) {
    m->release(s.blocks.back());
    s.blocks.pop_back();
    ++freed;
  }
  return freed;
}

// dst shares the first ceil(prefix_tokens / block_size) blocks of src (reference counts go up).
MLF_API int mlf_bm_fork(void* h, long long src, long long dst, int prefix_tokens) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(src);
  if (it == m->seqs.end() || m->seqs.count(dst)) return -1;
  const auto& s = it->second;
  if (prefix_tokens < 0 || prefix_tokens > s.tokens) prefix_tokens = s.tokens;
  const int nb = (prefix_tokens + m->block_size - 1) / m->block_size;
  SeqState d;
  d.tokens = prefix_tokens;
  for (int i = 0; i < nb; ++i) {
    d.blocks.push_back(s.blocks[i]);
    ++m->refcount[s.blocks[i]];
  }
  m->seqs[dst] = d;
  return nb;
}

MLF_API int mlf_bm_ref_count(void* h, int block) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  return (block >= 0 && block < m->total_blocks) ? m->refcount[block] : -1;
}

MLF_API int mlf_bm_seq_tokens(void* h, long long seq) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(seq);
  return it == m->seqs.end() ? -1 : it->second.tokens;
}

MLF_API int mlf_bm_seq_blocks(void* h, long long seq, int* out, int cap) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  auto it = m->seqs.find(seq);
  if (it == m->seqs.end()) return -1;
  const int n = (int)it->second.blocks.size();
  for (int i = 0; i < n && i < cap; ++i) out[i] = it->second.blocks[i];
  return n;
}

// Fills table[n_seqs][max_blocks] (padded with -1) and lens[n_seqs] for a batch in one call.
MLF_API int mlf_bm_build_tables(void* h, const long long* seqs, int n_seqs, int max_blocks, int* table, int* lens) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  for (int i = 0; i < n_seqs; ++i) {
    int* row = table + (long long)i * max_blocks;
    for (int j = 0; j < max_blocks; ++j) row[j] = -1;
    auto it = m->seqs.find(seqs[i]);
    if (it == m->seqs.end()) {
      lens[i] = 0;
      continue;
    }
    const auto& s = it->second;
    if ((int)s.blocks.size() > max_blocks) {
      set_error("sequence %lld has %d blocks, table holds %d", seqs[i], (int)s.blocks.size(), max_blocks);
      return -2;
    }
    memcpy(row, s.blocks.data(), s.blocks.size() * sizeof(int));
    lens[i] = s.tokens;
  }
  return 0;
}

// stats[0..7] = total, free, allocated, sequences, total_allocs, total_frees, failed_allocs, cow_copies
MLF_API void mlf_bm_stats(void* h, long long* stats) {
  auto* m = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  stats[0] = m->total_blocks;
  stats[1] = (long long)m->free_list.size();
  stats[2] = m->total_blocks - (long long)m->free_list.size();
  stats[3] = (long long)m->seqs.size();
  stats[4] = m->total_allocs;
  stats[5] = m->total_frees;
  stats[6] = m->failed_allocs;
  stats[7] = m->cow_copies;
}
