// Shared pieces of the tcgen05 GEMM kernels: kernel parameters, tile rasterisation and the
// fused epilogue applied to one 32-column chunk of an accumulator row.
#pragma once
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;

struct GemmKernelParams {
  int M, N, K;
  int a_mn, b_mn;
  int flags;
  float alpha;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  long long ldo, ld_aux_in, ld_aux_out;
  int tiles_m, tiles_n;
  int rot_m, rot_n;  // tile-order rotation (tiles), so locally owned rows come first
  int* err;
  // gather
  int gather_operand, world, rank, n_copy_ctas, rows_per_rank, flag_rows, row_bytes, total_rows;
  int copy_group;    // copy CTAs that share one gated chunk (n_copy_ctas is a multiple of it); consumers wait for this count
  const void* src[8];
  void* gathered;
  uint32_t* flags_ready;
  uint32_t* counters;
  const void* extra_segs;   // {src, dst, bytes} triples copied after the gated chunks, no flags
  int n_extra;
  // scatter
  int scatter_out, rows_per_owner;
  void* out_peer[8];
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int rot_m, int rot_n,
                                            int& tm, int& tn) {
  // Grouped rasterisation: 8 row-tiles share each column-tile while it is hot in L2.
  constexpr int GM = 8;
  const int per_group = GM * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gsz = min(GM, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
  tm += rot_m;
  if (tm >= tiles_m) tm -= tiles_m;
  tn += rot_n;
  if (tn >= tiles_n) tn -= tiles_n;
}

// One accumulator row chunk: r[0..31] are fp32 bit patterns of columns nb..nb+31 of row m.
// out_row points at the start of the output row (possibly in a peer's buffer).
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmKernelParams& p, const int m, const int nb,
                                                    const uint32_t (&r)[32], char* out_row, const bool out_fp32,
                                                    const bool swiglu, const bool dswiglu) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const int nvalid = min(32, p.N - nb);
        if (p.flags & MLF_EPI_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < nvalid) v[j] += __bfloat162float(p.bias[nb + j]);
        }
        if (p.flags & MLF_EPI_STORE_PRE) {
          __nv_bfloat16* ar = p.aux_out + (long long)m * p.ld_aux_out + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
              w.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
              w.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
              w.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
              reinterpret_cast<uint4*>(ar)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j) ar[j] = __float2bfloat16(v[j]);
          }
        }
        if (p.flags & MLF_EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        }
        if (p.flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL)) {
          const __nv_bfloat16* ar = p.aux_in + (long long)m * p.ld_aux_in + nb;
          float a[32];
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w = reinterpret_cast<const uint4*>(ar)[g];
              float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z),
                     f3 = unpack_bf16x2(w.w);
              a[8 * g + 0] = f0.x; a[8 * g + 1] = f0.y; a[8 * g + 2] = f1.x; a[8 * g + 3] = f1.y;
              a[8 * g + 4] = f2.x; a[8 * g + 5] = f2.y; a[8 * g + 6] = f3.x; a[8 * g + 7] = f3.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = j < nvalid ? __bfloat162float(ar[j]) : 0.f;
          }
          if (p.flags & MLF_EPI_RESIDUAL) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += a[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh(a[j]);
          }
        }
        if (swiglu) {
          // (gate, up) pairs -> 16 outputs at column nb/2
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + nb / 2;
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = silu(v[2 * j]) * v[2 * j + 1];
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              uint4 w;
              w.x = pack_bf16x2(o[8 * g + 0], o[8 * g + 1]);
              w.y = pack_bf16x2(o[8 * g + 2], o[8 * g + 3]);
              w.z = pack_bf16x2(o[8 * g + 4], o[8 * g + 5]);
              w.w = pack_bf16x2(o[8 * g + 6], o[8 * g + 7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid / 2; ++j) orow[j] = __float2bfloat16(o[j]);
          }
          return;
        }
        if (dswiglu) {
          // v = dL/dh for 32 hidden columns; aux_in holds (gate, up) pairs; out gets (dgate, dup)
          const __nv_bfloat16* ar = p.aux_in + (long long)m * p.ld_aux_in + 2 * nb;
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + 2 * nb;
          const bool vec = nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0) &&
                           ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float gu[8];
            if (vec) {
              uint4 w = reinterpret_cast<const uint4*>(ar)[g];
              float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z),
                     f3 = unpack_bf16x2(w.w);
              gu[0] = f0.x; gu[1] = f0.y; gu[2] = f1.x; gu[3] = f1.y;
              gu[4] = f2.x; gu[5] = f2.y; gu[6] = f3.x; gu[7] = f3.y;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                gu[j] = (4 * g + j / 2) < nvalid ? __bfloat162float(ar[8 * g + j]) : 0.f;
            }
            float o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float gate = gu[2 * j], up = gu[2 * j + 1], dh = v[4 * g + j];
              const float sg = 1.f / (1.f + __expf(-gate));
              o[2 * j] = dh * up * sg * (1.f + gate * (1.f - sg));
              o[2 * j + 1] = dh * gate * sg;
            }
            if (vec) {
              uint4 w;
              w.x = pack_bf16x2(o[0], o[1]);
              w.y = pack_bf16x2(o[2], o[3]);
              w.z = pack_bf16x2(o[4], o[5]);
              w.w = pack_bf16x2(o[6], o[7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if ((4 * g + j / 2) < nvalid) orow[8 * g + j] = __float2bfloat16(o[j]);
            }
          }
          return;
        }
        if (out_fp32) {
          float* orow = reinterpret_cast<float*>(out_row) + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              float4 w = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
              if (p.flags & MLF_EPI_ACCUM) {
                float4 o = reinterpret_cast<float4*>(orow)[g];
                w.x += o.x; w.y += o.y; w.z += o.z; w.w += o.w;
              }
              reinterpret_cast<float4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j)
              orow[j] = v[j] + ((p.flags & MLF_EPI_ACCUM) ? orow[j] : 0.f);
          }
        } else {
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (p.flags & MLF_EPI_ACCUM) {
                uint4 o = reinterpret_cast<uint4*>(orow)[g];
                float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z),
                       f3 = unpack_bf16x2(o.w);
                v[8 * g + 0] += f0.x; v[8 * g + 1] += f0.y; v[8 * g + 2] += f1.x; v[8 * g + 3] += f1.y;
                v[8 * g + 4] += f2.x; v[8 * g + 5] += f2.y; v[8 * g + 6] += f3.x; v[8 * g + 7] += f3.y;
              }
              uint4 w;
              w.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
              w.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
              w.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
              w.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j) {
              float x = v[j];
              if (p.flags & MLF_EPI_ACCUM) x += __bfloat162float(orow[j]);
              orow[j] = __float2bfloat16(x);
            }
          }
        }
      }

// ------------------------------------------------------------------------------------------
// copy role (gather side)
// ------------------------------------------------------------------------------------------
// One thread per copy CTA drives a ring of shared-memory buffers with bulk async copies:
// peer global -> shared (completion on an mbarrier), then shared -> local global (bulk group).
// kCopyLookahead loads of kCopyPiece bytes are kept in flight per CTA, which is what it takes
// to cover NVLink latency at full bandwidth with a handful of CTAs.
constexpr int kCopyPiece = 16384;
constexpr int kCopyBufs = 11;
constexpr int kCopyLookahead = 8;

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}

// Copy CTAs that share one gated chunk: enough that a chunk arrives quickly, few enough that each CTA moves a run of
// at least kCopyLookahead pieces per chunk (per-chunk work -- slice arithmetic, the publication fence -- is then small
// beside the copy). The result divides n_copy.
inline int copy_group_size(int n_copy, long long chunk_bytes) {
  long long g = chunk_bytes / ((long long)kCopyLookahead * kCopyPiece);
  if (g < 1) g = 1;
  if (g > n_copy) g = n_copy;
  while (n_copy % g) --g;
  return (int)g;
}

struct CopyCursor {
  int i;            // chunk iteration (rotated order)
  long long off;    // byte offset inside this CTA's slice of the chunk
  // slice of chunk iteration `cached_i` for this CTA, kept in registers: the segment table is read and
  // the slice bounds are divided out once per chunk, not once per piece
  int cached_i;
  int c;
  const char* src;
  char* dst;
  long long lo, hi;
};

struct CopyPiece {
  const char* src;
  char* dst;
  uint32_t bytes;
  int chunk;
  bool last_of_chunk;
  bool valid;
};

__device__ __forceinline__ void chunk_slice(const GemmKernelParams& p, int n_flags, int first_local, int i,
                                            int cta, int& c, const char*& src, char*& dst, long long& lo,
                                            long long& hi) {
  if (i >= n_flags) {
    // un-gated extra segment (prefetch for later kernels)
    const long long* sg = static_cast<const long long*>(p.extra_segs) + 3 * (i - n_flags);
    c = -1;
    src = reinterpret_cast<const char*>(sg[0]);
    dst = reinterpret_cast<char*>(sg[1]);
    const long long n16e = sg[2] / 16;
    const long long pere = (n16e + p.n_copy_ctas - 1) / p.n_copy_ctas;
    lo = min(n16e, pere * cta) * 16;
    hi = min(n16e, pere * (cta + 1)) * 16;
    return;
  }
  // gated chunk: the `copy_group` CTAs of this CTA's group split it; the groups take the chunks round-robin
  const int g = p.copy_group;
  const int mem = cta % g;
  c = first_local + i;
  if (c >= n_flags) c -= n_flags;
  const int row0 = c * p.flag_rows;
  const int rows = min(p.flag_rows, p.total_rows - row0);
  const int owner = min(row0 / p.rows_per_rank, p.world - 1);
  src = static_cast<const char*>(p.src[owner]) + (long long)(row0 - owner * p.rows_per_rank) * p.row_bytes;
  dst = static_cast<char*>(p.gathered) + (long long)row0 * p.row_bytes;
  if (src == dst) {
    // the owner's rows already sit in the gathered buffer (the shard is a region of it): nothing to move,
    // one zero-byte piece still publishes the chunk
    lo = hi = 0;
    return;
  }
  const long long n16 = (long long)rows * p.row_bytes / 16;
  const long long per = (n16 + g - 1) / g;
  lo = min(n16, per * mem) * 16;
  hi = min(n16, per * (mem + 1)) * 16;
}

// First chunk iteration of a copy CTA and the step to its next one: group k of n_copy_ctas / copy_group takes the
// gated iterations k, k + groups, ...; the un-gated extra segments that follow are split over all copy CTAs.
__device__ __forceinline__ int first_chunk_iter(const GemmKernelParams& p, int n_flags, int cta) {
  const int grp = cta / p.copy_group;
  return grp < n_flags ? grp : n_flags;
}
__device__ __forceinline__ int next_chunk_iter(const GemmKernelParams& p, int n_flags, int i) {
  if (i >= n_flags) return i + 1;
  const int nx = i + p.n_copy_ctas / p.copy_group;
  return nx < n_flags ? nx : n_flags;
}

// Returns the piece at the cursor and advances it. Chunks whose slice is empty for this CTA
// still yield one zero-byte piece so the chunk's completion counter is bumped.
__device__ __forceinline__ CopyPiece next_piece(const GemmKernelParams& p, int n_flags, int first_local,
                                                int cta, CopyCursor& cur) {
  CopyPiece pc;
  pc.valid = false;
  if (cur.i >= n_flags + p.n_extra) return pc;
  if (cur.cached_i != cur.i) {
    chunk_slice(p, n_flags, first_local, cur.i, cta, cur.c, cur.src, cur.dst, cur.lo, cur.hi);
    cur.cached_i = cur.i;
  }
  const long long pos = cur.lo + cur.off;
  const long long remain = cur.hi - pos;
  pc.valid = true;
  pc.chunk = cur.c;
  pc.bytes = (uint32_t)(remain > kCopyPiece ? kCopyPiece : (remain > 0 ? remain : 0));
  pc.src = cur.src + pos;
  pc.dst = cur.dst + pos;
  pc.last_of_chunk = remain <= kCopyPiece;
  if (pc.last_of_chunk) {
    cur.i = next_chunk_iter(p, n_flags, cur.i);
    cur.off = 0;
  } else {
    cur.off += kCopyPiece;
  }
  return pc;
}

// A gated chunk is published (its completion counter bumped, the ready flag set by the last copy CTA)
// once the stores of its last piece are complete. Waiting for that right away would drain the store
// pipeline at every chunk; instead the chunk is queued and published kCopySignalLag pieces later,
// when `cp.async.bulk.wait_group kCopySignalLag` guarantees that its group has completed.
constexpr int kCopySignalLag = 3;

__device__ __forceinline__ void publish_chunk(const GemmKernelParams& p, int chunk) {
  // The copy thread must not wait for an answer here: a returning atomic costs a round trip to L2 per chunk and CTA,
  // which at a megabyte per chunk is as long as the copy itself. The bulk stores of the chunk are complete (the
  // caller waited for their group); the proxy fence makes them visible to the generic proxy, and a releasing
  // reduction bumps the chunk's counter without returning. Consumers wait for the counter to reach copy_group.
  fence_proxy_async_all();
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&p.counters[chunk]) : "memory");
}

__device__ inline void gather_copy_role(const GemmKernelParams& p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + kCopyBufs * kCopyPiece;
  if (threadIdx.x != 0) return;
  for (int b = 0; b < kCopyBufs; ++b) mbar_init(bar0 + 8u * b, 1);
  mbar_fence_init();
  int abort_local = 0;
  volatile int* abort_flag = &abort_local;

  const int n_flags = p.gather_operand != 0 ? (p.total_rows + p.flag_rows - 1) / p.flag_rows : 0;
  const int first_local = p.gather_operand != 0 ? (p.rank * p.rows_per_rank) / p.flag_rows : 0;
  const int cta = blockIdx.x;
  const int i0 = first_chunk_iter(p, n_flags, cta);
  CopyCursor lc{i0, 0, -1, 0, nullptr, nullptr, 0, 0}, sc{i0, 0, -1, 0, nullptr, nullptr, 0, 0};
  int issued = 0;  // pieces whose load has been issued
  // pending publications: chunk id and the piece index whose commit closed the chunk
  int pend_chunk[8], pend_seq[8];
  int pend_head = 0, pend_tail = 0;
  // prologue: fill the lookahead window
  for (; issued < kCopyLookahead; ++issued) {
    CopyPiece pc = next_piece(p, n_flags, first_local, cta, lc);
    if (!pc.valid) break;
    const int slot = issued % kCopyBufs;
    if (pc.bytes) {
      mbar_expect_tx(bar0 + 8u * slot, pc.bytes);
      bulk_load(base + slot * kCopyPiece, pc.src, pc.bytes, bar0 + 8u * slot);
    } else {
      mbar_arrive(bar0 + 8u * slot);
    }
  }
  for (int i = 0;; ++i) {
    CopyPiece pc = next_piece(p, n_flags, first_local, cta, sc);
    if (!pc.valid) break;
    const int slot = i % kCopyBufs;
    const uint32_t ph = (i / kCopyBufs) & 1;
    if (!mbar_wait(bar0 + 8u * slot, ph, abort_flag, p.err, ERR_WAIT_CHUNK_FLAG)) break;
    if (pc.bytes) bulk_store(pc.dst, base + slot * kCopyPiece, pc.bytes);
    tma_store_commit();               // group i
    if (pc.last_of_chunk && pc.chunk >= 0) {
      pend_chunk[pend_tail & 7] = pc.chunk;
      pend_seq[pend_tail & 7] = i;
      ++pend_tail;
    }
    if (pend_head != pend_tail && i - pend_seq[pend_head & 7] >= kCopySignalLag) {
      tma_store_wait_all<kCopySignalLag>();     // every group up to i - kCopySignalLag is complete
      while (pend_head != pend_tail && i - pend_seq[pend_head & 7] >= kCopySignalLag) {
        publish_chunk(p, pend_chunk[pend_head & 7]);
        ++pend_head;
      }
    }
    // keep the window full: the slot about to be reused was read by the store issued
    // (kCopyBufs - kCopyLookahead) iterations ago at the latest.
    CopyPiece nx = next_piece(p, n_flags, first_local, cta, lc);
    if (nx.valid) {
      tma_store_wait_read<kCopyBufs - kCopyLookahead - 1>();
      const int nslot = issued % kCopyBufs;
      if (nx.bytes) {
        mbar_expect_tx(bar0 + 8u * nslot, nx.bytes);
        bulk_load(base + nslot * kCopyPiece, nx.src, nx.bytes, bar0 + 8u * nslot);
      } else {
        mbar_arrive(bar0 + 8u * nslot);
      }
      ++issued;
    }
  }
  tma_store_wait_all<0>();
  while (pend_head != pend_tail) {
    publish_chunk(p, pend_chunk[pend_head & 7]);
    ++pend_head;
  }
}


}  // namespace mlf
