// Paged-attention decode and KV-cache maintenance kernels.
//
// Cache layout: kv_cache[num_blocks][2 (K, V)][block_size][Hkv][128] bf16; block_table[B][max_blocks]
// maps a sequence's logical block to a physical block; seq_lens[B] counts cached tokens including
// the current one (the reference's block size is 16 tokens,
// src/MLFramework/Inference/ContinuousBatching/KVCache/KVCacheConfiguration.cs:6-32; block bookkeeping in
// src/MLFramework/Inference/PagedAttention/KVCacheBlockManager.cs:39-247 and BlockTable.cs:38-192).
//
// paged_attn_decode: one query token per sequence against its cached keys/values
// (the decode branch of StandardPagedAttentionKernel.ComputePagedAttention,
// src/MLFramework/Inference/PagedAttention/Kernels/StandardPagedAttentionKernel.cs:21-84, with the
// block-table gather folded in, which the reference leaves outside the kernel and stubs,
// PagedAttentionLayer.cs:368-389). The kernel is HBM-bound: a CTA owns one (sequence, kv head,
// split), stages K and V rows in shared memory with asynchronous 16-byte copies (16 lanes per token
// row) and shares every row between the G = Hq/Hkv query heads of the group. Sequences are split
// over grid.z (flash-decoding) and merged by a second small kernel.
//
// kv_cache_write: scatter new K/V rows into their slots (PagedAttentionLayer.UpdateKVCache :244-296).
// kv_gather: copy a sequence's pages into a contiguous buffer (for chunked prefill over a cached prefix).
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

constexpr int PD = 128;           // head dim
constexpr int P_THREADS = 128;
constexpr int P_SUB = 128;        // granularity of the host's split size
constexpr int P_CH = 64;          // tokens per staged chunk
constexpr int P_STAGES = 2;
constexpr int P_CH_BYTES = P_CH * PD * 2;               // 16 KB: one chunk of K (or V) rows of one kv head
constexpr int P_SMEM = 2 * P_STAGES * P_CH_BYTES;       // K ring + V ring
constexpr int P_MAXG = 8;         // max query heads per kv head

struct PagedDecodeParams {
  const __nv_bfloat16* q;         // [B, Hq, 128], row pitch ldq elements
  long long ldq;
  const __nv_bfloat16* cache;
  const int* block_table;         // [B, max_blocks]
  const int* seq_lens;            // [B]
  __nv_bfloat16* out;             // [B, Hq, 128]
  float* ws;                      // [B, Hkv, splits, G, 130] (m, l, o[128]) when splits > 1
  unsigned int* counters;         // [B, Hkv] finished splits (zero between launches); null: a separate merge launch
  int B, Hq, Hkv, G, block_size, bs_shift, max_blocks, num_blocks, split_tokens, splits;   // bs_shift: log2(block_size) or -1
  float scale_log2;
  int* err;
};

// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros (rows past the sequence end)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16, row) B(16x8, bf16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte column `c16` (0..15) of token row `row` inside a staged chunk: rows are
// 256 bytes, columns XOR-swizzled with the row so that the eight rows of an 8 x 8 matrix fetch
// (same column, consecutive rows) fall into eight different bank groups.
__device__ __forceinline__ uint32_t chunk_off(int row, int c16) { return (uint32_t)(row * 256 + ((c16 ^ (row & 7)) << 4)); }

// The split that finishes last for a (sequence, kv head) merges all splits' partial results:
// out = sum_s exp2(m_s - M) o_s / sum_s exp2(m_s - M) l_s, and leaves the counter at zero for the next launch.
template <int G>
__device__ __forceinline__ void finish_split(const PagedDecodeParams& p, int b, int hkv) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&p.counters[b * p.Hkv + hkv], 1u) == (unsigned)p.splits - 1u ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int d = threadIdx.x;               // P_THREADS == PD
  const long long sstride = (long long)G * (PD + 2);
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float* base = p.ws + ((((long long)b * p.Hkv + hkv) * p.splits) * G + g) * (PD + 2);
    float M = -INFINITY;
    for (int sp = 0; sp < p.splits; ++sp) M = fmaxf(M, __ldcg(base + sp * sstride));
    float L = 0.f, o = 0.f;
    for (int sp = 0; sp < p.splits; ++sp) {
      const float m = __ldcg(base + sp * sstride);
      if (m == -INFINITY) continue;
      const float w = exp2f(m - M);
      L += w * __ldcg(base + sp * sstride + 1);
      o += w * __ldcg(base + sp * sstride + 2 + d);
    }
    p.out[((long long)b * p.Hq + hkv * G + g) * PD + d] = __float2bfloat16(L > 0.f ? o / L : 0.f);
  }
  if (threadIdx.x == 0) p.counters[b * p.Hkv + hkv] = 0u;
}

// The kernel is bound by bytes in flight, not by arithmetic: K and V rows are staged through shared
// memory with asynchronous 16-byte copies (two chunks of 64 tokens of K and of V, up to 64 KB per
// CTA, in flight while the previous chunk is multiplied), so the amount outstanding does not depend
// on registers. The G query heads of the group are the (zero-padded) 16 rows of a warp-level
// m16n8k16 tensor-core product: one query token gives at most 8 rows, far below the 64-row minimum
// of the tcgen05 path, and this way a chunk costs a warp ~100 instructions instead of ~1000 scalar
// ones. Each warp owns 16 tokens of every chunk with its own running (max, sum, output); the four
// warps merge at the end. Each sequence divides its own length evenly over the launch's splits.
template <int G>
__global__ void __launch_bounds__(P_THREADS)
paged_decode_kernel(const PagedDecodeParams p) {
  extern __shared__ __align__(128) uint8_t p_dsm[];
  const int b = blockIdx.x, hkv = blockIdx.y, sp = blockIdx.z;
  // A length beyond what the row of the block table can describe would index past the table: it is
  // clamped to the table's capacity and reported, like every other rejected index in this file.
  int len = p.seq_lens[b];
  const long long cap = (long long)p.max_blocks * p.block_size;
  if (len < 0 || len > cap) {
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_INDEX);
    len = len < 0 ? 0 : (int)cap;
  }
  int per = (len + p.splits - 1) / p.splits;
  per = (per + P_CH - 1) / P_CH * P_CH;
  const int t_lo = sp * per;
  const int t_hi = min(len, t_lo + per);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tg = tid >> 4;        // loader: token group 0..7
  const int dl = tid & 15;        // loader: 16-byte column of the row

  float* ws = p.ws ? p.ws + ((((long long)b * p.Hkv + hkv) * p.splits + sp) * G) * (PD + 2) : nullptr;
  if (t_lo >= t_hi) {
    if (ws) {
      for (int i = tid; i < G * (PD + 2); i += P_THREADS) ws[i] = (i % (PD + 2)) == 0 ? -INFINITY : 0.f;
      if (p.counters) finish_split<G>(p, b, hkv);
    } else if (sp == 0) {
      for (int i = tid; i < G * PD; i += P_THREADS)
        p.out[((long long)b * p.Hq + hkv * G) * PD + i] = __float2bfloat16(0.f);
    }
    return;
  }
  const long long blk_stride = 2LL * p.block_size * p.Hkv * PD;   // elements per physical block
  const long long v_off = (long long)p.block_size * p.Hkv * PD;
  const int* bt = p.block_table + (long long)b * p.max_blocks;
  const uint32_t sK = smem_u32(p_dsm), sV = sK + P_STAGES * P_CH_BYTES;
  const int n_ch = (t_hi - t_lo + P_CH - 1) / P_CH;

  // one commit group per chunk (its K and V rows), also when the chunk does not exist, so that the
  // group arithmetic of the waits below is the same in every iteration
  auto issue = [&](int c) {
    if (c < n_ch) {
      const uint32_t stage = (c % P_STAGES) * P_CH_BYTES;
      const int tbase = t_lo + c * P_CH;
      int tt[P_CH / 8], lb[P_CH / 8], blk[P_CH / 8];
#pragma unroll
      for (int e = 0; e < P_CH / 8; ++e) {     // the table entries first: eight independent loads
        const int t = tbase + tg + 8 * e;
        tt[e] = t < t_hi ? t : t_lo;
        lb[e] = p.bs_shift >= 0 ? (tt[e] >> p.bs_shift) : (tt[e] / p.block_size);
        blk[e] = bt[lb[e]];
      }
#pragma unroll
      for (int e = 0; e < P_CH / 8; ++e) {
        const int i = tg + 8 * e;
        const int sz = tbase + i < t_hi ? 16 : 0;
        if (blk[e] < 0 || blk[e] >= p.num_blocks) { atomicCAS(p.err, 0, ERR_BAD_INDEX); blk[e] = 0; }
        const __nv_bfloat16* src = p.cache + blk[e] * blk_stride + ((long long)(tt[e] - lb[e] * p.block_size) * p.Hkv + hkv) * PD + dl * 8;
        const uint32_t off = stage + chunk_off(i, dl);
        cp_async16(sK + off, src, sz);
        cp_async16(sV + off, src + v_off, sz);
      }
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);

  // Q as the A operand: row = lane / 4 is the head of the group (rows >= G and rows 8..15 are zero)
  const int qrow = lane >> 2, qcol = (lane & 3) * 2;
  uint32_t qa[PD / 16][2];
#pragma unroll
  for (int ks = 0; ks < PD / 16; ++ks) {
    qa[ks][0] = qa[ks][1] = 0u;
    if (qrow < G) {
      const __nv_bfloat16* qp = p.q + (long long)b * p.ldq + (long long)(hkv * G + qrow) * PD + ks * 16 + qcol;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[PD / 8][4];
#pragma unroll
  for (int nt = 0; nt < PD / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;     // of row qrow, over this warp's tokens (l: this thread's columns only)

  for (int c = 0; c < n_ch; ++c) {
    const int cn = min(P_CH, t_hi - t_lo - c * P_CH);
    const uint32_t kst = sK + (c % P_STAGES) * P_CH_BYTES, vst = sV + (c % P_STAGES) * P_CH_BYTES;
    const int tok0 = warp * 16;              // this warp's 16 tokens of the chunk
    const bool active = tok0 < cn;           // warp-uniform
    cp_async_wait<1>();                      // chunk c: one younger group may still be in flight
    __syncthreads();
    float sacc[2][4];
    if (active) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < PD / 16; ks += 2) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t kb[4];                    // (b0, b1) of k-step ks and of k-step ks + 1
          ldsm_x4(kst + chunk_off(tok0 + nt * 8 + (lane & 7), ks * 2 + (lane >> 3)), kb);
          mma_16816(sacc[nt], qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
          mma_16816(sacc[nt], qa[ks + 1][0], 0u, qa[ks + 1][1], 0u, kb[2], kb[3]);
        }
      }
      // online softmax of row qrow: this thread holds columns nt * 8 + qcol + {0, 1}
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const bool valid = tok0 + nt * 8 + qcol + j < cn;
          sacc[nt][j] = valid ? sacc[nt][j] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, sacc[nt][j]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);           // finite: the warp has at least one valid token
      const float alpha = exp2f(m_run - m_new);
      m_run = m_new;
      float ps = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) { sacc[nt][j] = exp2f(sacc[nt][j] - m_new); ps += sacc[nt][j]; }
      l_run = l_run * alpha + ps;
#pragma unroll
      for (int nt = 0; nt < PD / 8; ++nt) { o[nt][0] *= alpha; o[nt][1] *= alpha; }
    }
    if (active) {
      // P (16 heads x 16 tokens) as the A operand; rows 8..15 stay zero
      const uint32_t pa0 = pack_bf16x2(sacc[0][0], sacc[0][1]), pa2 = pack_bf16x2(sacc[1][0], sacc[1][1]);
#pragma unroll
      for (int nt = 0; nt < PD / 8; nt += 2) {
        uint32_t vb[4];                      // (b0, b1) of output columns nt * 8.. and of (nt + 1) * 8..
        ldsm_x4_trans(vst + chunk_off(tok0 + (lane & 7) + ((lane >> 3) & 1) * 8, nt + (lane >> 4)), vb);
        mma_16816(o[nt], pa0, 0u, pa2, 0u, vb[0], vb[1]);
        mma_16816(o[nt + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
      }
    }
    __syncthreads();                         // the stage is free
    issue(c + 2);
  }
  cp_async_wait<0>();
  __syncthreads();
  // ---- merge the four warps (the staging rings are free now): s_red[warp][g][m, l, o[128]]
  float (*s_red)[G][PD + 2] = reinterpret_cast<float (*)[G][PD + 2]>(p_dsm);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (qrow < G) {
    if ((lane & 3) == 0) { s_red[warp][qrow][0] = m_run; s_red[warp][qrow][1] = l_run; }
#pragma unroll
    for (int nt = 0; nt < PD / 8; ++nt) {
      s_red[warp][qrow][2 + nt * 8 + qcol] = o[nt][0];
      s_red[warp][qrow][2 + nt * 8 + qcol + 1] = o[nt][1];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * PD; i += P_THREADS) {
    const int g = i / PD, d = i % PD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < P_THREADS / 32; ++w) M = fmaxf(M, s_red[w][g][0]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < P_THREADS / 32; ++w) {
      const float f = exp2f(s_red[w][g][0] - M);       // a warp without tokens has m = -inf, l = 0, o = 0
      acc += f * s_red[w][g][2 + d];
      l += f * s_red[w][g][1];
    }
    if (ws) {
      ws[g * (PD + 2) + 2 + d] = acc;
      if (d == 0) { ws[g * (PD + 2)] = M; ws[g * (PD + 2) + 1] = l; }
    } else {
      p.out[((long long)b * p.Hq + hkv * G + g) * PD + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    }
  }
  if (ws && p.counters) finish_split<G>(p, b, hkv);
}

// Merge the per-split partial results: out = sum_s exp2(m_s - M) o_s / sum_s exp2(m_s - M) l_s.
__global__ void __launch_bounds__(128)
paged_decode_merge_kernel(const float* ws, __nv_bfloat16* out, int B, int Hq, int Hkv, int G, int splits) {
  const int bh = blockIdx.x;      // b * Hq + h
  const int b = bh / Hq, h = bh % Hq;
  const int hkv = h / G, g = h % G;
  const int d = threadIdx.x;
  const float* base = ws + (((long long)b * Hkv + hkv) * splits * G + g) * (PD + 2);
  const long long sstride = (long long)G * (PD + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * sstride]);
  float L = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = base[s * sstride];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - M);
    L += w * base[s * sstride + 1];
    o += w * base[s * sstride + 2 + d];
  }
  out[((long long)b * Hq + h) * PD + d] = __float2bfloat16(L > 0.f ? o / L : 0.f);
}

// k, v: [T, Hkv, 128] (row pitch ldk / ldv elements); slot_mapping[T] = block * block_size + offset, < 0 skips.
__global__ void __launch_bounds__(256)
kv_cache_write_kernel(__nv_bfloat16* cache, const __nv_bfloat16* k, const __nv_bfloat16* v, const long long* slots, long long T,
                      int Hkv, int block_size, int num_blocks, long long ldk, long long ldv, int* err) {
  const int vec_per_tok = Hkv * PD / 8;
  const long long total = T * vec_per_tok;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_tok;
    const int c = (int)(i % vec_per_tok) * 8;
    const long long slot = slots[t];
    if (slot < 0) continue;
    const long long blk = slot / block_size;
    if (blk >= num_blocks) { atomicCAS(err, 0, ERR_BAD_INDEX); continue; }
    const int off = (int)(slot % block_size);
    __nv_bfloat16* kd = cache + blk * 2LL * block_size * Hkv * PD + (long long)off * Hkv * PD + c;
    __nv_bfloat16* vd = kd + (long long)block_size * Hkv * PD;
    *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<const uint4*>(k + t * ldk + c);
    *reinterpret_cast<uint4*>(vd) = *reinterpret_cast<const uint4*>(v + t * ldv + c);
  }
}

// One pass over packed QKV rows [T, (Hq + 2 Hkv) * 128] (pitch ld): rotary embedding (rotate-half, positions
// pos[T]) in place on the query and key heads, and the rotated keys plus the values written to their cache
// slots (slot < 0 skips the write). Replaces two rotary launches and the cache write of a serving step.
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(__nv_bfloat16* qkv, long long ld, const long long* pos, const long long* slots, __nv_bfloat16* cache, long long T,
                     int Hq, int Hkv, int block_size, int num_blocks, float theta, int* err) {
  const int heads = Hq + 2 * Hkv;
  const long long total = T * heads * 16;                    // 16 threads per head: 4 + 4 elements each
  const float log_theta = __logf(theta);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i & 15) * 4;                         // 0..60: pairs (d, d + 64)
    const long long th = i >> 4;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    __nv_bfloat16* row = qkv + t * ld + (long long)h * PD;
    uint2 lo = *reinterpret_cast<const uint2*>(row + d);
    uint2 hi = *reinterpret_cast<const uint2*>(row + d + 64);
    const bool is_v = h >= Hq + Hkv;
    if (!is_v) {
      const float p = (float)pos[t];
      const float2 a0 = unpack_bf16x2(lo.x), a1 = unpack_bf16x2(lo.y), b0 = unpack_bf16x2(hi.x), b1 = unpack_bf16x2(hi.y);
      float a[4] = {a0.x, a0.y, a1.x, a1.y}, b[4] = {b0.x, b0.y, b1.x, b1.y};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float inv_freq = __expf(-log_theta * (2.f * (d + j) / PD));
        float sn, cs;
        sincosf(p * inv_freq, &sn, &cs);
        const float x = a[j], y = b[j];
        a[j] = x * cs - y * sn;
        b[j] = y * cs + x * sn;
      }
      lo.x = pack_bf16x2(a[0], a[1]); lo.y = pack_bf16x2(a[2], a[3]);
      hi.x = pack_bf16x2(b[0], b[1]); hi.y = pack_bf16x2(b[2], b[3]);
      *reinterpret_cast<uint2*>(row + d) = lo;
      *reinterpret_cast<uint2*>(row + d + 64) = hi;
    }
    if (h >= Hq) {
      const long long slot = slots[t];
      if (slot < 0) continue;
      const long long blk = slot / block_size;
      if (blk >= num_blocks) { atomicCAS(err, 0, ERR_BAD_INDEX); continue; }
      const int off = (int)(slot % block_size);
      const int hk = is_v ? h - Hq - Hkv : h - Hq;
      __nv_bfloat16* dst = cache + blk * 2LL * block_size * Hkv * PD + (is_v ? (long long)block_size * Hkv * PD : 0) +
                           ((long long)off * Hkv + hk) * PD;
      *reinterpret_cast<uint2*>(dst + d) = lo;
      *reinterpret_cast<uint2*>(dst + d + 64) = hi;
    }
  }
}

// out_k / out_v [len, Hkv, 128] <- pages of one sequence.
__global__ void __launch_bounds__(256)
kv_gather_kernel(const __nv_bfloat16* cache, const int* block_table, int len, int Hkv, int block_size, int num_blocks,
                 __nv_bfloat16* out_k, __nv_bfloat16* out_v, int* err) {   // len <= table entries * block_size (checked by the launcher)
  const int vec_per_tok = Hkv * PD / 8;
  const long long total = (long long)len * vec_per_tok;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_tok);
    const int c = (int)(i % vec_per_tok) * 8;
    int blk = block_table[t / block_size];
    if (blk < 0 || blk >= num_blocks) { atomicCAS(err, 0, ERR_BAD_INDEX); blk = 0; }
    const __nv_bfloat16* ks = cache + blk * 2LL * block_size * Hkv * PD + (long long)(t % block_size) * Hkv * PD + c;
    *reinterpret_cast<uint4*>(out_k + (long long)t * Hkv * PD + c) = *reinterpret_cast<const uint4*>(ks);
    *reinterpret_cast<uint4*>(out_v + (long long)t * Hkv * PD + c) = *reinterpret_cast<const uint4*>(ks + (long long)block_size * Hkv * PD);
  }
}

// Greedy sampling: argmax over the first `vocab` columns of each row of bf16 logits (lowest index on ties).
// One CTA of 1024 threads per row; 16-byte loads when the rows are 16-byte aligned (vec != 0).
constexpr int AM_THREADS = 1024;
__global__ void __launch_bounds__(AM_THREADS)
argmax_rows_kernel(const __nv_bfloat16* logits, long long ld, int vocab, long long* out, int vec) {
  const long long r = blockIdx.x;
  const __nv_bfloat16* row = logits + r * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int done = 0;
  if (vec) {
    const int nv = vocab / 8;
    for (int i = threadIdx.x; i < nv; i += AM_THREADS) {
      const uint4 u = reinterpret_cast<const uint4*>(row)[i];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (f[j] > best || (f[j] == best && i * 8 + j < bi)) { best = f[j]; bi = i * 8 + j; }
    }
    done = nv * 8;
  }
  for (int i = done + threadIdx.x; i < vocab; i += AM_THREADS) {
    const float v = __bfloat162float(row[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  __shared__ float sv[AM_THREADS];
  __shared__ int si[AM_THREADS];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = AM_THREADS / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = sv[threadIdx.x + s];
      const int oi = si[threadIdx.x + s];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[r] = si[0] == 0x7fffffff ? 0 : si[0];
}

}  // namespace mlf

using namespace mlf;

// Workspace floats needed by mlf_paged_decode for a given split count.
MLF_API long long mlf_paged_decode_ws_elems(int B, int Hq, int splits) { return (long long)B * Hq * splits * (PD + 2); }

MLF_API int mlf_paged_decode_ld(const void* q, long long ldq, const void* cache, const int* block_table, const int* seq_lens, void* out,
                                float* ws, void* counters, int B, int Hq, int Hkv, int block_size, int max_blocks, int num_blocks,
                                int max_seq_len, int split_tokens, float scale, uint64_t stream);

MLF_API int mlf_paged_decode(const void* q, const void* cache, const int* block_table, const int* seq_lens, void* out, float* ws,
                             int B, int Hq, int Hkv, int block_size, int max_blocks, int num_blocks, int max_seq_len,
                             int split_tokens, float scale, uint64_t stream) {
  return mlf_paged_decode_ld(q, (long long)Hq * PD, cache, block_table, seq_lens, out, ws, nullptr, B, Hq, Hkv, block_size, max_blocks,
                             num_blocks, max_seq_len, split_tokens, scale, stream);
}

// q rows may sit inside a wider packed buffer: ldq = elements between consecutive sequences' query rows.
// counters (optional, B * Hkv zeroed uint32 that the kernel leaves zero): the last split of each (sequence, kv head)
// merges the splits inside the same launch; without it a second small kernel does.
MLF_API int mlf_paged_decode_ld(const void* q, long long ldq, const void* cache, const int* block_table, const int* seq_lens, void* out,
                                float* ws, void* counters, int B, int Hq, int Hkv, int block_size, int max_blocks, int num_blocks,
                                int max_seq_len, int split_tokens, float scale, uint64_t stream) {
  MLF_REQUIRE(ldq % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0, "paged_decode: query rows must be 4-byte aligned");
  MLF_REQUIRE(B > 0 && Hq % Hkv == 0, "paged_decode: bad head counts");
  const int G = Hq / Hkv;
  MLF_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, "paged_decode: group size %d not supported (1, 2, 4, 8)", G);
  if (split_tokens <= 0) split_tokens = 512;
  split_tokens = (split_tokens + P_SUB - 1) / P_SUB * P_SUB;
  int splits = (max_seq_len + split_tokens - 1) / split_tokens;
  if (splits < 1) splits = 1;
  MLF_REQUIRE(splits == 1 || ws != nullptr, "paged_decode: workspace required for %d splits", splits);
  PagedDecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ws = splits > 1 ? ws : nullptr;
  p.counters = splits > 1 ? static_cast<unsigned int*>(counters) : nullptr;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.block_size = block_size; p.max_blocks = max_blocks; p.num_blocks = num_blocks;
  p.split_tokens = split_tokens; p.splits = splits;
  p.bs_shift = -1;
  for (int sh = 0; sh < 16; ++sh) if ((1 << sh) == block_size) p.bs_shift = sh;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(B, Hkv, splits);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(paged_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    MLF_CHECK_CUDA(cudaFuncSetAttribute(paged_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    MLF_CHECK_CUDA(cudaFuncSetAttribute(paged_decode_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    MLF_CHECK_CUDA(cudaFuncSetAttribute(paged_decode_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    attr_set[dev & 63] = true;
  }
  switch (G) {
    case 1: paged_decode_kernel<1><<<grid, P_THREADS, P_SMEM, st>>>(p); break;
    case 2: paged_decode_kernel<2><<<grid, P_THREADS, P_SMEM, st>>>(p); break;
    case 4: paged_decode_kernel<4><<<grid, P_THREADS, P_SMEM, st>>>(p); break;
    default: paged_decode_kernel<8><<<grid, P_THREADS, P_SMEM, st>>>(p); break;
  }
  count_launch();
  if (splits > 1 && p.counters == nullptr) {
    paged_decode_merge_kernel<<<B * Hq, 128, 0, st>>>(ws, p.out, B, Hq, Hkv, G, splits);
    count_launch();
  }
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_kv_cache_write(void* cache, const void* k, const void* v, const long long* slots, long long T, int Hkv,
                               int block_size, int num_blocks, long long ldk, long long ldv, uint64_t stream) {
  if (T <= 0) return 0;
  long long g = (T * (Hkv * PD / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  kv_cache_write_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(cache), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), slots, T, Hkv,
      block_size, num_blocks, ldk, ldv, device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_rope_kv_write(void* qkv, long long ld, const long long* pos, const long long* slots, void* cache, long long T, int Hq,
                              int Hkv, int block_size, int num_blocks, float theta, uint64_t stream) {
  if (T <= 0) return 0;
  MLF_REQUIRE(ld % 4 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 7) == 0, "rope_kv_write: rows must be 8-byte aligned");
  long long g = (T * (Hq + 2 * Hkv) * 16 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  rope_kv_write_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), ld, pos, slots, static_cast<__nv_bfloat16*>(cache), T, Hq, Hkv, block_size, num_blocks, theta,
      device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_kv_gather(const void* cache, const int* block_table, int table_len, int len, int Hkv, int block_size, int num_blocks,
                          void* out_k, void* out_v, uint64_t stream) {
  if (len <= 0) return 0;
  MLF_REQUIRE((long long)len <= (long long)table_len * block_size,
              "kv_gather: %d tokens need more than the %d block-table entries given", len, table_len);
  long long g = ((long long)len * (Hkv * PD / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  kv_gather_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(cache), block_table, len, Hkv, block_size, num_blocks, static_cast<__nv_bfloat16*>(out_k),
      static_cast<__nv_bfloat16*>(out_v), device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_argmax_rows(const void* logits, long long rows, long long ld, int vocab, long long* out, uint64_t stream) {
  if (rows <= 0) return 0;
  const int vec = (ld % 8 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) ? 1 : 0;
  argmax_rows_kernel<<<(int)rows, AM_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(logits), ld,
                                                                                          vocab, out, vec);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
