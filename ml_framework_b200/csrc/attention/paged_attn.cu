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
// split) and streams K and V rows with 16-byte loads, 16 lanes per token row, sharing every
// loaded row between the G = Hq/Hkv query heads of the group. Long sequences are split over
// grid.z (flash-decoding) and merged by a second small kernel.
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
constexpr int P_SUB = 128;        // tokens per inner chunk
constexpr int P_MAXG = 8;         // max query heads per kv head

struct PagedDecodeParams {
  const __nv_bfloat16* q;         // [B, Hq, 128]
  const __nv_bfloat16* cache;
  const int* block_table;         // [B, max_blocks]
  const int* seq_lens;            // [B]
  __nv_bfloat16* out;             // [B, Hq, 128]
  float* ws;                      // [B, Hkv, splits, G, 130] (m, l, o[128]) when splits > 1
  int B, Hq, Hkv, G, block_size, max_blocks, num_blocks, split_tokens, splits;
  float scale_log2;
  int* err;
};

template <int G>
__global__ void __launch_bounds__(P_THREADS)
paged_decode_kernel(const PagedDecodeParams p) {
  const int b = blockIdx.x, hkv = blockIdx.y, sp = blockIdx.z;
  const int len = p.seq_lens[b];
  const int t_lo = sp * p.split_tokens;
  const int t_hi = min(len, t_lo + p.split_tokens);
  const int tid = threadIdx.x;
  const int tg = tid >> 4;        // token group 0..7
  const int dl = tid & 15;        // 16 lanes x 8 elements = 128
  __shared__ float s_q[G][PD];
  __shared__ float s_p[G][P_SUB];
  __shared__ float s_red[8][G][PD + 2];
  __shared__ float s_m[G], s_l[G], s_alpha[G];

  float* ws = p.ws ? p.ws + ((((long long)b * p.Hkv + hkv) * p.splits + sp) * G) * (PD + 2) : nullptr;
  if (t_lo >= t_hi) {
    if (ws) {
      for (int i = tid; i < G * (PD + 2); i += P_THREADS) ws[i] = (i % (PD + 2)) == 0 ? -INFINITY : 0.f;
    } else if (sp == 0) {
      for (int i = tid; i < G * PD; i += P_THREADS)
        p.out[((long long)b * p.Hq + hkv * G) * PD + i] = __float2bfloat16(0.f);
    }
    return;
  }
  for (int i = tid; i < G * PD; i += P_THREADS)
    s_q[i / PD][i % PD] = __bfloat162float(p.q[((long long)b * p.Hq + hkv * G) * PD + i]) * p.scale_log2;
  if (tid < G) { s_m[tid] = -INFINITY; s_l[tid] = 0.f; }
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
  __syncthreads();
  float qreg[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) qreg[g][j] = s_q[g][dl * 8 + j];

  const long long blk_stride = 2LL * p.block_size * p.Hkv * PD;   // elements per physical block
  const long long v_off = (long long)p.block_size * p.Hkv * PD;
  const int* bt = p.block_table + (long long)b * p.max_blocks;

  for (int c0 = t_lo; c0 < t_hi; c0 += P_SUB) {
    const int cn = min(P_SUB, t_hi - c0);
    // ---- scores for up to 128 tokens: 8 tokens per step, 16 lanes per token; the 16-byte loads of
    // four steps are issued together so that four rows per thread are in flight (the kernel is
    // bound by memory latency x bytes in flight, not by arithmetic)
#pragma unroll 1
    for (int i0 = tg; i0 < P_SUB; i0 += 32) {
      uint4 u[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + 8 * e;
        u[e] = make_uint4(0, 0, 0, 0);
        if (i < cn) {
          const int t = c0 + i;
          int blk = bt[t / p.block_size];
          if (blk < 0 || blk >= p.num_blocks) { atomicCAS(p.err, 0, ERR_BAD_INDEX); blk = 0; }
          u[e] = *reinterpret_cast<const uint4*>(p.cache + blk * blk_stride + ((long long)(t % p.block_size) * p.Hkv + hkv) * PD + dl * 8);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + 8 * e;
        float s[G];
        float k[8];
        const float2 a = unpack_bf16x2(u[e].x), bb = unpack_bf16x2(u[e].y), c = unpack_bf16x2(u[e].z), d = unpack_bf16x2(u[e].w);
        k[0] = a.x; k[1] = a.y; k[2] = bb.x; k[3] = bb.y; k[4] = c.x; k[5] = c.y; k[6] = d.x; k[7] = d.y;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          s[g] = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) s[g] += qreg[g][j] * k[j];
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
          if (dl == 0) s_p[g][i] = i < cn ? s[g] : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- online softmax bookkeeping: one warp per head (G <= 8 heads over 4 warps)
    for (int g = tid >> 5; g < G; g += P_THREADS / 32) {
      const int lane = tid & 31;
      float mx = -INFINITY;
      for (int i = lane; i < P_SUB; i += 32) mx = fmaxf(mx, s_p[g][i]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = s_m[g];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int i = lane; i < P_SUB; i += 32) {
        const float e = exp2f(s_p[g][i] - m_new);
        s_p[g][i] = e;
        sum += e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        const float alpha = exp2f(m_old - m_new);
        s_alpha[g] = alpha;
        s_l[g] = s_l[g] * alpha + sum;
        s_m[g] = m_new;
      }
    }
    __syncthreads();
    // ---- acc = acc * alpha + P V
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float al = s_alpha[g];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] *= al;
    }
#pragma unroll 1
    for (int i0 = tg; i0 < cn; i0 += 32) {
      uint4 u[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + 8 * e;
        u[e] = make_uint4(0, 0, 0, 0);
        if (i < cn) {
          const int t = c0 + i;
          int blk = bt[t / p.block_size];
          if (blk < 0 || blk >= p.num_blocks) blk = 0;
          u[e] = *reinterpret_cast<const uint4*>(p.cache + blk * blk_stride + v_off + ((long long)(t % p.block_size) * p.Hkv + hkv) * PD + dl * 8);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + 8 * e;
        if (i >= cn) break;
        float v[8];
        const float2 a = unpack_bf16x2(u[e].x), bb = unpack_bf16x2(u[e].y), c = unpack_bf16x2(u[e].z), d = unpack_bf16x2(u[e].w);
        v[0] = a.x; v[1] = a.y; v[2] = bb.x; v[3] = bb.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pw = s_p[g][i];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[g][j] += pw * v[j];
        }
      }
    }
    __syncthreads();
  }
  // ---- reduce the 8 token groups
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) s_red[tg][g][dl * 8 + j] = acc[g][j];
  __syncthreads();
  for (int i = tid; i < G * PD; i += P_THREADS) {
    const int g = i / PD, d = i % PD;
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) o += s_red[k][g][d];
    if (ws) {
      ws[g * (PD + 2) + 2 + d] = o;
      if (d == 0) { ws[g * (PD + 2)] = s_m[g]; ws[g * (PD + 2) + 1] = s_l[g]; }
    } else {
      const float l = s_l[g];
      p.out[((long long)b * p.Hq + hkv * G + g) * PD + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    }
  }
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

// out_k / out_v [len, Hkv, 128] <- pages of one sequence.
__global__ void __launch_bounds__(256)
kv_gather_kernel(const __nv_bfloat16* cache, const int* block_table, int len, int Hkv, int block_size, int num_blocks,
                 __nv_bfloat16* out_k, __nv_bfloat16* out_v, int* err) {
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

// Greedy sampling: argmax over the first `vocab` columns of each row of bf16 logits.
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const __nv_bfloat16* logits, long long ld, int vocab, long long* out) {
  const long long r = blockIdx.x;
  const __nv_bfloat16* row = logits + r * ld;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best) { best = v; bi = i; }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = sv[threadIdx.x + s];
      const int oi = si[threadIdx.x + s];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[r] = si[0];
}

}  // namespace mlf

using namespace mlf;

// Workspace floats needed by mlf_paged_decode for a given split count.
MLF_API long long mlf_paged_decode_ws_elems(int B, int Hq, int splits) { return (long long)B * Hq * splits * (PD + 2); }

MLF_API int mlf_paged_decode(const void* q, const void* cache, const int* block_table, const int* seq_lens, void* out, float* ws,
                             int B, int Hq, int Hkv, int block_size, int max_blocks, int num_blocks, int max_seq_len,
                             int split_tokens, float scale, uint64_t stream) {
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
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ws = splits > 1 ? ws : nullptr;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.block_size = block_size; p.max_blocks = max_blocks; p.num_blocks = num_blocks;
  p.split_tokens = split_tokens; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(B, Hkv, splits);
  switch (G) {
    case 1: paged_decode_kernel<1><<<grid, P_THREADS, 0, st>>>(p); break;
    case 2: paged_decode_kernel<2><<<grid, P_THREADS, 0, st>>>(p); break;
    case 4: paged_decode_kernel<4><<<grid, P_THREADS, 0, st>>>(p); break;
    default: paged_decode_kernel<8><<<grid, P_THREADS, 0, st>>>(p); break;
  }
  count_launch();
  if (splits > 1) {
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

MLF_API int mlf_kv_gather(const void* cache, const int* block_table, int len, int Hkv, int block_size, int num_blocks, void* out_k,
                          void* out_v, uint64_t stream) {
  if (len <= 0) return 0;
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
  argmax_rows_kernel<<<(int)rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(logits), ld,
                                                                                   vocab, out);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
