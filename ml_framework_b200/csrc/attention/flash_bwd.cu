// Self-attention backward for head_dim 128 on tcgen05 tensor cores.
//
// One CTA owns 128 key/value rows of one (batch, kv-head) and walks the 64-row query tiles
// that can see them (all heads of the GQA group). Everything is computed in the transposed
// orientation so each thread owns one key row and no operand is ever transposed in memory:
//   S^T  = K  Q^T        (M128 N64 K128)      dP^T = V dO^T      (M128 N64 K128)
//   P^T  = exp2(S^T c - lse)                  dS^T = P^T o (dP^T - D) * scale
//   dV  += P^T  dO       (M128 N128 K64)      dK  += dS^T Q      (M128 N128 K64)
//   dQ^T = K^T dS^T      (M128 N64 K128)  -> fp32 atomics into dq_accum (coalesced along d)
// K-major and MN-major shared-memory descriptors pick the orientation: a [rows][64 x bf16]
// 128B-swizzled block is read K-major when its rows index M/N and MN-major when they index K.
// TMEM: dK 128 | dV 128 | S^T 64 | dP^T 64 | dQ^T 64 columns.
//
// 192 threads: warp 0 TMA producer (K, V once; Q and dO tiles through a 2-stage ring), warp 1
// MMA issuer, warps 2..5 one key row per thread.
//
// The reference has no attention backward (its TP/attention layers are forward-only,
// src/MLFramework/Inference/PagedAttention/Layers/PagedAttentionLayer.cs:102-144); training the
// GPT and Llama configurations requires it.
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo);

constexpr int FB_BKV = 128;
constexpr int FB_BQ = 64;
constexpr int FB_D = 128;
constexpr int FB_THREADS = 192;
constexpr int FB_KV_BYTES = FB_BKV * FB_D * 2;   // 32 KB (two 16 KB column blocks)
constexpr int FB_Q_BYTES = FB_BQ * FB_D * 2;     // 16 KB (two 8 KB column blocks)
constexpr int FB_P_BYTES = FB_BKV * FB_BQ * 2;   // 16 KB
constexpr int FB_STAGE = 2 * FB_Q_BYTES;         // Q + dO
constexpr int FB_STATS_BYTES = 2 * 4 * 2 * FB_BQ * 4;  // [2 buffers][4 warps][lse 64 | delta 64] fp32
constexpr int FB_SMEM = 2 * FB_KV_BYTES + 2 * FB_STAGE + 2 * FB_P_BYTES + FB_STATS_BYTES + 256;
constexpr int FB_TMEM_COLS = 512;

struct FlashBwdParams {
  float* dq_accum;          // fp32 [tokens, Hq*128], zeroed by the launcher
  __nv_bfloat16* dk;        // [tokens, *] pitch lddk, Hkv heads
  __nv_bfloat16* dv;
  const float* lse;         // [B, Hq, S]
  const float* delta;       // [B, Hq, S]  rowsum(dO o O)
  long long lddk, lddv;
  int B, S, Hq, Hkv, causal;
  float scale, scale_log2;
  int* err;
};

// delta[b, h, s] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (token, head), two such rows per warp in flight.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* o, const __nv_bfloat16* dout, float* delta, const float* lse, float* lse2, int B, int S,
                  int H, long long ldo, long long lddo) {
  const long long total = (long long)B * S * H;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long w0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w0 < total; w0 += 2 * nwarps) {
    const long long w1 = w0 + nwarps;
    const bool two = w1 < total;
    const long long t0 = w0 / H, t1 = two ? w1 / H : t0;
    const int h0 = (int)(w0 % H), h1 = two ? (int)(w1 % H) : h0;
    const uint2 a0v = *reinterpret_cast<const uint2*>(o + t0 * ldo + h0 * FB_D + lane * 4);
    const uint2 g0v = *reinterpret_cast<const uint2*>(dout + t0 * lddo + h0 * FB_D + lane * 4);
    const uint2 a1v = *reinterpret_cast<const uint2*>(o + t1 * ldo + h1 * FB_D + lane * 4);
    const uint2 g1v = *reinterpret_cast<const uint2*>(dout + t1 * lddo + h1 * FB_D + lane * 4);
    float2 p0 = unpack_bf16x2(a0v.x), p1 = unpack_bf16x2(a0v.y), q0 = unpack_bf16x2(g0v.x), q1 = unpack_bf16x2(g0v.y);
    float s0 = p0.x * q0.x + p0.y * q0.y + p1.x * q1.x + p1.y * q1.y;
    p0 = unpack_bf16x2(a1v.x); p1 = unpack_bf16x2(a1v.y); q0 = unpack_bf16x2(g1v.x); q1 = unpack_bf16x2(g1v.y);
    float s1 = p0.x * q0.x + p0.y * q0.y + p1.x * q1.x + p1.y * q1.y;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, off);
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
    }
    if (lane < 2 && (lane == 0 || two)) {
      const long long t = lane ? t1 : t0;
      const int h = lane ? h1 : h0;
      const long long b = t / S, sidx = t % S;
      delta[(b * H + h) * S + sidx] = lane ? s1 : s0;
      if (lse2) lse2[(b * H + h) * S + sidx] = lse[(b * H + h) * S + sidx] * 1.4426950408889634f;
    }
  }
}

// out[t, c] (bf16, pitch ldo) = in[t, c] (fp32, pitch ldi); cols multiple of 4.
__global__ void __launch_bounds__(256)
cast_rows_f32_bf16_kernel(__nv_bfloat16* out, const float* in, long long rows, int cols, long long ldo, long long ldi) {
  const int vpr = cols / 4;
  const long long total = rows * vpr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = (int)(i % vpr) * 4;
    const float4 v = *reinterpret_cast<const float4*>(in + r * ldi + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + r * ldo + c) = o;
  }
}

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const FlashBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase;
  const uint32_t sV = sK + FB_KV_BYTES;
  const uint32_t sQdO = sV + FB_KV_BYTES;                 // stage s: Q at +s*FB_STAGE, dO right after Q
  const uint32_t sP = sQdO + 2 * FB_STAGE;
  const uint32_t sdS = sP + FB_P_BYTES;
  const uint32_t sStats = sdS + FB_P_BYTES;               // [2 stages][lse 64 | delta 64] fp32
  const uint32_t bars = sStats + FB_STATS_BYTES;
  // barriers: kv_full, q_full[2], q_empty[2], s_full, p_full, dq_full
  const uint32_t kv_full = bars;
  auto q_full = [&](int s) { return bars + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bars + 8u * (3 + s); };
  const uint32_t s_full = bars + 8u * 5;
  const uint32_t p_full = bars + 8u * 6;
  const uint32_t dq_full = bars + 8u * 7;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + (bars - sbase) + 8 * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  float* stats = reinterpret_cast<float*>(smem + (sStats - sbase));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kt = blockIdx.x;
  const int hkv = blockIdx.y;
  const int b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int k0 = kt * FB_BKV;
  const long long row_base = (long long)b * p.S;
  const int n_qt = (p.S + FB_BQ - 1) / FB_BQ;
  const int qt0 = p.causal ? (k0 / FB_BQ) : 0;
  const int per_head = n_qt - qt0;
  const int n_it = per_head * group;

  if ((sbase & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_INDEX);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), FB_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t_dK = tmem_base, t_dV = tmem_base + 128, t_S = tmem_base + 256, t_dP = tmem_base + 320,
                 t_dQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      const int krow = (int)(row_base + k0);
      mbar_expect_tx(kv_full, 2 * FB_KV_BYTES);
      tma_load_2d(sK, &tmK, hkv * FB_D, krow, kv_full);
      tma_load_2d(sK + FB_KV_BYTES / 2, &tmK, hkv * FB_D + 64, krow, kv_full);
      tma_load_2d(sV, &tmV, hkv * FB_D, krow, kv_full);
      tma_load_2d(sV + FB_KV_BYTES / 2, &tmV, hkv * FB_D + 64, krow, kv_full);
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        if (!mbar_wait(q_empty(s), ((it >> 1) & 1) ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        const int h = hkv * group + it / per_head;
        const int q0 = (qt0 + it % per_head) * FB_BQ;
        const int qrow = (int)(row_base + q0);
        const uint32_t sQ = sQdO + s * FB_STAGE, sdO = sQ + FB_Q_BYTES;
        mbar_expect_tx(q_full(s), FB_STAGE);
        tma_load_2d(sQ, &tmQ, h * FB_D, qrow, q_full(s));
        tma_load_2d(sQ + FB_Q_BYTES / 2, &tmQ, h * FB_D + 64, qrow, q_full(s));
        tma_load_2d(sdO, &tmdO, h * FB_D, qrow, q_full(s));
        tma_load_2d(sdO + FB_Q_BYTES / 2, &tmdO, h * FB_D + 64, qrow, q_full(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, FB_BQ, 0, 0);    // S^T, dP^T
      const uint32_t idesc_g = make_idesc_bf16(128, FB_D, 0, 1);     // dV, dK: B = dO / Q MN-major
      const uint32_t idesc_q = make_idesc_bf16(128, FB_BQ, 1, 1);    // dQ^T: A = K MN-major, B = dS^T MN-major
      auto issue_s = [&](int it) -> bool {
        const int s = it & 1;
        if (!mbar_wait(q_full(s), (it >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) return false;
        tc_fence_after_sync();
        const uint32_t sQ = sQdO + s * FB_STAGE, sdO = sQ + FB_Q_BYTES;
#pragma unroll
        for (int k = 0; k < FB_D / 16; ++k) {
          const uint32_t ao = (k >> 2) * (FB_KV_BYTES / 2) + (k & 3) * 32;
          const uint32_t bo = (k >> 2) * (FB_Q_BYTES / 2) + (k & 3) * 32;
          umma_bf16_ss(t_S, make_smem_desc_sw128(sK + ao, 16, 1024), make_smem_desc_sw128(sQ + bo, 16, 1024), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < FB_D / 16; ++k) {
          const uint32_t ao = (k >> 2) * (FB_KV_BYTES / 2) + (k & 3) * 32;
          const uint32_t bo = (k >> 2) * (FB_Q_BYTES / 2) + (k & 3) * 32;
          umma_bf16_ss(t_dP, make_smem_desc_sw128(sV + ao, 16, 1024), make_smem_desc_sw128(sdO + bo, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(s_full);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
      if (ok && n_it > 0) ok = issue_s(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t sQ = sQdO + s * FB_STAGE, sdO = sQ + FB_Q_BYTES;
        if (!mbar_wait(p_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < FB_BQ / 16; ++k)   // dV += P^T dO
          umma_bf16_ss(t_dV, make_smem_desc_sw128(sP + k * 32, 16, 1024),
                       make_smem_desc_sw128(sdO + k * 2048, FB_Q_BYTES / 2, 1024), idesc_g, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < FB_BQ / 16; ++k)   // dK += dS^T Q
          umma_bf16_ss(t_dK, make_smem_desc_sw128(sdS + k * 32, 16, 1024),
                       make_smem_desc_sw128(sQ + k * 2048, FB_Q_BYTES / 2, 1024), idesc_g, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < FB_BKV / 16; ++k)  // dQ^T = K^T dS^T
          umma_bf16_ss(t_dQ, make_smem_desc_sw128(sK + k * 2048, FB_KV_BYTES / 2, 1024),
                       make_smem_desc_sw128(sdS + k * 2048, FB_P_BYTES, 1024), idesc_q, k != 0);
        umma_commit(dq_full);
        umma_commit(q_empty(s));
        if (it + 1 < n_it) ok = issue_s(it + 1);
      }
    }
  } else {
    const int qd = warp & 3;
    const int r = qd * 32 + lane;          // key row in the tile == TMEM lane == d index for dQ^T
    const int kv_i = k0 + r;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int h = hkv * group + it / per_head;
      const int q0 = (qt0 + it % per_head) * FB_BQ;
      float* st = stats + ((it & 1) * 4 + qd) * 2 * FB_BQ;   // this warp's own copy
      {  // stage lse (log2 domain) and delta for this query tile: 4 values per lane
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int idx_in = lane + 32 * e;          // 0..127: [lse 64 | delta 64]
          const int c = idx_in & 63;
          const int qi = q0 + c;
          const long long idx = ((long long)b * p.Hq + h) * p.S + qi;
          float v = 0.f;
          if (qi < p.S) v = idx_in < 64 ? p.lse[idx] * 1.4426950408889634f : p.delta[idx];
          st[idx_in] = v;
        }
      }
      __syncwarp();
      if (!mbar_wait_warp(s_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      const bool need_mask = (p.causal && q0 < k0 + FB_BKV - 1) || (q0 + FB_BQ > p.S) || (k0 + FB_BKV > p.S);
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t ts[32], tp[32];
        tmem_ld_32x32b_x32(t_S + 32 * hlf + lane_off, ts);
        tmem_ld_32x32b_x32(t_dP + 32 * hlf + lane_off, tp);
        tmem_wait_ld();
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = 32 * hlf + 2 * i + e;
            float pr = exp2f(__uint_as_float(ts[2 * i + e]) * p.scale_log2 - st[c]);
            if (need_mask) {
              const int qi = q0 + c;
              if (qi >= p.S || kv_i >= p.S || (p.causal && qi < kv_i)) pr = 0.f;
            }
            pv[e] = pr;
            dv[e] = pr * (__uint_as_float(tp[2 * i + e]) - st[FB_BQ + c]) * p.scale;
          }
          pk[i] = pack_bf16x2(pv[0], pv[1]);
          dk_[i] = pack_bf16x2(dv[0], dv[1]);
        }
        const uint32_t prow = sP + r * 128, drow = sdS + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t off = ((4 * hlf + c) ^ (r & 7)) << 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + off), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                       "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(drow + off), "r"(dk_[4 * c]), "r"(dk_[4 * c + 1]),
                       "r"(dk_[4 * c + 2]), "r"(dk_[4 * c + 3]) : "memory");
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      if (!mbar_wait_warp(dq_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      // dQ^T: lane = d, columns = query index
      float* dq_col = p.dq_accum + (row_base + q0) * (long long)(p.Hq * FB_D) + h * FB_D + r;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(t_dQ + 32 * hlf + lane_off, t);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = 32 * hlf + i;
          if (q0 + c < p.S) atomicAdd(dq_col + (long long)c * (p.Hq * FB_D), __uint_as_float(t[i]));
        }
      }
      tc_fence_before_sync();
    }
    // `ok` and `n_it` are warp-uniform; the row test is not, so it only guards the stores:
    // tcgen05.ld is .sync.aligned and must be executed by the whole warp together.
    if (ok && n_it > 0) {
      // the last dq_full wait also covers the final dV / dK accumulations
      const bool row_ok = kv_i < p.S;
      __nv_bfloat16* dk_row = p.dk + (row_base + kv_i) * p.lddk + (long long)hkv * FB_D;
      __nv_bfloat16* dv_row = p.dv + (row_base + kv_i) * p.lddv + (long long)hkv * FB_D;
#pragma unroll
      for (int c = 0; c < FB_D / 32; ++c) {
        uint32_t a[32], g[32];
        tmem_ld_32x32b_x32(t_dK + 32 * c + lane_off, a);
        tmem_ld_32x32b_x32(t_dV + 32 * c + lane_off, g);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w, x;
            w.x = pack_bf16x2(__uint_as_float(a[8 * v + 0]), __uint_as_float(a[8 * v + 1]));
            w.y = pack_bf16x2(__uint_as_float(a[8 * v + 2]), __uint_as_float(a[8 * v + 3]));
            w.z = pack_bf16x2(__uint_as_float(a[8 * v + 4]), __uint_as_float(a[8 * v + 5]));
            w.w = pack_bf16x2(__uint_as_float(a[8 * v + 6]), __uint_as_float(a[8 * v + 7]));
            x.x = pack_bf16x2(__uint_as_float(g[8 * v + 0]), __uint_as_float(g[8 * v + 1]));
            x.y = pack_bf16x2(__uint_as_float(g[8 * v + 2]), __uint_as_float(g[8 * v + 3]));
            x.z = pack_bf16x2(__uint_as_float(g[8 * v + 4]), __uint_as_float(g[8 * v + 5]));
            x.w = pack_bf16x2(__uint_as_float(g[8 * v + 6]), __uint_as_float(g[8 * v + 7]));
            reinterpret_cast<uint4*>(dk_row + 32 * c)[v] = w;
            reinterpret_cast<uint4*>(dv_row + 32 * c)[v] = x;
          }
        }
      }
    } else if (ok && n_it == 0 && kv_i < p.S) {
      __nv_bfloat16* dk_row = p.dk + (row_base + kv_i) * p.lddk + (long long)hkv * FB_D;
      __nv_bfloat16* dv_row = p.dv + (row_base + kv_i) * p.lddv + (long long)hkv * FB_D;
      for (int c = 0; c < FB_D / 8; ++c) {
        reinterpret_cast<uint4*>(dk_row)[c] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(dv_row)[c] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, FB_TMEM_COLS);
  }
}

}  // namespace mlf

using namespace mlf;

namespace mlf {
int launch_flash_bwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                        float* dq_accum, void* dk, void* dv, const float* lse2, const float* delta, long long lddk, long long lddv,
                        int B, int S, int Hq, int Hkv, float scale, int causal, cudaStream_t st);
}

static int g_flash_bwd_ws = 1;
// 1 (default): sequences of at least 128 tokens (a multiple of 4) use the 128 x 128 warpgroup kernel; 0: the 128 x 64 kernel.
MLF_API void mlf_set_flash_bwd_ws(int on) { g_flash_bwd_ws = on; }

// Bytes of fp32 scratch the caller must provide: dq accumulator [B*S, Hq*128] + delta [B, Hq, S] +
// logsumexp in the log2 domain [B, Hq, S] + 256 floats of slack (the last tile's statistics are
// fetched as whole 512-byte pieces).
MLF_API long long mlf_flash_bwd_scratch_bytes(int B, int S, int Hq) {
  return ((long long)B * S * Hq * FB_D + 2 * (long long)B * Hq * S + 256) * 4;
}

// q/k/v/o/dout: bf16 token-major views (row pitches in elements). dq/dk/dv: bf16 outputs with
// their own pitches (may point into a packed dQKV buffer). lse from mlf_flash_fwd.
MLF_API int mlf_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                          void* dq, void* dk, void* dv, void* scratch, int B, int S, int Hq, int Hkv, long long ldq,
                          long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk,
                          long long lddv, float scale, int causal, uint64_t stream) {
  MLF_REQUIRE(B > 0 && S > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "flash_bwd: bad shape");
  MLF_REQUIRE(lddq % 4 == 0 && lddk % 8 == 0 && lddv % 8 == 0, "flash_bwd: gradient pitches must be multiples of 8");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * S;
  float* dq_accum = static_cast<float*>(scratch);
  float* delta = dq_accum + rows * Hq * FB_D;
  float* lse2 = delta + rows * Hq + 128;        // 16-byte aligned when S % 4 == 0; 128 floats of slack after each array
  const bool use_ws = g_flash_bwd_ws && S >= 128 && S % 4 == 0 && ((reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(lse2)) & 15) == 0;
  MLF_CHECK_CUDA(cudaMemsetAsync(dq_accum, 0, sizeof(float) * rows * Hq * FB_D, st));
  {
    MLF_REQUIRE(((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dout)) & 15) == 0 && ldo % 8 == 0 && lddo % 8 == 0,
                "flash_bwd: O and dO must be 16-byte aligned with pitches that are multiples of 8");
    const long long warps = rows * Hq;
    long long grid = (warps + 7) / 8;
    const long long cap = (long long)sm_count() * 8;
    if (grid > cap) grid = cap;
    attn_delta_kernel<<<(int)grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout),
                                                 delta, lse, use_ws ? lse2 : nullptr, B, S, Hq, ldo, lddo);
                                                 count_launch();
    MLF_CHECK_CUDA(cudaGetLastError());
  }
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if (use_ws) {
    if ((rc = cached_tmap_bf16(&tq, q, (uint64_t)Hq * FB_D, rows, ldq, 64, 128))) return rc;
    if ((rc = cached_tmap_bf16(&tk, k, (uint64_t)Hkv * FB_D, rows, ldk, 64, 128))) return rc;
    if ((rc = cached_tmap_bf16(&tv, v, (uint64_t)Hkv * FB_D, rows, ldv, 64, 128))) return rc;
    if ((rc = cached_tmap_bf16(&tdo, dout, (uint64_t)Hq * FB_D, rows, lddo, 64, 128))) return rc;
    if ((rc = launch_flash_bwd_ws(tq, tk, tv, tdo, dq_accum, dk, dv, lse2, delta, lddk, lddv, B, S, Hq, Hkv, scale, causal, st))) return rc;
  } else {
  if ((rc = cached_tmap_bf16(&tq, q, (uint64_t)Hq * FB_D, rows, ldq, 64, FB_BQ))) return rc;
  if ((rc = cached_tmap_bf16(&tk, k, (uint64_t)Hkv * FB_D, rows, ldk, 64, FB_BKV))) return rc;
  if ((rc = cached_tmap_bf16(&tv, v, (uint64_t)Hkv * FB_D, rows, ldv, 64, FB_BKV))) return rc;
  if ((rc = cached_tmap_bf16(&tdo, dout, (uint64_t)Hq * FB_D, rows, lddo, 64, FB_BQ))) return rc;
  FlashBwdParams p;
  p.dq_accum = dq_accum;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.lse = lse;
  p.delta = delta;
  p.lddk = lddk; p.lddv = lddv;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM));
    attr_set[dev & 63] = true;
  }
  dim3 grid((S + FB_BKV - 1) / FB_BKV, Hkv, B);
  flash_bwd_kernel<<<grid, FB_THREADS, FB_SMEM, st>>>(tq, tk, tv, tdo, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  }
  {
    const long long total = rows * (Hq * FB_D / 4);
    long long g = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (g > cap) g = cap;
    cast_rows_f32_bf16_kernel<<<(int)g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(dq), dq_accum, rows, Hq * FB_D, lddq,
                                                      (long long)Hq * FB_D);
                                                      count_launch();
    MLF_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
}
