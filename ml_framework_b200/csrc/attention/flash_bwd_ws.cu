// Self-attention backward, head_dim 128: 128 x 128 tiles, three warpgroups, P^T kept in tensor memory.
//
// One CTA owns 128 key/value rows of one (batch, kv-head) and walks the 128-row query tiles that can
// see them (all heads of the GQA group). Key-major ("transposed") orientation, so that each thread of the
// compute warpgroup owns one key row and dK / dV accumulate in place across the whole walk:
//   S^T  = K  Q^T        dP^T = V dO^T                 (M128 N128 K128, operands in shared memory)
//   P^T  = exp2(S^T c - lse)        -> packed bf16 into TENSOR MEMORY over S^T (A operand of dV)
//   dS^T = P^T o (dP^T - delta) c   -> packed bf16 into shared memory        (operand of dK and dQ)
//   dV  += P^T  dO       dK  += dS^T Q                 (M128 N128 K128)
//   dQ   = dS   K        (M = query rows)  -> read out by its own warpgroup into swizzled staging tiles
//                                            and added to the fp32 dQ buffer by TMA reduction stores
//                                            (per-thread reductions saturate the L2 atomic path and
//                                            the load/store unit the other warpgroup needs)
// The same 128B-swizzled tiles serve as K-major or MN-major operands through their descriptors, so
// nothing is ever transposed in memory.
//
// 384 threads: warps 0..3 control (warp 0 TMA producer, warp 1 MMA issuer), warps 4..7 compute
// (one key row per thread), warps 8..11 dQ read-out; the control warpgroup hands registers to the
// other two (setmaxnreg). TMEM (512 columns): dK | dV | S^T (then P^T) | dP^T (then dQ).
// Issue order on the tensor pipe: dV(i), S^T(i+1), dK(i), dQ(i), dP^T(i+1): the next tile's
// exponentials run while this tile's gradients are multiplied.
//
// The reference has no attention backward (its attention layers are forward-only,
// src/MLFramework/Inference/PagedAttention/Layers/PagedAttentionLayer.cs:102-144); training the
// GPT and Llama configurations requires it.
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

constexpr int G_T = 128;                       // tile edge (keys and queries)
constexpr int G_D = 128;
constexpr int G_THREADS = 384;
constexpr int G_TILE = G_T * G_D * 2;          // 32 KB: two 64-column blocks of 16 KB
constexpr int G_HALF = G_TILE / 2;
constexpr int G_STATS = 2 * G_T * 4;           // lse (log2 domain) | delta, fp32, per stage
constexpr int G_DQ_STG = G_T * 32 * 4;         // dQ staging tile: 128 rows x 32 fp32 columns, 128B-swizzled
constexpr int G_SMEM = 7 * G_TILE + 2 * G_STATS + 256;   // K, V, Q x 2, dO, dS, 2 staging tiles (= 1 tile)
constexpr int G_TMEM_COLS = 512;

struct FlashBwdWsParams {
  float* dq_accum;          // fp32 [tokens, Hq*128], zeroed by the launcher
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  const float* lse2;        // [B, Hq, S] logsumexp * log2(e)
  const float* delta;       // [B, Hq, S] rowsum(dO o O)
  long long lddk, lddv;
  int B, S, Hq, Hkv, causal;
  float scale, scale_log2;
  int* err;
};

__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

__global__ void __launch_bounds__(G_THREADS, 1)
flash_bwd_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmDQ, const FlashBwdWsParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase;
  const uint32_t sV = sK + G_TILE;
  auto sQ = [&](int s) { return sV + G_TILE + (uint32_t)s * G_TILE; };
  const uint32_t sdO = sV + 3u * G_TILE;                  // single buffer: reloaded once dV of the previous tile has read it
  const uint32_t sdS = sV + 4u * G_TILE;
  const uint32_t sStg = sV + 5u * G_TILE;                  // two dQ staging tiles of 16 KB
  const uint32_t sStats = sStg + G_TILE;                    // stage s at + s * G_STATS
  const uint32_t bars = sStats + 2 * G_STATS;
  // barriers: kv_full, q_full[2], q_empty[2], s_full, dp_full, p_full, ds_full, dq_full, dq_empty, do_full, do_empty, stg_bar
  const uint32_t kv_full = bars;
  auto q_full = [&](int s) { return bars + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bars + 8u * (3 + s); };
  const uint32_t s_full = bars + 8u * 5, dp_full = bars + 8u * 6, p_full = bars + 8u * 7, ds_full = bars + 8u * 8,
                 dq_full = bars + 8u * 9, dq_empty = bars + 8u * 10, do_full = bars + 8u * 11, do_empty = bars + 8u * 12,
                 stg_bar = bars + 8u * 13;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + (bars - sbase) + 8 * 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_kt = (p.S + G_T - 1) / G_T;
  // 1-D grid ordered by work: under a causal mask the first key tiles see the most query tiles
  const int per_kt = p.Hkv * p.B;
  const int kt = (int)blockIdx.x / per_kt;
  const int hkv = ((int)blockIdx.x % per_kt) % p.Hkv;
  const int b = ((int)blockIdx.x % per_kt) / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int k0 = kt * G_T;
  const long long row_base = (long long)b * p.S;
  const int qt0 = p.causal ? kt : 0;
  const int per_head = n_kt - qt0;           // query tiles per head (n_qt == n_kt: same tile edge)
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
    mbar_init(dp_full, 1);
    mbar_init(p_full, 128);
    mbar_init(ds_full, 128);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 128);
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(stg_bar, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), G_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t_dK = tmem_base, t_dV = tmem_base + 128, t_S = tmem_base + 256, t_dP = tmem_base + 384;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ===================== TMA producer =====================
      if (lane == 0) {
        const int krow = (int)(row_base + k0);
        mbar_expect_tx(kv_full, 2 * G_TILE);
        tma_load_2d(sK, &tmK, hkv * G_D, krow, kv_full);
        tma_load_2d(sK + G_HALF, &tmK, hkv * G_D + 64, krow, kv_full);
        tma_load_2d(sV, &tmV, hkv * G_D, krow, kv_full);
        tma_load_2d(sV + G_HALF, &tmV, hkv * G_D + 64, krow, kv_full);
        for (int it = 0; it < n_it; ++it) {
          const int s = it & 1;
          if (!mbar_wait(q_empty(s), ((it >> 1) & 1) ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          const int h = hkv * group + it / per_head;
          const int q0 = (qt0 + it % per_head) * G_T;
          const int qrow = (int)(row_base + q0);
          const long long sidx = ((long long)b * p.Hq + h) * p.S + q0;
          mbar_expect_tx(q_full(s), G_TILE + G_STATS);
          tma_load_2d(sQ(s), &tmQ, h * G_D, qrow, q_full(s));
          tma_load_2d(sQ(s) + G_HALF, &tmQ, h * G_D + 64, qrow, q_full(s));
          bulk_g2s(sStats + s * G_STATS, p.lse2 + sidx, G_T * 4, q_full(s));
          bulk_g2s(sStats + s * G_STATS + G_T * 4, p.delta + sidx, G_T * 4, q_full(s));
          if (!mbar_wait(do_empty, (it & 1) ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          mbar_expect_tx(do_full, G_TILE);
          tma_load_2d(sdO, &tmdO, h * G_D, qrow, do_full);
          tma_load_2d(sdO + G_HALF, &tmdO, h * G_D + 64, qrow, do_full);
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer =====================
      if (lane == 0) {
        const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);   // S^T, dP^T: both operands K-major
        const uint32_t idesc_kn = make_idesc_bf16(128, 128, 0, 1);   // dV, dK: B (dO / Q) MN-major
        const uint32_t idesc_nn = make_idesc_bf16(128, 128, 1, 1);   // dQ: A (dS) and B (K) MN-major
        auto issue_kk = [&](uint32_t d_tmem, uint32_t a, uint32_t bm) {
#pragma unroll
          for (int k = 0; k < G_D / 16; ++k) {
            const uint32_t off = (k >> 2) * G_HALF + (k & 3) * 32;
            umma_bf16_ss(d_tmem, make_smem_desc_sw128(a + off, 16, 1024), make_smem_desc_sw128(bm + off, 16, 1024), idesc_kk, k != 0);
          }
        };
        bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
        if (ok && n_it > 0) ok = mbar_wait(q_full(0), 0, abort_flag, p.err, ERR_WAIT_ATTN);
        if (ok && n_it > 0) {
          tc_fence_after_sync();
          issue_kk(t_S, sK, sQ(0));
          umma_commit(s_full);
          ok = mbar_wait(do_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
          if (ok) {
            tc_fence_after_sync();
            issue_kk(t_dP, sV, sdO);
            umma_commit(dp_full);
          }
        }
        for (int it = 0; it < n_it && ok; ++it) {
          const int s = it & 1;
          if (!mbar_wait(p_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < G_T / 16; ++k)     // dV += P^T dO   (A from tensor memory)
            umma_bf16_ts(t_dV, t_S + 8u * k, make_smem_desc_sw128(sdO + k * 2048, G_HALF, 1024), idesc_kn, (it | k) != 0);
          umma_commit(do_empty);                   // dO of this tile has been read (dP^T earlier, dV now)
          const bool more = it + 1 < n_it;
          if (more) {                              // S^T of the next tile goes in behind dV
            if (!mbar_wait(q_full(s ^ 1), ((it + 1) >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
            tc_fence_after_sync();
            issue_kk(t_S, sK, sQ(s ^ 1));
            umma_commit(s_full);
          }
          if (!mbar_wait(ds_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < G_T / 16; ++k)     // dK += dS^T Q
            umma_bf16_ss(t_dK, make_smem_desc_sw128(sdS + (k >> 2) * G_HALF + (k & 3) * 32, 16, 1024),
                         make_smem_desc_sw128(sQ(s) + k * 2048, G_HALF, 1024), idesc_kn, (it | k) != 0);
          if (it > 0) {                            // dQ lands where the previous dQ was: wait for its read-out
            if (!mbar_wait(dq_empty, (it - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
            tc_fence_after_sync();
          }
#pragma unroll
          for (int k = 0; k < G_T / 16; ++k)     // dQ = dS K
            umma_bf16_ss(t_dP, make_smem_desc_sw128(sdS + k * 2048, G_HALF, 1024),
                         make_smem_desc_sw128(sK + k * 2048, G_HALF, 1024), idesc_nn, k != 0);
          umma_commit(dq_full);
          umma_commit(q_empty(s));
          if (more) {                              // dP^T of the next tile needs the dQ columns back
            if (!mbar_wait(dq_empty, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
            if (!mbar_wait(do_full, (it + 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
            tc_fence_after_sync();
            issue_kk(t_dP, sV, sdO);
            umma_commit(dp_full);
          }
        }
      }
    }
  } else if (warp < 8) {
    // ===================== compute warpgroup: one key row per thread =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int kv_i = k0 + r;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int q0 = (qt0 + it % per_head) * G_T;
      const bool need_mask = (p.causal && q0 < k0 + G_T - 1) || (q0 + G_T > p.S) || (k0 + G_T > p.S);
      // the statistics arrive with Q / dO on q_full
      if (!mbar_wait_warp(q_full(s), (it >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      if (!mbar_wait_warp(s_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t pk[64];
      const uint32_t st_addr = sStats + s * G_STATS;     // shared-window address of this stage's statistics
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        // 64 columns at a time: S^T from tensor memory and the 64 row statistics from shared memory are
        // all requested up front (explicit shared-space vector loads, issued back to back) so that
        // their latencies overlap instead of preceding every group of four exponentials
        uint32_t sv[64];
        tmem_ld_32x32b_x32(t_S + 64 * hh + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32b_x32(t_S + 64 * hh + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        float4 ls[16];
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4)
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(ls[c4].x), "=f"(ls[c4].y), "=f"(ls[c4].z), "=f"(ls[c4].w)
                       : "r"(st_addr + (64 * hh + 4 * c4) * 4));
        tmem_wait_ld();
        if (need_mask) {                         // diagonal / ragged tiles only: masked scores become -inf, exp2 gives 0
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int qi = q0 + 64 * hh + i;
            if (qi >= p.S || kv_i >= p.S || (p.causal && qi < kv_i)) sv[i] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[4 * c4 + 0]), p.scale_log2, -ls[c4].x));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[4 * c4 + 1]), p.scale_log2, -ls[c4].y));
          const float p2 = exp2f(fmaf(__uint_as_float(sv[4 * c4 + 2]), p.scale_log2, -ls[c4].z));
          const float p3 = exp2f(fmaf(__uint_as_float(sv[4 * c4 + 3]), p.scale_log2, -ls[c4].w));
          pk[32 * hh + 2 * c4] = pack_bf16x2(p0, p1);
          pk[32 * hh + 2 * c4 + 1] = pack_bf16x2(p2, p3);
        }
      }
      tmem_st_32x32b_x32(t_S + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st_32x32b_x32(t_S + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      // dS^T from the rounded P^T (the same values dV is multiplied with)
      if (!mbar_wait_warp(dp_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t dp[64];
        tmem_ld_32x32b_x32(t_dP + 64 * hh + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
        tmem_ld_32x32b_x32(t_dP + 64 * hh + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
        float4 dls[16];
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4)
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(dls[c4].x), "=f"(dls[c4].y), "=f"(dls[c4].z), "=f"(dls[c4].w)
                       : "r"(st_addr + (G_T + 64 * hh + 4 * c4) * 4));
        tmem_wait_ld();
        uint32_t dsk[32];
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 dl = dls[c4];
          const uint32_t pa = pk[32 * hh + 2 * c4], pb = pk[32 * hh + 2 * c4 + 1];
          const float d0 = __uint_as_float(pa << 16) * (__uint_as_float(dp[4 * c4 + 0]) - dl.x) * p.scale;
          const float d1 = __uint_as_float(pa & 0xffff0000u) * (__uint_as_float(dp[4 * c4 + 1]) - dl.y) * p.scale;
          const float d2 = __uint_as_float(pb << 16) * (__uint_as_float(dp[4 * c4 + 2]) - dl.z) * p.scale;
          const float d3 = __uint_as_float(pb & 0xffff0000u) * (__uint_as_float(dp[4 * c4 + 3]) - dl.w) * p.scale;
          dsk[2 * c4] = pack_bf16x2(d0, d1);
          dsk[2 * c4 + 1] = pack_bf16x2(d2, d3);
        }
        const uint32_t drow = sdS + hh * G_HALF + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t off = ((uint32_t)(c ^ (r & 7))) << 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(drow + off), "r"(dsk[4 * c]), "r"(dsk[4 * c + 1]),
                       "r"(dsk[4 * c + 2]), "r"(dsk[4 * c + 3]) : "memory");
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(ds_full);
    }
    // the last dq_full also covers the final dV / dK accumulations
    if (ok && n_it > 0) ok = mbar_wait_warp(dq_full, (n_it - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN);
    if (ok && n_it > 0) {
      tc_fence_after_sync();
      const bool row_ok = kv_i < p.S;
      __nv_bfloat16* dk_row = p.dk + (row_base + kv_i) * p.lddk + (long long)hkv * G_D;
      __nv_bfloat16* dv_row = p.dv + (row_base + kv_i) * p.lddv + (long long)hkv * G_D;
#pragma unroll
      for (int c = 0; c < G_D / 32; ++c) {
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
    }
    tc_fence_before_sync();
  } else {
    // ===================== dQ read-out warpgroup: one query row per thread =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const bool elected = warp == 8 && lane == 0;
    uint32_t units = 0;                        // staging tiles handed to the copy engine so far
    for (int it = 0; it < n_it; ++it) {
      const int h = hkv * group + it / per_head;
      const int q0 = (qt0 + it % per_head) * G_T;
      if (!mbar_wait_warp(dq_full, it & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
      tc_fence_after_sync();
      uint32_t dq[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_dP + 32 * c + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dq[32 * c]));
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(dq_empty);
      // Rows past the end of this sequence would land in the next sequence's rows: they add zeros.
      const bool row_ok = q0 + r < p.S;
      bool ok = true;
#pragma unroll
      for (int u = 0; u < 4; ++u) {            // four 32-column units of 128 bytes per row
        const uint32_t buf = sStg + (units & 1u) * G_DQ_STG;
        const uint32_t rowaddr = buf + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t addr = rowaddr + (((uint32_t)c ^ (uint32_t)(r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(row_ok ? dq[32 * u + 4 * c] : 0u),
                       "r"(row_ok ? dq[32 * u + 4 * c + 1] : 0u), "r"(row_ok ? dq[32 * u + 4 * c + 2] : 0u),
                       "r"(row_ok ? dq[32 * u + 4 * c + 3] : 0u) : "memory");
        }
        fence_proxy_async_smem();
        if (elected) tma_store_wait_read<0>();  // the previous unit's tile has been read: its buffer is free after the meeting point
        mbar_arrive(stg_bar);
        if (!mbar_wait_warp(stg_bar, units & 1u, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
        if (elected) {
          asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                       ::"l"(reinterpret_cast<uint64_t>(&tmDQ)), "r"(buf), "r"(h * G_D + 32 * u), "r"((int)(row_base + q0))
                       : "memory");
          tma_store_commit();
        }
        ++units;
      }
      if (!ok) break;
    }
    if (elected) tma_store_wait_all<0>();
    tc_fence_before_sync();
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
    tmem_dealloc(tmem_base, G_TMEM_COLS);
  }
}

// Launches the main kernel only; the caller has zeroed dq_accum and filled lse2 / delta.
int launch_flash_bwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                        float* dq_accum, void* dk, void* dv, const float* lse2, const float* delta, long long lddk, long long lddv,
                        int B, int S, int Hq, int Hkv, float scale, int causal, cudaStream_t st) {
  FlashBwdWsParams p;
  p.dq_accum = dq_accum;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.lse2 = lse2;
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
    MLF_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM));
    attr_set[dev & 63] = true;
  }
  // fp32 dQ accumulator as a 2-D tensor [tokens, Hq * 128]: tiles of 32 columns x 128 rows, 128B swizzle
  CUtensorMap tdq;
  {
    const int rc = make_tmap_2d(&tdq, dq_accum, 4, (uint64_t)Hq * G_D, (uint64_t)B * S, (uint64_t)Hq * G_D, 32, 128, true);
    if (rc) return rc;
  }
  dim3 grid(((S + G_T - 1) / G_T) * Hkv * B);
  flash_bwd_ws_kernel<<<grid, G_THREADS, G_SMEM, st>>>(tq, tk, tv, tdo, tdq, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mlf
