// bf16 GEMM with CTA-pair tensor-core instructions (tcgen05.mma.cta_group::2).
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 output tile: each CTA
// stages its own 128 rows of A and its own half (128 columns) of B, and one tcgen05.mma issued by
// the leader CTA drives both tensor cores, each reading the peer's half of B from the peer's
// shared memory. Per SM and per k-block that is 16 KB of A + 16 KB of B for 128 x 256 x 64 of
// math, instead of 16 KB + 32 KB in the single-CTA kernel: the L2 -> shared-memory traffic, which
// bounds the single-CTA kernel near 63 % tensor-pipe utilisation, drops by a third. No load is
// shared between CTAs through the copy engine: every CTA fetches exactly the bytes it owns.
//
// Synchronisation (all barriers live at the same shared-memory offsets in both CTAs):
//   full[s]   in the leader, count 1: the leader's producer arrives with the byte count of both
//             CTAs' loads; every load of the pair completes on that barrier (2-SM form of the TMA
//             load). A peer load may land before the leader's arrive of the same phase, never in
//             an earlier phase: the peer refills a stage only after the MMAs that read it are done.
//   empty[s]  in each CTA: the leader commits twice after the k-block's MMAs, once to its own and
//             once to the peer's barrier (address translated with mapa).
//   tfull[a]  in each CTA (same double commit), tempty[a] in the leader, count 8: the four
//             epilogue warps of each CTA arrive (the peer's through a cluster-scope arrive).
// Every wait is bounded; a cluster barrier at the end keeps either CTA from exiting while the
// other may still touch its shared memory.
#include <cooperative_groups.h>

#include "gemm_common.cuh"

namespace mlf {

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo);

constexpr int T2_BN = 256;                       // tile columns (both CTAs)
constexpr int T2_BNH = 128;                      // columns of B staged per CTA
constexpr int T2_STAGE_A = BM * BK * 2;          // 16 KB
constexpr int T2_STAGE_B = T2_BNH * BK * 2;      // 16 KB
constexpr int T2_STAGE = T2_STAGE_A + T2_STAGE_B;
constexpr int T2_STAGES = 6;
constexpr int T2_STG_BYTES = 128 * 64 * 2;     // epilogue staging: 128 rows x 64 bf16 columns, 128B-swizzled
constexpr int T2_SMEM = T2_STAGES * T2_STAGE + 1024 /*barriers*/ + 2 * T2_STG_BYTES + 1024 /*align*/;
constexpr int T2_TMEM_COLS = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-SM TMA tile load: data lands in this CTA's shared memory, completion bytes are counted on the
// barrier at `bar_cluster_addr`, which may belong to the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* tm, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at a cluster address once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Output tensor maps of the row owners when the epilogue routes rows to peers (GEMM -> reduce-scatter).
struct alignas(64) PeerMaps {
  CUtensorMap m[8];
};

// TMA reduction store: global[tile] += shared[tile], element type taken from the tensor map (bf16).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tm, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmPre,
                         const __grid_constant__ CUtensorMap tmAux, const __grid_constant__ PeerMaps peer_maps,
                         const GemmKernelParams p, const int tma_epilogue, const int tma_aux, const int k_splits,
                         const int reduce_out) {
  // Copy CTAs come in whole clusters (their count is even) and never touch the cluster barrier.
  if ((int)blockIdx.x < p.n_copy_ctas) {
    gather_copy_role(p);
    return;
  }
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + T2_STAGES * T2_STAGE;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (T2_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * T2_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * T2_STAGES + 2 + a); };
  const uint32_t epi_bar = bar_base + 8u * (2 * T2_STAGES + 4);      // the four epilogue warps meet here (128 arrivals)
  const uint32_t aux_bar = bar_base + 8u * (2 * T2_STAGES + 5);      // aux_in tile landed in the staging buffer
  const uint32_t stg_base = bar_base + 1024u;                        // two staging buffers
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_al + T2_STAGES * T2_STAGE + 8 * (2 * T2_STAGES + 6));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();     // 0 = leader
  const uint32_t peer = rank ^ 1u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    mbar_init(epi_bar, 128);
    mbar_init(aux_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_ptr_smem), T2_TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                          // both CTAs' barriers are initialised before any remote arrive
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int pair = ((int)blockIdx.x - p.n_copy_ctas) >> 1;
  const int n_pairs = ((int)gridDim.x - p.n_copy_ctas) >> 1;
  // Work items: (tile, k-split). Splits of one tile are consecutive items, their partial products meet in
  // global memory through TMA reduction stores (the host cleared or kept `out` accordingly).
  const int num_tiles = p.tiles_m * p.tiles_n * k_splits;   // tiles of 256 x 256, times splits
  const int num_kb_all = (p.K + BK - 1) / BK;
  const int kb_per = (num_kb_all + k_splits - 1) / k_splits;

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int t = pair; t < num_tiles; t += n_pairs) {
        int tm, tn;
        tile_coords(t / k_splits, p.tiles_m, p.tiles_n, p.rot_m, p.rot_n, tm, tn);
        const int kb0 = (t % k_splits) * kb_per, kb1 = min(num_kb_all, kb0 + kb_per);
        if (kb0 >= kb1) continue;
        const int m0 = tm * 256 + (int)rank * BM;
        const int n0 = tn * T2_BN + (int)rank * T2_BNH;
        bool ok = true;
        if (p.gather_operand != 0) {
          // this CTA's 128 rows of the gathered operand must have landed
          const int r0 = p.gather_operand == 1 ? m0 : n0;
          const int r1 = min(p.total_rows, r0 + 128) - 1;
          for (int c = r0 / p.flag_rows; c <= r1 / p.flag_rows && ok; ++c)
            ok = wait_flag_ge_gpu(&p.counters[c], (uint32_t)p.copy_group, abort_flag, p.err, ERR_WAIT_CHUNK_FLAG);
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_SMEM_EMPTY)) { ok = false; break; }
          const uint32_t sa = smem_base + s * T2_STAGE;
          const uint32_t sb = sa + T2_STAGE_A;
          const uint32_t lead_full = mapa_u32(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * T2_STAGE);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmA, k0, m0, lead_full);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, m0 + 64 * j, k0, lead_full);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmB, k0, n0, lead_full);
          } else {
#pragma unroll
            for (int j = 0; j < T2_BNH / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmB, n0 + 64 * j, k0, lead_full);
          }
          if (++s == T2_STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA only) =====================
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_bf16(256, T2_BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_lbo = p.b_mn ? BK * 128 : 16, b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += n_pairs) {
        const int kb0 = (t % k_splits) * kb_per, kb1 = min(num_kb_all, kb0 + kb_per);
        if (kb0 >= kb1) continue;
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * T2_BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * T2_STAGE;
          const uint32_t sb = sa + T2_STAGE_A;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_bf16_ss_pair(d_tmem, ad, bd, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(mapa_u32(empty_bar(s), 0));
          umma_commit_pair(mapa_u32(empty_bar(s), 1));
          if (++s == T2_STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          umma_commit_pair(mapa_u32(tfull_bar(acc), 0));
          umma_commit_pair(mapa_u32(tfull_bar(acc), 1));
        }
        ++it;
      }
    }
  } else {
    // ===================== epilogue (warps 2..5 of both CTAs) =====================
    const int q = warp & 3;
    const bool out_fp32 = (p.flags & MLF_EPI_OUT_FP32) != 0;
    const bool swiglu = (p.flags & MLF_EPI_SWIGLU) != 0;
    const bool dswiglu = (p.flags & MLF_EPI_DSWIGLU) != 0;
    uint32_t epi_units = 0;
    int it = 0;
    for (int t = pair; t < num_tiles; t += n_pairs) {
      if ((t % k_splits) * kb_per >= min(num_kb_all, (t % k_splits) * kb_per + kb_per)) continue;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      int tm, tn;
      tile_coords(t / k_splits, p.tiles_m, p.tiles_n, p.rot_m, p.rot_n, tm, tn);
      const int m = tm * 256 + (int)rank * BM + q * 32 + lane;
      const int n0 = tn * T2_BN;
      if (!mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const bool row_ok = m < p.M;
      char* out_row = nullptr;
      if (row_ok) {
        const int esz = out_fp32 ? 4 : 2;
        if (p.scatter_out) {               // rows routed to their owner's partial buffer (possibly on a peer)
          const int owner = min(m / p.rows_per_owner, p.world - 1);
          const long long lr = (long long)p.rank * p.rows_per_owner + (m - owner * p.rows_per_owner);
          out_row = static_cast<char*>(p.out_peer[owner]) + lr * p.ldo * esz;
        } else {
          out_row = static_cast<char*>(p.out) + (long long)m * p.ldo * esz;
        }
      }
      if (tma_epilogue) {
        // Outputs leave through shared memory and TMA stores: each thread writes its row's 64
        // columns (128 bytes) into a swizzled staging tile, the four warps meet, one thread hands
        // the tile to the copy engine. Two staging tiles alternate; the elected thread makes sure
        // the previous store has finished reading before the meeting point that releases its tile.
        const int r = q * 32 + lane;
        const bool elected = warp == 2 && lane == 0;
        const int m_tile = tm * 256 + (int)rank * BM;
        bool ok = true;
        // aux_in (residual / dGELU input) comes in through the same staging tile, fetched by the copy
        // engine one unit ahead: unit u's tile may be overwritten once the store of unit u-2 has
        // finished reading, which the meeting point of unit u-1 guarantees.
        auto prefetch_aux = [&](uint32_t unit, int x, int y) {
          mbar_expect_tx(aux_bar, T2_STG_BYTES);
          tma_load_2d(stg_base + (unit & 1u) * T2_STG_BYTES, &tmAux, x, y, aux_bar);
        };
        if (tma_aux && elected && epi_units == 0) prefetch_aux(0, n0, m_tile);
        auto emit = [&](const float (&v)[64], const CUtensorMap* tmap, int x) -> bool {
          const uint32_t buf = stg_base + (epi_units & 1u) * T2_STG_BYTES;
          const uint32_t rowaddr = buf + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t addr = rowaddr + (((uint32_t)c ^ (uint32_t)(r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(v[8 * c], v[8 * c + 1])),
                         "r"(pack_bf16x2(v[8 * c + 2], v[8 * c + 3])), "r"(pack_bf16x2(v[8 * c + 4], v[8 * c + 5])),
                         "r"(pack_bf16x2(v[8 * c + 6], v[8 * c + 7])) : "memory");
          }
          fence_proxy_async_smem();
          if (elected) tma_store_wait_read<0>();
          mbar_arrive(epi_bar);
          if (!mbar_wait_warp(epi_bar, epi_units & 1u, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) return false;
          if (elected) {
            if (p.scatter_out) {                 // the whole 128-row block belongs to one owner (possibly a peer)
              const int owner = min(m_tile / p.rows_per_owner, p.world - 1);
              tma_store_2d(&peer_maps.m[owner], buf, x, p.rank * p.rows_per_owner + (m_tile - owner * p.rows_per_owner));
            } else if (reduce_out) {
              tma_reduce_add_2d(tmap, buf, x, m_tile);
            } else {
              tma_store_2d(tmap, buf, x, m_tile);
            }
            tma_store_commit();
            if (tma_aux) {                       // next unit: next column group of this tile, or the first of the next tile
              int nx = x + 64, ny = m_tile;
              bool have = nx < n0 + T2_BN && nx < p.N;
              if (!have && t + n_pairs < num_tiles) {
                int tm2, tn2;
                tile_coords((t + n_pairs) / k_splits, p.tiles_m, p.tiles_n, p.rot_m, p.rot_n, tm2, tn2);
                nx = tn2 * T2_BN;
                ny = tm2 * 256 + (int)rank * BM;
                have = true;
              }
              if (have) prefetch_aux(epi_units + 1, nx, ny);
            }
          }
          ++epi_units;
          return true;
        };
#pragma unroll 1
        for (int g = 0; g < T2_BN / 64 && ok; ++g) {
          const int nb = n0 + 64 * g;
          if (nb >= p.N) break;
          float v[64];
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            uint32_t t32[32];
            tmem_ld_32x32b_x32(tmem_base + acc * T2_BN + g * 64 + h2 * 32 + ((uint32_t)(q * 32) << 16), t32);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[32 * h2 + j] = __uint_as_float(t32[j]) * p.alpha;
          }
          const int nvalid = min(64, p.N - nb);
          if (p.flags & MLF_EPI_BIAS) {
            if (nvalid == 64 && ((reinterpret_cast<uintptr_t>(p.bias + nb) & 15) == 0)) {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(p.bias + nb) + c);
                const float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z), f3 = unpack_bf16x2(w.w);
                v[8 * c + 0] += f0.x; v[8 * c + 1] += f0.y; v[8 * c + 2] += f1.x; v[8 * c + 3] += f1.y;
                v[8 * c + 4] += f2.x; v[8 * c + 5] += f2.y; v[8 * c + 6] += f3.x; v[8 * c + 7] += f3.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (j < nvalid) v[j] += __bfloat162float(p.bias[nb + j]);
            }
          }
          if (p.flags & MLF_EPI_STORE_PRE) {
            ok = emit(v, &tmPre, nb);
            if (!ok) break;
          }
          if (p.flags & MLF_EPI_GELU) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = gelu_tanh(v[j]);
          }
          if (p.flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL)) {
            const bool resid = (p.flags & MLF_EPI_RESIDUAL) != 0;
            const __nv_bfloat16* ar = p.aux_in + (long long)m * p.ld_aux_in + nb;
            if (tma_aux) {
              if (!mbar_wait_warp(aux_bar, epi_units & 1u, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
              const uint32_t rowaddr = stg_base + (epi_units & 1u) * T2_STG_BYTES + r * 128;
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                uint4 w;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                             : "r"(rowaddr + (((uint32_t)c ^ (uint32_t)(r & 7)) << 4)));
                const float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z), f3 = unpack_bf16x2(w.w);
                const float a8[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[8 * c + j] = resid ? v[8 * c + j] + a8[j] : v[8 * c + j] * dgelu_tanh(a8[j]);
              }
            } else if (row_ok && nvalid == 64 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0)) {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const uint4 w = reinterpret_cast<const uint4*>(ar)[c];
                const float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z), f3 = unpack_bf16x2(w.w);
                const float a8[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[8 * c + j] = resid ? v[8 * c + j] + a8[j] : v[8 * c + j] * dgelu_tanh(a8[j]);
              }
            } else if (row_ok) {
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                const float a1 = j < nvalid ? __bfloat162float(ar[j]) : 0.f;
                v[j] = resid ? v[j] + a1 : v[j] * dgelu_tanh(a1);
              }
            }
          }
          ok = emit(v, &tmOut, nb);
        }
        if (!ok) break;
      } else {
#pragma unroll 1
      for (int c = 0; c < T2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * T2_BN + c * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_wait_ld();
        const int nb = n0 + c * 32;
        if (!row_ok || nb >= p.N) continue;
        gemm_epilogue_chunk(p, m, nb, r, out_row, out_fp32, swiglu, dswiglu);
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
      ++it;
    }
    if (tma_epilogue && warp == 2 && lane == 0) tma_store_wait_all<0>();   // shared memory stays valid until the copies have read it
  }

  // ===================== teardown =====================
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();                          // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, T2_TMEM_COLS);
  }
}

}  // namespace mlf

using namespace mlf;

// GEMM on CTA pairs, with the same in-kernel communication options as the single-CTA kernel (copy
// CTAs that gather an operand or prefetch extra segments; an epilogue that routes rows to their
// owners). Same arguments as mlf_gemm_bf16; returns -4 without launching when the problem is not a
// fit (the caller then uses the single-CTA kernel).
MLF_API int mlf_gemm_bf16_2cta(const MlfGemmArgs* a, uint64_t stream) {
  MLF_REQUIRE(a != nullptr, "null args");
  const MlfGemmComm* cm = a->comm;
  // fewer than 256 rows only as a plain product (optionally accumulated), where K is split over the pairs
  if (a->N < 256 || (a->M < 256 && ((a->flags & ~MLF_EPI_ACCUM) != 0 || cm != nullptr))) return -4;
  const bool gatherA = cm && cm->gather_operand == 1;
  const bool gatherB = cm && cm->gather_operand == 2;
  if (cm && cm->gather_operand && (cm->flag_rows <= 0 || cm->flag_rows % 128 != 0)) return -4;
  if (cm && cm->scatter_out && cm->rows_per_owner % 128 != 0) return -4;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  GemmKernelParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_mn = a->a_mn ? 1 : 0; p.b_mn = a->b_mn ? 1 : 0;
  p.flags = a->flags; p.alpha = a->alpha;
  p.out = a->out;
  p.bias = static_cast<const __nv_bfloat16*>(a->bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a->aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(a->aux_out);
  p.ldo = a->ldo; p.ld_aux_in = a->ld_aux_in; p.ld_aux_out = a->ld_aux_out;
  p.tiles_m = (a->M + 255) / 256;
  p.tiles_n = (a->N + T2_BN - 1) / T2_BN;
  p.err = device_status_word();
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  if ((a->flags & MLF_EPI_BIAS)) MLF_REQUIRE(a->bias, "MLF_EPI_BIAS without bias");
  if ((a->flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL | MLF_EPI_DSWIGLU))) MLF_REQUIRE(a->aux_in, "epilogue needs aux_in");
  if ((a->flags & MLF_EPI_STORE_PRE)) MLF_REQUIRE(a->aux_out, "MLF_EPI_STORE_PRE without aux_out");
  const int sms_all = a->max_ctas > 0 ? a->max_ctas : sm_count();
  const void* a_base = a->a;
  const void* b_base = a->b;
  int n_copy = 0;
  if (cm && (cm->gather_operand || cm->n_extra > 0)) {
    MLF_REQUIRE(cm->n_copy_ctas >= 1 && cm->n_copy_ctas + 2 < sms_all, "n_copy_ctas out of range");
    n_copy = (cm->n_copy_ctas + 1) & ~1;          // whole clusters
    p.n_copy_ctas = n_copy;
    p.copy_group = 1;
    p.extra_segs = cm->extra_segs;
    p.n_extra = cm->n_extra;
  }
  if (cm && cm->gather_operand) {
    MLF_REQUIRE(cm->world >= 1 && cm->world <= 8, "world %d out of range", cm->world);
    MLF_REQUIRE(cm->rows_per_rank % cm->flag_rows == 0, "rows_per_rank must be a multiple of flag_rows");
    MLF_REQUIRE(cm->row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
    MLF_REQUIRE(!(gatherA && a->a_mn) && !(gatherB && a->b_mn), "gathered operand must be K-major");
    p.gather_operand = cm->gather_operand;
    p.world = cm->world; p.rank = cm->rank;
    p.rows_per_rank = cm->rows_per_rank; p.flag_rows = cm->flag_rows; p.row_bytes = cm->row_bytes;
    p.copy_group = copy_group_size(n_copy, (long long)cm->flag_rows * cm->row_bytes);
    p.total_rows = gatherA ? a->M : a->N;
    for (int r = 0; r < 8; ++r) p.src[r] = cm->src[r];
    p.gathered = cm->gathered;
    p.flags_ready = cm->flags; p.counters = cm->counters;
    // start with the tiles whose rows are already local
    if (gatherA) { a_base = cm->gathered; p.rot_m = (cm->rank * cm->rows_per_rank) / 256; }
    else { b_base = cm->gathered; p.rot_n = (cm->rank * cm->rows_per_rank) / T2_BN; }
    if (p.rot_m >= p.tiles_m) p.rot_m = 0;
    if (p.rot_n >= p.tiles_n) p.rot_n = 0;
  }
  if (cm && cm->scatter_out) {
    MLF_REQUIRE(cm->world >= 1 && cm->world <= 8, "world %d out of range", cm->world);
    p.scatter_out = 1; p.rows_per_owner = cm->rows_per_owner;
    p.world = cm->world; p.rank = cm->rank;
    for (int r = 0; r < 8; ++r) p.out_peer[r] = cm->out_peer[r];
    p.rot_m = (((cm->rank + 1) % cm->world) * cm->rows_per_owner) / 256;   // remote traffic starts first
    if (p.rot_m >= p.tiles_m) p.rot_m = 0;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (!a->a_mn) rc = cached_tmap_bf16(&tmA, a_base, a->K, a->M, a->lda, BK, BM);
  else rc = cached_tmap_bf16(&tmA, a_base, a->M, a->K, a->lda, 64, BK);
  if (rc) return rc;
  if (!a->b_mn) rc = cached_tmap_bf16(&tmB, b_base, a->K, a->N, a->ldb, BK, T2_BNH);
  else rc = cached_tmap_bf16(&tmB, b_base, a->N, a->K, a->ldb, 64, BK);
  if (rc) return rc;
  // Outputs go through TMA stores when they are plain bf16 rows this GPU owns.
  CUtensorMap tmOut = tmA, tmPre = tmA, tmAux = tmA;
  PeerMaps peer_maps;                        // only read by the kernel when rows are routed
  memset(&peer_maps, 0, sizeof(peer_maps));
  int tma_epi = 0, tma_aux = 0;
  const bool scatter = cm && cm->scatter_out;
  const bool plain = (a->flags & ~MLF_EPI_ACCUM) == 0 && cm == nullptr;      // nothing but (optionally) out += product
  if (!(a->flags & (MLF_EPI_OUT_FP32 | MLF_EPI_SWIGLU | MLF_EPI_DSWIGLU)) && (!(a->flags & MLF_EPI_ACCUM) || plain) && a->ldo % 8 == 0 &&
      (scatter || (reinterpret_cast<uintptr_t>(a->out) & 15) == 0) &&
      (!(a->flags & MLF_EPI_STORE_PRE) || (a->ld_aux_out % 8 == 0 && (reinterpret_cast<uintptr_t>(a->aux_out) & 15) == 0))) {
    if (scatter) {
      for (int r = 0; r < cm->world; ++r) {
        MLF_REQUIRE((reinterpret_cast<uintptr_t>(cm->out_peer[r]) & 15) == 0, "partial buffers must be 16-byte aligned");
        rc = cached_tmap_bf16(&peer_maps.m[r], cm->out_peer[r], a->N, (uint64_t)cm->world * cm->rows_per_owner, a->ldo, 64, 128);
        if (rc) return rc;
      }
    } else {
      rc = cached_tmap_bf16(&tmOut, a->out, a->N, a->M, a->ldo, 64, 128);
      if (rc) return rc;
    }
    if (a->flags & MLF_EPI_STORE_PRE) {
      rc = cached_tmap_bf16(&tmPre, a->aux_out, a->N, a->M, a->ld_aux_out, 64, 128);
      if (rc) return rc;
    }
    tma_epi = 1;
    if ((a->flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL)) && !(a->flags & MLF_EPI_STORE_PRE) && a->ld_aux_in % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(a->aux_in) & 15) == 0) {
      rc = cached_tmap_bf16(&tmAux, a->aux_in, a->N, a->M, a->ld_aux_in, 64, 128);
      if (rc) return rc;
      tma_aux = 1;
    }
  }
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM));
    attr_set[dev & 63] = true;
  }
  const int sms = sms_all - n_copy;
  const int num_tiles = p.tiles_m * p.tiles_n;
  static int max_clusters[64] = {0};
  if (!max_clusters[dev & 63]) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = T2_SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_2cta_kernel, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
    max_clusters[dev & 63] = n;
  }
  int pairs = sms / 2;
  if (pairs > max_clusters[dev & 63]) pairs = max_clusters[dev & 63];
  if (pairs > num_tiles) pairs = num_tiles;
  if (pairs < 1) pairs = 1;
  // Split K when the tiles alone cannot fill the GPU (weight gradients of narrow layers: few tiles, long K).
  // Splits add their partial products into `out` with TMA reduction stores.
  int k_splits = 1;
  if (plain && tma_epi) {
    const int kb_all = (a->K + BK - 1) / BK;
    int avail = sms / 2;
    if (avail > max_clusters[dev & 63]) avail = max_clusters[dev & 63];
    double best = (double)((num_tiles + avail - 1) / avail);
    for (int ks = 2; ks <= 8; ++ks) {
      if (kb_all / ks < 8) break;
      const double cost = (double)((num_tiles * ks + avail - 1) / avail) / ks;
      if (cost < best * 0.9) { best = cost; k_splits = ks; }
    }
  }
  const int reduce_out = (k_splits > 1 || (a->flags & MLF_EPI_ACCUM)) ? 1 : 0;
  if (k_splits > 1 && !(a->flags & MLF_EPI_ACCUM))
    MLF_CHECK_CUDA(cudaMemset2DAsync(a->out, (size_t)a->ldo * 2, 0, (size_t)a->N * 2, (size_t)a->M, st));
  pairs = sms / 2;
  if (pairs > max_clusters[dev & 63]) pairs = max_clusters[dev & 63];
  if (pairs > num_tiles * k_splits) pairs = num_tiles * k_splits;
  if (pairs < 1) pairs = 1;
  gemm_tcgen05_2cta_kernel<<<n_copy + 2 * pairs, kGemmThreads, T2_SMEM, st>>>(tmA, tmB, tmOut, tmPre, tmAux, peer_maps, p, tma_epi, tma_aux,
                                                                              k_splits, reduce_out);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
