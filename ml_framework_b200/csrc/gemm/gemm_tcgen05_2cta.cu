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
constexpr int T2_SMEM = T2_STAGES * T2_STAGE + 1024 + 256;
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmKernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + T2_STAGES * T2_STAGE;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (T2_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * T2_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * T2_STAGES + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_al + T2_STAGES * T2_STAGE + 8 * (2 * T2_STAGES + 4));
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

  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;   // tiles of 256 x 256
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int t = pair; t < num_tiles; t += n_pairs) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, 0, 0, tm, tn);
        const int m0 = tm * 256 + (int)rank * BM;
        const int n0 = tn * T2_BN + (int)rank * T2_BNH;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
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
      for (int t = pair; t < num_tiles && ok; t += n_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * T2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * T2_STAGE;
          const uint32_t sb = sa + T2_STAGE_A;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_bf16_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(mapa_u32(empty_bar(s), 0));
          umma_commit_pair(mapa_u32(empty_bar(s), 1));
          if (++s == T2_STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          umma_commit_pair(mapa_u32(tfull_bar(acc), 0));
          umma_commit_pair(mapa_u32(tfull_bar(acc), 1));
        }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5 of both CTAs) =====================
    const int q = warp & 3;
    const bool out_fp32 = (p.flags & MLF_EPI_OUT_FP32) != 0;
    const bool swiglu = (p.flags & MLF_EPI_SWIGLU) != 0;
    const bool dswiglu = (p.flags & MLF_EPI_DSWIGLU) != 0;
    int it = 0;
    for (int t = pair; t < num_tiles; t += n_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, 0, 0, tm, tn);
      const int m = tm * 256 + (int)rank * BM + q * 32 + lane;
      const int n0 = tn * T2_BN;
      if (!mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const bool row_ok = m < p.M;
      char* out_row = row_ok ? static_cast<char*>(p.out) + (long long)m * p.ldo * (out_fp32 ? 4 : 2) : nullptr;
#pragma unroll 1
      for (int c = 0; c < T2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * T2_BN + c * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_wait_ld();
        const int nb = n0 + c * 32;
        if (!row_ok || nb >= p.N) continue;
        gemm_epilogue_chunk(p, m, nb, r, out_row, out_fp32, swiglu, dswiglu);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
    }
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

// Plain GEMM (no in-kernel communication) on CTA pairs. Same arguments as mlf_gemm_bf16; returns
// -4 without launching when the problem is not a fit (caller then uses the single-CTA kernel).
MLF_API int mlf_gemm_bf16_2cta(const MlfGemmArgs* a, uint64_t stream) {
  MLF_REQUIRE(a != nullptr, "null args");
  if (a->comm != nullptr || a->M < 256 || a->N < 256) return -4;
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
  CUtensorMap tmA, tmB;
  int rc;
  if (!a->a_mn) rc = cached_tmap_bf16(&tmA, a->a, a->K, a->M, a->lda, BK, BM);
  else rc = cached_tmap_bf16(&tmA, a->a, a->M, a->K, a->lda, 64, BK);
  if (rc) return rc;
  if (!a->b_mn) rc = cached_tmap_bf16(&tmB, a->b, a->K, a->N, a->ldb, BK, T2_BNH);
  else rc = cached_tmap_bf16(&tmB, a->b, a->N, a->K, a->ldb, 64, BK);
  if (rc) return rc;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM));
    attr_set[dev & 63] = true;
  }
  const int sms = a->max_ctas > 0 ? a->max_ctas : sm_count();
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
  gemm_tcgen05_2cta_kernel<<<2 * pairs, kGemmThreads, T2_SMEM, st>>>(tmA, tmB, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
