// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = alpha * A[M,K] * B[N,K]^T with fp32
// accumulation in TMEM and a fused epilogue.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: streams 128xBK A tiles and BNxBK B tiles into a ring of shared
//               memory stages (128-byte swizzle), one mbarrier pair (full/empty) per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               stage, commits the stage's "empty" barrier, and at the end of a tile commits the
//               accumulator's "full" barrier. It also owns TMEM allocation.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread), apply
//               bias / GELU / SwiGLU / residual / derivative factors, store bf16 or fp32.
//   Two accumulators (2*BN TMEM columns) let the epilogue of tile i overlap the main loop of
//   tile i+1.
//
// Operands may be K-major (the contraction index is contiguous in memory) or MN-major (the
// row/column index is contiguous), which covers forward (x*W^T), dgrad (dy*W) and wgrad
// (dy^T*x) without transposing anything in memory.
//
// Optional in-kernel communication (MlfGemmComm):
//   gather:  the first n_copy_ctas CTAs do not compute; they copy row chunks of one operand
//            from the peers' shards (plain peer loads over NVLink) into a local buffer and
//            publish per-chunk ready flags. The TMA producer of every compute CTA waits
//            (bounded) for the flags of the rows it is about to load. Tiles are visited in an
//            order that starts with the rows owned by this rank, so compute starts at once.
//            Copy CTAs have the lowest block indices, so they are resident before any CTA that
//            waits on them.
//   scatter: the epilogue routes each output row to the partial-sum buffer of the rank that
//            owns it (peer stores), visiting remote owners first.
//
// Reference behaviour covered: Tensor.Matmul (src/MLFramework/Tensor/TensorExtensions.cs:429),
// Linear.Forward (src/MLFramework/Modules/Linear.cs:81), TensorMathExtensions.MatMul with
// transposeA/transposeB (src/MLFramework/Layers/TensorParallel/TensorMathExtensions.cs:21),
// AllGatherOperation.AllGather (src/MLFramework/Distributed/FSDP/AllGatherOperation.cs:60) and
// RowParallelLinear's reduction (src/MLFramework/Layers/TensorParallel/RowParallelLinear.cs:154).
#include <unordered_map>
#include <mutex>

#include "gemm_common.cuh"

namespace mlf {

template <int BN>
struct GemmCfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;  // 512, 256, 128
  static constexpr int kSmemBytes = kStages * kStage + 1024 /*align*/ + 256 /*barriers*/;
};

// ------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmKernelParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;

  if ((int)blockIdx.x < p.n_copy_ctas) {
    gather_copy_role(p);
    return;
  }
  const int cta = blockIdx.x - p.n_copy_ctas;
  const int n_ctas = gridDim.x - p.n_copy_ctas;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * Cfg::kStage;
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem ptr, abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_al + kStages * Cfg::kStage + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, p.rot_m, p.rot_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        if (p.gather_operand != 0) {
          const int r0 = p.gather_operand == 1 ? m0 : n0;
          const int r1 = min(p.total_rows, r0 + (p.gather_operand == 1 ? BM : BN)) - 1;
          for (int c = r0 / p.flag_rows; c <= r1 / p.flag_rows && ok; ++c)
            ok = wait_flag_ge_gpu(&p.counters[c], (uint32_t)p.copy_group, abort_flag, p.err, ERR_WAIT_CHUNK_FLAG);
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + s * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
          mbar_expect_tx(full_bar(s), Cfg::kStage);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmA, k0, m0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmA, m0 + 64 * j, k0, full_bar(s));
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmB, k0, n0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmB, n0 + 64 * j, k0, full_bar(s));
          }
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      // K-major: 8-row groups 1024 B apart, K advance = 32 B inside the swizzle atom.
      // MN-major: 8-k-row groups 1024 B apart, 64-column blocks BK*128 B apart, K advance = 2048 B.
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, a_sbo = 1024, a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_lbo = p.b_mn ? BK * 128 : 16, b_sbo = 1024, b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, ERR_WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, a_sbo);
            const uint64_t bd = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, b_sbo);
            umma_bf16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool out_fp32 = (p.flags & MLF_EPI_OUT_FP32) != 0;
    const bool swiglu = (p.flags & MLF_EPI_SWIGLU) != 0;
    const bool dswiglu = (p.flags & MLF_EPI_DSWIGLU) != 0;
    int it = 0;
    for (int t = cta; t < num_tiles; t += n_ctas, ++it) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, p.rot_m, p.rot_n, tm, tn);
      const int m = tm * BM + q * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const bool row_ok = m < p.M;
      // output row pointer (possibly on a peer)
      char* out_row = nullptr;
      if (row_ok) {
        const int esz = out_fp32 ? 4 : 2;
        if (p.scatter_out) {
          const int owner = min(m / p.rows_per_owner, p.world - 1);
          const long long lr = (long long)p.rank * p.rows_per_owner + (m - owner * p.rows_per_owner);
          out_row = static_cast<char*>(p.out_peer[owner]) + lr * p.ldo * esz;
        } else {
          out_row = static_cast<char*>(p.out) + (long long)m * p.ldo * esz;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * BN + c * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_wait_ld();
        const int nb = n0 + c * 32;
        if (!row_ok || nb >= p.N) continue;
        gemm_epilogue_chunk(p, m, nb, r, out_row, out_fp32, swiglu, dswiglu);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  // ===================== teardown =====================
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // A wait expired somewhere in this CTA. Give copies and MMAs already in flight time to
    // land before shared memory and TMEM are released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct TmapKey {
  const void* base;
  uint64_t inner, outer, ld;
  uint32_t bi, bo;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && bi == o.bi && bo == o.bo;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1315423911u ^ k.inner;
    h = h * 1315423911u ^ k.outer;
    h = h * 1315423911u ^ k.ld;
    h = h * 1315423911u ^ ((uint64_t)k.bi << 32 | k.bo);
    return h;
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
static std::mutex g_tmap_mu;

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo) {
  TmapKey k{base, inner, outer, ld, bi, bo};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmaps.find(k);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return 0;
    }
  }
  int rc = make_tmap_2d(out, base, 2, inner, outer, ld, bi, bo, true);
  if (rc) return rc;
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  if (g_tmaps.size() > 8192) g_tmaps.clear();
  g_tmaps.emplace(k, *out);
  return 0;
}

template <int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmKernelParams& p,
                       int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  gemm_tcgen05_kernel<BN><<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(tmA, tmB, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mlf

using namespace mlf;

MLF_API int mlf_gemm_bf16_2cta(const MlfGemmArgs* a, uint64_t stream);

static int g_use_2cta = 1;
// Selects the CTA-pair kernel for large plain GEMMs (tile_n == 0). tile_n == 512 always selects it.
MLF_API void mlf_set_gemm_2cta(int on) { g_use_2cta = on; }
MLF_API int mlf_get_gemm_2cta() { return g_use_2cta; }
static int g_small_m_split = 1;
// Routes plain GEMMs with M <= 256 and a large weight to the split-K CTA-pair kernel.
MLF_API void mlf_set_gemm_small_m_split(int on) { g_small_m_split = on; }

MLF_API int mlf_gemm_fewrow(const void* x, const void* w, void* out, int M, int N, int K, long long ldx, long long ldw, long long ldo,
                            int accumulate, int max_ctas, uint64_t stream);
static int g_fewrow = 1;
// Routes plain products with at most 128 rows against a K-major weight to the weight-as-M stream-K kernel.
MLF_API void mlf_set_gemm_fewrow(int on) { g_fewrow = on; }

MLF_API int mlf_gemm_bf16(const MlfGemmArgs* a, uint64_t stream) {
  MLF_REQUIRE(a != nullptr, "null args");
  if (g_fewrow && a->tile_n == 0 && a->comm == nullptr && (a->flags & ~MLF_EPI_ACCUM) == 0 && !a->a_mn && !a->b_mn && a->M <= 128 &&
      a->N >= 1024 && a->K >= 512 && a->alpha == 1.0f) {
    const int rcf = mlf_gemm_fewrow(a->a, a->b, a->out, a->M, a->N, a->K, a->lda, a->ldb, a->ldo, (a->flags & MLF_EPI_ACCUM) ? 1 : 0,
                                    a->max_ctas, stream);
    if (rcf != -4) return rcf;
  }
  // CTA pairs for everything with at least 16 pair tiles (split-K fills the GPU when tiles alone cannot).
  // Few rows against a large weight (a decode step: M <= 256) is a weight-streaming problem: one row of
  // tiles cannot occupy the GPU, so the pair kernel splits K and every SM streams a slice of the weight.
  const bool plain_out = (a->flags & ~MLF_EPI_ACCUM) == 0 && a->comm == nullptr;
  const bool small_m = g_small_m_split && a->tile_n == 0 && plain_out && a->M <= 256 && a->N >= 1024 && a->K >= 1024;
  if (a->tile_n == 512 || small_m ||
      (g_use_2cta && a->tile_n == 0 && a->M >= 512 && a->N >= 512 && (long long)((a->M + 255) / 256) * ((a->N + 255) / 256) >= 16)) {
    const int rc2 = mlf_gemm_bf16_2cta(a, stream);
    if (rc2 != -4) return rc2;
  }
  MLF_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "bad GEMM shape %d %d %d", a->M, a->N, a->K);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const MlfGemmComm* cm = a->comm;
  const bool gatherA = cm && cm->gather_operand == 1;
  const bool gatherB = cm && cm->gather_operand == 2;

  int BN = a->tile_n;
  const int sms = a->max_ctas > 0 ? a->max_ctas : sm_count();
  if (BN == 0) {
    const long long tm = (a->M + BM - 1) / BM;
    if (tm * ((a->N + 255) / 256) >= sms || a->N >= 4096) BN = 256;
    else if (tm * ((a->N + 127) / 128) >= sms) BN = 128;
    else BN = 64;
    if ((a->flags & (MLF_EPI_SWIGLU)) && BN < 64) BN = 64;
  }
  if (BN == 512) BN = 256;
  MLF_REQUIRE(BN == 64 || BN == 128 || BN == 256, "tile_n must be 64, 128, 256 or 512 (CTA pair)");

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
  p.tiles_m = (a->M + BM - 1) / BM;
  p.tiles_n = (a->N + BN - 1) / BN;
  p.err = device_status_word();
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  if ((a->flags & MLF_EPI_BIAS)) MLF_REQUIRE(a->bias, "MLF_EPI_BIAS without bias");
  if ((a->flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL | MLF_EPI_DSWIGLU)))
    MLF_REQUIRE(a->aux_in, "epilogue needs aux_in");
  if ((a->flags & MLF_EPI_STORE_PRE)) MLF_REQUIRE(a->aux_out, "MLF_EPI_STORE_PRE without aux_out");

  const void* a_base = a->a;
  const void* b_base = a->b;
  int n_copy = 0;
  if (cm && !cm->gather_operand && cm->n_extra > 0) {
    MLF_REQUIRE(cm->n_copy_ctas >= 1 && cm->n_copy_ctas < sms, "n_copy_ctas out of range");
    p.n_copy_ctas = n_copy = cm->n_copy_ctas;
    p.copy_group = 1;
    p.extra_segs = cm->extra_segs;
    p.n_extra = cm->n_extra;
  }
  if (cm && cm->gather_operand) {
    MLF_REQUIRE(cm->world >= 1 && cm->world <= 8, "world %d out of range", cm->world);
    MLF_REQUIRE(cm->n_copy_ctas >= 1 && cm->n_copy_ctas < sms, "n_copy_ctas out of range");
    p.extra_segs = cm->extra_segs;
    p.n_extra = cm->n_extra;
    MLF_REQUIRE(cm->flag_rows > 0 && cm->flag_rows % (gatherA ? BM : BN) == 0,
                "flag_rows %d must be a multiple of the tile extent %d", cm->flag_rows, gatherA ? BM : BN);
    MLF_REQUIRE(cm->rows_per_rank % cm->flag_rows == 0, "rows_per_rank must be a multiple of flag_rows");
    MLF_REQUIRE(cm->row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
    MLF_REQUIRE(!(gatherA && a->a_mn) && !(gatherB && a->b_mn), "gathered operand must be K-major");
    p.gather_operand = cm->gather_operand;
    p.world = cm->world; p.rank = cm->rank;
    p.n_copy_ctas = n_copy = cm->n_copy_ctas;
    p.copy_group = copy_group_size(n_copy, (long long)cm->flag_rows * cm->row_bytes);
    p.rows_per_rank = cm->rows_per_rank; p.flag_rows = cm->flag_rows; p.row_bytes = cm->row_bytes;
    p.total_rows = gatherA ? a->M : a->N;
    for (int r = 0; r < 8; ++r) p.src[r] = cm->src[r];
    p.gathered = cm->gathered;
    p.flags_ready = cm->flags; p.counters = cm->counters;
    if (gatherA) { a_base = cm->gathered; p.rot_m = (cm->rank * cm->rows_per_rank) / BM; }
    else { b_base = cm->gathered; p.rot_n = (cm->rank * cm->rows_per_rank) / BN; }
    if (p.rot_m >= p.tiles_m) p.rot_m = 0;
    if (p.rot_n >= p.tiles_n) p.rot_n = 0;
  }
  if (cm && cm->scatter_out) {
    MLF_REQUIRE(cm->world >= 1 && cm->world <= 8, "world %d out of range", cm->world);
    MLF_REQUIRE(cm->rows_per_owner % BM == 0, "rows_per_owner must be a multiple of %d", BM);
    p.scatter_out = 1; p.rows_per_owner = cm->rows_per_owner;
    p.world = cm->world; p.rank = cm->rank;
    for (int r = 0; r < 8; ++r) p.out_peer[r] = cm->out_peer[r];
    // start with the rows of the next rank so remote traffic starts first
    p.rot_m = (((cm->rank + 1) % cm->world) * cm->rows_per_owner) / BM;
    if (p.rot_m >= p.tiles_m) p.rot_m = 0;
  }

  CUtensorMap tmA, tmB;
  int rc;
  if (!a->a_mn) rc = cached_tmap_bf16(&tmA, a_base, a->K, a->M, a->lda, BK, BM);
  else rc = cached_tmap_bf16(&tmA, a_base, a->M, a->K, a->lda, 64, BK);
  if (rc) return rc;
  if (!a->b_mn) rc = cached_tmap_bf16(&tmB, b_base, a->K, a->N, a->ldb, BK, BN);
  else rc = cached_tmap_bf16(&tmB, b_base, a->N, a->K, a->ldb, 64, BK);
  if (rc) return rc;

  const int num_tiles = p.tiles_m * p.tiles_n;
  int grid = num_tiles < (sms - n_copy) ? num_tiles : (sms - n_copy);
  grid += n_copy;
  if (BN == 256) return launch_gemm<256>(tmA, tmB, p, grid, st);
  if (BN == 128) return launch_gemm<128>(tmA, tmB, p, grid, st);
  return launch_gemm<64>(tmA, tmB, p, grid, st);
}
