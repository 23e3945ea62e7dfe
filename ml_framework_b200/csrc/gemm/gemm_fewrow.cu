// Few-row bf16 GEMM for decode steps: out[M, N] (+)= x[M, K] * W[N, K]^T with M <= 128 token rows.
//
// A decode step streams the whole weight once for a handful of rows, so the kernel is built around the weight
// stream, not around the rows:
//   * operands are swapped on the tensor core: 128 WEIGHT rows are the M dimension of tcgen05.mma and the token
//     rows are its N dimension (BT = 32, 64 or 128), so a 16 KB weight tile costs one M128 x N(BT) x K64 step
//     instead of a 128 x 256 one -- the tensor time per weight byte drops with the row count instead of being
//     fixed by a 128-row token tile that is mostly padding;
//   * the (weight tile, k block) grid is cut into equal contiguous runs, one per SM (stream-K): every SM streams
//     the same number of 16 KB weight tiles through an 8-deep (6 for BT = 128) TMA ring whatever N and K are;
//   * a run that covers part of a tile's K range adds its partial product into `out` with a TMA reduction store
//     (bf16 add at L2), so tiles shared by two SMs need no second pass. `out` is zeroed first unless the call
//     accumulates into it (residual stream).
// The accumulator tile comes out of tensor memory transposed (lane = weight row n, column = token m); the epilogue
// warps write it into 128B-swizzled staging tiles [BT token rows x 64 columns] from which the copy engine adds it
// into out[m, n0 .. n0 + 127]. Rows m >= M and columns n >= N are clipped by the tensor maps (zero-filled on load).
//
// Warp roles as in the other tcgen05 GEMMs: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2..5
// epilogue; two accumulators so that a run's epilogue overlaps the next run's products. Every wait is bounded.
//
// Reference behaviour covered: the per-token projections of the decode phase
// (src/MLFramework/Inference/PagedAttention/Phases/DecodeOrchestrator.cs:28-66 drives one token per sequence through
// the model's linear layers, Linear.Forward src/MLFramework/Modules/Linear.cs:81).
#include "gemm_common.cuh"

namespace mlf {

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo);

constexpr int FR_WT = 128;                         // weight rows per tile (MMA M)
constexpr int FR_STAGE_W = FR_WT * BK * 2;         // 16 KB

template <int BT>
struct FewRowCfg {
  static constexpr int kStageX = BT * BK * 2;
  static constexpr int kStage = FR_STAGE_W + kStageX;
  static constexpr int kStages = BT == 128 ? 5 : 8;
  static constexpr int kStgBox = BT * 128;         // staging box: BT token rows x 64 bf16 columns
  static constexpr int kTmemCols = BT == 32 ? 64 : 2 * BT;   // two accumulators, at least 32 columns each
  static constexpr int kSmemBytes = kStages * kStage + 2 * kStgBox + 1024 /*align*/ + 256 /*barriers*/;
};

struct FewRowParams {
  int M, N, K;
  int num_kb;            // k blocks per weight tile
  long long units;       // weight tiles x k blocks
  int* err;
};

__device__ __forceinline__ void fr_reduce_add_2d(const CUtensorMap* tm, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}

template <int BT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_fewrow_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const __grid_constant__ CUtensorMap tmOut, const FewRowParams p) {
  using Cfg = FewRowCfg<BT>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t stg_base = smem_base + kStages * Cfg::kStage;          // 1024-aligned: stages are multiples of 1 KB
  const uint32_t bar_base = stg_base + 2 * Cfg::kStgBox;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  const uint32_t epi_bar = bar_base + 8u * (2 * kStages + 4);            // meeting point of the four epilogue warps
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_al + (bar_base - smem_base) + 8 * (2 * kStages + 5));
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
      mbar_init(tempty_bar(a), 4);
    }
    mbar_init(epi_bar, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmOut);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  constexpr int kAccCols = BT < 32 ? 32 : BT;

  // this CTA's run of (tile, k block) units
  const long long u_begin = p.units * (long long)blockIdx.x / gridDim.x;
  const long long u_end = p.units * (long long)(blockIdx.x + 1) / gridDim.x;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (long long u = u_begin; u < u_end; ++u) {
        const int tile = (int)(u / p.num_kb);
        const int kb = (int)(u - (long long)tile * p.num_kb);
        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_SMEM_EMPTY)) break;
        const uint32_t sw = smem_base + s * Cfg::kStage;
        mbar_expect_tx(full_bar(s), Cfg::kStage);
        tma_load_2d(sw, &tmW, kb * BK, tile * FR_WT, full_bar(s));
        tma_load_2d(sw + FR_STAGE_W, &tmX, kb * BK, 0, full_bar(s));
        if (++s == kStages) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(FR_WT, BT, 0, 0);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (long long u = u_begin; u < u_end && ok; ++it) {
        const int tile = (int)(u / p.num_kb);
        const int kb0 = (int)(u - (long long)tile * p.num_kb);
        const long long seg_end = min(u_end, (long long)(tile + 1) * p.num_kb);
        const int n_kb = (int)(seg_end - u);
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int i = 0; i < n_kb; ++i) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, ERR_WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_base + s * Cfg::kStage;
          const uint32_t sx = sw + FR_STAGE_W;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sw + k * UMMA_K * 2, 16, 1024);
            const uint64_t bd = make_smem_desc_sw128(sx + k * UMMA_K * 2, 16, 1024);
            umma_bf16_ss(d_tmem, ad, bd, idesc, (i | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        (void)kb0;
        if (ok) umma_commit(tfull_bar(acc));
        u = seg_end;
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int n_loc = q * 32 + lane;              // weight row of this thread inside the tile
    const int half = n_loc >> 6;                  // staging box (64 output columns each)
    const int col = n_loc & 63;
    const bool elected = warp == 2 && lane == 0;
    int it = 0;
    uint32_t meets = 0;                             // uses of the meeting point (its phase parity)
    bool ok = true;
    // The four warps meet on an mbarrier with a bounded wait, not on a hardware barrier: should one warp give up
    // (a wait elsewhere in the CTA ran out), the others time out here too and unwind instead of waiting for ever.
    auto meet = [&]() -> bool {
      mbar_arrive(epi_bar);
      const bool good = mbar_wait_warp(epi_bar, meets & 1u, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      ++meets;
      return good;
    };
    for (long long u = u_begin; u < u_end && ok; ++it) {
      const int tile = (int)(u / p.num_kb);
      const long long seg_end = min(u_end, (long long)(tile + 1) * p.num_kb);
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait_warp(tfull_bar(acc), acc_ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      // the staging tiles are free once the previous run's reduction stores have read them
      if (elected) tma_store_wait_read<0>();
      if (!meet()) break;
      const uint32_t box = stg_base + half * Cfg::kStgBox;
      const uint32_t cb = (uint32_t)(col >> 3), ce = (uint32_t)(col & 7) * 2u;
#pragma unroll 1
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * kAccCols + c * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t m = (uint32_t)(c * 32 + j);
          const uint32_t addr = box + m * 128u + ((cb ^ (m & 7u)) << 4) + ce;
          const __nv_bfloat16 v = __float2bfloat16(__uint_as_float(r[j]));
          asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const uint16_t*>(&v)) : "memory");
        }
      }
      // the accumulator is free for the MMA warp as soon as it has been read
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      fence_proxy_async_smem();
      if (!meet()) break;
      if (elected) {
        fr_reduce_add_2d(&tmOut, stg_base, tile * FR_WT, 0);
        if (tile * FR_WT + 64 < p.N) fr_reduce_add_2d(&tmOut, stg_base + Cfg::kStgBox, tile * FR_WT + 64, 0);
        tma_store_commit();
      }
      u = seg_end;
    }
    if (elected) tma_store_wait_all<0>();
  }

  // ===================== teardown =====================
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BT>
static int launch_fewrow(const CUtensorMap& tmW, const CUtensorMap& tmX, const CUtensorMap& tmOut, const FewRowParams& p, int ctas,
                         cudaStream_t st) {
  using Cfg = FewRowCfg<BT>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(gemm_fewrow_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  gemm_fewrow_kernel<BT><<<ctas, kGemmThreads, Cfg::kSmemBytes, st>>>(tmW, tmX, tmOut, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mlf

using namespace mlf;

// Returns -4 when the shape or the alignment is not one this route handles (the caller falls back).
MLF_API int mlf_gemm_fewrow(const void* x, const void* w, void* out, int M, int N, int K, long long ldx, long long ldw, long long ldo,
                            int accumulate, int max_ctas, uint64_t stream) {
  if (M < 1 || M > 128 || N < 128 || K < 64) return -4;
  if (ldx % 8 || ldw % 8 || ldo % 8 || K % 8) return -4;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return -4;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int BT = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  FewRowParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_kb = (K + BK - 1) / BK;
  const int tiles = (N + FR_WT - 1) / FR_WT;
  p.units = (long long)tiles * p.num_kb;
  p.err = device_status_word();
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  CUtensorMap tmW, tmX, tmOut;
  int rc = cached_tmap_bf16(&tmW, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK, FR_WT);
  if (rc) return rc;
  rc = cached_tmap_bf16(&tmX, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, BK, (uint32_t)BT);
  if (rc) return rc;
  rc = cached_tmap_bf16(&tmOut, out, (uint64_t)N, (uint64_t)M, (uint64_t)ldo, 64, (uint32_t)BT);
  if (rc) return rc;
  int ctas = max_ctas > 0 ? max_ctas : sm_count();
  // a run shorter than 8 k blocks is all prologue and epilogue: use fewer SMs for small weights
  const long long max_useful = (p.units + 7) / 8;
  if (ctas > max_useful) ctas = (int)max_useful;
  if (ctas < 1) ctas = 1;
  if (!accumulate) MLF_CHECK_CUDA(cudaMemset2DAsync(out, (size_t)ldo * 2, 0, (size_t)N * 2, (size_t)M, st));
  if (BT == 32) return launch_fewrow<32>(tmW, tmX, tmOut, p, ctas, st);
  if (BT == 64) return launch_fewrow<64>(tmW, tmX, tmOut, p, ctas, st);
  return launch_fewrow<128>(tmW, tmX, tmOut, p, ctas, st);
}
