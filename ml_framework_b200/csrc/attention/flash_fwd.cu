// Causal / full self-attention forward for head_dim 128 on tcgen05 tensor cores
// (FlashAttention-style online softmax; nothing of size S x S ever reaches HBM).
//
// One CTA = 128 query rows of one (batch, head); two CTAs share an SM so one CTA's softmax
// overlaps the other's tensor-core work. 192 threads:
//   warp 0      TMA producer: Q once, then K and V tiles of 64 keys through a 2-stage ring
//   warp 1      MMA issuer:   S = Q K^T (M128 N64 K128) into a double-buffered TMEM tile,
//                             PV = P V  (M128 N128 K64) into a second TMEM tile
//   warps 2..5  softmax: one query row per thread straight out of TMEM (no shuffles), running
//               max / sum in the log2 domain, P written as bf16 into 128B-swizzled shared memory
//               as the A operand of the PV product. The output accumulates in TMEM across key
//               tiles (PV issued with accumulate); it is only rescaled (TMEM load, multiply, TMEM
//               store) when a row's maximum has grown by more than 2^8 since the last rescale, so
//               the common iteration touches TMEM only to read S.
// Q/K/V are addressed through 2-D tensor maps over [tokens, features], so packed QKV
// buffers (row pitch 3*H*128) and GQA layouts need no copies. The same kernel serves training
// (contiguous sequences) and prefill; the paged variant lives in paged_attn.cu.
//
// Math reference: StandardPagedAttentionKernel.ComputePagedAttention
// (src/MLFramework/Inference/PagedAttention/Kernels/StandardPagedAttentionKernel.cs:21-84;
// causal rule :219-255: query i sees keys <= start + i).
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo);

constexpr int FA_BQ = 128;
constexpr int FA_BKV = 64;
constexpr int FA_D = 128;
constexpr int FA_THREADS = 192;
constexpr int FA_Q_BYTES = FA_BQ * FA_D * 2;         // 32 KB, two 64-column blocks of 16 KB
constexpr int FA_K_BYTES = FA_BKV * FA_D * 2;        // 16 KB, two blocks of 8 KB
constexpr int FA_V_BYTES = FA_K_BYTES;
constexpr int FA_P_BYTES = FA_BQ * FA_BKV * 2;       // 16 KB
constexpr int FA_STAGES = 2;
constexpr int FA_SMEM = FA_Q_BYTES + FA_STAGES * (FA_K_BYTES + FA_V_BYTES) + FA_P_BYTES + 128;
constexpr int FA_TMEM_COLS = 256;  // S0 (64) | S1 (64) | PV (128)

struct FlashFwdParams {
  __nv_bfloat16* out;   // [tokens, Hq*128] with pitch ldo
  float* lse;           // [B, Hq, S] natural-log logsumexp of the scaled scores
  long long ldo;
  int B, S, Hq, Hkv;
  int causal;
  float scale_log2;     // softmax scale * log2(e)
  int* err;
};

__global__ void __launch_bounds__(FA_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase;
  const uint32_t sKV = sQ + FA_Q_BYTES;
  const uint32_t sP = sKV + FA_STAGES * (FA_K_BYTES + FA_V_BYTES);
  const uint32_t bars = sP + FA_P_BYTES;
  // barriers: q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], p_full, pv_full  -> 11 x 8 B
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto v_full = [&](int s) { return bars + 8u * (3 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (5 + s); };
  auto s_full = [&](int b) { return bars + 8u * (7 + b); };
  const uint32_t p_full = bars + 8u * 9;
  const uint32_t pv_full = bars + 8u * 10;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + (bars - sbase) + 8 * 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_qt = (p.S + FA_BQ - 1) / FA_BQ;
  const int qt = n_qt - 1 - (int)blockIdx.x;  // longest rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qt * FA_BQ;
  const long long row_base = (long long)b * p.S;
  int n_kv = (p.S + FA_BKV - 1) / FA_BKV;
  if (p.causal) n_kv = min(n_kv, (q0 + FA_BQ + FA_BKV - 1) / FA_BKV);

  if ((sbase & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_INDEX);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
      mbar_init(s_full(s), 1);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tS = tmem_base;         // + 64 * buffer
  const uint32_t tPV = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FA_Q_BYTES);
      tma_load_2d(sQ, &tmQ, h * FA_D, (int)(row_base + q0), q_full);
      tma_load_2d(sQ + FA_Q_BYTES / 2, &tmQ, h * FA_D + 64, (int)(row_base + q0), q_full);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(kv_empty(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        const uint32_t sK = sKV + s * (FA_K_BYTES + FA_V_BYTES);
        const uint32_t sV = sK + FA_K_BYTES;
        const int krow = (int)(row_base + j * FA_BKV);
        mbar_expect_tx(k_full(s), FA_K_BYTES);
        tma_load_2d(sK, &tmK, hkv * FA_D, krow, k_full(s));
        tma_load_2d(sK + FA_K_BYTES / 2, &tmK, hkv * FA_D + 64, krow, k_full(s));
        mbar_expect_tx(v_full(s), FA_V_BYTES);
        tma_load_2d(sV, &tmV, hkv * FA_D, krow, v_full(s));
        tma_load_2d(sV + FA_V_BYTES / 2, &tmV, hkv * FA_D + 64, krow, v_full(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, FA_BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, FA_D, 0, 1);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(k_full(s), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) return false;
        tc_fence_after_sync();
        const uint32_t sK = sKV + s * (FA_K_BYTES + FA_V_BYTES);
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(sQ + (k >> 2) * (FA_Q_BYTES / 2) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sK + (k >> 2) * (FA_K_BYTES / 2) + (k & 3) * 32, 16, 1024);
          umma_bf16_ss(tS + 64 * (j & 1), ad, bd, idesc_s, k != 0);
        }
        umma_commit(s_full(j & 1));
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        if (!mbar_wait(v_full(s), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        tc_fence_after_sync();
        const uint32_t sV = sKV + s * (FA_K_BYTES + FA_V_BYTES) + FA_K_BYTES;
#pragma unroll
        for (int k = 0; k < FA_BKV / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(sP + k * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sV + k * 2048, FA_V_BYTES / 2, 1024);
          umma_bf16_ss(tPV, ad, bd, idesc_pv, (j | k) != 0);
        }
        umma_commit(pv_full);
        umma_commit(kv_empty(s));
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;         // row inside the tile
    const int qi = q0 + r;               // query position in the sequence
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m_used = 0.f;                  // the maximum P and O are currently expressed against
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_warp(s_full(j & 1), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = j * FA_BKV;
      const bool need_mask = (p.causal && k0 + FA_BKV - 1 > q0) || (k0 + FA_BKV > p.S);
      const uint32_t tSj = tS + 64 * (j & 1) + lane_off;
      // pass 1: row maximum of this tile
      float mx = -INFINITY;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tSj + 32 * hlf, t);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(t[i]);
          if (need_mask) {
            const int kj = k0 + 32 * hlf + i;
            if (kj >= p.S || (p.causal && kj > qi)) v = -INFINITY;
          }
          mx = fmaxf(mx, v * p.scale_log2);
        }
      }
      bool pv_waited = false;
      if (j == 0) {
        m_used = mx == -INFINITY ? 0.f : mx;
      } else {
        const bool grow = mx > m_used + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          // rescale the accumulator in TMEM; PV of the previous tile must have landed first
          if (!mbar_wait_warp(pv_full, (j - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
          pv_waited = true;
          tc_fence_after_sync();
          const float f = grow ? exp2f(m_used - mx) : 1.f;
#pragma unroll
          for (int c = 0; c < FA_D / 32; ++c) {
            uint32_t t[32];
            tmem_ld_32x32b_x32(tPV + c * 32 + lane_off, t);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * f);
            tmem_st_32x32b_x32(tPV + c * 32 + lane_off, t);
          }
          tmem_wait_st();
          l *= f;
          if (grow) m_used = mx;
        }
      }
      if (j > 0 && !pv_waited) {
        // P's shared-memory tile is still being read by the previous PV product until this fires
        if (!mbar_wait_warp(pv_full, (j - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      }
      // pass 2: P = exp2(S*c - m_used) as bf16 into 128B-swizzled shared memory
      float rs = 0.f;
      const uint32_t rowaddr = sP + r * 128;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tSj + 32 * hlf, t);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float v0 = __uint_as_float(t[2 * i]) * p.scale_log2 - m_used;
          float v1 = __uint_as_float(t[2 * i + 1]) * p.scale_log2 - m_used;
          if (need_mask) {
            const int kj = k0 + 32 * hlf + 2 * i;
            if (kj >= p.S || (p.causal && kj > qi)) v0 = -INFINITY;
            if (kj + 1 >= p.S || (p.causal && kj + 1 > qi)) v1 = -INFINITY;
          }
          const float p0 = exp2f(v0), p1 = exp2f(v1);
          rs += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t addr = rowaddr + (((4 * hlf + c) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                       "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                       : "memory");
        }
      }
      l += rs;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
    }
    if (ok && n_kv > 0) ok = mbar_wait_warp(pv_full, (n_kv - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN);
    if (ok) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qi < p.S;
      __nv_bfloat16* orow = p.out + (row_base + qi) * p.ldo + (long long)h * FA_D;
#pragma unroll
      for (int c = 0; c < FA_D / 32; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tPV + c * 32 + lane_off, t);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(t[8 * v + 0]) * inv, __uint_as_float(t[8 * v + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(t[8 * v + 2]) * inv, __uint_as_float(t[8 * v + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(t[8 * v + 4]) * inv, __uint_as_float(t[8 * v + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(t[8 * v + 6]) * inv, __uint_as_float(t[8 * v + 7]) * inv);
            reinterpret_cast<uint4*>(orow + 32 * c)[v] = w;
          }
        }
      }
      if (row_ok && p.lse) p.lse[((long long)b * p.Hq + h) * p.S + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
    }
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
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

}  // namespace mlf

using namespace mlf;

MLF_API int mlf_flash_fwd_ws(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq,
                             int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
                             uint64_t stream);

static int g_flash_ws = 1;
// 1 (default): sequences of at least 256 tokens use the two-tile ping-pong kernel; 0: always the single-tile kernel.
MLF_API void mlf_set_flash_ws(int on) { g_flash_ws = on; }

// q: [B*S, *] bf16 with Hq heads of 128 starting at q and row pitch ldq (elements); k, v likewise
// with Hkv heads. out: [B*S, Hq*128] pitch ldo. lse: fp32 [B, Hq, S] or null.
MLF_API int mlf_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq,
                          int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
                          uint64_t stream) {
  MLF_REQUIRE(B > 0 && S > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "flash_fwd: bad shape");
  MLF_REQUIRE(ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "flash_fwd: out must be 16-byte aligned");
  if (g_flash_ws && S >= 256 && scale > 0.f)
    return mlf_flash_fwd_ws(q, k, v, out, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, causal, stream);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv;
  int rc;
  const uint64_t rows = (uint64_t)B * S;
  if ((rc = cached_tmap_bf16(&tq, q, (uint64_t)Hq * FA_D, rows, ldq, 64, FA_BQ))) return rc;
  if ((rc = cached_tmap_bf16(&tk, k, (uint64_t)Hkv * FA_D, rows, ldk, 64, FA_BKV))) return rc;
  if ((rc = cached_tmap_bf16(&tv, v, (uint64_t)Hkv * FA_D, rows, ldv, 64, FA_BKV))) return rc;
  FlashFwdParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.ldo = ldo;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    attr_set[dev & 63] = true;
  }
  dim3 grid((S + FA_BQ - 1) / FA_BQ, Hq, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, st>>>(tq, tk, tv, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
