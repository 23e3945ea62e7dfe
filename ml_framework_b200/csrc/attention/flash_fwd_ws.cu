// Self-attention forward, head_dim 128: two 128-row query tiles per CTA, ping-ponged.
//
// One CTA = 256 query rows of one (batch, head) as two tiles of 128. 384 threads in three warpgroups;
// the control warpgroup hands most of its registers to the softmax warpgroups (setmaxnreg):
//   warp 0        TMA producer: both Q tiles once, then K and V tiles of 128 keys through 2-stage rings
//   warp 1        MMA issuer (one thread). Per key tile j and query tile t:
//                   S_t = Q_t K_j^T   (M128 N128 K128, operands in shared memory)  -> TMEM S_t
//                   O_t += P_t V_j    (M128 N128 K128, P read from TENSOR MEMORY, V from shared memory)
//                 issued in the order PV_0(j), S_0(j+1), PV_1(j), S_1(j+1) so that the tensor pipe
//                 works on one tile while the other tile's softmax runs
//   warps 4..7    softmax of tile 0: one query row per thread; reads S_0 from TMEM into registers,
//                 running max / sum in the log2 domain, writes P_0 as packed bf16 back over S_0
//   warps 8..11   softmax of tile 1
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each; P_t occupies the first 64
// columns of S_t. The MMAs of one thread execute in issue order, so S_t(j+1) overwrites P_t(j)
// only after PV_t(j) has read it. O is rescaled lazily: only when a row's maximum has grown by
// more than 2^8 since the value P and O are expressed against (then O_t is read, scaled and
// written back by its softmax warps, after PV_t(j-1) has completed).
// Per SM and key tile: 4 x 128x128x128 of tensor work against 2 x 16384 exponentials.
//
// Math reference: StandardPagedAttentionKernel.ComputePagedAttention
// (src/MLFramework/Inference/PagedAttention/Kernels/StandardPagedAttentionKernel.cs:21-84;
// causal rule :219-255).
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t bi, uint32_t bo);

constexpr int W_BQ = 128;                       // rows per query tile
constexpr int W_BKV = 128;
constexpr int W_D = 128;
constexpr int W_THREADS = 384;   // warps 0..3 control (TMA, MMA, two idle), 4..7 softmax of tile 0, 8..11 softmax of tile 1
constexpr int W_TILE_BYTES = 128 * 128 * 2;     // 32 KB: two 64-column blocks of 16 KB
constexpr int W_STAGES = 2;
constexpr int W_SMEM = 2 * W_TILE_BYTES + 2 * W_STAGES * W_TILE_BYTES + 256;
constexpr int W_TMEM_COLS = 512;

struct FlashWsParams {
  __nv_bfloat16* out;
  float* lse;
  long long ldo;
  int B, S, Hq, Hkv;           // S: query rows per sequence
  int Skv, qoff;               // key/value rows per sequence; query row i sits at position i + qoff (= Skv - S)
  int causal;
  float scale_log2;
  int* err;
  // paged keys / values: the K and V tensor maps then cover the KV cache as token rows
  // [num_blocks * 2 * 16, Hkv * 128] (K rows of block b start at row b * 32, V rows at b * 32 + 16) with a box of
  // 16 rows, and every 128-key tile is fetched page by page through this sequence's row of the block table
  const int* block_table;      // [B, max_blocks] physical block ids, or null for contiguous K / V
  int max_blocks, num_blocks;
};

constexpr int W_PAGE = 16;                      // tokens per KV-cache block on the paged path
constexpr int W_PAGE_BYTES = W_PAGE * 128;      // one page of one 64-column half: 16 rows of 128 bytes

__global__ void __launch_bounds__(W_THREADS, 1)
flash_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FlashWsParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase;                                  // 2 tiles
  const uint32_t sK = sQ + 2 * W_TILE_BYTES;                  // W_STAGES tiles
  const uint32_t sV = sK + W_STAGES * W_TILE_BYTES;           // W_STAGES tiles
  const uint32_t bars = sV + W_STAGES * W_TILE_BYTES;
  // barriers: q_full[2] k_full[2] v_full[2] k_empty[2] v_empty[2] s_full[2] p_full[2] pv_done[2]
  auto q_full = [&](int t) { return bars + 8u * t; };
  auto k_full = [&](int s) { return bars + 8u * (2 + s); };
  auto v_full = [&](int s) { return bars + 8u * (4 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (6 + s); };
  auto v_empty = [&](int s) { return bars + 8u * (8 + s); };
  auto s_full = [&](int t) { return bars + 8u * (10 + t); };
  auto p_full = [&](int t) { return bars + 8u * (12 + t); };
  auto pv_done = [&](int t) { return bars + 8u * (14 + t); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + (bars - sbase) + 8 * 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_pairs = (p.S + 2 * W_BQ - 1) / (2 * W_BQ);
  // 1-D grid ordered by work: all (batch, head) of the longest query pair first, the shortest last
  const int hb = p.Hq * p.B;
  const int pair = p.causal ? n_pairs - 1 - (int)blockIdx.x / hb : (int)blockIdx.x / hb;
  const int h = ((int)blockIdx.x % hb) % p.Hq;
  const int b = ((int)blockIdx.x % hb) / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = pair * 2 * W_BQ;
  const long long row_base = (long long)b * p.S;
  const long long kv_row_base = (long long)b * p.Skv;
  // key tiles each query tile needs
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qs = q0 + t * W_BQ;
    int n = (p.Skv + W_BKV - 1) / W_BKV;
    if (p.causal) n = min(n, (qs + p.qoff + W_BQ + W_BKV - 1) / W_BKV);
    n_t[t] = qs < p.S ? n : 0;
  }
  const int n_kv = max(n_t[0], n_t[1]);

  if ((sbase & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_INDEX);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full(i), 1);
      mbar_init(k_full(i), 1);
      mbar_init(v_full(i), 1);
      mbar_init(k_empty(i), 1);
      mbar_init(v_empty(i), 1);
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), 128);
      mbar_init(pv_done(i), 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), W_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  auto tS = [&](int t) { return tmem_base + 128u * t; };
  auto tO = [&](int t) { return tmem_base + 256u + 128u * t; };

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      for (int t = 0; t < 2; ++t) {
        mbar_expect_tx(q_full(t), W_TILE_BYTES);
        const int qrow = (int)(row_base + q0 + t * W_BQ);
        tma_load_2d(sQ + t * W_TILE_BYTES, &tmQ, h * W_D, qrow, q_full(t));
        tma_load_2d(sQ + t * W_TILE_BYTES + W_TILE_BYTES / 2, &tmQ, h * W_D + 64, qrow, q_full(t));
      }
      const int* bt = p.block_table ? p.block_table + (long long)b * p.max_blocks : nullptr;
      const int seq_pages = (p.Skv + W_PAGE - 1) / W_PAGE;
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int krow = (int)(kv_row_base + j * W_BKV);
        int blk[W_BKV / W_PAGE];
        if (bt) {
          // the eight table entries of this tile first (independent loads); pages past the end of the sequence
          // repeat its first page: their keys are masked, they only have to be readable
#pragma unroll
          for (int g = 0; g < W_BKV / W_PAGE; ++g) {
            const int pg = j * (W_BKV / W_PAGE) + g;
            blk[g] = bt[pg < seq_pages && pg < p.max_blocks ? pg : 0];
          }
#pragma unroll
          for (int g = 0; g < W_BKV / W_PAGE; ++g)
            if (blk[g] < 0 || blk[g] >= p.num_blocks) { atomicCAS(p.err, 0, ERR_BAD_INDEX); blk[g] = 0; }
        }
        if (!mbar_wait(k_empty(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(k_full(s), W_TILE_BYTES);
        if (bt) {
#pragma unroll
          for (int g = 0; g < W_BKV / W_PAGE; ++g) {
            const uint32_t dst = sK + s * W_TILE_BYTES + g * W_PAGE_BYTES;
            tma_load_2d(dst, &tmK, hkv * W_D, blk[g] * 2 * W_PAGE, k_full(s));
            tma_load_2d(dst + W_TILE_BYTES / 2, &tmK, hkv * W_D + 64, blk[g] * 2 * W_PAGE, k_full(s));
          }
        } else {
          tma_load_2d(sK + s * W_TILE_BYTES, &tmK, hkv * W_D, krow, k_full(s));
          tma_load_2d(sK + s * W_TILE_BYTES + W_TILE_BYTES / 2, &tmK, hkv * W_D + 64, krow, k_full(s));
        }
        if (!mbar_wait(v_empty(s), ph ^ 1u, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(v_full(s), W_TILE_BYTES);
        if (bt) {
#pragma unroll
          for (int g = 0; g < W_BKV / W_PAGE; ++g) {
            const uint32_t dst = sV + s * W_TILE_BYTES + g * W_PAGE_BYTES;
            tma_load_2d(dst, &tmV, hkv * W_D, (blk[g] * 2 + 1) * W_PAGE, v_full(s));
            tma_load_2d(dst + W_TILE_BYTES / 2, &tmV, hkv * W_D + 64, (blk[g] * 2 + 1) * W_PAGE, v_full(s));
          }
        } else {
          tma_load_2d(sV + s * W_TILE_BYTES, &tmV, hkv * W_D, krow, v_full(s));
          tma_load_2d(sV + s * W_TILE_BYTES + W_TILE_BYTES / 2, &tmV, hkv * W_D + 64, krow, v_full(s));
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, W_BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, W_D, 0, 1);
      auto issue_s = [&](int t, int j) {
        const uint32_t q = sQ + t * W_TILE_BYTES, k = sK + (j & 1) * W_TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < W_D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (W_TILE_BYTES / 2) + (kk & 3) * 32;
          umma_bf16_ss(tS(t), make_smem_desc_sw128(q + off, 16, 1024), make_smem_desc_sw128(k + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(s_full(t));
      };
      auto issue_pv = [&](int t, int j) {
        const uint32_t v = sV + (j & 1) * W_TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < W_BKV / 16; ++kk)
          umma_bf16_ts(tO(t), tS(t) + 8u * kk, make_smem_desc_sw128(v + kk * 2048, W_TILE_BYTES / 2, 1024), idesc_pv, (j | kk) != 0);
        umma_commit(pv_done(t));
      };
      bool ok = true;
      // prologue: S_0(0), S_1(0)
      if (n_kv > 0) {
        ok = mbar_wait(k_full(0), 0, abort_flag, p.err, ERR_WAIT_ATTN);
        for (int t = 0; t < 2 && ok; ++t) {
          if (n_t[t] == 0) continue;
          ok = mbar_wait(q_full(t), 0, abort_flag, p.err, ERR_WAIT_ATTN);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(t, 0);
        }
        if (ok) umma_commit(k_empty(0));          // K_0 consumed by both tiles' S
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        bool k_next_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < n_t[t]) {
            if (!mbar_wait(p_full(t), j & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
            if (!mbar_wait(v_full(s), ph, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
            tc_fence_after_sync();
            issue_pv(t, j);
          }
          if (j + 1 < n_t[t]) {
            if (!k_next_ready) {
              if (!mbar_wait(k_full((j + 1) & 1), ((j + 1) >> 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
              k_next_ready = true;
              tc_fence_after_sync();
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        umma_commit(v_empty(s));                               // V_j consumed by both tiles' PV
        if (j + 1 < n_kv) umma_commit(k_empty((j + 1) & 1));   // K_{j+1} consumed by both tiles' S
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ===================== softmax warpgroups =====================
    const int t = (warp - 4) >> 2;            // query tile of this warpgroup
    const int q = warp & 3;                   // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;
    const int qi = q0 + t * W_BQ + r;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int n_mine = n_t[t];
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait_warp(s_full(t), j & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = j * W_BKV;
      const bool need_mask = (p.causal && k0 + W_BKV - 1 > q0 + t * W_BQ + p.qoff) || (k0 + W_BKV > p.Skv);
      uint32_t sv[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(tS(t) + 32 * c + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sv[32 * c]));
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kj = k0 + i;
          if (kj >= p.Skv || (p.causal && kj > qi + p.qoff)) sv[i] = __float_as_uint(-INFINITY);
        }
      }
      if (j == 0) {
        // first tile: the reference maximum comes from a pass of its own
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          m0 = fmax3(m0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          m1 = fmax3(m1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
          m2 = fmax3(m2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
          m3 = fmax3(m3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
        }
        const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scale_log2;   // scale > 0: max commutes with the scaling
        m_used = mx == -INFINITY ? 0.f : mx;
      }
      // One fused pass: P = exp2(S * c - m_used) against the maximum the row is ALREADY expressed
      // against, while the tile's own maximum is computed on the side (the maximum runs on the
      // integer/compare pipe under the shadow of the exponentials). If some row's maximum has
      // grown by more than 2^8 the pass is repeated once after O, l and m_used have been brought
      // up to date; S is still in registers. Exponents stay below 2^8 in every accepted pass.
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t pk[64];
      float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float s0 = __uint_as_float(sv[2 * i]), s1 = __uint_as_float(sv[2 * i + 1]);
        if (i & 1) m1 = fmax3(m1, s0, s1); else m0 = fmax3(m0, s0, s1);
        const float p0 = exp2f(fmaf(s0, p.scale_log2, -m_used));
        const float p1 = exp2f(fmaf(s1, p.scale_log2, -m_used));
        rs0 += p0;
        rs1 += p1;
        pk[i] = pack_bf16x2(p0, p1);
      }
      const float mx = fmaxf(m0, m1) * p.scale_log2;
      const bool grow = j > 0 && mx > m_used + 8.f;
      if (__any_sync(0xffffffffu, grow)) {
        if (!mbar_wait_warp(pv_done(t), (j - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        const float f = grow ? exp2f(m_used - mx) : 1.f;
#pragma unroll
        for (int c = 0; c < W_D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tO(t) + c * 32 + lane_off, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st_32x32b_x32(tO(t) + c * 32 + lane_off, o);
        }
        l *= f;
        if (grow) m_used = mx;
        rs0 = 0.f;
        rs1 = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_used));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_used));
          rs0 += p0;
          rs1 += p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
      }
      tmem_st_32x32b_x32(tS(t) + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st_32x32b_x32(tS(t) + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      l += rs0 + rs1;
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(p_full(t));
    }
    if (ok && n_mine > 0) ok = mbar_wait_warp(pv_done(t), (n_mine - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN);
    if (ok && n_mine > 0) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qi < p.S;
      __nv_bfloat16* orow = p.out + (row_base + qi) * p.ldo + (long long)h * W_D;
#pragma unroll
      for (int c = 0; c < W_D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tO(t) + c * 32 + lane_off, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
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
    tmem_dealloc(tmem_base, W_TMEM_COLS);
  }
}

}  // namespace mlf

using namespace mlf;

// Queries [B * Sq rows] against keys / values [B * Skv rows], Skv >= Sq: query row i of a sequence sits at
// position i + (Skv - Sq), i.e. the queries are the LAST Sq positions (a prompt chunk attending to its cached
// prefix plus itself). Skv == Sq is plain self-attention.
MLF_API int mlf_flash_fwd_prefix(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Skv, int Hq,
                                 int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
                                 uint64_t stream) {
  const int S = Sq;
  MLF_REQUIRE(B > 0 && S > 0 && Skv >= Sq && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "flash_fwd: bad shape");
  MLF_REQUIRE(scale > 0.f, "flash_fwd: softmax scale must be positive");
  MLF_REQUIRE(ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "flash_fwd: out must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv;
  int rc;
  const uint64_t rows = (uint64_t)B * S, kv_rows = (uint64_t)B * Skv;
  if ((rc = cached_tmap_bf16(&tq, q, (uint64_t)Hq * W_D, rows, ldq, 64, W_BQ))) return rc;
  if ((rc = cached_tmap_bf16(&tk, k, (uint64_t)Hkv * W_D, kv_rows, ldk, 64, W_BKV))) return rc;
  if ((rc = cached_tmap_bf16(&tv, v, (uint64_t)Hkv * W_D, kv_rows, ldv, 64, W_BKV))) return rc;
  FlashWsParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.ldo = ldo;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.Skv = Skv; p.qoff = Skv - Sq;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  p.block_table = nullptr;
  p.max_blocks = p.num_blocks = 0;
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM));
    attr_set[dev & 63] = true;
  }
  dim3 grid(((S + 2 * W_BQ - 1) / (2 * W_BQ)) * Hq * B);
  flash_fwd_ws_kernel<<<grid, W_THREADS, W_SMEM, st>>>(tq, tk, tv, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Prefill attention whose keys and values are read straight out of the paged KV cache: queries [B * Sq rows] are the
// LAST Sq positions of sequences of Skv cached tokens each (the chunk's own K / V are already in the cache), and
// every 128-key tile is fetched page by page through the sequence's row of the block table by the kernel's TMA
// producer - no gather of the cached prefix into a contiguous buffer. cache: [num_blocks, 2, 16, Hkv, 128] bf16;
// block_table: int32 [B, max_blocks]. The reference walks the block table per token
// (src/MLFramework/Inference/PagedAttention/Layers/PagedAttentionLayer.cs:332-389, Phases/PrefillOrchestrator.cs:62-78).
MLF_API int mlf_flash_fwd_paged(const void* q, const void* cache, const int* block_table, void* out, float* lse, int B, int Sq, int Skv,
                                int Hq, int Hkv, long long ldq, long long ldo, int num_blocks, int block_size, int max_blocks, float scale,
                                int causal, uint64_t stream) {
  MLF_REQUIRE(B > 0 && Sq > 0 && Skv >= Sq && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "flash_fwd_paged: bad shape");
  MLF_REQUIRE(block_size == W_PAGE, "flash_fwd_paged: the block size must be %d tokens", W_PAGE);
  MLF_REQUIRE(block_table != nullptr && num_blocks > 0 && (long long)max_blocks * W_PAGE >= Skv,
              "flash_fwd_paged: %d table entries cannot describe %d tokens", max_blocks, Skv);
  MLF_REQUIRE(scale > 0.f, "flash_fwd_paged: softmax scale must be positive");
  MLF_REQUIRE(ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "flash_fwd_paged: out must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tq, tkv;
  int rc;
  if ((rc = cached_tmap_bf16(&tq, q, (uint64_t)Hq * W_D, (uint64_t)B * Sq, ldq, 64, W_BQ))) return rc;
  if ((rc = cached_tmap_bf16(&tkv, cache, (uint64_t)Hkv * W_D, (uint64_t)num_blocks * 2 * W_PAGE, (uint64_t)Hkv * W_D, 64, W_PAGE))) return rc;
  FlashWsParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.ldo = ldo;
  p.B = B; p.S = Sq; p.Hq = Hq; p.Hkv = Hkv;
  p.Skv = Skv; p.qoff = Skv - Sq;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_status_word();
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  MLF_REQUIRE(p.err != nullptr, "no device status word");
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM));
    attr_set[dev & 63] = true;
  }
  dim3 grid(((Sq + 2 * W_BQ - 1) / (2 * W_BQ)) * Hq * B);
  flash_fwd_ws_kernel<<<grid, W_THREADS, W_SMEM, st>>>(tq, tkv, tkv, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Same arguments as mlf_flash_fwd.
MLF_API int mlf_flash_fwd_ws(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq,
                             int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
                             uint64_t stream) {
  return mlf_flash_fwd_prefix(q, k, v, out, lse, B, S, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, causal, stream);
}
