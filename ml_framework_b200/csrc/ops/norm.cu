// LayerNorm and RMSNorm, forward and backward, bf16 activations with fp32 statistics.
//
// One warp owns one row at a time and keeps it in registers as packed bf16 (NV 16-byte
// vectors per lane), so x is read from HBM exactly once per pass. The backward pass adds the
// per-row contributions to gamma/beta gradients into a per-CTA shared-memory accumulator with
// shared atomics and writes one partial per CTA; a second tiny kernel sums the partials. The wide
// model dimensions (2048 and 4096) use a backward kernel with whole-CTA rows instead.
//
// The reference has no norm kernels (its AMP rules only name layernorm as an fp32 op,
// src/MLFramework/Amp/DefaultAmpRules.cs:48-110); these are required by the GPT and Llama
// model families.
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// D = NV * 256. rms != 0 selects RMSNorm (no mean subtraction, no beta).
template <int NV>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, float eps, int rms) {
  constexpr int D = NV * 256;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_cta) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
    uint4 xv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) xv[i] = xr[i * 32 + lane];
    float s = 0.f;
    if (!rms) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float f[8];
        unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += f[j];
      }
      s = warp_sum(s) * (1.f / D);
    }
    const float mean = rms ? 0.f : s;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = f[j] - mean;
        ss += d * d;
      }
    }
    const float rstd = rsqrtf(warp_sum(ss) * (1.f / D) + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(gamma);
    const uint4* br = reinterpret_cast<const uint4*>(beta);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8], g[8], b[8];
      unpack8(xv[i], f);
      unpack8(gr[i * 32 + lane], g);
      if (beta) unpack8(br[i * 32 + lane], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * g[j] + (beta ? b[j] : 0.f);
      yr[i * 32 + lane] = pack8(f);
    }
  }
}

// Forward for D = NVT * 2048 with whole-CTA rows: 256 threads own 8 * NVT fixed columns each (gamma / beta in
// registers), R rows are loaded together, and the row sums meet across the eight warps through shared memory.
// Few rows (a decode step: 64 x 4096) then still occupy one CTA per row group instead of one warp per row.
template <int NVT, int R>
__global__ void __launch_bounds__(256, 3)
norm_fwd_cta_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                    const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                    float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, float eps, int rms) {
  constexpr int D = NVT * 2048;
  __shared__ float red[2][2][8][R];          // [iteration parity][sum | centred squares][warp][row]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float g[NVT][8], bt[NVT][8];
#pragma unroll
  for (int v = 0; v < NVT; ++v) {
    unpack8(reinterpret_cast<const uint4*>(gamma)[v * 256 + tid], g[v]);
    if (beta) unpack8(reinterpret_cast<const uint4*>(beta)[v * 256 + tid], bt[v]);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) bt[v][j] = 0.f;
    }
  }
  const float inv_d = 1.f / D;
  int par = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, par ^= 1) {
    uint4 xv[R][NVT];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long base = (long long)(row0 + r < rows ? row0 + r : row0) * (D / 8);
#pragma unroll
      for (int v = 0; v < NVT; ++v) xv[r][v] = reinterpret_cast<const uint4*>(x)[base + v * 256 + tid];
    }
    float mean[R];
    if (!rms) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float sm = 0.f;
#pragma unroll
        for (int v = 0; v < NVT; ++v) {
          float f[8];
          unpack8(xv[r][v], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) sm += f[j];
        }
        sm = warp_sum(sm);
        if (lane == 0) red[par][0][warp][r] = sm;
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[par][0][w][r];
        mean[r] = t * inv_d;
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) mean[r] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < NVT; ++v) {
        float f[8];
        unpack8(xv[r][v], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = f[j] - mean[r];
          ss = fmaf(d, d, ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[par][1][warp][r] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) break;
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[par][1][w][r];
      const float rstd = rsqrtf(t * inv_d + eps);
      if (tid == 0) {
        if (mean_out) mean_out[row0 + r] = mean[r];
        if (rstd_out) rstd_out[row0 + r] = rstd;
      }
#pragma unroll
      for (int v = 0; v < NVT; ++v) {
        float f[8];
        unpack8(xv[r][v], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = fmaf((f[j] - mean[r]) * rstd, g[v][j], bt[v][j]);
        reinterpret_cast<uint4*>(y)[(long long)(row0 + r) * (D / 8) + v * 256 + tid] = pack8(f);
      }
    }
  }
}

// Backward. Each warp walks rows with a grid stride. Gamma / beta gradient contributions are kept
// per lane in registers when they fit (MODE 0: D <= 2048, row cached in registers too; MODE 1:
// RMSNorm up to D = 5120, row re-read from L1/L2 for the second pass) and only folded into a
// per-CTA shared-memory accumulator once per kernel. MODE 2 (everything else) adds every row's
// contribution to shared memory directly.
template <int NV, int MODE>
__global__ void __launch_bounds__(256)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ partials /* [grid, 2, D] */, int rows, int rms,
                const __nv_bfloat16* __restrict__ dx_add /* optional: added to dx (gradient of a skip connection) */) {
  constexpr int D = NV * 256;
  constexpr int NK = MODE == 0 ? NV : 1;          // cached row vectors
  constexpr int NG = MODE <= 1 ? NV : 1;          // register dgamma partials
  constexpr int NB = MODE == 0 ? NV : 1;          // register dbeta partials
  extern __shared__ float acc[];  // [2][D]
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  float dg[NG][8], db[NB][8];
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[i][j] = 0.f;
#pragma unroll
  for (int i = 0; i < NB; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) db[i][j] = 0.f;
  for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_cta) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + (long long)row * D);
    uint4 xv[NK], dv[NK];
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < NK; ++i) {
        xv[i] = xr[i * 32 + lane];
        dv[i] = dr[i * 32 + lane];
      }
    }
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8], d[8], g[8];
      unpack8(MODE == 0 ? xv[MODE == 0 ? i : 0] : xr[i * 32 + lane], f);
      unpack8(MODE == 0 ? dv[MODE == 0 ? i : 0] : dr[i * 32 + lane], d);
      unpack8(gr[i * 32 + lane], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (f[j] - mean) * rstd;
        const float dxh = d[j] * g[j];
        c1 += dxh;
        c2 += dxh * xh;
        if (MODE <= 1) dg[MODE <= 1 ? i : 0][j] += d[j] * xh;
        if (MODE == 0) db[MODE == 0 ? i : 0][j] += d[j];
      }
    }
    c1 = rms ? 0.f : warp_sum(c1) * (1.f / D);
    c2 = warp_sum(c2) * (1.f / D);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (long long)row * D);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[8], d[8], g[8], o[8];
      unpack8(MODE == 0 ? xv[MODE == 0 ? i : 0] : xr[i * 32 + lane], f);
      unpack8(MODE == 0 ? dv[MODE == 0 ? i : 0] : dr[i * 32 + lane], d);
      unpack8(gr[i * 32 + lane], g);
      const int col = (i * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (f[j] - mean) * rstd;
        o[j] = rstd * (d[j] * g[j] - c1 - xh * c2);
        if (MODE == 2) {
          atomicAdd(&acc[col + j], d[j] * xh);
          if (!rms) atomicAdd(&acc[D + col + j], d[j]);
        }
        if (MODE == 1 && !rms) atomicAdd(&acc[D + col + j], d[j]);
      }
      if (dx_add) {
        float e[8];
        unpack8(reinterpret_cast<const uint4*>(dx_add + (long long)row * D)[i * 32 + lane], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += e[j];
      }
      dxr[i * 32 + lane] = pack8(o);
    }
  }
  if (MODE <= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&acc[col + j], dg[MODE <= 1 ? i : 0][j]);
        if (MODE == 0 && !rms) atomicAdd(&acc[D + col + j], db[MODE == 0 ? i : 0][j]);
      }
    }
  }
  __syncthreads();
  float* po = partials + (long long)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) po[i] = acc[i];
}

// Backward for D = NVT * 2048 (the model widths 2048 and 4096): a CTA of 256 threads owns
// R rows at a time and every thread a fixed set of 8 * NVT columns, so gamma sits in registers as
// fp32, the gamma / beta gradient partials need only 16 * NVT registers, and R rows of x and dy
// (R * 12 KB per CTA at D = 2048) are in flight per CTA while several CTAs share an SM. The two row
// sums meet across the eight warps through a double-buffered shared array: one barrier per R rows.
template <int NVT, int R>
__global__ void __launch_bounds__(256, 2)
norm_bwd_cta_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                    const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                    const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                    float* __restrict__ partials /* [grid, 2, D] */, int rows, int rms,
                    const __nv_bfloat16* __restrict__ dx_add /* optional: added to dx */) {
  constexpr int D = NVT * 2048;
  __shared__ float red[2][8][2 * R];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float g[NVT][8], dg[NVT][8], db[NVT][8];
#pragma unroll
  for (int v = 0; v < NVT; ++v) {
    unpack8(reinterpret_cast<const uint4*>(gamma)[v * 256 + tid], g[v]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[v][j] = db[v][j] = 0.f;
  }
  const float inv_d = 1.f / D;
  int buf = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, buf ^= 1) {
    uint4 xv[R][NVT], dv[R][NVT], ev[R][NVT];
    float mean[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool ok = row0 + r < rows;
      const long long base = (long long)(ok ? row0 + r : row0) * (D / 8);
#pragma unroll
      for (int v = 0; v < NVT; ++v) {
        xv[r][v] = reinterpret_cast<const uint4*>(x)[base + v * 256 + tid];
        dv[r][v] = ok ? reinterpret_cast<const uint4*>(dy)[base + v * 256 + tid] : make_uint4(0, 0, 0, 0);
        ev[r][v] = dx_add ? reinterpret_cast<const uint4*>(dx_add)[base + v * 256 + tid] : make_uint4(0, 0, 0, 0);
      }
      mean[r] = rms ? 0.f : mean_in[ok ? row0 + r : row0];
      rstd[r] = rstd_in[ok ? row0 + r : row0];
    }
    float c[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float c1 = 0.f, c2 = 0.f;
      const float nm = -mean[r] * rstd[r];
#pragma unroll
      for (int v = 0; v < NVT; ++v) {
        float f[8], d[8];
        unpack8(xv[r][v], f);
        unpack8(dv[r][v], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = fmaf(f[j], rstd[r], nm);
          const float dxh = d[j] * g[v][j];
          c1 += dxh;
          c2 = fmaf(dxh, xh, c2);
          dg[v][j] = fmaf(d[j], xh, dg[v][j]);
          db[v][j] += d[j];
        }
      }
      c[2 * r] = warp_sum(c1);
      c[2 * r + 1] = warp_sum(c2);
    }
    if (lane < 2 * R) {
      float mine = c[0];
#pragma unroll
      for (int k = 1; k < 2 * R; ++k) mine = lane == k ? c[k] : mine;
      red[buf][warp][lane] = mine;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[buf][w][k];
      c[k] = t * inv_d;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) break;
      const float c1 = rms ? 0.f : c[2 * r], c2 = c[2 * r + 1];
      const float nm = -mean[r] * rstd[r];
#pragma unroll
      for (int v = 0; v < NVT; ++v) {
        float f[8], d[8], e[8], o[8];
        unpack8(xv[r][v], f);
        unpack8(dv[r][v], d);
        unpack8(ev[r][v], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = fmaf(f[j], rstd[r], nm);
          o[j] = fmaf(rstd[r], fmaf(d[j], g[v][j], -c1) - xh * c2, e[j]);
        }
        reinterpret_cast<uint4*>(dx)[(long long)(row0 + r) * (D / 8) + v * 256 + tid] = pack8(o);
      }
    }
  }
  float* po = partials + (long long)blockIdx.x * 2 * D;
#pragma unroll
  for (int v = 0; v < NVT; ++v) {
    float4* pg = reinterpret_cast<float4*>(po + (v * 256 + tid) * 8);
    float4* pb = reinterpret_cast<float4*>(po + D + (v * 256 + tid) * 8);
    pg[0] = make_float4(dg[v][0], dg[v][1], dg[v][2], dg[v][3]);
    pg[1] = make_float4(dg[v][4], dg[v][5], dg[v][6], dg[v][7]);
    pb[0] = make_float4(db[v][0], db[v][1], db[v][2], db[v][3]);
    pb[1] = make_float4(db[v][4], db[v][5], db[v][6], db[v][7]);
  }
}

// dgamma[c] = sum_g partials[g][0][c]; dbeta likewise. 32 columns x 32 partial-lanes per CTA (a few hundred
// partial rows: the kernel is pure load latency, so the rows are spread over 32 warps).
constexpr int NF_WARPS = 32;
__global__ void __launch_bounds__(NF_WARPS * 32)
norm_bwd_finalize_kernel(const float* __restrict__ partials, int nparts, int D, void* dgamma, void* dbeta,
                         int out_fp32, int accumulate) {
  __shared__ float sg[NF_WARPS][33], sb[NF_WARPS][33];
  const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float g = 0.f, b = 0.f;
  if (c < D) {
#pragma unroll 4
    for (int p = pl; p < nparts; p += NF_WARPS) {
      g += partials[(long long)p * 2 * D + c];
      if (dbeta) b += partials[(long long)p * 2 * D + D + c];
    }
  }
  sg[pl][cl] = g;
  sb[pl][cl] = b;
  __syncthreads();
  if (pl != 0 || c >= D) return;
#pragma unroll
  for (int k = 1; k < NF_WARPS; ++k) { g += sg[k][cl]; b += sb[k][cl]; }
  if (out_fp32) {
    float* dgp = static_cast<float*>(dgamma);
    dgp[c] = g + (accumulate ? dgp[c] : 0.f);
    if (dbeta) {
      float* dbp = static_cast<float*>(dbeta);
      dbp[c] = b + (accumulate ? dbp[c] : 0.f);
    }
  } else {
    __nv_bfloat16* dgp = static_cast<__nv_bfloat16*>(dgamma);
    dgp[c] = __float2bfloat16(g + (accumulate ? __bfloat162float(dgp[c]) : 0.f));
    if (dbeta) {
      __nv_bfloat16* dbp = static_cast<__nv_bfloat16*>(dbeta);
      dbp[c] = __float2bfloat16(b + (accumulate ? __bfloat162float(dbp[c]) : 0.f));
    }
  }
}

template <int NV>
static int launch_fwd(const void* x, const void* g, const void* b, void* y, float* mean, float* rstd, int rows,
                      float eps, int rms, cudaStream_t st) {
  const int grid = min((rows + 7) / 8, sm_count() * 8);
  norm_fwd_kernel<NV><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g),
                                            static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), mean,
                                            rstd, rows, eps, rms);
                                            count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <int NV>
static int launch_bwd(const void* x, const void* dy, const void* g, const float* mean, const float* rstd, void* dx,
                      float* partials, int grid, int rows, int rms, const void* dx_add, cudaStream_t st) {
  constexpr int smem = 2 * NV * 256 * 4;
  constexpr int MODE = NV <= 8 ? 0 : (NV <= 20 ? 1 : 2);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && !attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(norm_bwd_kernel<NV, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev & 63] = true;
  }
  norm_bwd_kernel<NV, MODE><<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x),
                                               static_cast<const __nv_bfloat16*>(dy),
                                               static_cast<const __nv_bfloat16*>(g), mean, rstd,
                                               static_cast<__nv_bfloat16*>(dx), partials, rows, rms,
                                               static_cast<const __nv_bfloat16*>(dx_add));
                                               count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mlf

using namespace mlf;

#define MLF_NORM_DISPATCH(NVVAL, CALL)                      \
  switch (NVVAL) {                                          \
    case 1: return CALL(1); case 2: return CALL(2); case 3: return CALL(3); case 4: return CALL(4); \
    case 6: return CALL(6); case 8: return CALL(8); case 12: return CALL(12); case 16: return CALL(16); \
    case 20: return CALL(20); case 24: return CALL(24); case 32: return CALL(32);                   \
    default: break;                                         \
  }

// y = norm(x) * gamma (+ beta). D must be a multiple of 256 from {256..1024, 1536, 2048, 3072,
// 4096, 5120, 6144, 8192}. mean/rstd (fp32 [rows]) may be null for inference.
MLF_API int mlf_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                         int rows, int D, float eps, int rms, uint64_t stream) {
  MLF_REQUIRE(D % 256 == 0, "norm: D=%d must be a multiple of 256", D);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 2048 || D == 4096) {
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gamma);
    const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(beta);
    __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
    const int cap = 4 * sm_count();
    if (D == 2048) {
      const int r = rows >= 4 * cap ? 4 : (rows >= 2 * cap ? 2 : 1);      // few rows: one row per CTA, more CTAs
      const int grid = min((rows + r - 1) / r, cap);
      if (r == 4) norm_fwd_cta_kernel<1, 4><<<grid, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, eps, rms);
      else if (r == 2) norm_fwd_cta_kernel<1, 2><<<grid, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, eps, rms);
      else norm_fwd_cta_kernel<1, 1><<<grid, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, eps, rms);
    } else {
      const int r = rows >= 2 * cap ? 2 : 1;
      const int grid = min((rows + r - 1) / r, cap);
      if (r == 2) norm_fwd_cta_kernel<2, 2><<<grid, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, eps, rms);
      else norm_fwd_cta_kernel<2, 1><<<grid, 256, 0, st>>>(xp, gp, bp, yp, mean, rstd, rows, eps, rms);
    }
    count_launch();
    MLF_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
#define CALL(NV) launch_fwd<NV>(x, gamma, beta, y, mean, rstd, rows, eps, rms, st)
  MLF_NORM_DISPATCH(D / 256, CALL)
#undef CALL
  set_error("norm: unsupported D=%d", D);
  return -2;
}

// CTAs of the backward kernel: whole-CTA rows for the wide model dimensions, warp rows otherwise.
static int norm_bwd_grid(int rows, int D, bool* cta_rows) {
  const bool wide = D == 2048 || D == 4096;
  if (cta_rows) *cta_rows = wide;
  if (wide) {
    const int r = D == 2048 ? 4 : 2;
    return min((rows + r - 1) / r, 2 * sm_count());
  }
  return min((rows + 7) / 8, sm_count());
}

// Number of fp32 elements the caller must provide as `partials` scratch for mlf_norm_bwd.
MLF_API long long mlf_norm_bwd_scratch_elems(int rows, int D) {
  return (long long)norm_bwd_grid(rows, D, nullptr) * 2 * D;
}

// dx_add (optional, bf16 [rows, D]) is added to dx: the gradient arriving over a skip connection that
// branched off the normalised tensor's input, so that the sum needs no pass of its own.
MLF_API int mlf_norm_bwd_add(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                             void* dx, void* dgamma, void* dbeta, float* partials, int rows, int D, int rms,
                             int grads_fp32, int accumulate, const void* dx_add, uint64_t stream) {
  MLF_REQUIRE(D % 256 == 0, "norm: D=%d must be a multiple of 256", D);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  bool cta_rows = false;
  const int grid = norm_bwd_grid(rows, D, &cta_rows);
  int rc = -2;
  bool matched = true;
  if (cta_rows) {
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* dyp = static_cast<const __nv_bfloat16*>(dy);
    const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gamma);
    __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(dx);
    const __nv_bfloat16* addp = static_cast<const __nv_bfloat16*>(dx_add);
    switch (D / 2048) {
      case 1: norm_bwd_cta_kernel<1, 4><<<grid, 256, 0, st>>>(xp, dyp, gp, mean, rstd, dxp, partials, rows, rms, addp); break;
      default: norm_bwd_cta_kernel<2, 2><<<grid, 256, 0, st>>>(xp, dyp, gp, mean, rstd, dxp, partials, rows, rms, addp); break;
    }
    count_launch();
    MLF_CHECK_CUDA(cudaGetLastError());
    rc = 0;
  } else
  switch (D / 256) {
#define CASE(NV) case NV: rc = launch_bwd<NV>(x, dy, gamma, mean, rstd, dx, partials, grid, rows, rms, dx_add, st); break;
    CASE(1) CASE(2) CASE(3) CASE(4) CASE(6) CASE(8) CASE(12) CASE(16) CASE(20) CASE(24) CASE(32)
#undef CASE
    default: matched = false;
  }
  MLF_REQUIRE(matched, "norm: unsupported D=%d", D);
  if (rc) return rc;
  norm_bwd_finalize_kernel<<<(D + 31) / 32, NF_WARPS * 32, 0, st>>>(partials, grid, D, dgamma, rms ? nullptr : dbeta,
                                                            grads_fp32, accumulate);
                                                            count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_norm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                         void* dx, void* dgamma, void* dbeta, float* partials, int rows, int D, int rms,
                         int grads_fp32, int accumulate, uint64_t stream) {
  return mlf_norm_bwd_add(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, partials, rows, D, rms, grads_fp32, accumulate, nullptr, stream);
}
