// Shared pieces of the tcgen05 GEMM kernels: kernel parameters, tile rasterisation and the
// fused epilogue applied to one 32-column chunk of an accumulator row.
#pragma once
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;

struct GemmKernelParams {
  int M, N, K;
  int a_mn, b_mn;
  int flags;
  float alpha;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  long long ldo, ld_aux_in, ld_aux_out;
  int tiles_m, tiles_n;
  int rot_m, rot_n;  // tile-order rotation (tiles), so locally owned rows come first
  int* err;
  // gather
  int gather_operand, world, rank, n_copy_ctas, rows_per_rank, flag_rows, row_bytes, total_rows;
  const void* src[8];
  void* gathered;
  uint32_t* flags_ready;
  uint32_t* counters;
  const void* extra_segs;   // {src, dst, bytes} triples copied after the gated chunks, no flags
  int n_extra;
  // scatter
  int scatter_out, rows_per_owner;
  void* out_peer[8];
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int rot_m, int rot_n,
                                            int& tm, int& tn) {
  // Grouped rasterisation: 8 row-tiles share each column-tile while it is hot in L2.
  constexpr int GM = 8;
  const int per_group = GM * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gsz = min(GM, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
  tm += rot_m;
  if (tm >= tiles_m) tm -= tiles_m;
  tn += rot_n;
  if (tn >= tiles_n) tn -= tiles_n;
}

// One accumulator row chunk: r[0..31] are fp32 bit patterns of columns nb..nb+31 of row m.
// out_row points at the start of the output row (possibly in a peer's buffer).
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmKernelParams& p, const int m, const int nb,
                                                    const uint32_t (&r)[32], char* out_row, const bool out_fp32,
                                                    const bool swiglu, const bool dswiglu) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const int nvalid = min(32, p.N - nb);
        if (p.flags & MLF_EPI_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < nvalid) v[j] += __bfloat162float(p.bias[nb + j]);
        }
        if (p.flags & MLF_EPI_STORE_PRE) {
          __nv_bfloat16* ar = p.aux_out + (long long)m * p.ld_aux_out + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
              w.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
              w.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
              w.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
              reinterpret_cast<uint4*>(ar)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j) ar[j] = __float2bfloat16(v[j]);
          }
        }
        if (p.flags & MLF_EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        }
        if (p.flags & (MLF_EPI_RESIDUAL | MLF_EPI_DGELU_MUL)) {
          const __nv_bfloat16* ar = p.aux_in + (long long)m * p.ld_aux_in + nb;
          float a[32];
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w = reinterpret_cast<const uint4*>(ar)[g];
              float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z),
                     f3 = unpack_bf16x2(w.w);
              a[8 * g + 0] = f0.x; a[8 * g + 1] = f0.y; a[8 * g + 2] = f1.x; a[8 * g + 3] = f1.y;
              a[8 * g + 4] = f2.x; a[8 * g + 5] = f2.y; a[8 * g + 6] = f3.x; a[8 * g + 7] = f3.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = j < nvalid ? __bfloat162float(ar[j]) : 0.f;
          }
          if (p.flags & MLF_EPI_RESIDUAL) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += a[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh(a[j]);
          }
        }
        if (swiglu) {
          // (gate, up) pairs -> 16 outputs at column nb/2
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + nb / 2;
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = silu(v[2 * j]) * v[2 * j + 1];
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              uint4 w;
              w.x = pack_bf16x2(o[8 * g + 0], o[8 * g + 1]);
              w.y = pack_bf16x2(o[8 * g + 2], o[8 * g + 3]);
              w.z = pack_bf16x2(o[8 * g + 4], o[8 * g + 5]);
              w.w = pack_bf16x2(o[8 * g + 6], o[8 * g + 7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid / 2; ++j) orow[j] = __float2bfloat16(o[j]);
          }
          return;
        }
        if (dswiglu) {
          // v = dL/dh for 32 hidden columns; aux_in holds (gate, up) pairs; out gets (dgate, dup)
          const __nv_bfloat16* ar = p.aux_in + (long long)m * p.ld_aux_in + 2 * nb;
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + 2 * nb;
          const bool vec = nvalid == 32 && ((reinterpret_cast<uintptr_t>(ar) & 15) == 0) &&
                           ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float gu[8];
            if (vec) {
              uint4 w = reinterpret_cast<const uint4*>(ar)[g];
              float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z),
                     f3 = unpack_bf16x2(w.w);
              gu[0] = f0.x; gu[1] = f0.y; gu[2] = f1.x; gu[3] = f1.y;
              gu[4] = f2.x; gu[5] = f2.y; gu[6] = f3.x; gu[7] = f3.y;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                gu[j] = (4 * g + j / 2) < nvalid ? __bfloat162float(ar[8 * g + j]) : 0.f;
            }
            float o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float gate = gu[2 * j], up = gu[2 * j + 1], dh = v[4 * g + j];
              const float sg = 1.f / (1.f + __expf(-gate));
              o[2 * j] = dh * up * sg * (1.f + gate * (1.f - sg));
              o[2 * j + 1] = dh * gate * sg;
            }
            if (vec) {
              uint4 w;
              w.x = pack_bf16x2(o[0], o[1]);
              w.y = pack_bf16x2(o[2], o[3]);
              w.z = pack_bf16x2(o[4], o[5]);
              w.w = pack_bf16x2(o[6], o[7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if ((4 * g + j / 2) < nvalid) orow[8 * g + j] = __float2bfloat16(o[j]);
            }
          }
          return;
        }
        if (out_fp32) {
          float* orow = reinterpret_cast<float*>(out_row) + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              float4 w = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
              if (p.flags & MLF_EPI_ACCUM) {
                float4 o = reinterpret_cast<float4*>(orow)[g];
                w.x += o.x; w.y += o.y; w.z += o.z; w.w += o.w;
              }
              reinterpret_cast<float4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j)
              orow[j] = v[j] + ((p.flags & MLF_EPI_ACCUM) ? orow[j] : 0.f);
          }
        } else {
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out_row) + nb;
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (p.flags & MLF_EPI_ACCUM) {
                uint4 o = reinterpret_cast<uint4*>(orow)[g];
                float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z),
                       f3 = unpack_bf16x2(o.w);
                v[8 * g + 0] += f0.x; v[8 * g + 1] += f0.y; v[8 * g + 2] += f1.x; v[8 * g + 3] += f1.y;
                v[8 * g + 4] += f2.x; v[8 * g + 5] += f2.y; v[8 * g + 6] += f3.x; v[8 * g + 7] += f3.y;
              }
              uint4 w;
              w.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
              w.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
              w.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
              w.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
              reinterpret_cast<uint4*>(orow)[g] = w;
            }
          } else {
            for (int j = 0; j < nvalid; ++j) {
              float x = v[j];
              if (p.flags & MLF_EPI_ACCUM) x += __bfloat162float(orow[j]);
              orow[j] = __float2bfloat16(x);
            }
          }
        }
      }

}  // namespace mlf
