// fp32 operator kernels of the mobile inference runtime: conv2d, pooling, batch-norm (+ReLU),
// row softmax, fully connected, element-wise ReLU.
//
// The reference's mobile runtime encodes these as GPU compute dispatches without shader source
// (src/MobileRuntime/Backends/Metal/Shaders/Metal{Conv2D,MaxPool2D,BatchNorm,Softmax,FullyConnected,Relu}
// Shader.cs: 16x16x1 thread groups over the output plane for conv, 256 threads for softmax) and
// as CPU loops (src/MobileRuntime/Tensors/TensorOperations.cs). Here the same operator set runs as
// CUDA kernels over NCHW fp32 tensors. The conv kernel keeps the 16 x 16 output tile of the reference's
// dispatch shape, stages the input patch of one input channel slab in shared memory and computes
// 8 output channels per thread so every staged input value is used 8 x kh x kw times.
#include <float.h>

#include "../common/host.h"
#include "../mlf_api.h"

namespace mlf {

constexpr int CT = 16;        // output tile edge
constexpr int COC = 8;        // output channels per CTA
constexpr int CIC = 8;        // input channels staged per step
constexpr int CMAXK = 7;      // largest kernel edge of the tiled path

struct ConvParams {
  int N, C, H, W, O, KH, KW, OH, OW, stride, pad, dil, groups, relu;
};

// grid: (tiles_x * tiles_y, ceil(O_per_group / COC) * groups, N)
__global__ void __launch_bounds__(CT * CT) conv2d_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                         const float* __restrict__ w, const float* __restrict__ bias, ConvParams p) {
  extern __shared__ float sm[];
  const int tiles_x = (p.OW + CT - 1) / CT;
  const int tx = threadIdx.x % CT, ty = threadIdx.x / CT;
  const int ox0 = (blockIdx.x % tiles_x) * CT, oy0 = (blockIdx.x / tiles_x) * CT;
  const int o_per_g = p.O / p.groups, c_per_g = p.C / p.groups;
  const int oc_blocks = (o_per_g + COC - 1) / COC;
  const int g = blockIdx.y / oc_blocks;
  const int oc0 = g * o_per_g + (blockIdx.y % oc_blocks) * COC;
  const int oc_end = min(oc0 + COC, (g + 1) * o_per_g);
  const int n = blockIdx.z;
  const int pw = (CT - 1) * p.stride + (p.KW - 1) * p.dil + 1;   // staged patch width / height
  const int ph = (CT - 1) * p.stride + (p.KH - 1) * p.dil + 1;
  float* s_in = sm;                                  // [CIC][ph][pw]
  float* s_w = sm + CIC * ph * pw;                   // [COC][CIC][KH*KW]
  const int ix0 = ox0 * p.stride - p.pad, iy0 = oy0 * p.stride - p.pad;
  float acc[COC];
#pragma unroll
  for (int k = 0; k < COC; ++k) acc[k] = 0.f;

  for (int c0 = 0; c0 < c_per_g; c0 += CIC) {
    const int nc = min(CIC, c_per_g - c0);
    for (int i = threadIdx.x; i < nc * ph * pw; i += CT * CT) {
      const int c = i / (ph * pw), r = (i / pw) % ph, x = i % pw;
      const int iy = iy0 + r, ix = ix0 + x;
      float v = 0.f;
      if (iy >= 0 && iy < p.H && ix >= 0 && ix < p.W) v = in[(((long long)n * p.C + g * c_per_g + c0 + c) * p.H + iy) * p.W + ix];
      s_in[i] = v;
    }
    const int kk = p.KH * p.KW;
    for (int i = threadIdx.x; i < COC * nc * kk; i += CT * CT) {
      const int oc = i / (nc * kk), c = (i / kk) % nc, k = i % kk;
      s_w[(oc * CIC + c) * kk + k] = (oc0 + oc < oc_end) ? w[((long long)(oc0 + oc) * c_per_g + c0 + c) * kk + k] : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < nc; ++c)
      for (int ky = 0; ky < p.KH; ++ky)
        for (int kx = 0; kx < p.KW; ++kx) {
          const float v = s_in[(c * ph + ty * p.stride + ky * p.dil) * pw + tx * p.stride + kx * p.dil];
#pragma unroll
          for (int k = 0; k < COC; ++k) acc[k] += v * s_w[(k * CIC + c) * kk + ky * p.KW + kx];
        }
    __syncthreads();
  }
  const int ox = ox0 + tx, oy = oy0 + ty;
  if (ox < p.OW && oy < p.OH) {
#pragma unroll
    for (int k = 0; k < COC; ++k) {
      if (oc0 + k >= oc_end) break;
      float v = acc[k] + (bias ? bias[oc0 + k] : 0.f);
      if (p.relu) v = fmaxf(v, 0.f);
      out[(((long long)n * p.O + oc0 + k) * p.OH + oy) * p.OW + ox] = v;
    }
  }
}

// mode 0 = max, 1 = average over the in-bounds part of the window, 2 = average over the full k x k window (padding counts as zeros)
__global__ void __launch_bounds__(256) pool2d_kernel(float* __restrict__ out, const float* __restrict__ in, int NC, int H, int W, int OH,
                                                     int OW, int k, int stride, int pad, int mode) {
  const long long total = (long long)NC * OH * OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = (int)(i % OW), oy = (int)((i / OW) % OH);
    const long long nc = i / ((long long)OW * OH);
    float m = -FLT_MAX, s = 0.f;
    int cnt = 0;
    for (int ky = 0; ky < k; ++ky) {
      const int iy = oy * stride - pad + ky;
      if (iy < 0 || iy >= H) continue;
      for (int kx = 0; kx < k; ++kx) {
        const int ix = ox * stride - pad + kx;
        if (ix < 0 || ix >= W) continue;
        const float v = in[(nc * H + iy) * W + ix];
        m = fmaxf(m, v);
        s += v;
        ++cnt;
      }
    }
    out[i] = mode == 0 ? m : (mode == 1 ? (cnt ? s / cnt : 0.f) : s / (float)(k * k));
  }
}

// y = (x - mean) * gamma / sqrt(var + eps) + beta, optional ReLU; NCHW, per channel
__global__ void __launch_bounds__(256) batchnorm_kernel(float* __restrict__ out, const float* __restrict__ in, const float* gamma,
                                                        const float* beta, const float* mean, const float* var, float eps, int C,
                                                        int HW, long long total, int relu) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)((i / HW) % C);
    const float s = (gamma ? gamma[c] : 1.f) * rsqrtf(var[c] + eps);
    float v = (in[i] - mean[c]) * s + (beta ? beta[c] : 0.f);
    out[i] = relu ? fmaxf(v, 0.f) : v;
  }
}

// one warp per row
__global__ void __launch_bounds__(256) softmax_rows_kernel(float* __restrict__ out, const float* __restrict__ in, long long rows, int cols) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* x = in + row * cols;
  float m = -FLT_MAX;
  for (int c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += __expf(x[c] - m);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float inv = 1.f / s;
  for (int c = lane; c < cols; c += 32) out[row * cols + c] = __expf(x[c] - m) * inv;
}

// y[b, o] = act(sum_i x[b, i] * w[o, i] + bias[o]); one warp per (b, o); fp32 (batch sizes of a mobile model are tiny)
__global__ void __launch_bounds__(256) fc_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                                 const float* __restrict__ bias, int B, int I, int O, int relu) {
  const long long idx = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (idx >= (long long)B * O) return;
  const int b = (int)(idx / O), o = (int)(idx % O), lane = threadIdx.x & 31;
  float s = 0.f;
  if ((I & 3) == 0) {
    const float4* xv = reinterpret_cast<const float4*>(x + (long long)b * I);
    const float4* wv = reinterpret_cast<const float4*>(w + (long long)o * I);
    for (int i = lane; i < I / 4; i += 32) {
      const float4 a = xv[i], c = wv[i];
      s += a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w;
    }
  } else {
    for (int i = lane; i < I; i += 32) s += x[(long long)b * I + i] * w[(long long)o * I + i];
  }
  for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
  if (lane == 0) {
    s += bias ? bias[o] : 0.f;
    out[idx] = relu ? fmaxf(s, 0.f) : s;
  }
}

static int m_grid(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mlf

using namespace mlf;

MLF_API int mlf_conv2d_f32(float* out, const float* in, const float* w, const float* bias, int N, int C, int H, int W, int O, int KH,
                           int KW, int stride, int pad, int dil, int groups, int relu, uint64_t stream) {
  MLF_REQUIRE(N > 0 && C > 0 && O > 0 && groups > 0 && C % groups == 0 && O % groups == 0, "conv2d: bad channel / group counts");
  MLF_REQUIRE(KH >= 1 && KW >= 1 && KH <= CMAXK && KW <= CMAXK, "conv2d: kernel edge must be 1..%d", CMAXK);
  MLF_REQUIRE(stride >= 1 && stride <= 4 && dil >= 1 && dil <= 2 && pad >= 0, "conv2d: stride 1..4, dilation 1..2");
  ConvParams p{N, C, H, W, O, KH, KW, (H + 2 * pad - dil * (KH - 1) - 1) / stride + 1, (W + 2 * pad - dil * (KW - 1) - 1) / stride + 1,
               stride, pad, dil, groups, relu};
  MLF_REQUIRE(p.OH > 0 && p.OW > 0, "conv2d: empty output");
  const int pw = (CT - 1) * stride + (KW - 1) * dil + 1, ph = (CT - 1) * stride + (KH - 1) * dil + 1;
  const size_t smem = sizeof(float) * ((size_t)CIC * ph * pw + (size_t)COC * CIC * KH * KW);
  MLF_REQUIRE(smem <= 200 * 1024, "conv2d: staged patch of %zu bytes exceeds shared memory", smem);
  if (smem > 48 * 1024) MLF_CHECK_CUDA(cudaFuncSetAttribute(conv2d_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int o_per_g = O / groups;
  dim3 grid(((p.OW + CT - 1) / CT) * ((p.OH + CT - 1) / CT), ((o_per_g + COC - 1) / COC) * groups, N);
  conv2d_kernel<<<grid, CT * CT, smem, reinterpret_cast<cudaStream_t>(stream)>>>(out, in, w, bias, p);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_pool2d_f32(float* out, const float* in, int NC, int H, int W, int k, int stride, int pad, int mode, uint64_t stream) {
  MLF_REQUIRE(NC > 0 && k >= 1 && stride >= 1 && pad >= 0 && pad < k, "pool2d: bad arguments");
  const int OH = (H + 2 * pad - k) / stride + 1, OW = (W + 2 * pad - k) / stride + 1;
  MLF_REQUIRE(OH > 0 && OW > 0, "pool2d: empty output");
  pool2d_kernel<<<m_grid((long long)NC * OH * OW), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, in, NC, H, W, OH, OW, k, stride, pad, mode);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_batchnorm_f32(float* out, const float* in, const float* gamma, const float* beta, const float* mean, const float* var,
                              float eps, int N, int C, int HW, int relu, uint64_t stream) {
  MLF_REQUIRE(N > 0 && C > 0 && HW > 0 && mean && var, "batchnorm: bad arguments");
  const long long total = (long long)N * C * HW;
  batchnorm_kernel<<<m_grid(total), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, in, gamma, beta, mean, var, eps, C, HW, total, relu);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_softmax_rows_f32(float* out, const float* in, long long rows, int cols, uint64_t stream) {
  MLF_REQUIRE(rows > 0 && cols > 0, "softmax: bad shape");
  softmax_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, in, rows, cols);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_fc_f32(float* out, const float* x, const float* w, const float* bias, int B, int I, int O, int relu, uint64_t stream) {
  MLF_REQUIRE(B > 0 && I > 0 && O > 0, "fc: bad shape");
  MLF_REQUIRE((I & 3) != 0 || (((uintptr_t)x | (uintptr_t)w) & 15u) == 0, "fc: operands must be 16-byte aligned when I %% 4 == 0");
  const long long n = (long long)B * O;
  fc_kernel<<<(unsigned)((n + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, x, w, bias, B, I, O, relu);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
