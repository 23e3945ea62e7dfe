// Optimizer, mixed-precision and loss kernels.
//
//   adamw            fused AdamW over a flat shard: fp32 master weights + m + v, gradient in bf16
//                    or fp32, unscale by a device-resident inverse loss scale, skip when a
//                    device-resident found-inf flag is set, write the bf16 working copy.
//                    Update rule and order (decay first, then the Adam step) follow
//                    src/MLFramework/Optimizers/Adam.cs:167-213.
//   sgd              momentum SGD (config-1 style training on the GPU).
//   amp_unscale_check  multiply gradients by 1/scale in place, raise found_inf on NaN/Inf, and
//                    accumulate sum of squares (src/MLFramework/Amp/DynamicLossScaler.cs:149-220,
//                    331-363; src/MLFramework/Amp/GradientUtils.cs:17-187).
//   scaler_update    dynamic loss-scale state machine on the device (no host sync):
//                    src/MLFramework/Amp/DynamicLossScaler.cs:227-269.
//   clip_scale       gradient scaling by min(1, max_norm / norm) from a device-resident norm
//                    (src/MLFramework/Amp/GradientClipper.cs:60-153).
//   cross_entropy    fused softmax cross-entropy forward + backward: one pass over bf16 logits
//                    kept in shared memory, gradient written in place.
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

template <typename G>
__device__ __forceinline__ float load_grad(const G* g, long long i);
template <>
__device__ __forceinline__ float load_grad<float>(const float* g, long long i) { return g[i]; }
template <>
__device__ __forceinline__ float load_grad<__nv_bfloat16>(const __nv_bfloat16* g, long long i) { return __bfloat162float(g[i]); }

struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
};

template <typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, float* __restrict__ vmax,
             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_out, long long n, AdamWArgs a,
             const float* inv_scale_ptr, const int* found_inf) {
  if (found_inf && *found_inf) return;
  const float gs = a.grad_scale * (inv_scale_ptr ? *inv_scale_ptr : 1.f);
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float4 x4 = vmax ? reinterpret_cast<float4*>(vmax)[i] : make_float4(0, 0, 0, 0);
    float p[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
    float xx[4] = {x4.x, x4.y, x4.z, x4.w};
    float g[4];
    if (sizeof(G) == 2) {
      uint2 u = reinterpret_cast<const uint2*>(grad)[i];
      float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y);
      g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y;
    } else {
      float4 g4 = reinterpret_cast<const float4*>(grad)[i];
      g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gs;
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      float vh = vv[j];
      if (vmax) { xx[j] = fmaxf(xx[j], vv[j]); vh = xx[j]; }
      p[j] -= a.lr * a.weight_decay * p[j];
      p[j] -= a.lr * (mm[j] / a.bc1) / (sqrtf(vh / a.bc2) + a.eps);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (vmax) reinterpret_cast<float4*>(vmax)[i] = make_float4(xx[0], xx[1], xx[2], xx[3]);
    if (param_out) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(param_out)[i] = o;
    }
  }
  for (long long i = nvec * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gj = load_grad<G>(grad, i) * gs;
    float mm = a.beta1 * m[i] + (1.f - a.beta1) * gj;
    float vv = a.beta2 * v[i] + (1.f - a.beta2) * gj * gj;
    float vh = vv;
    if (vmax) { vmax[i] = fmaxf(vmax[i], vv); vh = vmax[i]; }
    float p = master[i];
    p -= a.lr * a.weight_decay * p;
    p -= a.lr * (mm / a.bc1) / (sqrtf(vh / a.bc2) + a.eps);
    master[i] = p; m[i] = mm; v[i] = vv;
    if (param_out) param_out[i] = __float2bfloat16(p);
  }
}

template <typename G>
__global__ void __launch_bounds__(256)
sgd_kernel(float* master, float* mom, const G* grad, __nv_bfloat16* param_out, long long n, float lr, float momentum,
           float weight_decay, float grad_scale, const float* inv_scale_ptr, const int* found_inf) {
  if (found_inf && *found_inf) return;
  const float gs = grad_scale * (inv_scale_ptr ? *inv_scale_ptr : 1.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = load_grad<G>(grad, i) * gs + weight_decay * master[i];
    if (mom) { g = momentum * mom[i] + g; mom[i] = g; }
    const float p = master[i] - lr * g;
    master[i] = p;
    if (param_out) param_out[i] = __float2bfloat16(p);
  }
}

// In place: g *= inv_scale; found_inf |= any non-finite; sumsq += sum(g^2) (after unscale).
template <typename G>
__global__ void __launch_bounds__(256)
amp_unscale_check_kernel(G* grad, long long n, const float* inv_scale_ptr, float inv_scale, int* found_inf, float* sumsq,
                         int write_back) {
  const float s = inv_scale * (inv_scale_ptr ? *inv_scale_ptr : 1.f);
  float acc = 0.f;
  bool bad = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = load_grad<G>(grad, i) * s;
    if (!isfinite(g)) bad = true;
    acc += g * g;
    if (write_back) {
      if (sizeof(G) == 2) reinterpret_cast<__nv_bfloat16*>(grad)[i] = __float2bfloat16(g);
      else reinterpret_cast<float*>(grad)[i] = g;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(found_inf, 1);
  if (sumsq && (threadIdx.x & 31) == 0 && isfinite(acc)) atomicAdd(sumsq, acc);
}

// Read-only check of bf16 gradients (no write-back): 16-byte loads, four per thread in flight.
__global__ void __launch_bounds__(256)
amp_check_bf16_vec_kernel(const __nv_bfloat16* grad, long long n, const float* inv_scale_ptr, float inv_scale, int* found_inf,
                          float* sumsq) {
  const float s = inv_scale * (inv_scale_ptr ? *inv_scale_ptr : 1.f);
  const long long nvec = n / 8;
  const uint4* gv = reinterpret_cast<const uint4*>(grad);
  float acc = 0.f;
  bool bad = false;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += 4 * stride) {
    uint4 u[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) u[k] = i + k * stride < nvec ? gv[i + k * stride] : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t w[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // a bf16 is non-finite when its exponent bits are all ones
        bad |= ((w[j] & 0x7f800000u) == 0x7f800000u) | ((w[j] & 0x00007f80u) == 0x00007f80u);
        if (sumsq) {
          const float2 f = unpack_bf16x2(w[j]);
          acc = fmaf(f.x * s, f.x * s, acc);
          acc = fmaf(f.y * s, f.y * s, acc);
        }
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * 8)) {
    const float g = __bfloat162float(grad[nvec * 8 + threadIdx.x]) * s;
    if (!isfinite(g)) bad = true;
    acc += g * g;
  }
  if (!isfinite(s)) bad = true;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(found_inf, 1);
  if (sumsq && (threadIdx.x & 31) == 0 && isfinite(acc)) atomicAdd(sumsq, acc);
}

// state: scale[0], growth_tracker (int) ; found_inf is reset to 0 afterwards.
__global__ void scaler_update_kernel(float* scale, int* tracker, int* found_inf, float growth, float backoff,
                                     int interval, float min_scale, float max_scale, int* skipped_steps) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float s = *scale;
  if (*found_inf) {
    s *= backoff;
    *tracker = 0;
    if (skipped_steps) *skipped_steps += 1;
  } else {
    const int t = *tracker + 1;
    if (t >= interval) { s *= growth; *tracker = 0; }
    else *tracker = t;
  }
  s = fminf(fmaxf(s, min_scale), max_scale);
  *scale = s;
  *found_inf = 0;
}

template <typename G>
__global__ void __launch_bounds__(256)
clip_scale_kernel(G* grad, long long n, const float* sumsq, float max_norm, float eps) {
  const float norm = sqrtf(*sumsq);
  const float c = fminf(1.f, max_norm / (norm + eps));
  if (c >= 1.f) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if (sizeof(G) == 2) reinterpret_cast<__nv_bfloat16*>(grad)[i] = __float2bfloat16(load_grad<G>(grad, i) * c);
    else reinterpret_cast<float*>(grad)[i] = load_grad<G>(grad, i) * c;
  }
}

// ------------------------------------------------------------------------------------------
// fused cross-entropy: one CTA per row. logits bf16 [T, ld], first V columns valid.
// loss_rows[t] = logsumexp - logit[target]; logits <- (softmax - onehot) * gscale (pad cols 0).
// target < 0 (ignore) gives loss 0 and a zero gradient row.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
cross_entropy_kernel(__nv_bfloat16* logits, const long long* targets, float* loss_rows, float* loss_sum, int T, int V,
                     long long ld, float gscale, const float* gscale_ptr, float loss_weight, int cache_row, int* err) {
  extern __shared__ uint4 row_cache[];  // ld bf16 values when cache_row != 0
  __shared__ float red_a[16], red_b[16];
  const int t = blockIdx.x;
  __nv_bfloat16* row = logits + (long long)t * ld;
  const int nvec = V / 8;
  const long long tgt = targets[t];
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  // pass 1: online max / sum-exp
  float mx = -FLT_MAX, se = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[i];
    if (cache_row) row_cache[i] = u;
    float f[8];
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > mx) { se *= __expf(mx - lm); mx = lm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(row[i]);
    if (f > mx) { se *= __expf(mx - f); mx = f; }
    se += __expf(f - mx);
  }
  // CTA reduce (max, then rescaled sums)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, se, o);
    const float nm = fmaxf(mx, om);
    se = se * __expf(mx - nm) + os * __expf(om - nm);
    mx = nm;
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { red_a[w] = mx; red_b[w] = se; }
  __syncthreads();
  float gm = red_a[0], gsum = red_b[0];
  for (int k = 1; k < nw; ++k) {
    const float nm = fmaxf(gm, red_a[k]);
    gsum = gsum * __expf(gm - nm) + red_b[k] * __expf(red_a[k] - nm);
    gm = nm;
  }
  const float lse = gm + __logf(gsum);
  const bool ignore = tgt < 0;
  if (!ignore && tgt >= V) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_INDEX);
  }
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignore && tgt < V) l = lse - __bfloat162float(row[tgt]);
    if (loss_rows) loss_rows[t] = l;
    if (loss_sum) atomicAdd(loss_sum, l * loss_weight);
  }
  __syncthreads();  // row[tgt] read before anyone overwrites it
  // pass 2: gradient in place
  const float inv = 1.f / gsum;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 u = cache_row ? row_cache[i] : reinterpret_cast<const uint4*>(row)[i];
    float f[8];
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = ignore ? 0.f : __expf(f[j] - gm) * inv;
      if (!ignore && (long long)(i * 8 + j) == tgt) g -= 1.f;
      f[j] = g * gs;
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]); o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    reinterpret_cast<uint4*>(row)[i] = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < (int)ld; i += blockDim.x) {
    float g = 0.f;
    if (i < V && !ignore) {
      g = __expf(__bfloat162float(row[i]) - gm) * inv;
      if ((long long)i == tgt) g -= 1.f;
    }
    row[i] = __float2bfloat16(g * gs);
  }
}

static inline int ew_grid2(long long n) {
  long long g = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace mlf

using namespace mlf;

// grad_dtype: 0 fp32, 1 bf16. vmax null unless amsgrad. param_out (bf16) may be null.
MLF_API int mlf_adamw(float* master, float* m, float* v, float* vmax, const void* grad, int grad_dtype, void* param_out,
                      long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                      float grad_scale, const float* inv_scale_ptr, const int* found_inf, uint64_t stream) {
  if (n <= 0) return 0;
  MLF_REQUIRE(step >= 1, "adamw: step must be >= 1");
  AdamWArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), grad_scale};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = ew_grid2(n / 4 + 1);
  if (grad_dtype == 1)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, m, v, vmax, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param_out, n, a, inv_scale_ptr, found_inf);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(master, m, v, vmax, (const float*)grad, (__nv_bfloat16*)param_out, n, a, inv_scale_ptr, found_inf);
    count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_sgd(float* master, float* mom, const void* grad, int grad_dtype, void* param_out, long long n, float lr,
                    float momentum, float weight_decay, float grad_scale, const float* inv_scale_ptr, const int* found_inf,
                    uint64_t stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (grad_dtype == 1)
    sgd_kernel<__nv_bfloat16><<<ew_grid2(n), 256, 0, st>>>(master, mom, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param_out, n, lr, momentum, weight_decay, grad_scale, inv_scale_ptr, found_inf);
  else
    sgd_kernel<float><<<ew_grid2(n), 256, 0, st>>>(master, mom, (const float*)grad, (__nv_bfloat16*)param_out, n, lr, momentum, weight_decay, grad_scale, inv_scale_ptr, found_inf);
    count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_amp_unscale_check(void* grad, int grad_dtype, long long n, const float* inv_scale_ptr, float inv_scale,
                                  int* found_inf, float* sumsq, int write_back, uint64_t stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (grad_dtype == 1 && !write_back && (reinterpret_cast<uintptr_t>(grad) & 15) == 0)
    amp_check_bf16_vec_kernel<<<ew_grid2(n / 32 + 1), 256, 0, st>>>((const __nv_bfloat16*)grad, n, inv_scale_ptr, inv_scale, found_inf, sumsq);
  else if (grad_dtype == 1)
    amp_unscale_check_kernel<__nv_bfloat16><<<ew_grid2(n), 256, 0, st>>>((__nv_bfloat16*)grad, n, inv_scale_ptr, inv_scale, found_inf, sumsq, write_back);
  else
    amp_unscale_check_kernel<float><<<ew_grid2(n), 256, 0, st>>>((float*)grad, n, inv_scale_ptr, inv_scale, found_inf, sumsq, write_back);
    count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_scaler_update(float* scale, int* tracker, int* found_inf, float growth, float backoff, int interval,
                              float min_scale, float max_scale, int* skipped_steps, uint64_t stream) {
  scaler_update_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(scale, tracker, found_inf, growth, backoff, interval, min_scale, max_scale, skipped_steps);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_clip_scale(void* grad, int grad_dtype, long long n, const float* sumsq, float max_norm, float eps, uint64_t stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (grad_dtype == 1) clip_scale_kernel<__nv_bfloat16><<<ew_grid2(n), 256, 0, st>>>((__nv_bfloat16*)grad, n, sumsq, max_norm, eps);
  else clip_scale_kernel<float><<<ew_grid2(n), 256, 0, st>>>((float*)grad, n, sumsq, max_norm, eps);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
// logits are overwritten with the gradient. ld must be a multiple of 8; V <= ld.
MLF_API int mlf_cross_entropy(void* logits, const long long* targets, float* loss_rows, float* loss_sum, int T, int V,
                              long long ld, float gscale, const float* gscale_ptr, float loss_weight, uint64_t stream) {
  MLF_REQUIRE(ld % 8 == 0 && V <= ld, "cross_entropy: need V <= ld and ld %% 8 == 0 (V=%d ld=%lld)", V, ld);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)ld * 2;
  const int cache = smem <= 200 * 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    MLF_CHECK_CUDA(cudaFuncSetAttribute(cross_entropy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[dev & 63] = true;
  }
  cross_entropy_kernel<<<T, 512, cache ? smem : 0, st>>>((__nv_bfloat16*)logits, targets, loss_rows, loss_sum, T, V, ld, gscale,
                                                         gscale_ptr, loss_weight, cache, device_status_word());
                                                         count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
