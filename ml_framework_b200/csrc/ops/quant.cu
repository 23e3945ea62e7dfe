// int8 quantisation kernels: quantise, dequantise, fake-quantise (with straight-through mask) and
// min/max observation. Element-wise and bandwidth-bound: 16-byte loads, one pass, per-tensor or
// per-channel (row or column) parameters.
//
// Semantics follow the reference's operations (src/MLFramework/Quantization/Operations/
// QuantizationOperations.cs, DequantizationOperations.cs, PerChannelOperations.cs and
// QAT/FakeQuantize.cs, StraightThroughEstimator.cs):
//   q = clamp(round(x / scale) + zero_point, qmin, qmax);   x' = (q - zero_point) * scale
// Rounding is round-half-to-even (cvt.rni), which is what a float -> int8 conversion on the tensor
// cores' input path does as well.
#include <cuda_bf16.h>
#include <float.h>

#include "../common/host.h"
#include "../mlf_api.h"

namespace mlf {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// axis: -1 per tensor (scale[0]), 0 per row (scale[row]), 1 per column (scale[col])
__device__ __forceinline__ int qparam_index(int axis, long long row, int col) { return axis < 0 ? 0 : (axis == 0 ? (int)row : col); }

// MODE 0: quantise to int8; 1: fake-quantise to T (+ optional mask of in-range elements)
template <typename T, int MODE>
__global__ void __launch_bounds__(256) quant_kernel(void* out_, unsigned char* mask, const T* in, long long rows, int cols,
                                                    const float* scale, const int* zp, int axis, int qmin, int qmax) {
  constexpr int V = 4;
  const int vec_per_row = (cols + V - 1) / V;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c0 = (int)(i % vec_per_row) * V;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int c = c0 + j;
      if (c >= cols) break;
      const int qi = qparam_index(axis, r, c);
      const float s = scale[qi];
      const int z = zp ? zp[qi] : 0;
      const float x = ldf(in + r * cols + c);
      int q = __float2int_rn(x / s) + z;
      const bool inside = q >= qmin && q <= qmax;
      q = min(max(q, qmin), qmax);
      if (MODE == 0) {
        static_cast<signed char*>(out_)[r * cols + c] = (signed char)q;
      } else {
        stf(static_cast<T*>(out_) + r * cols + c, (float)(q - z) * s);
        if (mask) mask[r * cols + c] = inside ? 1 : 0;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dequant_kernel(T* out, const signed char* in, long long rows, int cols, const float* scale,
                                                      const int* zp, int axis) {
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i % cols);
    const int qi = qparam_index(axis, r, c);
    stf(out + i, (float)((int)in[i] - (zp ? zp[qi] : 0)) * scale[qi]);
  }
}

// Order-preserving float <-> int encoding so that integer atomics give float min / max.
__device__ __forceinline__ int f2ord(float f) { int i = __float_as_int(f); return i >= 0 ? i : i ^ 0x7fffffff; }
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__global__ void minmax_init_kernel(int* acc) { acc[0] = f2ord(FLT_MAX); acc[1] = f2ord(-FLT_MAX); }
template <typename T>
__global__ void __launch_bounds__(256) minmax_kernel(int* acc, const T* in, long long n) {
  float lo = FLT_MAX, hi = -FLT_MAX;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = ldf(in + i);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&acc[0], f2ord(lo));
    atomicMax(&acc[1], f2ord(hi));
  }
}
__global__ void minmax_finish_kernel(float* out, const int* acc) { out[0] = ord2f(acc[0]); out[1] = ord2f(acc[1]); }

static int q_grid(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mlf

using namespace mlf;

// dtype: 0 = fp32, 1 = bf16
MLF_API int mlf_quantize_i8(void* out, const void* in, int dtype, long long rows, int cols, const float* scale, const int* zp,
                            int axis, int qmin, int qmax, uint64_t stream) {
  MLF_REQUIRE(rows > 0 && cols > 0 && scale != nullptr, "quantize: bad arguments");
  MLF_REQUIRE(qmin >= -128 && qmax <= 127 && qmin < qmax, "quantize: range [%d, %d] does not fit int8", qmin, qmax);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = q_grid(rows * ((cols + 3) / 4));
  if (dtype == 0) quant_kernel<float, 0><<<g, 256, 0, st>>>(out, nullptr, (const float*)in, rows, cols, scale, zp, axis, qmin, qmax);
  else quant_kernel<__nv_bfloat16, 0><<<g, 256, 0, st>>>(out, nullptr, (const __nv_bfloat16*)in, rows, cols, scale, zp, axis, qmin, qmax);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_dequantize_i8(void* out, const void* in, int dtype, long long rows, int cols, const float* scale, const int* zp,
                              int axis, uint64_t stream) {
  MLF_REQUIRE(rows > 0 && cols > 0 && scale != nullptr, "dequantize: bad arguments");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = q_grid(rows * cols);
  if (dtype == 0) dequant_kernel<float><<<g, 256, 0, st>>>((float*)out, (const signed char*)in, rows, cols, scale, zp, axis);
  else dequant_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((__nv_bfloat16*)out, (const signed char*)in, rows, cols, scale, zp, axis);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_fake_quant(void* out, void* mask, const void* in, int dtype, long long rows, int cols, const float* scale,
                           const int* zp, int axis, int qmin, int qmax, uint64_t stream) {
  MLF_REQUIRE(rows > 0 && cols > 0 && scale != nullptr, "fake_quant: bad arguments");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = q_grid(rows * ((cols + 3) / 4));
  if (dtype == 0) quant_kernel<float, 1><<<g, 256, 0, st>>>(out, (unsigned char*)mask, (const float*)in, rows, cols, scale, zp, axis, qmin, qmax);
  else quant_kernel<__nv_bfloat16, 1><<<g, 256, 0, st>>>(out, (unsigned char*)mask, (const __nv_bfloat16*)in, rows, cols, scale, zp, axis, qmin, qmax);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
// out[0] = min, out[1] = max of n elements. scratch: 2 ints.
MLF_API int mlf_minmax(float* out, const void* in, int dtype, long long n, int* scratch, uint64_t stream) {
  MLF_REQUIRE(n > 0 && scratch != nullptr, "minmax: bad arguments");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  minmax_init_kernel<<<1, 1, 0, st>>>(scratch);
  if (dtype == 0) minmax_kernel<float><<<q_grid(n), 256, 0, st>>>(scratch, (const float*)in, n);
  else minmax_kernel<__nv_bfloat16><<<q_grid(n), 256, 0, st>>>(scratch, (const __nv_bfloat16*)in, n);
  minmax_finish_kernel<<<1, 1, 0, st>>>(out, scratch);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
