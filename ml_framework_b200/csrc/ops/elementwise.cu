// Bandwidth-bound element-wise, reduction, activation and embedding kernels.
//
// Covers the device operations behind the reference's HAL kernel table
// (src/MLFramework/HAL/CUDA/CudaKernels.cs:20-138: add/subtract/multiply/divide, relu/sigmoid/
// tanh, sum/max/min, copy/fill), the tanh-GELU of its TP MLP factory
// (src/MLFramework/Layers/TensorParallel/TPMLPFactory.cs:113-140), plus SwiGLU, RoPE, embedding
// and bias-gradient kernels the GPT/Llama model families need. All kernels use 16-byte
// accesses and a grid sized to the SM count.
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

enum { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_MAX = 4, OP_MIN = 5 };
enum { UOP_RELU = 0, UOP_SIGMOID = 1, UOP_TANH = 2, UOP_GELU = 3, UOP_SILU = 4, UOP_EXP = 5, UOP_NEG = 6,
       UOP_SQRT = 7, UOP_LOG = 8, UOP_ABS = 9 };

__device__ __forceinline__ float apply_bin(int op, float a, float b) {
  switch (op) {
    case OP_ADD: return a + b;
    case OP_SUB: return a - b;
    case OP_MUL: return a * b;
    case OP_DIV: return a / b;
    case OP_MAX: return fmaxf(a, b);
    default: return fminf(a, b);
  }
}
__device__ __forceinline__ float apply_un(int op, float a) {
  switch (op) {
    case UOP_RELU: return fmaxf(a, 0.f);
    case UOP_SIGMOID: return 1.f / (1.f + __expf(-a));
    case UOP_TANH: return tanhf(a);
    case UOP_GELU: return gelu_tanh(a);
    case UOP_SILU: return silu(a);
    case UOP_EXP: return __expf(a);
    case UOP_NEG: return -a;
    case UOP_SQRT: return sqrtf(a);
    case UOP_LOG: return __logf(a);
    default: return fabsf(a);
  }
}

template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  using V = float4;
  __device__ static void load(const float* p, float (&f)[4]) { float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ static void store(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
  __device__ static float ld1(const float* p) { return *p; }
  __device__ static void st1(float* p, float v) { *p = v; }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

// out = a (op) b, or a (op) scalar when b == nullptr.
template <typename T>
__global__ void __launch_bounds__(256) ew_binary_kernel(T* out, const T* a, const T* b, float scalar, long long n, int op) {
  constexpr int N = Vec<T>::N;
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[N], y[N];
    Vec<T>::load(a + i * N, x);
    if (b) Vec<T>::load(b + i * N, y);
#pragma unroll
    for (int j = 0; j < N; ++j) x[j] = apply_bin(op, x[j], b ? y[j] : scalar);
    Vec<T>::store(out + i * N, x);
  }
  for (long long i = nvec * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    Vec<T>::st1(out + i, apply_bin(op, Vec<T>::ld1(a + i), b ? Vec<T>::ld1(b + i) : scalar));
}

template <typename T>
__global__ void __launch_bounds__(256) ew_unary_kernel(T* out, const T* a, long long n, int op) {
  constexpr int N = Vec<T>::N;
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[N];
    Vec<T>::load(a + i * N, x);
#pragma unroll
    for (int j = 0; j < N; ++j) x[j] = apply_un(op, x[j]);
    Vec<T>::store(out + i * N, x);
  }
  for (long long i = nvec * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    Vec<T>::st1(out + i, apply_un(op, Vec<T>::ld1(a + i)));
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* out, float value, long long n) {
  constexpr int N = Vec<T>::N;
  const long long nvec = n / N;
  float x[N];
#pragma unroll
  for (int j = 0; j < N; ++j) x[j] = value;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    Vec<T>::store(out + i * N, x);
  for (long long i = nvec * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    Vec<T>::st1(out + i, value);
}

// Full reduction, stage 1: per-CTA partial (sum / max / min) -> partials[blockIdx.x].
// red: 0 sum, 1 max, 2 min.
template <typename T>
__global__ void __launch_bounds__(256) reduce_stage1_kernel(const T* a, long long n, float* partials, int red) {
  constexpr int N = Vec<T>::N;
  float acc = red == 0 ? 0.f : (red == 1 ? -FLT_MAX : FLT_MAX);
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[N];
    Vec<T>::load(a + i * N, x);
#pragma unroll
    for (int j = 0; j < N; ++j) acc = red == 0 ? acc + x[j] : (red == 1 ? fmaxf(acc, x[j]) : fminf(acc, x[j]));
  }
  for (long long i = nvec * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = Vec<T>::ld1(a + i);
    acc = red == 0 ? acc + v : (red == 1 ? fmaxf(acc, v) : fminf(acc, v));
  }
  __shared__ float sm[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = red == 0 ? acc + other : (red == 1 ? fmaxf(acc, other) : fminf(acc, other));
  }
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = sm[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = red == 0 ? r + sm[w] : (red == 1 ? fmaxf(r, sm[w]) : fminf(r, sm[w]));
    partials[blockIdx.x] = r;
  }
}
__global__ void reduce_stage2_kernel(const float* partials, int n, float* out, int red, float scale) {
  float acc = red == 0 ? 0.f : (red == 1 ? -FLT_MAX : FLT_MAX);
  for (int i = threadIdx.x; i < n; i += 32) {
    const float v = partials[i];
    acc = red == 0 ? acc + v : (red == 1 ? fmaxf(acc, v) : fminf(acc, v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = red == 0 ? acc + other : (red == 1 ? fmaxf(acc, other) : fminf(acc, other));
  }
  if (threadIdx.x == 0) *out = red == 0 ? acc * scale : acc;
}

// ------------------------------------------------------------------------------------------
// activations with their derivatives (bf16)
// ------------------------------------------------------------------------------------------
// dx = dy * gelu'(x)
__global__ void __launch_bounds__(256) gelu_bwd_kernel(__nv_bfloat16* dx, const __nv_bfloat16* dy, const __nv_bfloat16* x, long long n) {
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[8], g[8];
    Vec<__nv_bfloat16>::load(x + i * 8, a);
    Vec<__nv_bfloat16>::load(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= dgelu_tanh(a[j]);
    Vec<__nv_bfloat16>::store(dx + i * 8, g);
  }
}

// SwiGLU with gate and up stored as two halves of a row: gu[r, 0:F] = gate, gu[r, F:2F] = up,
// or interleaved (gate, up) pairs when `interleaved` != 0. out[r, F] = silu(gate) * up.
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(__nv_bfloat16* out, const __nv_bfloat16* gu, long long rows, int F, int interleaved) {
  const long long total = rows * F / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (F / 8);
    const int c = (int)(i % (F / 8)) * 8;
    float g[8], u[8], o[8];
    if (!interleaved) {
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + c, g);
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + F + c, u);
    } else {
      float p0[8], p1[8];
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + 2 * c, p0);
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + 2 * c + 8, p1);
#pragma unroll
      for (int j = 0; j < 4; ++j) { g[j] = p0[2 * j]; u[j] = p0[2 * j + 1]; g[4 + j] = p1[2 * j]; u[4 + j] = p1[2 * j + 1]; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu(g[j]) * u[j];
    Vec<__nv_bfloat16>::store(out + r * F + c, o);
  }
}
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(__nv_bfloat16* dgu, const __nv_bfloat16* dout, const __nv_bfloat16* gu, long long rows, int F, int interleaved) {
  const long long total = rows * F / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (F / 8);
    const int c = (int)(i % (F / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    Vec<__nv_bfloat16>::load(dout + r * F + c, d);
    if (!interleaved) {
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + c, g);
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + F + c, u);
    } else {
      float p0[8], p1[8];
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + 2 * c, p0);
      Vec<__nv_bfloat16>::load(gu + r * 2 * F + 2 * c + 8, p1);
#pragma unroll
      for (int j = 0; j < 4; ++j) { g[j] = p0[2 * j]; u[j] = p0[2 * j + 1]; g[4 + j] = p1[2 * j]; u[4 + j] = p1[2 * j + 1]; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
      du[j] = d[j] * g[j] * sg;
    }
    if (!interleaved) {
      Vec<__nv_bfloat16>::store(dgu + r * 2 * F + c, dg);
      Vec<__nv_bfloat16>::store(dgu + r * 2 * F + F + c, du);
    } else {
      float p0[8], p1[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { p0[2 * j] = dg[j]; p0[2 * j + 1] = du[j]; p1[2 * j] = dg[4 + j]; p1[2 * j + 1] = du[4 + j]; }
      Vec<__nv_bfloat16>::store(dgu + r * 2 * F + 2 * c, p0);
      Vec<__nv_bfloat16>::store(dgu + r * 2 * F + 2 * c + 8, p1);
    }
  }
}

// ------------------------------------------------------------------------------------------
// column sum (bias gradient): db[n] = sum_m dy[m, n]; dy bf16 [M, N] with pitch ld.
// One launch, no atomics on the data: each CTA owns 256 columns x a slab of rows and writes its fp32
// partial sums to part[slab][N]; the CTA that finishes last for a column block (a counter per block,
// reset by that CTA) adds the slabs in slab order and writes bf16. The order of the additions is
// fixed, so the result is the same from run to run.
// ------------------------------------------------------------------------------------------
constexpr int CS_COLS = 256;     // columns per CTA: a warp reads 512 contiguous bytes of a row
__global__ void __launch_bounds__(256) colsum_kernel(__nv_bfloat16* __restrict__ db, const __nv_bfloat16* __restrict__ dy,
                                                     float* __restrict__ part, unsigned int* __restrict__ counters, int M, int N,
                                                     long long ld, int rows_per_cta, int accumulate) {
  const int col0 = blockIdx.x * CS_COLS;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(M, r0 + rows_per_cta);
  const int cl = (threadIdx.x & 31) * 8;  // 32 threads x 8 columns = 256 columns
  const int rl = threadIdx.x >> 5;        // 8 row lanes
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col0 + cl + 8 <= N) {
    for (int r = r0 + rl; r < r1; r += 32) {           // four 16-byte loads per thread in flight
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        u[k] = r + 8 * k < r1 ? *reinterpret_cast<const uint4*>(dy + (long long)(r + 8 * k) * ld + col0 + cl) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_bf16x2(u[k].x), b = unpack_bf16x2(u[k].y), c = unpack_bf16x2(u[k].z), d = unpack_bf16x2(u[k].w);
        s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
      }
    }
  } else {
    for (int r = r0 + rl; r < r1; r += 8)
      for (int j = 0; j < 8; ++j)
        if (col0 + cl + j < N) s[j] += __bfloat162float(dy[(long long)r * ld + col0 + cl + j]);
  }
  __shared__ float sm[8][CS_COLS + 1];
  __shared__ int s_last;
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[rl][cl + j] = s[j];
  __syncthreads();
  {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += sm[r][threadIdx.x];
    if (col0 + threadIdx.x < N) part[(long long)blockIdx.y * N + col0 + threadIdx.x] = t;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[blockIdx.x], 1u) == gridDim.y - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (col0 + threadIdx.x < N) {
    float t = 0.f;
    for (int y = 0; y < (int)gridDim.y; ++y) t += __ldcg(part + (long long)y * N + col0 + threadIdx.x);
    __nv_bfloat16* o = db + col0 + threadIdx.x;
    *o = __float2bfloat16(t + (accumulate ? __bfloat162float(*o) : 0.f));
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0u;      // ready for the next launch on this stream
}
__global__ void cast_f32_to_bf16_kernel(__nv_bfloat16* out, const float* in, long long n, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i] + (accumulate ? __bfloat162float(out[i]) : 0.f));
}

// ------------------------------------------------------------------------------------------
// embedding: out[t, :] = wte[ids[t], :] (+ wpe[pos[t], :]); D multiple of 8
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embedding_fwd_kernel(__nv_bfloat16* out, const long long* ids, const long long* pos,
                                                            const __nv_bfloat16* wte, const __nv_bfloat16* wpe,
                                                            long long T, int D, int vocab, int max_pos, int* err) {
  const int vec_per_row = D / 8;
  const long long total = T * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    long long id = ids[t];
    if (id < 0 || id >= vocab) { atomicCAS(err, 0, ERR_BAD_INDEX); id = 0; }
    float a[8];
    Vec<__nv_bfloat16>::load(wte + id * D + c, a);
    if (wpe) {
      long long p = pos ? pos[t] : 0;
      if (p < 0 || p >= max_pos) { atomicCAS(err, 0, ERR_BAD_INDEX); p = 0; }
      float b[8];
      Vec<__nv_bfloat16>::load(wpe + p * D + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    Vec<__nv_bfloat16>::store(out + t * D + c, a);
  }
}
// dW[ids[t], :] += dout[t, :] into an fp32 accumulator (atomics; rows repeat).
__global__ void __launch_bounds__(256) embedding_bwd_kernel(float* dw, const __nv_bfloat16* dout, const long long* ids,
                                                            long long T, int D, int vocab) {
  const int vec_per_row = D / 8;
  const long long total = T * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float a[8];
    Vec<__nv_bfloat16>::load(dout + t * D + c, a);
    float* dst = dw + id * D + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, a[j]);
  }
}

// ------------------------------------------------------------------------------------------
// RoPE (rotate-half convention): x [T, H, Dh] bf16 in place; pos [T]; inverse != 0 applies the
// transposed rotation (backward). theta is the base (500000 for Llama 3 style models).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16* x, const long long* pos, long long T, int H, int Dh,
                                                   long long row_stride, float theta, int inverse) {
  const int half = Dh / 2;
  const long long total = T * H * half;
  const float log_theta = __logf(theta);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % half);
    const long long th = i / half;
    const int h = (int)(th % H);
    const long long t = th / H;
    const float inv_freq = __expf(-log_theta * (2.f * d / Dh));
    float s, c;
    sincosf((float)pos[t] * inv_freq, &s, &c);
    if (inverse) s = -s;
    __nv_bfloat16* p = x + t * row_stride + (long long)h * Dh;
    const float a = __bfloat162float(p[d]), b = __bfloat162float(p[d + half]);
    p[d] = __float2bfloat16(a * c - b * s);
    p[d + half] = __float2bfloat16(b * c + a * s);
  }
}

static inline int ew_grid(long long work_items) {
  long long g = (work_items + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace mlf

using namespace mlf;

// dtype: 0 = fp32, 1 = bf16. b may be null (then `scalar` is the right-hand operand).
MLF_API int mlf_ew_binary(void* out, const void* a, const void* b, float scalar, long long n, int op, int dtype, uint64_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (n <= 0) return 0;
  if (dtype == 0) ew_binary_kernel<float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((float*)out, (const float*)a, (const float*)b, scalar, n, op);
  else ew_binary_kernel<__nv_bfloat16><<<ew_grid(n / 8 + 1), 256, 0, st>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, scalar, n, op);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_ew_unary(void* out, const void* a, long long n, int op, int dtype, uint64_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (n <= 0) return 0;
  if (dtype == 0) ew_unary_kernel<float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((float*)out, (const float*)a, n, op);
  else ew_unary_kernel<__nv_bfloat16><<<ew_grid(n / 8 + 1), 256, 0, st>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, n, op);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_fill(void* out, float value, long long n, int dtype, uint64_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (n <= 0) return 0;
  if (dtype == 0) fill_kernel<float><<<ew_grid(n / 4 + 1), 256, 0, st>>>((float*)out, value, n);
  else fill_kernel<__nv_bfloat16><<<ew_grid(n / 8 + 1), 256, 0, st>>>((__nv_bfloat16*)out, value, n);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
// red: 0 sum, 1 max, 2 min, 3 mean. scratch: fp32 [1024]. out: fp32 scalar on the device.
MLF_API int mlf_reduce_all(float* out, const void* a, long long n, int red, int dtype, float* scratch, uint64_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  MLF_REQUIRE(n > 0, "reduce over an empty tensor");
  const int grid = min(1024, ew_grid(n / 8 + 1));
  const int r = red == 3 ? 0 : red;
  if (dtype == 0) reduce_stage1_kernel<float><<<grid, 256, 0, st>>>((const float*)a, n, scratch, r);
  else reduce_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, n, scratch, r);
  count_launch();
  reduce_stage2_kernel<<<1, 32, 0, st>>>(scratch, grid, out, r, red == 3 ? 1.f / (float)n : 1.f);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_gelu_bwd(void* dx, const void* dy, const void* x, long long n, uint64_t stream) {
  MLF_REQUIRE(n % 8 == 0, "gelu_bwd: n must be a multiple of 8");
  gelu_bwd_kernel<<<ew_grid(n / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)dx, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, n);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_swiglu_fwd(void* out, const void* gu, long long rows, int F, int interleaved, uint64_t stream) {
  MLF_REQUIRE(F % 8 == 0, "swiglu: F must be a multiple of 8");
  swiglu_fwd_kernel<<<ew_grid(rows * F / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, rows, F, interleaved);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_swiglu_bwd(void* dgu, const void* dout, const void* gu, long long rows, int F, int interleaved, uint64_t stream) {
  MLF_REQUIRE(F % 8 == 0, "swiglu: F must be a multiple of 8");
  swiglu_bwd_kernel<<<ew_grid(rows * F / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)dgu, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, rows, F, interleaved);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
static void colsum_shape(int M, int N, int& col_ctas, int& row_ctas, int& rows_per_cta) {
  col_ctas = (N + CS_COLS - 1) / CS_COLS;
  row_ctas = (sm_count() * 6 + col_ctas - 1) / col_ctas;      // six CTAs fit per SM (40 registers): one full wave
  if (row_ctas > (M + 31) / 32) row_ctas = (M + 31) / 32;
  if (row_ctas < 1) row_ctas = 1;
  rows_per_cta = ((M + row_ctas - 1) / row_ctas + 31) / 32 * 32;
  row_ctas = (M + rows_per_cta - 1) / rows_per_cta;
}
// Scratch layout of mlf_colsum: ceil(N / 256) counters (uint32, zero before the first use; the kernel
// leaves them zero), padded to 256 bytes, then row_ctas x N floats of partial sums.
MLF_API long long mlf_colsum_scratch_bytes(int M, int N) {
  int c, r, rp;
  colsum_shape(M, N, c, r, rp);
  return (((long long)c * 4 + 255) / 256) * 256 + (long long)r * N * 4;
}
// db (bf16 [N]) = column sums of dy (+ db when accumulate). One launch; calls that share a scratch
// buffer must be ordered on one stream.
MLF_API int mlf_colsum(void* db, const void* dy, int M, int N, long long ld, void* scratch, int accumulate, uint64_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  MLF_REQUIRE(ld % 8 == 0, "colsum: pitch must be a multiple of 8 elements");
  MLF_REQUIRE(scratch != nullptr && M > 0 && N > 0, "colsum: bad arguments");
  int col_ctas, row_ctas, rows_per_cta;
  colsum_shape(M, N, col_ctas, row_ctas, rows_per_cta);
  unsigned int* counters = static_cast<unsigned int*>(scratch);
  float* part = reinterpret_cast<float*>(static_cast<char*>(scratch) + (((long long)col_ctas * 4 + 255) / 256) * 256);
  colsum_kernel<<<dim3(col_ctas, row_ctas), 256, 0, st>>>((__nv_bfloat16*)db, (const __nv_bfloat16*)dy, part, counters, M, N, ld,
                                                          rows_per_cta, accumulate);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_embedding_fwd(void* out, const long long* ids, const long long* pos, const void* wte, const void* wpe,
                              long long T, int D, int vocab, int max_pos, uint64_t stream) {
  MLF_REQUIRE(D % 8 == 0, "embedding: D must be a multiple of 8");
  embedding_fwd_kernel<<<ew_grid(T * (D / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (__nv_bfloat16*)out, ids, pos, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, T, D, vocab, max_pos, device_status_word());
      count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_embedding_bwd(float* dw, const void* dout, const long long* ids, long long T, int D, int vocab, uint64_t stream) {
  MLF_REQUIRE(D % 8 == 0, "embedding: D must be a multiple of 8");
  embedding_bwd_kernel<<<ew_grid(T * (D / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dw, (const __nv_bfloat16*)dout, ids, T, D, vocab);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_cast_f32_to_bf16(void* out, const float* in, long long n, int accumulate, uint64_t stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<ew_grid(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)out, in, n, accumulate);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_rope(void* x, const long long* pos, long long T, int H, int Dh, long long row_stride, float theta, int inverse, uint64_t stream) {
  MLF_REQUIRE(Dh % 2 == 0, "rope: head dim must be even");
  rope_kernel<<<ew_grid(T * H * (Dh / 2)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)x, pos, T, H, Dh, row_stride, theta, inverse);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
