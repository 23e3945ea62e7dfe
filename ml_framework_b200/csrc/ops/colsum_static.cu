// Allocation-free column sum: see colsum_static.h for the contract.
#include "colsum_static.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../common/host.h"

namespace {

constexpr int kMaxCols = 65536;
constexpr int kMaxDevices = 64;

// Work buffer: fp32 partial sums meet here through atomics. One instance per device (each device
// that loads this module gets its own copy of a __device__ variable).
static __device__ __align__(256) float g_colsum_acc[kMaxCols];

float* g_acc_ptr[kMaxDevices] = {nullptr};
int g_sms[kMaxDevices] = {0};
std::mutex g_setup_mutex;

__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

// Each CTA owns 64 columns and a slab of rows: 8 threads x 8 columns wide, 32 row lanes deep.
__global__ void __launch_bounds__(256) colsum_static_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ acc,
                                                            int M, int N, long long ld, int rows_per_cta) {
  const int col0 = blockIdx.x * 64;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(M, r0 + rows_per_cta);
  const int cl = (threadIdx.x & 7) * 8;
  const int rl = threadIdx.x >> 3;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col0 + cl + 8 <= N) {
    for (int r = r0 + rl; r < r1; r += 32) {
      const uint4 u = *reinterpret_cast<const uint4*>(dy + (long long)r * ld + col0 + cl);
      const float2 a = bf16x2_to_f2(u.x), b = bf16x2_to_f2(u.y), c = bf16x2_to_f2(u.z), d = bf16x2_to_f2(u.w);
      s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
    }
  } else {
    for (int r = r0 + rl; r < r1; r += 32)
      for (int j = 0; j < 8; ++j)
        if (col0 + cl + j < N) s[j] += __bfloat162float(dy[(long long)r * ld + col0 + cl + j]);
  }
  __shared__ float sm[32][65];
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[rl][cl + j] = s[j];
  __syncthreads();
  if (threadIdx.x < 64) {
    float t = 0.f;
#pragma unroll 8
    for (int r = 0; r < 32; ++r) t += sm[r][threadIdx.x];
    if (col0 + threadIdx.x < N) atomicAdd(&acc[col0 + threadIdx.x], t);
  }
}

__global__ void colsum_static_finish_kernel(__nv_bfloat16* __restrict__ db, const float* __restrict__ acc, int N, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) db[i] = __float2bfloat16(acc[i] + (accumulate ? __bfloat162float(db[i]) : 0.f));
}

// Once per device, with that device current: the device address of the work buffer.
int setup_current_device(int* dev_out, float** ptr_out) {
  int dev = 0;
  MLF_CHECK_CUDA(cudaGetDevice(&dev));
  MLF_REQUIRE(dev >= 0 && dev < kMaxDevices, "colsum_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_acc_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_acc);
    if (e != cudaSuccess || ptr == nullptr) {
      mlf::set_error("colsum_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return -1;
    }
    int sms = 0;
    MLF_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_sms[dev] = sms > 0 ? sms : 1;
    g_acc_ptr[dev] = ptr;
  }
  *dev_out = dev;
  *ptr_out = g_acc_ptr[dev];
  return 0;
}

}  // namespace

MLF_API int mlf_colsum_static_max_cols(void) { return kMaxCols; }

MLF_API int mlf_colsum_static_setup(void) {
  int dev;
  float* acc;
  return setup_current_device(&dev, &acc);
}

MLF_API int mlf_colsum_static(void* db, const void* dy, int M, int N, long long ld, int accumulate, uint64_t stream) {
  MLF_REQUIRE(db != nullptr && dy != nullptr, "colsum_static: null pointer");
  MLF_REQUIRE(M > 0 && N > 0, "colsum_static: bad shape %d x %d", M, N);
  MLF_REQUIRE(N <= kMaxCols, "colsum_static: N = %d exceeds the built-in work buffer of %d columns; use mlf_colsum with a caller buffer",
              N, kMaxCols);
  MLF_REQUIRE(ld % 8 == 0 && ld >= N, "colsum_static: pitch %lld must be a multiple of 8 and at least N", ld);
  MLF_REQUIRE((reinterpret_cast<uintptr_t>(dy) & 15u) == 0, "colsum_static: dy must be 16-byte aligned");
  int dev;
  float* acc;
  const int rc = setup_current_device(&dev, &acc);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // The buffer keeps the previous call's sums: clear the part this call accumulates into.
  MLF_CHECK_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)N, st));
  const int col_ctas = (N + 63) / 64;
  int row_ctas = (g_sms[dev] * 4 + col_ctas - 1) / col_ctas;
  if (row_ctas > (M + 31) / 32) row_ctas = (M + 31) / 32;
  if (row_ctas < 1) row_ctas = 1;
  const int rows_per_cta = ((M + row_ctas - 1) / row_ctas + 31) / 32 * 32;
  row_ctas = (M + rows_per_cta - 1) / rows_per_cta;
  colsum_static_kernel<<<dim3(col_ctas, row_ctas), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), acc, M, N, ld, rows_per_cta);
  colsum_static_finish_kernel<<<(N + 255) / 256, 256, 0, st>>>(static_cast<__nv_bfloat16*>(db), acc, N, accumulate);
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
