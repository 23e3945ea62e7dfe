#include "host.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

namespace mlf {

static thread_local char g_err[1024] = {0};
static std::atomic<long long> g_launches{0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  (void)cudaGetLastError();   // a recoverable failure (e.g. out of memory) must not be reported again by the next launch check
  set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return -1;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Driver entry points need a context bound to the calling thread. Threads that have only ever
// received device pointers (autograd worker threads, for instance) may not have one yet; a
// cudaSetDevice on the thread's current device binds the primary context.
static void ensure_context() {
  static thread_local bool ready = false;
  if (ready) return;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    cudaSetDevice(dev);
    cudaFree(nullptr);
  }
  ready = true;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld, uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  ensure_context();
  EncodeTiledFn fn = get_encode_fn();
  MLF_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled entry point not available");
  MLF_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base %p not 16-byte aligned", base);
  MLF_REQUIRE((ld * elem_bytes) % 16 == 0, "TMA row pitch %llu bytes not a multiple of 16",
              (unsigned long long)(ld * elem_bytes));
  MLF_REQUIRE(box_inner <= 256 && box_outer <= 256, "TMA box too large");
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                              : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MLF_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d (inner=%llu outer=%llu ld=%llu box=%ux%u)",
              (int)r, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld,
              box_inner, box_outer);
  return 0;
}

static int* g_status[64] = {nullptr};
static int g_sms[64] = {0};
static std::mutex g_mu;

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    // offset 8: the wait budget in cycles read by the bounded waits (0 = the compiled default)
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sms[dev] = n > 0 ? n : 148;
  }
  return g_sms[dev];
}

}  // namespace mlf

MLF_API const char* mlf_last_error() { return mlf::g_err; }

// Reads and clears the device status word (synchronises the device). 0 = no kernel reported a
// timed-out wait or a rejected index since the last call.
MLF_API int mlf_read_status(int clear) {
  int* p = mlf::device_status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (clear && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

MLF_API int mlf_sm_count() { return mlf::sm_count(); }

// Cycle budget of every bounded device-side wait on the current device (mbarrier, chunk flag and
// peer flag waits). 0 restores the compiled default (~1.5 s). Takes effect for kernels launched
// after the call; synchronises the device.
MLF_API int mlf_set_wait_budget_cycles(long long cycles) {
  MLF_REQUIRE(cycles >= 0, "set_wait_budget_cycles: negative budget");
  int* p = mlf::device_status_word();
  MLF_REQUIRE(p != nullptr, "set_wait_budget_cycles: no status block");
  MLF_CHECK_CUDA(cudaDeviceSynchronize());
  MLF_CHECK_CUDA(cudaMemcpy(reinterpret_cast<char*>(p) + 8, &cycles, sizeof(cycles), cudaMemcpyHostToDevice));
  return 0;
}

// Kernels launched by this library in this process so far.
MLF_API long long mlf_launch_count() { return mlf::g_launches.load(std::memory_order_relaxed); }
