// Host-side helpers shared by the kernel launchers: TMA tensor-map construction (through the
// driver entry point, so the library needs no link-time dependency on libcuda), a per-device
// status word that kernels write when a bounded wait expires, and error reporting for the
// C ABI (every exported function returns 0 on success, a negative code on failure, and
// leaves a message readable through mlf_last_error()).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MLF_API extern "C" __attribute__((visibility("default")))

namespace mlf {

void set_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

// 2-D bf16/fp32 tensor map. `inner` is the contiguous extent (elements), `outer` the number of
// rows, `ld` the row pitch in elements. box_* is the tile copied by one TMA instruction.
// swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (box_inner * elemsize must then be 128 bytes).
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld, uint32_t box_inner, uint32_t box_outer, bool swizzle128);

// Device status word for the current device (allocated once per device, zero-initialised).
int* device_status_word();

int sm_count();

// Number of kernels launched by this library since load (incremented by the launchers).
void count_launch(int n = 1);

}  // namespace mlf

#define MLF_CHECK_CUDA(expr)                                  \
  do {                                                        \
    int _rc = ::mlf::check_cuda((expr), #expr);               \
    if (_rc) return _rc;                                      \
  } while (0)

#define MLF_REQUIRE(cond, ...)       \
  do {                               \
    if (!(cond)) {                   \
      ::mlf::set_error(__VA_ARGS__); \
      return -2;                     \
    }                                \
  } while (0)
