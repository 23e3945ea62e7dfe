// Column sums of a bf16 matrix through a C entry point that allocates nothing.
//
// This entry point has no counterpart in the reference project. It exists for host programs that
// call the library's C symbols directly and have no device allocator to hand: a C or C++ service
// that links the shared object without PyTorch has no caching allocator, and one that sits in a
// latency-critical loop cannot afford cudaMalloc / cudaFree, which synchronise the whole device.
// mlf_colsum() makes its caller supply a work buffer (mlf_colsum_scratch_bytes); this variant keeps
// its work buffer inside the library instead.
//
// Contract
//   * db    bf16 [N]        out: db[n] = sum_m dy[m, n]   (added to the old db when accumulate != 0)
//   * dy    bf16 [M, N]     row pitch `ld` elements, ld a multiple of 8, base 16-byte aligned
//   * N <= mlf_colsum_static_max_cols() (65536). A larger N returns -2 and mlf_last_error() says so;
//     nothing is launched.
//   * The work buffer is one file-scope __device__ array per device (256 KB), shared by every call
//     on that device and keeping whatever the last call left in it. Each call clears the first N
//     floats on `stream` before it accumulates, so calls issued in order on one stream are
//     independent. Two calls that may overlap in time on the same device (different streams or
//     host threads without ordering between them) race on the buffer: serialise them.
//   * The first call on each device looks up the array's device address (once per device, with that
//     device current). That lookup is set-up work, not stream work: make the first call, or call
//     mlf_colsum_static_setup(), before any stream capture begins on that device.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
#pragma once
#include <cstdint>

#ifdef __cplusplus
extern "C" {
#endif
int mlf_colsum_static_max_cols(void);
int mlf_colsum_static_setup(void);
int mlf_colsum_static(void* db, const void* dy, int M, int N, long long ld, int accumulate, uint64_t stream);
#ifdef __cplusplus
}
#endif
